"""Host-side sharding of the attention path over the GPUs of one box.

Two ways the path shards (one process per GPU, torch.distributed for the plumbing):

* lane-parallel -- whole request lanes are assigned to GPUs and each GPU runs the ordinary
  batched decode; there is no data-path collective.  Because the split-KV partition function
  depends only on a lane's own context, every lane's output is bit-identical to its solo run on
  any GPU.
* split-KV -- one long lane's keys are cut into contiguous ranges, one per GPU; each GPU reduces
  its range to one 258-float record per head ([numerator | max | sum], the reference's partition
  record, src/backend/metal/kernels/attention.metal:1086-1108), the records are all-gathered
  (16 x 258 x 4 = 16512 bytes per rank) and every rank runs the same log-sum-exp combine.
"""
from __future__ import annotations

from typing import Callable, List, Sequence, Tuple

from . import split_buffer_bytes as tb_split_buffer_bytes

RECORD_FLOATS = 258
Q_HEADS = 16


def assign_lanes(contexts: Sequence[int], world: int) -> List[List[int]]:
    """Greedy longest-first assignment of whole lanes to `world` GPUs.

    Returns, per rank, the lane indices it owns (in assignment order).  Deterministic: ties go
    to the lower lane index and the lower rank."""
    if world <= 0:
        raise ValueError("world must be positive")
    loads = [0] * world
    owned: List[List[int]] = [[] for _ in range(world)]
    for lane in sorted(range(len(contexts)), key=lambda i: (-contexts[i], i)):
        rank = loads.index(min(loads))
        loads[rank] += contexts[lane]
        owned[rank].append(lane)
    return owned


def split_kv_ranges(n_keys: int, world: int) -> List[Tuple[int, int]]:
    """Contiguous key ranges [begin, end) per rank, 16-key aligned except the last end."""
    if n_keys <= 0 or world <= 0:
        raise ValueError("n_keys and world must be positive")
    per = -(-n_keys // world)
    per = (per + 15) // 16 * 16
    ranges = []
    for r in range(world):
        begin = min(r * per, n_keys)
        ranges.append((begin, min(begin + per, n_keys)))
    return ranges


def split_kv_decode(dist, world: int, partial: Callable[[], "object"], gathered, combine: Callable[[object], None]):
    """One split-KV decode step on this rank: local partial records -> all-gather -> combine.

    `partial()` returns this rank's record tensor [16][258] f32 (a rank whose range is empty
    returns max = -inf, sum = 0 records, which the combine weighs with 0); `gathered` is the
    [world][16][258] receive buffer; `combine(gathered)` merges in rank order."""
    rec = partial()
    if world > 1:
        dist.all_gather_into_tensor(gathered.view(-1), rec.reshape(-1))
    else:
        gathered.view(-1).copy_(rec.reshape(-1))
    combine(gathered)
    return gathered


class PeerExchange:
    """Peer buffers of the collective-free split-KV merge: per rank one buffer holding
    [2 parities][world][16][258] f32 records followed by [2][world] u32 flags and the device step
    counter (tatara_split_buffer_bytes), mapped into every process through CUDA IPC (handles
    exchanged once with all_gather_object).  Use EITHER step() (host-numbered epochs, two calls per
    step) OR tatara_attn_decode_split with pointer_array (device-numbered steps, one call) on one
    exchange: both write the same flags."""

    RECORD_BYTES = Q_HEADS * RECORD_FLOATS * 4

    def __init__(self, ctx, dist, rank: int, world: int):
        self.ctx, self.rank, self.world = ctx, rank, world
        self.gather_bytes = world * self.RECORD_BYTES
        self.flags_offset = 2 * self.gather_bytes
        nbytes = tb_split_buffer_bytes(world)                # ... then the device step counter
        self.own_ptr, handle = ctx.peer_buffer_create(nbytes)
        handles = [None] * world
        if world > 1:
            dist.all_gather_object(handles, handle)
        else:
            handles[0] = handle
        self.ptrs = [self.own_ptr if r == rank else ctx.peer_buffer_open(handles[r]) for r in range(world)]
        self.pointer_array = ctx.pointer_array(self.ptrs)     # argument of tatara_attn_decode_split
        self.epoch = 0

    def step(self, push, combine_wait):
        """push(peer_gather, peer_flags, epoch) then combine_wait(gather_ptr, flags_ptr, epoch)."""
        self.epoch += 1
        parity = self.epoch & 1
        gathers = [p + parity * self.gather_bytes for p in self.ptrs]
        flags = [p + self.flags_offset + parity * self.world * 4 for p in self.ptrs]
        push(gathers, flags, self.epoch)
        combine_wait(gathers[self.rank], flags[self.rank], self.epoch)

    def close(self, dist=None, sync=None):
        """Releases the mappings in three phases: (1) after `sync()` has drained this rank's stream (no
        kernel of this rank still stores into a peer's buffer) every rank closes the mappings it
        imported; (2) all ranks meet at a barrier; (3) each rank frees the buffer it exported.
        Freeing an exported buffer while another process still has it mapped is undefined."""
        if sync is not None:
            sync()
        for r, p in enumerate(self.ptrs):
            if r != self.rank:
                self.ctx.peer_buffer_close(p, owned=False)
        if dist is not None and self.world > 1:
            dist.barrier()
        if self.ptrs:
            self.ctx.peer_buffer_close(self.ptrs[self.rank], owned=True)
        self.ptrs = []

"""Synthetic workloads of bench.py (shapes and distributions of the benchmark configs).

Device tensors are created with torch (memory + streams only); every timed operation is a call
into libtatara_b200.so through the C ABI.
"""
from __future__ import annotations

import json
import os

import numpy as np

import tatara_b200 as tb
from tatara_b200 import sharding

ROOT = os.path.dirname(os.path.abspath(__file__))


WAVE_BENCH_SRC = os.path.join(ROOT, "bench_wave_loop.cpp")
WAVE_BENCH_EXE = os.path.join(ROOT, "bench_wave_loop")


def build_wave_loop_bench():
    """Compiles bench_wave_loop.cpp (the timing program of the owner's wave loop: plain C++ above the
    C ABI and the header-only host layer) next to bench.py; a no-op when it is up to date."""
    import subprocess
    pkg = os.path.dirname(os.path.abspath(tb.__file__))
    host = os.path.join(pkg, "host")
    deps = [WAVE_BENCH_SRC, tb.LIB_PATH] + [os.path.join(host, f) for f in os.listdir(host) if f.endswith(".hpp")]
    if os.path.exists(WAVE_BENCH_EXE) and all(os.path.getmtime(d) <= os.path.getmtime(WAVE_BENCH_EXE) for d in deps):
        return WAVE_BENCH_EXE
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cuda = os.path.dirname(os.path.dirname(nvcc))
    cmd = ["g++", "-std=c++17", "-O2", "-pthread", "-o", WAVE_BENCH_EXE, WAVE_BENCH_SRC, f"-I{cuda}/include", f"-I{ROOT}",
           f"-L{pkg}", "-ltatara_b200", f"-L{cuda}/lib64", "-lcudart", f"-Wl,-rpath,{pkg}", f"-Wl,-rpath,{cuda}/lib64"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"g++ failed for bench_wave_loop:\n{res.stdout}\n{res.stderr}")
    return WAVE_BENCH_EXE


def measured_peaks():
    """Roofline denominators: the driver-measured peaks of this pool, else the stated fallback."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def decode_bytes(n_keys: int) -> int:
    """Algorithmic bytes of one decode-attention step: K+V rows of n keys + q, gate, out."""
    return n_keys * 2048 + 3 * 8192


def prefill_flops(rows: int, base: int = 0) -> float:
    """Causal QK^T + PV flops: 4 * 256 * 16 heads * visible (row, key) pairs."""
    pairs = rows * base + rows * (rows + 1) // 2
    return 4.0 * 256 * 16 * pairs


def _rope_rows(torch, x, positions):
    """Rotate dims 0..63 of x [n, heads, 256] (f32) at `positions` (theta base 1e7)."""
    div = torch.pow(torch.tensor(1.0e7, dtype=torch.float64, device=x.device),
                    torch.arange(32, dtype=torch.float64, device=x.device) / 32).float()
    theta = positions.float()[:, None] / div[None, :]
    c, s = torch.cos(theta)[:, None, :], torch.sin(theta)[:, None, :]
    lo, hi = x[..., :32].clone(), x[..., 32:64].clone()
    x[..., :32] = lo * c - hi * s
    x[..., 32:64] = hi * c + lo * s
    return x


def device_cache(torch, n_keys, capacity, seed):
    """K, V planes [2][capacity][256] bf16: unit-RMS rotated keys, N(0,1) values."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    keys = torch.zeros((2, capacity, 256), dtype=torch.bfloat16, device="cuda")
    values = torch.zeros((2, capacity, 256), dtype=torch.bfloat16, device="cuda")
    chunk = 32768
    for start in range(0, n_keys, chunk):
        stop = min(start + chunk, n_keys)
        x = torch.randn((stop - start, 2, 256), generator=g, device="cuda")
        x = x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-6)
        x = _rope_rows(torch, x.to(torch.bfloat16).float(), torch.arange(start, stop, device="cuda"))
        keys[:, start:stop] = x.to(torch.bfloat16).transpose(0, 1)
        values[:, start:stop] = torch.randn((2, stop - start, 256), generator=g, device="cuda").to(torch.bfloat16)
    return keys, values


def device_query(torch, positions, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    pos = torch.as_tensor(positions, device="cuda")
    x = torch.randn((len(positions), 16, 256), generator=g, device="cuda")
    x = x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-6)
    q = _rope_rows(torch, x.to(torch.bfloat16).float(), pos).to(torch.bfloat16)
    gate = torch.randn((len(positions), 16, 256), generator=g, device="cuda").to(torch.bfloat16)
    return q, gate


L2_BYTES = 126 * 1000 * 1000


def replicas_for(bytes_per_step: int) -> int:
    """Distinct input sets to rotate through so that consecutive timed steps never find their
    inputs in the 126 MB L2 (a step streaming more than twice the L2 needs only one)."""
    if bytes_per_step >= 2 * L2_BYTES:
        return 1
    return -(-2 * L2_BYTES // bytes_per_step) + 1


class DecodeCase:
    """One lane at `n_keys` attended keys; `replicas` independent caches are rotated step to step."""

    def __init__(self, ctx, torch, n_keys, seed=0, replicas=None):
        self.ctx, self.torch, self.n = ctx, torch, n_keys
        self.capacity = n_keys
        self.replicas = replicas_for(n_keys * 2048) if replicas is None else replicas
        self.caches = []
        for r in range(self.replicas):
            if r == 0:
                self.caches.append(device_cache(torch, n_keys, n_keys, seed))
            else:   # same distribution; a permuted copy is enough to defeat the cache
                k0, v0 = self.caches[0]
                self.caches.append((k0.roll(r * 17, dims=1).contiguous(), v0.roll(r * 17, dims=1).contiguous()))
        q, gate = device_query(torch, [n_keys - 1], seed + 1)
        self.q, self.gate = q[0].contiguous(), gate[0].contiguous()
        self.out = torch.zeros((16, 256), dtype=torch.bfloat16, device="cuda")
        self.scratch = torch.empty(tb.decode_scratch_bytes(n_keys, 1) // 4, dtype=torch.float32, device="cuda")
        # end-to-end leg: the token's projection row lives in pinned host memory
        g = torch.Generator().manual_seed(seed + 2)
        self.h_proj = torch.randn((1, 9216), generator=g).to(torch.bfloat16).pin_memory()
        self.d_proj = torch.zeros((1, 9216), dtype=torch.bfloat16, device="cuda")
        self.h_out = torch.zeros((16, 256), dtype=torch.bfloat16).pin_memory()
        self.q2 = torch.zeros((1, 16, 256), dtype=torch.bfloat16, device="cuda")
        self.g2 = torch.zeros_like(self.q2)
        self.ones = torch.ones(256, dtype=torch.bfloat16, device="cuda")

    def step(self, i=0):
        keys, values = self.caches[i % self.replicas]
        self.ctx.attn_decode(self.q, self.gate, keys, values, self.n - 1, self.capacity, self.out, self.scratch)

    def step_e2e(self, i=0):
        keys, values = self.caches[i % self.replicas]
        self.d_proj.copy_(self.h_proj, non_blocking=True)
        self.ctx.attn_qk_rope(self.d_proj, self.ones, self.ones, self.q2, self.g2, keys, values,
                              self.n - 1, self.capacity, 1)
        self.ctx.attn_decode(self.q2, self.g2, keys, values, self.n - 1, self.capacity, self.out, self.scratch)
        self.h_out.copy_(self.out, non_blocking=True)

    def step_e2e_mapped(self, i=0):
        """step_e2e without the two copy nodes: qk_rope loads the projection row from the pinned host buffer and
        the merge kernel stores the attended row into the pinned host buffer (pinned memory is device-visible)."""
        keys, values = self.caches[i % self.replicas]
        self.ctx.attn_qk_rope(self.h_proj, self.ones, self.ones, self.q2, self.g2, keys, values,
                              self.n - 1, self.capacity, 1)
        self.ctx.attn_decode(self.q2, self.g2, keys, values, self.n - 1, self.capacity, self.h_out, self.scratch)

    def token_graph(self, mapped_host=False):
        """One decode token end to end as ONE CUDA graph: pinned H2D of the projection row, qk_rope and decode
        attention through the device-table entry points (nothing about the token is a kernel argument), D2H of the
        attended row.  Returns a callable that replays it (one graph launch per token, as an engine would).
        mapped_host=True drops the two copy nodes: qk_rope loads the projection row straight from the pinned
        host buffer and the combine kernel stores the attended row straight into the pinned host buffer (pinned
        memory is mapped into the device's address space), so the host<->device transfers ride inside the two
        kernels instead of waiting on the copy engine."""
        torch = self.torch
        keys, values = self.caches[0]
        table = tb.Context.device_lanes(tb.Context.attn_lanes([(0, self.n - 1)]))
        stream = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()

        def body():
            if mapped_host:
                proj, out = self.h_proj, self.h_out
            else:
                proj, out = self.d_proj, self.out
                self.d_proj.copy_(self.h_proj, non_blocking=True)
            self.ctx.attn_qk_rope_batch_indirect(proj, self.ones, self.ones, self.q2, self.g2, keys, values,
                                                 self.capacity, table, 1)
            self.ctx.attn_decode_batch_indirect(self.q2, self.g2, keys, values, table, 1, self.capacity, out,
                                                self.scratch)
            if not mapped_host:
                self.h_out.copy_(self.out, non_blocking=True)

        with torch.cuda.stream(stream):
            body()
            stream.synchronize()
            with torch.cuda.graph(graph, stream=stream):
                body()
        torch.cuda.synchronize()
        self._graph_keepalive = getattr(self, '_graph_keepalive', []) + [(graph, table, stream)]
        return lambda i=0: graph.replay()

    def free(self):
        del self.caches, self.scratch
        self.torch.cuda.empty_cache()


class SplitCase:
    """Config 4a: ONE lane of `n_keys` keys, its key axis cut into contiguous ranges, one per rank.

    Every rank draws the whole lane from the same seed (so that each can also run the unsplit decode
    as the check) and attends only its own range [begin, end) of it; the records cross NVLink.  Two
    forms of the step: `step` = tatara_attn_decode_split (one submission: partitions, merge + peer
    stores + flag, bounded wait + merge in rank order; replayable as a graph), and `step_nccl` =
    partial records -> all_gather -> combine (the library-collective form)."""

    def __init__(self, ctx, torch, dist, n_keys, rank, world):
        self.ctx, self.torch, self.dist, self.n, self.rank, self.world = ctx, torch, dist, n_keys, rank, world
        self.begin, self.end = sharding.split_kv_ranges(n_keys, world)[rank]
        self.keys, self.values = device_cache(torch, n_keys, n_keys, 31)
        q, gate = device_query(torch, [n_keys - 1], 32)
        self.q, self.gate = q[0].contiguous(), gate[0].contiguous()
        self.out = torch.zeros((16, 256), dtype=torch.bfloat16, device="cuda")
        self.out_nccl = torch.zeros_like(self.out)
        self.rec = torch.zeros((16, 258), device="cuda")
        self.allrec = torch.zeros((world, 16, 258), device="cuda")
        self.scratch = torch.empty(tb.decode_scratch_bytes(n_keys, 1) // 4, dtype=torch.float32, device="cuda")
        self.px = sharding.PeerExchange(ctx, dist, rank, world)
        g = torch.Generator().manual_seed(33)
        self.h_proj = torch.randn((1, 9216), generator=g).to(torch.bfloat16).pin_memory()
        self.d_proj = torch.zeros((1, 9216), dtype=torch.bfloat16, device="cuda")
        self.h_out = torch.zeros((16, 256), dtype=torch.bfloat16).pin_memory()
        self.q2 = torch.zeros((1, 16, 256), dtype=torch.bfloat16, device="cuda")
        self.g2 = torch.zeros_like(self.q2)
        self.ones = torch.ones(256, dtype=torch.bfloat16, device="cuda")

    def step(self, i=0):
        self.ctx.attn_decode_split(self.q, self.gate, self.keys, self.values, self.begin, self.end, self.n,
                                   self.px.pointer_array, self.rank, self.out, self.scratch)

    def step_kernel_only(self, i=0):
        self.ctx.attn_decode_partial(self.q, self.keys, self.values, self.begin, self.end, self.n, self.rec, self.scratch)

    def step_nccl(self, i=0):
        self.ctx.attn_decode_partial(self.q, self.keys, self.values, self.begin, self.end, self.n, self.rec, self.scratch)
        self.dist.all_gather_into_tensor(self.allrec.view(-1), self.rec.view(-1))
        # all-gather layout [rank][head][258]: head stride 258, part stride 16*258
        self.ctx.attn_combine(self.allrec, self.world, 258, 16 * 258, self.gate, self.out_nccl)

    def step_collective_only(self, i=0):
        self.dist.all_gather_into_tensor(self.allrec.view(-1), self.rec.view(-1))

    def step_e2e(self, i=0):
        """The step from host buffers: pinned H2D of the token's projection row, qk_rope at the lane's
        last position (the rank that owns that position attends the row it appends), the split step,
        D2H of the attended row -- on every rank."""
        self.d_proj.copy_(self.h_proj, non_blocking=True)
        self.ctx.attn_qk_rope(self.d_proj, self.ones, self.ones, self.q2, self.g2, self.keys, self.values,
                              self.n - 1, self.n, 1)
        self.ctx.attn_decode_split(self.q2, self.g2, self.keys, self.values, self.begin, self.end, self.n,
                                   self.px.pointer_array, self.rank, self.out, self.scratch)
        self.h_out.copy_(self.out, non_blocking=True)

    def check(self):
        """Split results against the unsplit decode of the same lane on this GPU (tolerance of the
        parity tests: max-abs 2e-2, cosine 0.9999), peer form against NCCL form (same records, same
        rank-order merge: equal bits); worst case over the ranks."""
        torch, dist = self.torch, self.dist
        unsplit = torch.zeros_like(self.out)
        self.out.zero_()
        self.out_nccl.zero_()
        self.step()
        self.step_nccl()
        self.ctx.attn_decode(self.q, self.gate, self.keys, self.values, self.n - 1, self.n, unsplit, self.scratch)
        self.ctx.sync()     # raises if a bounded wait ran out

        def distance(a, b):
            a, b = a.float().flatten(), b.float().flatten()
            cos = torch.dot(a, b) / (a.norm() * b.norm()).clamp_min(1e-30)
            return float((a - b).abs().max()), float(cos)

        pe, pc = distance(self.out, unsplit)
        ne, nc = distance(self.out_nccl, unsplit)
        t = torch.tensor([pe, ne, -pc, -nc, 0.0 if torch.equal(self.out, self.out_nccl) else 1.0], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        pe, ne, pc, nc, differ = (float(x) for x in t)
        return {"peer_max_abs": pe, "peer_cosine": -pc, "nccl_max_abs": ne, "nccl_cosine": -nc,
                "matches_unsplit": bool(pe <= 2e-2 and -pc >= 0.9999 and ne <= 2e-2 and -nc >= 0.9999),
                "peer_equals_nccl_bits": differ == 0.0,
                "checked": "every rank: split out vs tatara_attn_decode of the whole lane; worst over ranks"}

    def close(self):
        self.px.close(self.dist, sync=self.ctx.sync)


class Workloads:
    def __init__(self, ctx, torch, rank=0, world=1):
        self.ctx, self.torch, self.rank, self.world = ctx, torch, rank, world
        self._flush = None

    def traffic_hint(self):
        """DRAM bytes (read + write) per launch of attn_decode_partition_kernel at the headline
        context, from an ncu capture at 65 536 keys (134.280448 MB read + 4.332800 MB written),
        scaled by keys (traffic is proportional to keys) to 262 144."""
        return int((134.280448e6 + 4.332800e6) * 4)

    def decode_setup(self, n_keys):
        return DecodeCase(self.ctx, self.torch, n_keys, seed=self.rank * 100)

    # ---- config 4b: 32 independent lanes, contexts uniform in [4096, 32768]
    def lanes32(self, timed, steps, warmup):
        torch = self.torch
        rng = np.random.default_rng(0)
        contexts = [int(c) for c in rng.integers(4096, 32769, size=32)]
        owned = sharding.assign_lanes(contexts, self.world)      # greedy longest-first, whole lanes
        mine = owned[self.rank]
        loads = [sum(contexts[l] for l in r) for r in owned]
        cap = 32768
        n = len(mine)
        kpool = torch.randn((n, 2, cap, 256), device="cuda", dtype=torch.float32).to(torch.bfloat16) if n else None
        vpool = torch.randn((n, 2, cap, 256), device="cuda", dtype=torch.float32).to(torch.bfloat16) if n else None
        q, gate = device_query(torch, [contexts[i] - 1 for i in mine], 7)
        out = torch.zeros((n, 16, 256), dtype=torch.bfloat16, device="cuda")
        scratch = torch.empty(tb.decode_scratch_bytes(cap, n) // 4, dtype=torch.float32, device="cuda")
        lanes = tb.Context.attn_lanes([(i * 2 * cap * 256, contexts[lane] - 1) for i, lane in enumerate(mine)])

        def step(i=0):
            self.ctx.attn_decode_batch(q, gate, kpool, vpool, lanes, cap, out, scratch)

        ms = timed(step, steps, warmup)
        total_bytes = sum(c * 2048 + 3 * 8192 for c in contexts)
        res = {"lanes": 32, "contexts": "uniform[4096,32768] seed 0", "ms": ms, "lanes_per_s": 32 / (ms * 1e-3),
               "gbs": total_bytes / (ms * 1e-3) / 1e9, "total_kv_bytes": total_bytes,
               "max_rank_keys": max(loads)}
        # bit-identity: EVERY local lane alone gives the bits it got inside the batch
        if n:
            step()
            self.ctx.sync()
            batched = out.clone()
            solo = torch.zeros((16, 256), dtype=torch.bfloat16, device="cuda")
            solo_scratch = torch.empty(tb.decode_scratch_bytes(cap, 1) // 4, dtype=torch.float32, device="cuda")
            same = 0
            for i in range(n):
                solo.zero_()
                self.ctx.attn_decode(q[i], gate[i], kpool[i], vpool[i], contexts[mine[i]] - 1, cap, solo, solo_scratch)
                self.ctx.sync()
                same += int(torch.equal(solo, batched[i]))
            res["lanes_checked_alone_vs_batched"] = n
            res["lane_bits_identical_alone_vs_batched"] = bool(same == n)
        del kpool, vpool
        torch.cuda.empty_cache()
        return res

    # ---- config 1: GDN decode step, 4 lanes
    def gdn_step(self, timed, steps, warmup, n=4):
        torch = self.torch
        g = torch.Generator(device="cuda").manual_seed(11)
        bf = torch.bfloat16
        nbytes = n * (2 * 2097152 + 2 * 49152 + 24704 + 8192) + 65536
        reps = replicas_for(nbytes)
        proj = torch.randn((n, 12352), generator=g, device="cuda").to(bf)
        conv_w = (0.5 * torch.randn((8192, 4), generator=g, device="cuda")).to(bf)
        a_log = torch.log(1 + 15 * torch.rand(32, generator=g, device="cuda")).to(bf)
        dt_bias = (0.5 * torch.randn(32, generator=g, device="cuda")).to(bf)
        norm_w = torch.ones(128, device="cuda").to(bf)
        conv_pool = torch.randn((reps, n, 2, 3, 8192), generator=g, device="cuda").to(bf)
        rec_pool = 0.02 * torch.randn((reps, n, 2, 32, 128, 128), generator=g, device="cuda")
        y = torch.zeros((n, 4096), dtype=bf, device="cuda")
        gated = torch.zeros_like(y)
        cs, rs = 3 * 8192, 32 * 128 * 128
        tables = [tb.Context.gdn_lanes([((2 * i + a) * cs, (2 * i + b) * cs, (2 * i + a) * rs, (2 * i + b) * rs)
                                        for i in range(n)]) for a, b in ((0, 1), (1, 0))]

        def step(i=0):
            r = i % reps
            self.ctx.gdn_decode_batch(proj, conv_w, a_log, dt_bias, norm_w, conv_pool[r], rec_pool[r],
                                      tables[(i // reps) & 1], y, gated)

        ms = timed(step, max(steps, 2 * reps), max(warmup, reps))
        # the per-lane register data path on the same inputs (TATARA_POLICY_GDN_DECODE_FORM = 1), for comparison
        self.ctx.set_policy(tb.POLICY_GDN_DECODE_FORM, 1)
        try:
            ms_regs = timed(step, max(steps, 2 * reps), max(warmup, reps))
        finally:
            self.ctx.set_policy(tb.POLICY_GDN_DECODE_FORM, 0)
        # the step letting its successor be staged early (TATARA_POLICY_GDN_STEP_EARLY_DEPENDENTS = 1: the caller
        # promises that the next kernels do not read this call's state before their own dependency wait; true
        # here, every step works on another state set, and in a layer walk; the owner's wave loop sets it)
        self.ctx.set_policy(tb.POLICY_GDN_STEP_EARLY_DEPENDENTS, 1)
        try:
            ms_early = timed(step, max(steps, 2 * reps), max(warmup, reps))
        finally:
            self.ctx.set_policy(tb.POLICY_GDN_STEP_EARLY_DEPENDENTS, 0)
        return {"lanes": n, "us": ms * 1e3, "bytes": nbytes, "gbs": nbytes / (ms * 1e-3) / 1e9,
                "early_dependents_us": ms_early * 1e3, "register_form_us": ms_regs * 1e3,
                "l2": f"{reps} rotating state sets (> 2x L2)",
                "kernel": "gdn_decode_fused_kernel<bulk copies> (1 launch per step)"}

    # ---- config 3: GDN prefill, 16384 rows
    def gdn_prefill(self, timed, rows=16384):
        torch = self.torch
        g = torch.Generator(device="cuda").manual_seed(12)
        bf = torch.bfloat16
        x = torch.randn((rows, 32, 128), generator=g, device="cuda")
        x = x / x.norm(dim=-1, keepdim=True)
        qk = torch.cat([(x[:, :16] / 128 ** 0.5).reshape(rows, 2048), x[:, 16:].reshape(rows, 2048)], 1).to(bf).contiguous()
        v = torch.randn((rows, 4096), generator=g, device="cuda").to(bf)
        a = torch.randn((rows, 32), generator=g, device="cuda")
        a_log = torch.log(1 + 15 * torch.rand(32, generator=g, device="cuda"))
        decay = torch.exp(-torch.exp(a_log)[None, :] * torch.nn.functional.softplus(a)).contiguous()
        beta = torch.sigmoid(torch.randn((rows, 32), generator=g, device="cuda")).contiguous()
        s0 = torch.zeros((32, 128, 128), device="cuda")
        s1 = torch.zeros_like(s0)
        y = torch.zeros((rows, 4096), dtype=bf, device="cuda")
        out = {}
        scratch = torch.empty(tb.gdn_prefill_scratch_bytes(rows), dtype=torch.uint8, device="cuda")
        for chunk, form, name in ((64, 0, "chunk64"), (64, 2, "chunk64_two_launches"), (64, 1, "chunk64_register_form"),
                                  (1, 0, "sequential_scan")):
            try:
                self.ctx.set_policy(tb.POLICY_GDN_CHUNK_FORM, form)
                ms = timed(lambda i=0: self.ctx.gdn_prefill(qk, v, decay, beta, s0, y, s1, rows, chunk, scratch), 5, 3)
                out[name] = {"ms": ms, "tokens_per_s": rows / (ms * 1e-3),
                             "tflops_chunked_form": 94.5e9 * rows / 16384 / (ms * 1e-3) / 1e12,
                             "gbs_algorithmic": (rows * 24704 + 2097152 + 65536) / (ms * 1e-3) / 1e9}
            except tb.TataraError as e:
                out[name] = {"unavailable": str(e)}
        self.ctx.set_policy(tb.POLICY_GDN_CHUNK_FORM, 0)
        out["rows"] = rows
        out["forms"] = ("chunk64: tcgen05 MMAs, state in tensor memory (transition form), one launch in which the scan of "
                        "early chunks runs beside the preparation of later ones; chunk64_two_launches: the same kernels one "
                        "after the other; chunk64_register_form: mma.sync, state in registers; same inputs, same scratch")
        return out

    # ---- config 2: causal prefill attention, 16384 rows from position 0
    def prefill(self, timed, peaks, rows=16384, steps=5, sampler=None):
        torch = self.torch
        try:
            keys, values = device_cache(torch, rows, rows, 21)
            q, gate = device_query(torch, list(range(rows)), 22)
            out = torch.zeros((rows, 16, 256), dtype=torch.bfloat16, device="cuda")
            clocks = None
            if sampler is not None:
                with sampler as cs:
                    ms = timed(lambda i=0: self.ctx.attn_prefill(q, gate, keys, values, 0, rows, rows, out), steps, 3,
                               hold_s=1.0)
                clocks = cs.summary()
            else:
                ms = timed(lambda i=0: self.ctx.attn_prefill(q, gate, keys, values, 0, rows, rows, out), steps, 3)
            # the one-CTA kernel on the same inputs (TATARA_POLICY_ATTN_PREFILL_FORM = 1), timed the same way
            # (after the same hold of its own graph when the clocks are being sampled: under the power cap
            # the SM clock settles some 20 % below a short burst's)
            self.ctx.set_policy(tb.POLICY_ATTN_PREFILL_FORM, 1)
            try:
                if sampler is not None:
                    ms_single = timed(lambda i=0: self.ctx.attn_prefill(q, gate, keys, values, 0, rows, rows, out), steps, 3,
                                      hold_s=1.0)
                else:
                    ms_single = timed(lambda i=0: self.ctx.attn_prefill(q, gate, keys, values, 0, rows, rows, out), steps, 3)
            finally:
                self.ctx.set_policy(tb.POLICY_ATTN_PREFILL_FORM, 0)
        except tb.TataraError as e:
            return {"unavailable": str(e)}
        tf = prefill_flops(rows) / (ms * 1e-3) / 1e12
        return {"rows": rows, "ms": ms, "tflops": tf, "clocks": clocks, "frac_of_measured_bf16_burst": tf / peaks["bf16_tflops"],
                "frac_of_measured_bf16_sustained": tf / peaks["bf16_tflops_sustained"],
                "kernel": "attn_prefill_pair_kernel (CTA pairs, cta_group::2)",
                "single_cta_form": {"ms": ms_single, "tflops": prefill_flops(rows) / (ms_single * 1e-3) / 1e12},
                "l2": "Q/gate/out 402 MB > L2"}

    # ---- the projections on either side of the layers (affine Q4, group 64)
    def project(self, timed, peaks, steps, warmup, rows=16384):
        """Exact-row policy at decode sizes (1, 4, 8, 16 rows; bound by the Q4 weight stream, then by FMA rate)
        and tensor-unit policy at the prefill size, for the three call sites of the model."""
        torch = self.torch
        g = torch.Generator(device="cuda").manual_seed(13)
        bf = torch.bfloat16
        sites = {"attn_project": ((8192, 512, 512), 2048), "gdn_project": ((8192, 4096, 32, 32), 2048),
                 "out_projection": ((2048,), 4096)}
        out = {}
        for name, (sizes, k) in sites.items():
            n = sum(sizes)
            wbytes = n * k // 2 + 2 * n * (k // 64) * 2
            reps = replicas_for(wbytes)
            sets = []
            for _ in range(reps):
                held = [(torch.randint(-2 ** 31, 2 ** 31 - 1, (m, k // 8), generator=g, device="cuda", dtype=torch.int32),
                         (0.35 * 0.32 / k ** 0.5 * (1 + 0.2 * (2 * torch.rand((m, k // 64), generator=g, device="cuda") - 1))).to(bf),
                         (-0.35 * 2.4 / k ** 0.5 * (1 + 0.1 * torch.randn((m, k // 64), generator=g, device="cuda"))).to(bf))
                        for m in sizes]
                sets.append((held, tb.Context.q4_matrices(held)))
            res = {"n": n, "k": k, "q4_weight_bytes": wbytes}
            for r in (1, 4, 8, 16):
                x = torch.randn((r, k), generator=g, device="cuda").to(bf)
                y = torch.zeros((r, n), dtype=bf, device="cuda")
                ms = timed(lambda i=0: self.ctx.q4_project(x, sets[i % reps][1], k, y), max(steps, 2 * reps), max(warmup, reps))
                res[f"exact_rows{r}"] = {"us": ms * 1e3, "weight_gbs": wbytes / (ms * 1e-3) / 1e9,
                                         "gflops": 2.0 * r * n * k / (ms * 1e-3) / 1e9}
            # tensor-unit policy: dequantise once (load-time step, timed separately), then the GEMM
            w = torch.zeros((n, k), dtype=bf, device="cuda")
            ms = timed(lambda i=0: self.ctx.q4_dequantize(sets[0][1], k, w), 5, 3)
            res["dequantize_us"] = ms * 1e3
            x = torch.randn((rows, k), generator=g, device="cuda").to(bf)
            y = torch.zeros((rows, n), dtype=bf, device="cuda")
            try:
                ms = timed(lambda i=0: self.ctx.project_dense(x, w, y), 5, 3)
                tf = 2.0 * rows * n * k / (ms * 1e-3) / 1e12
                res[f"dense_rows{rows}"] = {"ms": ms, "tflops": tf, "frac_of_measured_bf16_burst": tf / peaks["bf16_tflops"],
                                            "bytes": 2 * (rows * k + n * k + rows * n)}
            except tb.TataraError as e:
                res[f"dense_rows{rows}"] = {"unavailable": str(e)}
            del sets, x, y, w
            torch.cuda.empty_cache()
            out[name] = res
        out["l2"] = "exact-row: rotating weight sets (> 2x L2 between reuse); dense: input + output > L2"
        return out

    # ---- decode layer slices: projection -> layer kernels -> output projection, one token
    def layer_slices(self, timed, steps, warmup, lanes=1, context=32768):
        """The kernels of this library that one decode token runs in one layer, chained in stream order:
        attention layer = attn_project (exact row) -> qk_rope -> decode attention -> out_projection;
        gated-delta layer = gdn_project -> fused conv/recurrence/gate-norm -> out_projection.
        Residual, norms and the MoE between them are not part of this library."""
        torch = self.torch
        g = torch.Generator(device="cuda").manual_seed(21)
        bf = torch.bfloat16

        def q4(sizes, k):
            held = [(torch.randint(-2 ** 31, 2 ** 31 - 1, (m, k // 8), generator=g, device="cuda", dtype=torch.int32),
                     (0.35 * 0.32 / k ** 0.5 * (1 + 0.2 * (2 * torch.rand((m, k // 64), generator=g, device="cuda") - 1))).to(bf),
                     (-0.35 * 2.4 / k ** 0.5 * (1 + 0.1 * torch.randn((m, k // 64), generator=g, device="cuda"))).to(bf))
                    for m in sizes]
            return held, tb.Context.q4_matrices(held)

        x = torch.randn((lanes, 2048), generator=g, device="cuda").to(bf)
        hidden = torch.zeros((lanes, 2048), dtype=bf, device="cuda")
        out = {"lanes": lanes, "context": context}
        # attention layer: per-lane caches in one pool, rotated replicas so that K/V never sit in L2
        cap = context + 1
        per_lane = 2 * cap * 256
        reps = replicas_for(lanes * context * 2048)
        kpool = torch.randn((reps, lanes, per_lane), generator=g, device="cuda").to(bf)
        vpool = torch.randn((reps, lanes, per_lane), generator=g, device="cuda").to(bf)
        attn_w = [q4((8192, 512, 512), 2048) for _ in range(4)]
        out_w = [q4((2048,), 4096) for _ in range(4)]
        proj = torch.zeros((lanes, 9216), dtype=bf, device="cuda")
        qb, gb = torch.zeros((lanes, 4096), dtype=bf, device="cuda"), torch.zeros((lanes, 4096), dtype=bf, device="cuda")
        attended = torch.zeros((lanes, 4096), dtype=bf, device="cuda")
        ones = torch.ones(256, dtype=bf, device="cuda")
        table = tb.Context.attn_lanes([(i * per_lane, context - 1) for i in range(lanes)])
        scratch = torch.empty(tb.decode_scratch_bytes(cap, lanes) // 4, dtype=torch.float32, device="cuda")

        def attn_layer(i=0):
            r, w = i % reps, i % 4
            self.ctx.q4_project(x, attn_w[w][1], 2048, proj)
            self.ctx.attn_qk_rope_batch(proj, ones, ones, qb, gb, kpool[r], vpool[r], cap, table)
            self.ctx.attn_decode_batch(qb, gb, kpool[r], vpool[r], table, cap, attended, scratch)
            self.ctx.q4_project(attended, out_w[w][1], 4096, hidden)

        ms = timed(attn_layer, max(steps, 2 * reps), max(warmup, reps))
        kv = lanes * context * 2048
        wbytes = 10616832 + 4718592
        out["attention_layer"] = {"us": ms * 1e3, "bytes": kv + wbytes, "gbs": (kv + wbytes) / (ms * 1e-3) / 1e9,
                                  "kernels": "q4_project, attn_qk_rope, attn_decode_partition, attn_combine, q4_project"}
        del kpool, vpool
        torch.cuda.empty_cache()
        # gated-delta layer
        nb = lanes * (2 * 2097152 + 2 * 49152)
        reps = replicas_for(nb + 14229504 + 4718592)
        conv_pool = torch.randn((reps, lanes, 2, 3, 8192), generator=g, device="cuda").to(bf)
        rec_pool = 0.02 * torch.randn((reps, lanes, 2, 32, 128, 128), generator=g, device="cuda")
        gdn_w = [q4((8192, 4096, 32, 32), 2048) for _ in range(4)]
        gproj = torch.zeros((lanes, 12352), dtype=bf, device="cuda")
        conv_w = (0.5 * torch.randn((8192, 4), generator=g, device="cuda")).to(bf)
        a_log = torch.log(1 + 15 * torch.rand(32, generator=g, device="cuda")).to(bf)
        dt_bias = (0.5 * torch.randn(32, generator=g, device="cuda")).to(bf)
        norm_w = torch.ones(128, device="cuda").to(bf)
        y, gated = torch.zeros((lanes, 4096), dtype=bf, device="cuda"), torch.zeros((lanes, 4096), dtype=bf, device="cuda")
        cs, rs = 3 * 8192, 32 * 128 * 128
        tables = [tb.Context.gdn_lanes([((2 * i + a) * cs, (2 * i + b) * cs, (2 * i + a) * rs, (2 * i + b) * rs)
                                        for i in range(lanes)]) for a, b in ((0, 1), (1, 0))]

        def gdn_layer(i=0):
            r, w = i % reps, i % 4
            self.ctx.q4_project(x, gdn_w[w][1], 2048, gproj)
            self.ctx.gdn_decode_batch(gproj, conv_w, a_log, dt_bias, norm_w, conv_pool[r], rec_pool[r],
                                      tables[(i // reps) & 1], y, gated)
            self.ctx.q4_project(gated, out_w[w][1], 4096, hidden)

        ms = timed(gdn_layer, max(steps, 2 * reps), max(warmup, reps))
        gb_ = nb + 14229504 + 4718592
        out["gated_delta_layer"] = {"us": ms * 1e3, "bytes": gb_, "gbs": gb_ / (ms * 1e-3) / 1e9,
                                    "kernels": "q4_project, gdn_decode_fused, q4_project"}
        if reps >= 2:   # consecutive steps work on different state sets: the step may stage its successor early
            self.ctx.set_policy(tb.POLICY_GDN_STEP_EARLY_DEPENDENTS, 1)
            try:
                ms = timed(gdn_layer, max(steps, 2 * reps), max(warmup, reps))
            finally:
                self.ctx.set_policy(tb.POLICY_GDN_STEP_EARLY_DEPENDENTS, 0)
            out["gated_delta_layer"]["early_dependents_us"] = ms * 1e3
        out["l2"] = "caches / states rotate through replicas (> 2x L2 between reuse); 4 weight sets (62 MB) rotate"
        return out

    # ---- state snapshot: the canonical prefix payload of the 40-layer schedule in one launch
    def state_copy(self, timed, peaks, positions=65536, capacity=65536):
        """60 gated-delta segments (48 KiB / 2 MiB) + 40 packed K/V head prefixes of `positions` rows, slot ->
        arena, as tatara_state_copy executes them: bytes moved = 2 x payload (read + write)."""
        torch = self.torch
        seg = positions * 512
        payload = 30 * (49152 + 2097152) + 40 * seg
        slot_attn = [torch.empty(2 * capacity * 512, dtype=torch.uint8, device="cuda") for _ in range(20)]   # K, V per layer
        slot_gdn = torch.empty(30 * (49152 + 2097152), dtype=torch.uint8, device="cuda")
        arena = torch.empty(payload, dtype=torch.uint8, device="cuda")
        entries, at = [], 0
        for l in range(30):
            for n in (49152, 2097152):
                entries.append((slot_gdn.data_ptr() + at, arena.data_ptr() + at, n))
                at += n
        for plane in slot_attn:
            for head in range(2):
                entries.append((plane.data_ptr() + head * capacity * 512, arena.data_ptr() + at, seg))
                at += seg
        segs = tb.Context.copy_segments(entries)
        ms = timed(lambda i=0: self.ctx.state_copy(segs), 5, 3)
        gbs = 2 * payload / (ms * 1e-3) / 1e9
        del slot_attn, slot_gdn, arena
        torch.cuda.empty_cache()
        return {"positions": positions, "segments": len(entries), "payload_bytes": payload, "ms": ms, "gbs_read_plus_write": gbs,
                "frac_of_measured_hbm": gbs / peaks["hbm_gbs"], "l2": "payload 1.4 GB > L2"}

    # ---- config 4a: one lane at 262144 split along KV over the ranks
    def split_setup(self, dist, n_keys):
        return SplitCase(self.ctx, self.torch, dist, n_keys, self.rank, self.world)

    # ---- single-workload runs (profiling)
    # ---- the engine's wave loop over a 40-layer stack (native program above the C ABI)
    def wave_loop(self, lanes=8, context=16384, tokens=40):
        """Runs bench_wave_loop (bench_wave_loop.cpp): 8 streams join through the owner loop to
        `context` positions, then full decode waves are timed with the host clock; the same waves walked
        eagerly with host tables beside them."""
        import json
        import subprocess
        exe = WAVE_BENCH_EXE
        if not os.path.exists(exe):
            raise RuntimeError("bench_wave_loop is not built: run __graft_entry__.build()")
        self.torch.cuda.empty_cache()
        res = subprocess.run([exe, "--lanes", str(lanes), "--context", str(context), "--tokens", str(tokens)],
                             capture_output=True, text=True, timeout=150)
        if res.returncode != 0:
            raise RuntimeError(f"wave_bench failed ({res.returncode}): {res.stderr[-400:]}")
        return json.loads(res.stdout.strip().splitlines()[-1])

    def run_only(self, which, args, timed, steps, warmup):
        if which == "decode":
            d = self.decode_setup(args.context)
            ms = timed(d.step, steps, warmup)
            return {"workload": f"decode_attn_ctx{args.context}", "us": ms * 1e3, "replicas": d.replicas,
                    "gbs": (args.context * 2048 + 24576) / (ms * 1e-3) / 1e9}
        if which == "gdn_step":
            return self.gdn_step(timed, steps, warmup, n=args.lanes)
        if which == "lanes32":
            return self.lanes32(timed, steps, warmup)
        if which == "gdn_prefill":
            return self.gdn_prefill(timed, rows=args.rows)
        if which == "layers":
            return self.layer_slices(timed, steps, warmup, lanes=args.lanes if args.lanes != 4 else 1, context=min(args.context, 65536))
        if which == "wave":
            return self.wave_loop(lanes=args.lanes if args.lanes != 4 else 8, context=min(args.context, 16384))
        if which == "state_copy":
            return self.state_copy(timed, measured_peaks())
        if which == "project":
            return self.project(timed, measured_peaks(), steps, warmup, rows=args.rows)
        if which == "prefill":
            return self.prefill(timed, measured_peaks(), rows=args.rows, steps=steps)
        raise ValueError(which)

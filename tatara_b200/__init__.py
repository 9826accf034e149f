"""tatara_b200 -- B200 (sm_100a) attention + Gated DeltaNet operators behind a C ABI.

The product is ``libtatara_b200.so`` (hand-written CUDA, C ABI declared in
``include/tatara_b200.h``).  This module is only the loader plus a thin ctypes wrapper used by
the tests and the benchmark; torch appears solely as the owner of device memory and streams.
There is no CPU path: if the library is missing, importing :func:`lib` raises.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtatara_b200.so")
HEADER_PATH = os.path.join(os.path.dirname(_HERE), "include", "tatara_b200.h")

Q_HEADS, KV_HEADS, HEAD_DIM = 16, 2, 256
ATTN_PROJ = 9216
GDN_PROJ, GDN_CONV, GDN_QK, GDN_V, GDN_HEADS, GDN_DIM = 12352, 8192, 4096, 4096, 32, 128
RECORD_FLOATS = 258
MAX_LANES = 256

STATUS_NAMES = ["None", "InvalidBuffer", "ContextOutOfRange", "StateSlotMismatch",
                "InvalidStreamGroup", "InvalidDispatchExtent", "InvalidDevice", "ScratchTooSmall",
                "DeviceWaitTimeout", "CudaError"]


class TataraError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"tatara_b200 status {status} ({STATUS_NAMES[status] if status < len(STATUS_NAMES) else '?'}): {message}")
        self.status = status


class AttnLane(ctypes.Structure):
    _fields_ = [("kv_offset", ctypes.c_uint64), ("context", ctypes.c_uint32), ("reserved", ctypes.c_uint32)]


class Q4Matrix(ctypes.Structure):
    _fields_ = [("words", ctypes.c_void_p), ("scales", ctypes.c_void_p), ("biases", ctypes.c_void_p),
                ("rows", ctypes.c_uint32), ("reserved", ctypes.c_uint32)]


class CopySegment(ctypes.Structure):
    _fields_ = [("src", ctypes.c_void_p), ("dst", ctypes.c_void_p), ("bytes", ctypes.c_uint64)]


class GdnLane(ctypes.Structure):
    _fields_ = [("conv_in", ctypes.c_uint64), ("conv_out", ctypes.c_uint64),
                ("rec_in", ctypes.c_uint64), ("rec_out", ctypes.c_uint64)]


_lib = None


def lib() -> ctypes.CDLL:
    """Loads libtatara_b200.so; raises if it has not been built (no fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m tatara_b200.build` "
                "(nvcc, sm_100a).  tatara_b200 has no CPU or PyTorch fallback.")
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.tatara_status_name.restype = ctypes.c_char_p
        _lib.tatara_last_error_string.restype = ctypes.c_char_p
        _lib.tatara_last_error_string.argtypes = [ctypes.c_void_p]
        _lib.tatara_attn_decode_scratch_bytes.restype = ctypes.c_uint64
        _lib.tatara_ctx_launch_count.restype = ctypes.c_uint64
        _lib.tatara_ctx_launch_count.argtypes = [ctypes.c_void_p]
        _lib.tatara_attn_partition_keys.restype = ctypes.c_uint32
        _lib.tatara_gdn_prefill_scratch_bytes.restype = ctypes.c_uint64
        _lib.tatara_attn_partitions.restype = ctypes.c_uint32
        _lib.tatara_split_buffer_bytes.restype = ctypes.c_uint64
        _lib.tatara_ctx_get_policy.restype = ctypes.c_uint64
    return _lib


POLICY_DECODE_L2_PREFETCH_KEYS = 0
POLICY_GDN_CHUNK_FORM = 1
POLICY_ATTN_PREFILL_FORM = 2
POLICY_GDN_DECODE_FORM = 3
POLICY_DECODE_FUSED_MERGE = 4
POLICY_Q4_ROW_FORM = 5
POLICY_GDN_STEP_EARLY_DEPENDENTS = 6


def split_buffer_bytes(world: int) -> int:
    return int(lib().tatara_split_buffer_bytes(ctypes.c_uint32(world)))


def partition_keys(n_keys: int) -> int:
    return int(lib().tatara_attn_partition_keys(ctypes.c_uint32(n_keys)))


def partitions(n_keys: int) -> int:
    return int(lib().tatara_attn_partitions(ctypes.c_uint32(n_keys)))


def decode_scratch_bytes(max_keys: int, lanes: int = 1) -> int:
    return int(lib().tatara_attn_decode_scratch_bytes(ctypes.c_uint32(max_keys), ctypes.c_uint32(lanes)))


def _ptr(t):
    """Device pointer of a torch tensor (or None / int passthrough)."""
    if t is None:
        return ctypes.c_void_p(0)
    if isinstance(t, int):
        return ctypes.c_void_p(t)
    return ctypes.c_void_p(t.data_ptr())


_u32 = ctypes.c_uint32
_u64 = ctypes.c_uint64


class Context:
    """One tatara_ctx on one device.  Methods mirror the C entry points one to one and raise
    :class:`TataraError` on a non-zero status; tensor arguments are torch CUDA tensors."""

    def __init__(self, device: int = 0):
        self._h = ctypes.c_void_p()
        st = lib().tatara_ctx_create(ctypes.c_int(device), ctypes.byref(self._h))
        if st != 0:
            raise TataraError(st, f"tatara_ctx_create(device={device})")
        self.device = device

    def close(self):
        if self._h:
            lib().tatara_ctx_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass

    def _check(self, st: int):
        if st != 0:
            raise TataraError(st, lib().tatara_last_error_string(self._h).decode())

    @staticmethod
    def _stream(stream):
        if stream is None:
            import torch
            stream = torch.cuda.current_stream()
        return ctypes.c_void_p(stream if isinstance(stream, int) else stream.cuda_stream)

    @property
    def launches(self) -> int:
        return int(lib().tatara_ctx_launch_count(self._h))

    def sync(self, stream=None):
        self._check(lib().tatara_ctx_sync(self._h, self._stream(stream)))

    # ---- attention
    def attn_qk_rope(self, projection, q_weight, k_weight, q_out, gate_out, keys, values, position,
                     capacity, rows, stream=None):
        self._check(lib().tatara_attn_qk_rope(self._h, self._stream(stream), _ptr(projection),
                                              _ptr(q_weight), _ptr(k_weight), _ptr(q_out), _ptr(gate_out),
                                              _ptr(keys), _ptr(values), _u32(position), _u32(capacity),
                                              _u32(rows)))

    @staticmethod
    def attn_lanes(entries):
        arr = (AttnLane * len(entries))()
        for i, (off, ctxt) in enumerate(entries):
            arr[i].kv_offset, arr[i].context, arr[i].reserved = off, ctxt, 0
        return arr

    @staticmethod
    def gdn_lanes(entries):
        arr = (GdnLane * len(entries))()
        for i, (ci, co, ri, ro) in enumerate(entries):
            arr[i].conv_in, arr[i].conv_out, arr[i].rec_in, arr[i].rec_out = ci, co, ri, ro
        return arr

    def attn_qk_rope_batch(self, projection, q_weight, k_weight, q_out, gate_out, keys_pool,
                           values_pool, capacity, lanes, projection_stride=ATTN_PROJ,
                           query_stride=Q_HEADS * HEAD_DIM, stream=None):
        self._check(lib().tatara_attn_qk_rope_batch(
            self._h, self._stream(stream), _ptr(projection), _ptr(q_weight), _ptr(k_weight), _ptr(q_out),
            _ptr(gate_out), _ptr(keys_pool), _ptr(values_pool), _u32(capacity), lanes, _u32(len(lanes)),
            _u32(projection_stride), _u32(query_stride)))

    def attn_decode(self, q, gate, keys, values, context, capacity, out, scratch, stream=None):
        self._check(lib().tatara_attn_decode(self._h, self._stream(stream), _ptr(q), _ptr(gate), _ptr(keys),
                                             _ptr(values), _u32(context), _u32(capacity), _ptr(out),
                                             _ptr(scratch), _u64(scratch.numel() * scratch.element_size())))

    def attn_decode_static(self, q, gate, keys, values, context, capacity, out, stream=None):
        """Decode attention with the library's built-in record scratch (no allocation, <= 65536 keys)."""
        self._check(lib().tatara_attn_decode_static(self._h, self._stream(stream), _ptr(q), _ptr(gate),
                                                    _ptr(keys), _ptr(values), _u32(context), _u32(capacity),
                                                    _ptr(out)))

    def attn_decode_batch(self, q, gate, keys_pool, values_pool, lanes, capacity, out, scratch,
                          query_stride=Q_HEADS * HEAD_DIM, stream=None):
        self._check(lib().tatara_attn_decode_batch(
            self._h, self._stream(stream), _ptr(q), _ptr(gate), _ptr(keys_pool), _ptr(values_pool), lanes,
            _u32(len(lanes)), _u32(capacity), _u32(query_stride), _ptr(out), _ptr(scratch),
            _u64(scratch.numel() * scratch.element_size())))

    def attn_decode_partial(self, q, keys, values, key_begin, key_end, capacity, records_out, scratch,
                            stream=None):
        self._check(lib().tatara_attn_decode_partial(
            self._h, self._stream(stream), _ptr(q), _ptr(keys), _ptr(values), _u32(key_begin), _u32(key_end),
            _u32(capacity), _ptr(records_out), _ptr(scratch), _u64(scratch.numel() * scratch.element_size())))

    def attn_combine(self, records, nparts, head_stride, part_stride, gate, out, stream=None):
        self._check(lib().tatara_attn_combine(self._h, self._stream(stream), _ptr(records), _u32(nparts),
                                              _u64(head_stride), _u64(part_stride), _ptr(gate), _ptr(out)))

    # ---- split-KV over peer memory
    def peer_buffer_create(self, nbytes):
        """Returns (device pointer, 64-byte IPC handle) of a zero-filled peer buffer."""
        ptr = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        self._check(lib().tatara_peer_buffer_create(self._h, _u64(nbytes), ctypes.byref(ptr), handle))
        return ptr.value, handle.raw

    def peer_buffer_open(self, handle):
        ptr = ctypes.c_void_p()
        self._check(lib().tatara_peer_buffer_open(self._h, ctypes.c_char_p(handle), ctypes.byref(ptr)))
        return ptr.value

    def peer_buffer_close(self, ptr, owned):
        self._check(lib().tatara_peer_buffer_close(self._h, ctypes.c_void_p(ptr), ctypes.c_int(1 if owned else 0)))

    def attn_decode_partial_push(self, q, keys, values, key_begin, key_end, capacity, peer_gather, peer_flags,
                                 rank, epoch, scratch, stream=None):
        world = len(peer_gather)
        pg = (ctypes.c_void_p * world)(*peer_gather)
        pf = (ctypes.c_void_p * world)(*peer_flags)
        self._check(lib().tatara_attn_decode_partial_push(
            self._h, self._stream(stream), _ptr(q), _ptr(keys), _ptr(values), _u32(key_begin), _u32(key_end),
            _u32(capacity), pg, pf, _u32(rank), _u32(world), _u32(epoch), _ptr(scratch),
            _u64(scratch.numel() * scratch.element_size())))

    def attn_decode_split(self, q, gate, keys, values, key_begin, key_end, capacity, peer_buffers, rank,
                          out, scratch, wait_limit_us=1000000, stream=None):
        """peer_buffers: a ctypes array of `world` device pointers (Context.pointer_array), built once."""
        self._check(lib().tatara_attn_decode_split(
            self._h, self._stream(stream), _ptr(q), _ptr(gate), _ptr(keys), _ptr(values), _u32(key_begin),
            _u32(key_end), _u32(capacity), peer_buffers, _u32(rank), _u32(len(peer_buffers)), _u32(wait_limit_us),
            _ptr(out), _ptr(scratch), _u64(scratch.numel() * scratch.element_size())))

    @staticmethod
    def pointer_array(pointers):
        return (ctypes.c_void_p * len(pointers))(*pointers)

    def set_policy(self, policy: int, value: int):
        self._check(lib().tatara_ctx_set_policy(self._h, ctypes.c_int(policy), _u64(value)))

    def get_policy(self, policy: int) -> int:
        return int(lib().tatara_ctx_get_policy(self._h, ctypes.c_int(policy)))

    def attn_combine_wait(self, gather_ptr, flags_ptr, world, epoch, gate, out, wait_limit_us=1000000, stream=None):
        self._check(lib().tatara_attn_combine_wait(self._h, self._stream(stream), ctypes.c_void_p(gather_ptr),
                                                   ctypes.c_void_p(flags_ptr), _u32(world), _u32(epoch),
                                                   _u32(wait_limit_us), _ptr(gate), _ptr(out)))

    def attn_prefill(self, query, gate, keys, values, context_base, rows, capacity, out, stream=None):
        self._check(lib().tatara_attn_prefill(self._h, self._stream(stream), _ptr(query), _ptr(gate),
                                              _ptr(keys), _ptr(values), _u32(context_base), _u32(rows),
                                              _u32(capacity), _ptr(out)))

    def attn_prefill_control(self, query, gate, keys, values, context_base, rows, capacity, out, scratch,
                             stream=None):
        self._check(lib().tatara_attn_prefill_control(
            self._h, self._stream(stream), _ptr(query), _ptr(gate), _ptr(keys), _ptr(values),
            _u32(context_base), _u32(rows), _u32(capacity), _ptr(out), _ptr(scratch),
            _u64(scratch.numel() * scratch.element_size())))

    # ---- gated deltanet
    def gdn_prepare(self, projection, conv_in, conv_weights, qk, value, z, conv_out, rows, stream=None):
        self._check(lib().tatara_gdn_prepare(self._h, self._stream(stream), _ptr(projection), _ptr(conv_in),
                                             _ptr(conv_weights), _ptr(qk), _ptr(value), _ptr(z),
                                             _ptr(conv_out), _u32(rows)))

    def gdn_gates(self, projection, a_log, dt_bias, decay, beta, rows, projection_stride=GDN_PROJ,
                  stream=None):
        self._check(lib().tatara_gdn_gates(self._h, self._stream(stream), _ptr(projection),
                                           _u32(projection_stride), _ptr(a_log), _ptr(dt_bias), _ptr(decay),
                                           _ptr(beta), _u32(rows)))

    def gdn_step(self, qk, value, projection, a_log, dt_bias, state_in, y, state_out, stream=None):
        self._check(lib().tatara_gdn_step(self._h, self._stream(stream), _ptr(qk), _ptr(value),
                                          _ptr(projection), _ptr(a_log), _ptr(dt_bias), _ptr(state_in),
                                          _ptr(y), _ptr(state_out)))

    def gdn_gate_norm(self, y, z, weight, out, rows, stream=None):
        self._check(lib().tatara_gdn_gate_norm(self._h, self._stream(stream), _ptr(y), _ptr(z), _ptr(weight),
                                               _ptr(out), _u32(rows)))

    def gdn_decode_batch(self, projection, conv_weights, a_log, dt_bias, norm_weight, conv_pool, rec_pool,
                         lanes, y, gated, projection_stride=GDN_PROJ, stream=None):
        self._check(lib().tatara_gdn_decode_batch(
            self._h, self._stream(stream), _ptr(projection), _u32(projection_stride), _ptr(conv_weights),
            _ptr(a_log), _ptr(dt_bias), _ptr(norm_weight), _ptr(conv_pool), _ptr(rec_pool), lanes,
            _u32(len(lanes)), _ptr(y), _ptr(gated)))

    def gdn_prefill(self, qk, value, decay, beta, state_in, y, state_out, rows, chunk=64, scratch=None,
                    stream=None):
        nbytes = 0 if scratch is None else scratch.numel() * scratch.element_size()
        self._check(lib().tatara_gdn_prefill(self._h, self._stream(stream), _ptr(qk), _ptr(value),
                                             _ptr(decay), _ptr(beta), _ptr(state_in), _ptr(y),
                                             _ptr(state_out), _u32(rows), _u32(chunk), _ptr(scratch),
                                             _u64(nbytes)))

    # ---- lane tables in device memory (CUDA-graph replay)
    @staticmethod
    def device_lanes(table):
        """A ctypes lane table (attn_lanes / gdn_lanes) as a device tensor of its bytes."""
        import torch
        raw = bytes(table)
        return torch.frombuffer(bytearray(raw), dtype=torch.uint8).cuda()

    def attn_qk_rope_batch_indirect(self, projection, q_weight, k_weight, q_out, gate_out, keys_pool, values_pool,
                                    capacity, lanes_device, n_lanes, projection_stride=ATTN_PROJ,
                                    query_stride=Q_HEADS * HEAD_DIM, stream=None):
        self._check(lib().tatara_attn_qk_rope_batch_indirect(
            self._h, self._stream(stream), _ptr(projection), _ptr(q_weight), _ptr(k_weight), _ptr(q_out),
            _ptr(gate_out), _ptr(keys_pool), _ptr(values_pool), _u32(capacity), _ptr(lanes_device), _u32(n_lanes),
            _u32(projection_stride), _u32(query_stride)))

    def attn_decode_batch_indirect(self, q, gate, keys_pool, values_pool, lanes_device, n_lanes, capacity, out, scratch,
                                   query_stride=Q_HEADS * HEAD_DIM, stream=None):
        self._check(lib().tatara_attn_decode_batch_indirect(
            self._h, self._stream(stream), _ptr(q), _ptr(gate), _ptr(keys_pool), _ptr(values_pool), _ptr(lanes_device),
            _u32(n_lanes), _u32(capacity), _u32(query_stride), _ptr(out), _ptr(scratch),
            _u64(scratch.numel() * scratch.element_size())))

    def gdn_decode_batch_indirect(self, projection, conv_weights, a_log, dt_bias, norm_weight, conv_pool, rec_pool,
                                  lanes_device, n_lanes, y, gated, projection_stride=GDN_PROJ, stream=None):
        self._check(lib().tatara_gdn_decode_batch_indirect(
            self._h, self._stream(stream), _ptr(projection), _u32(projection_stride), _ptr(conv_weights),
            _ptr(a_log), _ptr(dt_bias), _ptr(norm_weight), _ptr(conv_pool), _ptr(rec_pool), _ptr(lanes_device),
            _u32(n_lanes), _ptr(y), _ptr(gated)))

    def lanes_advance(self, attn_lanes_device, n_attn, gdn_lanes_device, n_gdn, stream=None):
        self._check(lib().tatara_lanes_advance(self._h, self._stream(stream), _ptr(attn_lanes_device), _u32(n_attn),
                                               _ptr(gdn_lanes_device), _u32(n_gdn)))

    # ---- speculative-decode support: GDN tape and replay
    def gdn_prepare_tape(self, projection, conv_in, conv_weights, qk, value, z, conv_out, rows, conv_tape, tape_layer,
                         stream=None):
        self._check(lib().tatara_gdn_prepare_tape(self._h, self._stream(stream), _ptr(projection), _ptr(conv_in),
                                                  _ptr(conv_weights), _ptr(qk), _ptr(value), _ptr(z), _ptr(conv_out),
                                                  _u32(rows), _ptr(conv_tape), _u32(tape_layer)))

    def gdn_prefill_tape(self, qk, value, decay, beta, state_in, y, state_out, rows, tape, tape_layer, stream=None):
        self._check(lib().tatara_gdn_prefill_tape(self._h, self._stream(stream), _ptr(qk), _ptr(value), _ptr(decay),
                                                  _ptr(beta), _ptr(state_in), _ptr(y), _ptr(state_out), _u32(rows),
                                                  _ptr(tape), _u32(tape_layer)))

    def gdn_tape_replay(self, tape, state_in, state_out, steps, tape_layer, stream=None):
        self._check(lib().tatara_gdn_tape_replay(self._h, self._stream(stream), _ptr(tape), _ptr(state_in),
                                                 _ptr(state_out), _u32(steps), _u32(tape_layer)))

    # ---- affine-Q4 projections
    @staticmethod
    def q4_matrices(triples):
        """(words [n][k/8] int32, scales [n][k/64] bf16, biases) device tensors -> tatara_q4_matrix[]."""
        arr = (Q4Matrix * len(triples))()
        for i, (w, s, b) in enumerate(triples):
            arr[i] = Q4Matrix(w.data_ptr(), s.data_ptr(), b.data_ptr(), w.shape[0], 0)
        return arr

    def q4_project(self, x, matrices, k, out, n_rows=None, x_stride=None, out_stride=None, stream=None):
        n_rows = x.shape[0] if n_rows is None else n_rows
        self._check(lib().tatara_q4_project(
            self._h, self._stream(stream), _ptr(x), _u64(x.stride(0) if x_stride is None else x_stride),
            _u32(n_rows), matrices, _u32(len(matrices)), _u32(k), _ptr(out),
            _u64(out.stride(0) if out_stride is None else out_stride)))

    def q4_dequantize(self, matrices, k, weights, stream=None):
        self._check(lib().tatara_q4_dequantize(self._h, self._stream(stream), matrices, _u32(len(matrices)),
                                               _u32(k), _ptr(weights)))

    def project_dense(self, x, weights, out, n_rows=None, stream=None):
        n_rows = x.shape[0] if n_rows is None else n_rows
        self._check(lib().tatara_project_dense(
            self._h, self._stream(stream), _ptr(x), _u64(x.stride(0)), _u32(n_rows), _ptr(weights),
            _u32(weights.shape[0]), _u32(weights.shape[1]), _ptr(out), _u64(out.stride(0))))

    # ---- state snapshots
    @staticmethod
    def copy_segments(entries):
        """[(src address, dst address, bytes)] -> tatara_copy_segment[]."""
        arr = (CopySegment * len(entries))()
        for i, (src, dst, n) in enumerate(entries):
            arr[i] = CopySegment(src, dst, n)
        return arr

    def state_copy(self, segments, stream=None):
        self._check(lib().tatara_state_copy(self._h, self._stream(stream), segments, _u32(len(segments))))


def gdn_tape_bytes() -> int:
    f = lib().tatara_gdn_tape_bytes
    f.restype = ctypes.c_uint64
    return int(f())


def gdn_conv_tape_bytes() -> int:
    f = lib().tatara_gdn_conv_tape_bytes
    f.restype = ctypes.c_uint64
    return int(f())


def gdn_prefill_scratch_bytes(rows: int) -> int:
    return int(lib().tatara_gdn_prefill_scratch_bytes(ctypes.c_uint32(rows)))

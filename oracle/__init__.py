"""ctypes binding of the CPU oracle (``oracle/tatara_oracle.cpp``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()`` and by
the ``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``.  The product package
``tatara_b200`` never imports this module.

All tensors are numpy arrays: bf16 values travel as ``uint16`` bit patterns, f32 as
``float32``.  Layouts are the reference engine's (see the C++ source for citations).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libtatara_oracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libtatara_ref.so")


def reference_root() -> str | None:
    """The reference checkout: $TATARA_REFERENCE_ROOT, else a directory named `reference` beside
    this repository (where the build container keeps it); None where neither exists."""
    for root in (os.environ.get("TATARA_REFERENCE_ROOT"),
                 os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")):
        if root and os.path.exists(os.path.join(root, "tests", "native", "kernel_reference.cpp")):
            return root
    return None


_u16p = ctypes.POINTER(ctypes.c_uint16)
_u32p = ctypes.POINTER(ctypes.c_uint32)
_f32p = ctypes.POINTER(ctypes.c_float)
_u32 = ctypes.c_uint32
_int = ctypes.c_int


def build(with_reference: bool | None = None) -> None:
    """Compile the oracle (and, where the reference tree is present, its CPU model)."""
    subprocess.check_call(["make", "-s", "-C", _HERE, "all"])
    root = reference_root()
    if with_reference is None:
        with_reference = root is not None
    if with_reference:
        if root is None:
            raise RuntimeError("the reference checkout was not found: set TATARA_REFERENCE_ROOT")
        subprocess.check_call(["make", "-s", "-C", _HERE, "ref", f"REFERENCE_ROOT={root}"])


def _p(a: np.ndarray, ty):
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be C-contiguous"
    return a.ctypes.data_as(ty)


def _u16(a):
    assert a.dtype == np.uint16
    return _p(a, _u16p)


def _f32(a):
    assert a.dtype == np.float32
    return _p(a, _f32p)


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build(with_reference=False)
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.orc_f32_from_bf16.restype = ctypes.c_float
        _lib.orc_rope_divisor.restype = ctypes.c_float
        _lib.orc_bf16_from_f32.argtypes = [ctypes.c_float]
        _lib.orc_bf16_from_f32.restype = ctypes.c_uint16
        _lib.orc_q4_dot.restype = ctypes.c_float
    return _lib


def hardware_threads() -> int:
    return int(lib().orc_hardware_threads())


# ---------------------------------------------------------------- bf16 helpers
def bf16_from_f32(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bit patterns (vectorised; Inf/NaN pass through)."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    special = (b & 0x7F800000) == 0x7F800000
    r = (b + 0x7FFF + ((b >> 16) & 1)) >> 16
    return np.where(special, b >> 16, r).astype(np.uint16)


def f32_from_bf16(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# ---------------------------------------------------------------- attention
def attn_qk_rope(projection, q_weight, k_weight, keys, values, position, capacity):
    """projection [rows][9216]; appends into keys/values in place; returns (q, gate) [rows][16][256]."""
    rows = projection.shape[0]
    q = np.zeros((rows, 16, 256), np.uint16)
    gate = np.zeros((rows, 16, 256), np.uint16)
    lib().orc_attn_qk_rope(_u16(projection), _u16(q_weight), _u16(k_weight), _u16(q), _u16(gate),
                           _u16(keys), _u16(values), _u32(position), _u32(capacity), _u32(rows))
    return q, gate


def attn_decode(q, gate, keys, values, context, capacity, threads=1):
    out = np.zeros((16, 256), np.uint16)
    lib().orc_attn_decode(_u16(q), _u16(gate), _u16(keys), _u16(values), _u32(context),
                          _u32(capacity), _u16(out), _int(threads))
    return out


def attn_partial(q, keys, values, key_begin, key_end, capacity, threads=1):
    rec = np.zeros((16, 258), np.float32)
    lib().orc_attn_partial(_u16(q), _u16(keys), _u16(values), _u32(key_begin), _u32(key_end),
                           _u32(capacity), _f32(rec), _u32(258), _int(threads))
    return rec


def attn_combine(records, gate):
    """records [16][nparts][258] -> out [16][256]."""
    assert records.shape[0] == 16 and records.shape[2] == 258
    out = np.zeros((16, 256), np.uint16)
    lib().orc_attn_combine(_f32(records), _u32(records.shape[1]), _u16(gate), _u16(out))
    return out


def attn_prefill(query, gate, keys, values, context_base, capacity, row_list=None, threads=1):
    """query/gate [rows][16][256]; returns out [rows][16][256] (only listed rows are written)."""
    rows = query.shape[0]
    out = np.zeros((rows, 16, 256), np.uint16)
    if row_list is None:
        rl, n = None, 0
    else:
        row_list = np.ascontiguousarray(row_list, dtype=np.uint32)
        rl, n = _p(row_list, _u32p), len(row_list)
    lib().orc_attn_prefill(_u16(query), _u16(gate), _u16(keys), _u16(values), _u32(context_base),
                           _u32(rows), _u32(capacity), rl, _u32(n), _u16(out), _int(threads))
    return out


# ---------------------------------------------------------------- gated deltanet
def gdn_prepare(projection, conv_state, conv_weights):
    """projection [rows][12352] -> (qk, value, z [rows][4096], new_conv_state [3][8192])."""
    rows = projection.shape[0]
    qk = np.zeros((rows, 4096), np.uint16)
    value = np.zeros((rows, 4096), np.uint16)
    z = np.zeros((rows, 4096), np.uint16)
    new_state = np.zeros((3, 8192), np.uint16)
    lib().orc_gdn_prepare(_u16(projection), _u16(conv_state), _u16(conv_weights), _u16(qk),
                          _u16(value), _u16(z), _u16(new_state), _u32(rows))
    return qk, value, z, new_state


def gdn_gates(projection, a_log, dt_bias):
    rows = projection.shape[0]
    decay = np.zeros((rows, 32), np.float32)
    beta = np.zeros((rows, 32), np.float32)
    lib().orc_gdn_gates(_u16(projection), _u32(projection.shape[1]), _u16(a_log), _u16(dt_bias),
                        _f32(decay), _f32(beta), _u32(rows))
    return decay, beta


def gdn_scan(qk, value, decay, beta, state_in, threads=1):
    """Sequential scan over rows; returns (y [rows][4096], state_out [32][128][128])."""
    rows = qk.shape[0]
    y = np.zeros((rows, 4096), np.uint16)
    state_out = np.zeros((32, 128, 128), np.float32)
    lib().orc_gdn_scan(_u16(qk), _u16(value), _f32(decay), _f32(beta), _f32(state_in), _u16(y),
                       _f32(state_out), _u32(rows), _int(threads))
    return y, state_out


def gdn_gate_norm(y, z, weight):
    rows = y.shape[0]
    out = np.zeros((rows, 4096), np.uint16)
    lib().orc_gdn_gate_norm(_u16(y), _u16(z), _u16(weight), _u16(out), _u32(rows))
    return out


TAPE_ROWS, TAPE_LAYERS = 16, 40


def gdn_tape_floats() -> int:
    f = lib().orc_gdn_tape_floats
    f.restype = ctypes.c_uint64
    return int(f())


def gdn_scan_tape(qk, value, decay, beta, state_in, tape, tape_layer, threads=1):
    """Sequential scan of rows <= 16 that also fills `tape` (f32, gdn_tape_floats()) for `tape_layer`."""
    rows = qk.shape[0]
    y = np.zeros((rows, 4096), np.uint16)
    state_out = np.zeros((32, 128, 128), np.float32)
    lib().orc_gdn_scan_tape(_u16(qk), _u16(value), _f32(decay), _f32(beta), _f32(state_in), _u16(y), _f32(state_out),
                            _u32(rows), _f32(tape), _u32(tape_layer), _int(threads))
    return y, state_out


def gdn_tape_replay(tape, state_in, steps, tape_layer, threads=1):
    state_out = np.zeros((32, 128, 128), np.float32)
    lib().orc_gdn_tape_replay(_f32(tape), _f32(state_in), _f32(state_out), _u32(steps), _u32(tape_layer), _int(threads))
    return state_out


def gdn_conv_tape(projection, conv_state, conv_tape, tape_layer):
    """Fills conv_tape [40][16][3][8192] u16 for `tape_layer` with the conv tail after every row."""
    lib().orc_gdn_conv_tape(_u16(projection), _u16(conv_state), _u32(projection.shape[0]), _u16(conv_tape), _u32(tape_layer))


def _u32a(a):
    assert a.dtype == np.uint32
    return _p(a, ctypes.POINTER(ctypes.c_uint32))


def q4_dot(x, words, scales, biases, fused=True) -> float:
    """One affine-Q4 output row over x[k]: words [k/8] u32, scales/biases [k/64] bf16 bits."""
    return float(lib().orc_q4_dot(_u16(x), _u32a(words), _u16(scales), _u16(biases), _u32(x.shape[0]),
                                  _int(1 if fused else 0)))


def q4_project(x, words, scales, biases, fused=True, threads=1):
    """Exact-row projection of x [rows][k] through one Q4 matrix (words [n][k/8]) -> bf16 [rows][n]."""
    rows, k = x.shape
    n = words.shape[0]
    out = np.zeros((rows, n), np.uint16)
    lib().orc_q4_project(_u16(x), _u32(k), _u32(rows), _u32a(words), _u16(scales), _u16(biases), _u32(n),
                         _u32(k), _u16(out), _u32(n), _int(1 if fused else 0), _int(threads))
    return out


def q4_dequantize(words, scales, biases):
    """bf16(q*scale + bias) weights [n][k] of the tensor-unit policy."""
    n, k = words.shape[0], words.shape[1] * 8
    out = np.zeros((n, k), np.uint16)
    lib().orc_q4_dequantize(_u32a(words), _u16(scales), _u16(biases), _u32(n), _u32(k), _u16(out))
    return out


def project_dense(x, weights, threads=1):
    """bf16 x [rows][k] times bf16 weights [n][k], f32 accumulation in k order -> bf16 [rows][n]."""
    rows, k = x.shape
    n = weights.shape[0]
    out = np.zeros((rows, n), np.uint16)
    lib().orc_project_dense(_u16(x), _u32(k), _u32(rows), _u16(weights), _u32(n), _u32(k), _u16(out), _u32(n),
                            _int(threads))
    return out


# ---------------------------------------------------------------- reference CPU model
_ref = None


def reference_available() -> bool:
    return os.path.exists(_REF_PATH)


def ref() -> ctypes.CDLL:
    """The reference's own CPU model (oracle/_ref); only where it was built."""
    global _ref
    if _ref is None:
        _ref = ctypes.CDLL(_REF_PATH)
    return _ref


def ref_q4_dot(x, words, scales, biases, fused=True) -> float:
    f = ref().ref_q4_dot
    f.restype = ctypes.c_float
    return float(f(_u16(x), _u32a(words), _u16(scales), _u16(biases), _u32(x.shape[0]), _int(1 if fused else 0)))


def ref_attn_qk_rope(projection, q_weight, k_weight, keys, values, position, capacity):
    q = np.zeros((16, 256), np.uint16)
    gate = np.zeros((16, 256), np.uint16)
    ref().ref_attn_qk_rope(_u16(projection), _u16(q_weight), _u16(k_weight), _u16(q), _u16(gate),
                           _u16(keys), _u16(values), _u32(position), _u32(capacity))
    return q, gate


def ref_attn_decode(q, gate, keys, values, context, capacity):
    out = np.zeros((16, 256), np.uint16)
    ref().ref_attn_decode(_u16(q), _u16(gate), _u16(keys), _u16(values), _u32(context),
                          _u32(capacity), _u16(out))
    return out


def ref_attn_split(q, gate, keys, values, context, capacity):
    nparts = (context + 1 + 255) // 256
    rec = np.zeros((16, nparts, 258), np.float32)
    out = np.zeros((16, 256), np.uint16)
    ref().ref_attn_split(_u16(q), _u16(gate), _u16(keys), _u16(values), _u32(context),
                         _u32(capacity), _f32(rec), _u16(out))
    return rec, out


def ref_gdn_prepare(projection, conv_state, conv_weights):
    qk = np.zeros(4096, np.uint16)
    value = np.zeros(4096, np.uint16)
    z = np.zeros(4096, np.uint16)
    new_state = np.zeros((3, 8192), np.uint16)
    ref().ref_gdn_prepare(_u16(projection), _u16(conv_state), _u16(conv_weights), _u16(qk),
                          _u16(value), _u16(z), _u16(new_state))
    return qk, value, z, new_state


def ref_gdn_gates(projection, a_log, dt_bias):
    decay = np.zeros(32, np.float32)
    beta = np.zeros(32, np.float32)
    ref().ref_gdn_gates(_u16(projection), _u16(a_log), _u16(dt_bias), _f32(decay), _f32(beta))
    return decay, beta


def ref_gdn_step(qk, value, decay, beta, state_in):
    y = np.zeros(4096, np.uint16)
    state_out = np.zeros((32, 128, 128), np.float32)
    ref().ref_gdn_step(_u16(qk), _u16(value), _f32(decay), _f32(beta), _f32(state_in), _u16(y),
                       _f32(state_out))
    return y, state_out


def ref_gdn_gate_norm(y, z, weight):
    out = np.zeros(4096, np.uint16)
    ref().ref_gdn_gate_norm(_u16(y), _u16(z), _u16(weight), _u16(out))
    return out

"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configs.

Everything is numpy; bf16 tensors are ``uint16`` bit patterns in the reference engine's
layouts.  Used by the tests, the smoke entry and ``bench.py`` -- no dataset is involved.

Attention (16 query heads, 2 KV heads, head_dim 256):
  raw q/k ~ N(0,1) per head, RMS-normalised to unit RMS (weight 1), RoPE on dims 0..63
  (theta base 1e7, rotate-half pairs d / d+32), v ~ N(0,1), gate logits ~ N(0,1).
Gated DeltaNet (16 qk heads, 32 v heads, head_dim 128, conv width 4):
  conv state and the current qkv row ~ N(0,1); conv weights ~ N(0, 0.5);
  b ~ N(0,1) (beta = sigmoid(b)); A_log = log U(1,16); a + dt_bias ~ N(0,1);
  recurrent state ~ N(0, 0.02) f32.
"""
from __future__ import annotations

import numpy as np

Q_HEADS, KV_HEADS, HEAD_DIM = 16, 2, 256
ATTN_PROJ = 9216
GDN_PROJ, GDN_CONV, GDN_QK, GDN_V, GDN_HEADS, GDN_DIM = 12352, 8192, 4096, 4096, 32, 128
ROPE_PAIRS, ROPE_BASE = 32, 1.0e7


def to_bf16(x: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    special = (b & 0x7F800000) == 0x7F800000
    r = (b + 0x7FFF + ((b >> 16) & 1)) >> 16
    return np.where(special, b >> 16, r).astype(np.uint16)


def from_bf16(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def normal_bf16(rng: np.random.Generator, shape, std: float = 1.0) -> np.ndarray:
    return to_bf16(rng.standard_normal(shape, dtype=np.float32) * np.float32(std))


def rope_divisors() -> np.ndarray:
    return np.power(ROPE_BASE, np.arange(ROPE_PAIRS, dtype=np.float64) / ROPE_PAIRS).astype(np.float32)


def normed_roped(rng: np.random.Generator, positions: np.ndarray, heads: int) -> np.ndarray:
    """[len(positions)][heads][256] bf16: unit-RMS N(0,1) vectors rotated at `positions`."""
    n = len(positions)
    x = rng.standard_normal((n, heads, HEAD_DIM), dtype=np.float32)
    x /= np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + 1e-6)
    x = from_bf16(to_bf16(x))
    theta = positions.astype(np.float32)[:, None] / rope_divisors()[None, :]
    c, s = np.cos(theta)[:, None, :], np.sin(theta)[:, None, :]
    lo, hi = x[..., :32].copy(), x[..., 32:64].copy()
    x[..., :32] = lo * c - hi * s
    x[..., 32:64] = hi * c + lo * s
    return to_bf16(x)


def attn_projection(rng: np.random.Generator, rows: int) -> np.ndarray:
    """Raw attention projection rows [rows][9216] ~ N(0,1) (input of qk_rope)."""
    return normal_bf16(rng, (rows, ATTN_PROJ))


def attn_weights(rng: np.random.Generator, unit: bool = True):
    """(q_norm weight, k_norm weight) [256] bf16; unit weights match the benchmark configs."""
    if unit:
        w = np.full(HEAD_DIM, 0x3F80, np.uint16)
        return w, w.copy()
    return (to_bf16(1.0 + 0.1 * rng.standard_normal(HEAD_DIM).astype(np.float32)),
            to_bf16(1.0 + 0.1 * rng.standard_normal(HEAD_DIM).astype(np.float32)))


def attn_cache(rng: np.random.Generator, n_keys: int, capacity: int, chunk: int = 16384):
    """Lane KV cache planes K, V [2][capacity][256] bf16 with positions 0..n_keys-1 filled."""
    keys = np.zeros((KV_HEADS, capacity, HEAD_DIM), np.uint16)
    values = np.zeros((KV_HEADS, capacity, HEAD_DIM), np.uint16)
    for start in range(0, n_keys, chunk):
        stop = min(start + chunk, n_keys)
        k = normed_roped(rng, np.arange(start, stop), KV_HEADS)
        keys[:, start:stop] = k.transpose(1, 0, 2)
        values[:, start:stop] = normal_bf16(rng, (KV_HEADS, stop - start, HEAD_DIM))
    return keys, values


def attn_query(rng: np.random.Generator, positions: np.ndarray):
    """(q, gate) [len(positions)][16][256] bf16."""
    q = normed_roped(rng, np.asarray(positions), Q_HEADS)
    gate = normal_bf16(rng, q.shape)
    return q, gate


def gdn_weights(rng: np.random.Generator):
    """(conv_weights [8192][4], a_log [32], dt_bias [32], norm_weight [128]) bf16."""
    conv_w = normal_bf16(rng, (GDN_CONV, 4), std=0.5)
    a_log = to_bf16(np.log(rng.uniform(1.0, 16.0, GDN_HEADS)).astype(np.float32))
    dt_bias = normal_bf16(rng, GDN_HEADS, std=0.5)
    norm_w = to_bf16(1.0 + 0.1 * rng.standard_normal(GDN_DIM).astype(np.float32))
    return conv_w, a_log, dt_bias, norm_w


def gdn_projection(rng: np.random.Generator, rows: int) -> np.ndarray:
    """[rows][12352] = q 2048 | k 2048 | v 4096 | z 4096 | b 32 | a 32, all ~ N(0,1)."""
    return normal_bf16(rng, (rows, GDN_PROJ))


def gdn_state(rng: np.random.Generator, zero: bool = False):
    """(conv_state [3][8192] bf16 ~ N(0,1), recurrent state [32][128][128] f32 ~ N(0,0.02))."""
    conv = normal_bf16(rng, (3, GDN_CONV))
    if zero:
        return conv, np.zeros((GDN_HEADS, GDN_DIM, GDN_DIM), np.float32)
    rec = (rng.standard_normal((GDN_HEADS, GDN_DIM, GDN_DIM), dtype=np.float32) * np.float32(0.02))
    return conv, rec


def q4_matrix(rng: np.random.Generator, n: int, k: int, gain: float = 0.35):
    """An affine-Q4 group-64 weight matrix of n output rows over k inputs.

    words [n][k/8] u32 (nibble j of word w is column 8w + j), scales and biases [n][k/64] bf16 bits.
    Nibbles are uniform in 0..15; scale ~ 0.32 gain/sqrt(k) (1 +- 0.2) and bias ~ -7.5 scale (1 +- 0.1),
    the shape a min/max group quantiser gives weights of standard deviation ~ gain/sqrt(k); a
    unit-variance input row then projects to outputs of standard deviation ~ 1.5 gain (0.5 at the
    default gain, so that one bf16 step of the largest outputs stays below the 2e-2 gate).
    """
    words = rng.integers(0, 1 << 32, size=(n, k // 8), dtype=np.uint64).astype(np.uint32)
    sigma = gain / np.sqrt(k)
    scale = 0.32 * sigma * (1.0 + 0.2 * rng.uniform(-1, 1, size=(n, k // 64)))
    bias = -7.5 * scale * (1.0 + 0.1 * rng.standard_normal((n, k // 64)))
    return words, to_bf16(scale.astype(np.float32)), to_bf16(bias.astype(np.float32))


def hidden_rows(rng: np.random.Generator, rows: int, k: int) -> np.ndarray:
    """RMS-normalised hidden rows [rows][k] bf16 bits (unit variance)."""
    return normal_bf16(rng, (rows, k))

"""Seeded inputs of the golden cases (shared by make_golden.py and the tests)."""
import zlib

import numpy as np

import oracle
from tatara_b200 import synthetic as syn

CAP = 512
CONTEXTS = [0, 4, 200, 300, 511]


def checksum(*arrays) -> np.ndarray:
    c = 0
    for a in arrays:
        c = zlib.crc32(np.ascontiguousarray(a).tobytes(), c)
    return np.array([c], np.uint64)


def attention_cases():
    for context in CONTEXTS:
        rng = np.random.default_rng(7000 + context)
        w = syn.attn_weights(rng, unit=False)
        keys = np.zeros((2, CAP, 256), np.uint16)
        values = np.zeros_like(keys)
        oracle.attn_qk_rope(syn.attn_projection(rng, context + 1), w[0], w[1], keys, values, 0, CAP)
        q, gate = syn.attn_query(rng, np.array([context]))
        yield f"attn/{context}", (q[0], gate[0], keys, values, context)


def rope_cases():
    for position in [0, 1, 300, 511]:
        rng = np.random.default_rng(7100 + position)
        qw, kw = syn.attn_weights(rng, unit=False)
        yield f"rope/{position}", (syn.attn_projection(rng, 1)[0], qw, kw, position)


def gdn_chain(steps: int = 4):
    rng = np.random.default_rng(7200)
    weights = syn.gdn_weights(rng)
    conv, state = syn.gdn_state(rng)
    projections = [syn.gdn_projection(rng, 1)[0] for _ in range(steps)]
    return weights, conv, state, projections


def q4_cases():
    """(name, x[k], words[k/8], scales[k/64], biases[k/64]) single-row dots at the three widths in use."""
    for k in (512, 2048, 4096):
        rng = np.random.default_rng(7300 + k)
        words, scales, biases = syn.q4_matrix(rng, 8, k)
        x = syn.hidden_rows(rng, 1, k)[0]
        for row in range(8):
            yield f"q4/{k}/{row}", (x, words[row].copy(), scales[row].copy(), biases[row].copy())

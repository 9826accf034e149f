"""The restated oracle against the reference's own CPU model (oracle/_ref), bit for bit.

Runs only where the reference tree was present at build time (oracle/_ref exists); the
committed golden vectors (tests/test_oracle_golden.py) carry the same pin everywhere else.
Shapes follow the reference's fixture probes: capacity 512, contexts 0 / 4 / 200 / 300
(tools/native/attention_fixture_probe.cpp:27-36) and a 4-step GDN chain
(tools/native/gdn_fixture_probe.cpp:44, 805-851).
"""
import ctypes

import numpy as np
import pytest

import oracle
from tatara_b200 import synthetic as syn

pytestmark = pytest.mark.skipif(not oracle.reference_available(),
                                reason="oracle/_ref not built (reference tree absent)")

CAP = 512


def _filled_cache(rng, n, weights):
    keys = np.zeros((2, CAP, 256), np.uint16)
    values = np.zeros((2, CAP, 256), np.uint16)
    proj = syn.attn_projection(rng, n)
    oracle.attn_qk_rope(proj, weights[0], weights[1], keys, values, 0, CAP)
    return keys, values


def test_bf16_rounding_matches_reference():
    rng = np.random.default_rng(1)
    x = rng.standard_normal(4096).astype(np.float32) * np.float32(1e3)
    ours = syn.to_bf16(x)
    for v, b in zip(x[:512], ours[:512]):
        assert oracle.ref().ref_bf16_from_f32(oracle.ctypes.c_float(float(v))) == int(b)
    # ties-to-even and Inf (tests/native/kernel_reference_test.cpp:15-35)
    ties = np.array([0x3F808000, 0x3F818000, 0x7F800000], np.uint32).view(np.float32)
    assert list(syn.to_bf16(ties)) == [0x3F80, 0x3F82, 0x7F80]


@pytest.mark.parametrize("position", [0, 4, 200, 300, 511])
def test_qk_rope_bit_exact(position):
    rng = np.random.default_rng(100 + position)
    proj = syn.attn_projection(rng, 1)
    qw, kw = syn.attn_weights(rng, unit=False)
    k1 = np.zeros((2, CAP, 256), np.uint16); v1 = np.zeros_like(k1)
    k2 = np.zeros_like(k1); v2 = np.zeros_like(k1)
    q, g = oracle.attn_qk_rope(proj, qw, kw, k1, v1, position, CAP)
    rq, rg = oracle.ref_attn_qk_rope(proj[0], qw, kw, k2, v2, position, CAP)
    assert np.array_equal(q[0], rq) and np.array_equal(g[0], rg)
    assert np.array_equal(k1, k2) and np.array_equal(v1, v2)


@pytest.mark.parametrize("context", [0, 4, 200, 255, 256, 300, 511])
def test_decode_bit_exact(context):
    rng = np.random.default_rng(200 + context)
    w = syn.attn_weights(rng, unit=False)
    keys, values = _filled_cache(rng, context + 1, w)
    q, gate = syn.attn_query(rng, np.array([context]))
    ours = oracle.attn_decode(q[0], gate[0], keys, values, context, CAP)
    theirs = oracle.ref_attn_decode(q[0], gate[0], keys, values, context, CAP)
    assert np.array_equal(ours, theirs)


@pytest.mark.parametrize("context", [4, 255, 256, 300, 511])
def test_partial_and_combine_bit_exact(context):
    rng = np.random.default_rng(300 + context)
    w = syn.attn_weights(rng)
    keys, values = _filled_cache(rng, context + 1, w)
    q, gate = syn.attn_query(rng, np.array([context]))
    ref_rec, ref_out = oracle.ref_attn_split(q[0], gate[0], keys, values, context, CAP)
    nparts = ref_rec.shape[1]
    rec = np.zeros_like(ref_rec)
    for p in range(nparts):
        rec[:, p] = oracle.attn_partial(q[0], keys, values, p * 256, min(context + 1, (p + 1) * 256), CAP)
    assert np.array_equal(rec.view(np.uint32), ref_rec.view(np.uint32))
    assert np.array_equal(oracle.attn_combine(rec, gate[0]), ref_out)


def test_gdn_chain_bit_exact():
    rng = np.random.default_rng(400)
    conv_w, a_log, dt_bias, norm_w = syn.gdn_weights(rng)
    conv, state = syn.gdn_state(rng)
    rconv, rstate = conv.copy(), state.copy()
    for step in range(4):
        proj = syn.gdn_projection(rng, 1)
        qk, v, z, conv = oracle.gdn_prepare(proj, conv, conv_w)
        rqk, rv, rz, rconv = oracle.ref_gdn_prepare(proj[0], rconv, conv_w)
        assert np.array_equal(qk[0], rqk) and np.array_equal(v[0], rv) and np.array_equal(z[0], rz)
        assert np.array_equal(conv, rconv)
        decay, beta = oracle.gdn_gates(proj, a_log, dt_bias)
        rdecay, rbeta = oracle.ref_gdn_gates(proj[0], a_log, dt_bias)
        assert np.array_equal(decay[0].view(np.uint32), rdecay.view(np.uint32))
        assert np.array_equal(beta[0].view(np.uint32), rbeta.view(np.uint32))
        y, state = oracle.gdn_scan(qk, v, decay, beta, state)
        ry, rstate = oracle.ref_gdn_step(rqk, rv, rdecay, rbeta, rstate)
        assert np.array_equal(y[0], ry)
        assert np.array_equal(state.view(np.uint32), rstate.view(np.uint32))
        out = oracle.gdn_gate_norm(y, z, norm_w)
        assert np.array_equal(out[0], oracle.ref_gdn_gate_norm(ry, rz, norm_w))


def test_gdn_block_prepare_equals_stepwise():
    """Block conv over rows == one position at a time (prefill_gdn.metal:1-3)."""
    rng = np.random.default_rng(401)
    conv_w, *_ = syn.gdn_weights(rng)
    conv, _ = syn.gdn_state(rng)
    proj = syn.gdn_projection(rng, 7)
    qk, v, z, new_conv = oracle.gdn_prepare(proj, conv, conv_w)
    c = conv
    for r in range(7):
        rqk, rv, rz, c = oracle.ref_gdn_prepare(proj[r], c, conv_w)
        assert np.array_equal(qk[r], rqk) and np.array_equal(v[r], rv) and np.array_equal(z[r], rz)
    assert np.array_equal(new_conv, c)


@pytest.mark.parametrize("k", [512, 2048, 4096])
def test_q4_dot_bit_exact(k):
    """q4_dot_reference (kernel_reference.cpp:388-442), adjacent-pairs tree, both chain orders; inputs from
    the reference's banded bf16 generator as in kernel_reference_test.cpp:165-184 and from the bench's."""
    rng = np.random.default_rng(k)
    for trial in range(40):
        if trial % 2:
            n = k + k // 8 * 2 + 2 * (k // 64)
            band = np.zeros(n, np.uint16)
            oracle.ref().ref_xorshift_banded(ctypes.c_uint64(trial + 1), band.ctypes.data_as(oracle._u16p),
                                             ctypes.c_uint32(n))
            x, rest = band[:k].copy(), band[k:]
            words = rest[: k // 4].copy().view(np.uint32)
            scales, biases = rest[k // 4: k // 4 + k // 64].copy(), rest[k // 4 + k // 64:].copy()
        else:
            w, s, b = syn.q4_matrix(rng, 1, k)
            words, scales, biases = w[0], s[0], b[0]
            x = syn.hidden_rows(rng, 1, k)[0]
        for fused in (True, False):
            a = np.float32(oracle.q4_dot(x, words, scales, biases, fused))
            r = np.float32(oracle.ref_q4_dot(x, words, scales, biases, fused))
            assert a.view(np.uint32) == r.view(np.uint32), (trial, fused, a, r)

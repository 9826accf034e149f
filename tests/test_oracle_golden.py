"""The CPU oracle against the committed golden vectors and the reference's known-answer tests.

tests/golden/reference_vectors.npz holds outputs of the reference's own CPU model
(tests/native/kernel_reference.cpp) on the seeded cases of tests/golden/cases.py; the
oracle must reproduce them bit for bit.  The closed forms below restate
tests/native/kernel_reference_test.cpp:15-35, 198-229, 257-275.
"""
import os
import sys

import numpy as np
import pytest

import oracle
from tatara_b200 import synthetic as syn

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import cases  # noqa: E402

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.npz"))


def test_bf16_known_answers():
    vals = np.array([0.0, 1.0, -2.0], np.float32)
    assert list(syn.to_bf16(vals)) == [0x0000, 0x3F80, 0xC000]
    ties = np.array([0x3F808000, 0x3F818000, 0x7F800000], np.uint32).view(np.float32)
    assert list(syn.to_bf16(ties)) == [0x3F80, 0x3F82, 0x7F80]
    lib = oracle.lib()
    # flush-to-zero of subnormal inputs and results (kernel_reference_test.cpp:37-54)
    assert lib.orc_bf16_mul(0x0001, 0x7F00) == 0x0000
    assert lib.orc_bf16_mul(0x3F80, 0x8014) == 0x8000
    assert lib.orc_bf16_mul(0x0080, 0x3F00) == 0x0000
    assert lib.orc_bf16_mul(0x8080, 0x3F00) == 0x8000


@pytest.mark.parametrize("name_inputs", list(cases.attention_cases()), ids=lambda c: c[0])
def test_attention_golden(name_inputs):
    name, (q, gate, keys, values, context) = name_inputs
    assert cases.checksum(q, gate, keys, values) == GOLD[f"{name}/checksum"]
    assert np.array_equal(oracle.attn_decode(q, gate, keys, values, context, cases.CAP),
                          GOLD[f"{name}/decode"])
    rec = GOLD[f"{name}/records"]
    ours = np.stack([oracle.attn_partial(q, keys, values, p * 256, min(context + 1, p * 256 + 256),
                                         cases.CAP) for p in range(rec.shape[1])], axis=1)
    assert np.array_equal(ours.view(np.uint32), rec.view(np.uint32))
    assert np.array_equal(oracle.attn_combine(ours, gate), GOLD[f"{name}/split"])
    # the reference gates partitioned == single kernel byte-equal
    # (tools/native/attention_fixture_probe.cpp:869-878) only on its device; on the CPU model
    # the two families agree to one bf16 step.
    a = syn.from_bf16(GOLD[f"{name}/split"]); b = syn.from_bf16(GOLD[f"{name}/decode"])
    assert np.max(np.abs(a - b)) <= 0.015625


@pytest.mark.parametrize("name_inputs", list(cases.rope_cases()), ids=lambda c: c[0])
def test_rope_golden(name_inputs):
    name, (proj, qw, kw, position) = name_inputs
    assert cases.checksum(proj, qw, kw) == GOLD[f"{name}/checksum"]
    keys = np.zeros((2, cases.CAP, 256), np.uint16); values = np.zeros_like(keys)
    q, _ = oracle.attn_qk_rope(proj[None], qw, kw, keys, values, position, cases.CAP)
    assert np.array_equal(q[0], GOLD[f"{name}/q"])
    assert np.array_equal(keys[:, position], GOLD[f"{name}/k"])
    assert np.array_equal(values[:, position], GOLD[f"{name}/v"])


def test_gdn_chain_golden():
    weights, conv, state, projections = cases.gdn_chain()
    conv_w, a_log, dt_bias, norm_w = weights
    assert cases.checksum(conv_w, a_log, dt_bias, norm_w, *projections) == GOLD["gdn/checksum"]
    for step, proj in enumerate(projections):
        qk, v, z, conv = oracle.gdn_prepare(proj[None], conv, conv_w)
        decay, beta = oracle.gdn_gates(proj[None], a_log, dt_bias)
        y, state = oracle.gdn_scan(qk, v, decay, beta, state)
        gated = oracle.gdn_gate_norm(y, z, norm_w)
        assert np.array_equal(qk[0], GOLD[f"gdn/{step}/qk"])
        assert np.array_equal(decay[0].view(np.uint32), GOLD[f"gdn/{step}/decay"].view(np.uint32))
        assert np.array_equal(beta[0].view(np.uint32), GOLD[f"gdn/{step}/beta"].view(np.uint32))
        assert np.array_equal(y[0], GOLD[f"gdn/{step}/y"])
        assert np.array_equal(gated[0], GOLD[f"gdn/{step}/gated"])
    assert np.array_equal(conv, GOLD["gdn/final_conv"])
    assert np.array_equal(state[3].view(np.uint32), GOLD["gdn/final_state_head3"].view(np.uint32))
    assert np.array_equal(state.astype(np.float64).sum(axis=2), GOLD["gdn/final_state_rowsum"])


def test_scan_equals_repeated_steps():
    """One block scan == the same steps one dispatch at a time (prefill_gdn.metal:198-203)."""
    rng = np.random.default_rng(11)
    _, state = syn.gdn_state(rng)
    conv_w, a_log, dt_bias, _ = syn.gdn_weights(rng)
    conv, _ = syn.gdn_state(rng)
    proj = syn.gdn_projection(rng, 5)
    qk, v, _, _ = oracle.gdn_prepare(proj, conv, conv_w)
    decay, beta = oracle.gdn_gates(proj, a_log, dt_bias)
    y_blk, s_blk = oracle.gdn_scan(qk, v, decay, beta, state, threads=4)
    s = state
    for r in range(5):
        y, s = oracle.gdn_scan(qk[r:r + 1], v[r:r + 1], decay[r:r + 1], beta[r:r + 1], s)
        assert np.array_equal(y[0], y_blk[r])
    assert np.array_equal(s.view(np.uint32), s_blk.view(np.uint32))


def test_attention_context0_closed_form():
    """Context 0, zero gate: out = bf16(v * 0.5) (kernel_reference_test.cpp:257-275)."""
    rng = np.random.default_rng(3)
    keys = syn.normal_bf16(rng, (2, 8, 256)); values = syn.normal_bf16(rng, (2, 8, 256))
    q = syn.normal_bf16(rng, (16, 256)); gate = np.zeros((16, 256), np.uint16)
    out = oracle.attn_decode(q, gate, keys, values, 0, 8)
    for h in range(16):
        want = syn.to_bf16(syn.from_bf16(values[h // 8, 0]) * np.float32(0.5))
        assert np.array_equal(out[h], want)


def test_gdn_identity_closed_form():
    """Zero q/k, beta 0, decay 1: state unchanged, output 0 (kernel_reference_test.cpp:198-229)."""
    rng = np.random.default_rng(4)
    state = syn.from_bf16(syn.normal_bf16(rng, (32, 128, 128)))
    qk = np.zeros((1, 4096), np.uint16); v = syn.normal_bf16(rng, (1, 4096))
    y, s = oracle.gdn_scan(qk, v, np.ones((1, 32), np.float32), np.zeros((1, 32), np.float32), state)
    assert np.array_equal(s, state) and not y.any()


def test_prefill_rows_equal_decode_steps():
    """Prefill row r == a decode step at context_base + r over the same cache."""
    rng = np.random.default_rng(5)
    keys, values = syn.attn_cache(rng, 300, 320)
    q, gate = syn.attn_query(rng, np.arange(290, 300))
    out = oracle.attn_prefill(q, gate, keys, values, 290, 320, row_list=[0, 3, 9], threads=2)
    for r in (0, 3, 9):
        assert np.array_equal(out[r], oracle.attn_decode(q[r], gate[r], keys, values, 290 + r, 320))


@pytest.mark.parametrize("name_inputs", list(cases.q4_cases()), ids=lambda c: c[0])
def test_q4_dot_golden(name_inputs):
    """Affine-Q4 row dot, both chain orders of the reference's CPU model (kernel_reference.cpp:388-442)."""
    name, (x, words, scales, biases) = name_inputs
    assert cases.checksum(x, words, scales, biases) == GOLD[f"{name}/checksum"]
    for order, fused in (("fused", True), ("separate", False)):
        got = np.float32(oracle.q4_dot(x, words, scales, biases, fused))
        assert got.view(np.uint32) == GOLD[f"{name}/{order}"].view(np.uint32)[0]


def test_q4_closed_forms():
    """Known answers: all-zero nibbles leave sum*bias; nibble value v at every column gives
    (v*scale + bias) * sum(x) when the arithmetic is exact (small integers, power-of-two scales)."""
    k = 512
    x = syn.to_bf16(np.ones(k, np.float32))
    scales = syn.to_bf16(np.full(k // 64, 0.5, np.float32))
    biases = syn.to_bf16(np.full(k // 64, -2.0, np.float32))
    for v in (0, 1, 7, 15):
        words = np.full(k // 8, v * 0x11111111, np.uint32)
        for fused in (True, False):
            assert oracle.q4_dot(x, words, scales, biases, fused) == (v * 0.5 - 2.0) * k
    # dequantised weights of the tensor-unit policy
    w = syn.from_bf16(oracle.q4_dequantize(np.full((1, k // 8), 0x76543210, np.uint32), scales[None], biases[None]))
    assert np.array_equal(w[0, :8], np.arange(8) * 0.5 - 2.0)


def test_q4_project_policies_agree_within_rounding():
    """Exact-row and tensor-unit policies differ only by the bf16 rounding of the dequantised weights."""
    rng = np.random.default_rng(5)
    words, scales, biases = syn.q4_matrix(rng, 48, 2048)
    x = syn.hidden_rows(rng, 3, 2048)
    exact = syn.from_bf16(oracle.q4_project(x, words, scales, biases))
    dense = syn.from_bf16(oracle.project_dense(x, oracle.q4_dequantize(words, scales, biases)))
    assert np.abs(exact - dense).max() <= 2e-2
    assert np.dot(exact.ravel(), dense.ravel()) / np.linalg.norm(exact) / np.linalg.norm(dense) >= 0.9999
    assert 0.2 < exact.std() < 2.0


def _band(rng, rows):
    """A verify band: prepared q/k/v rows, gates, conv state, initial state (the GDN step's distributions)."""
    conv_w, a_log, dt_bias, _ = syn.gdn_weights(rng)
    conv, state = syn.gdn_state(rng)
    proj = syn.gdn_projection(rng, rows)
    qk, v, z, new_conv = oracle.gdn_prepare(proj, conv, conv_w)
    decay, beta = oracle.gdn_gates(proj, a_log, dt_bias)
    return proj, conv, conv_w, qk, v, decay, beta, state


def test_gdn_tape_replay_reaches_the_scan_state():
    """Replay of r taped rows onto the pre-band state has the bits of the scan after r rows
    (the generation pin of gdn_tape_replay_blk, prefill_gdn.metal:529-534); the taped scan's own
    outputs are those of the plain scan; layers do not share tape cells."""
    rng = np.random.default_rng(31)
    rows = 16
    proj, conv, conv_w, qk, v, decay, beta, state = _band(rng, rows)
    tape = np.full(oracle.gdn_tape_floats(), np.float32(7.5))
    y, out = oracle.gdn_scan_tape(qk, v, decay, beta, state, tape, tape_layer=39, threads=4)
    y_plain, out_plain = oracle.gdn_scan(qk, v, decay, beta, state, threads=4)
    assert np.array_equal(y, y_plain) and np.array_equal(out, out_plain)
    for r in (0, 1, 5, 16):
        want = state if r == 0 else oracle.gdn_scan(qk[:r], v[:r], decay[:r], beta[:r], state, threads=4)[1]
        assert np.array_equal(oracle.gdn_tape_replay(tape, state, r, 39, threads=4).view(np.uint32), want.view(np.uint32))
    # geometry: layer 39 wrote the last 1/40 of each region and nothing else
    key_off, gate_off = 40 * 16 * 32 * 128, 40 * 16 * 32 * 128 + 40 * 16 * 16 * 128
    touched = tape != np.float32(7.5)
    assert touched[39 * 16 * 32 * 128:key_off].all() and not touched[:39 * 16 * 32 * 128].any()
    assert not touched[key_off:key_off + 39 * 16 * 16 * 128].any() and not touched[gate_off:gate_off + 39 * 16 * 64].any()
    assert np.array_equal(tape[gate_off + 39 * 16 * 64:].reshape(16, 32, 2)[:, :, 0], decay)


def test_gdn_conv_tape_rows_are_the_conv_state_after_each_row():
    rng = np.random.default_rng(32)
    proj, conv, conv_w, *_ = _band(rng, 9)
    conv_tape = np.zeros((40, 16, 3, 8192), np.uint16)
    oracle.gdn_conv_tape(proj, conv, conv_tape, 2)
    for r in range(9):
        assert np.array_equal(conv_tape[2, r], oracle.gdn_prepare(proj[:r + 1], conv, conv_w)[3])
    assert not conv_tape[2, 9:].any() and not conv_tape[:2].any() and not conv_tape[3:].any()

"""GPU parity of the Gated DeltaNet operators against the CPU oracle, through the C ABI."""
import os
import sys

import numpy as np
import pytest
import torch

import oracle
import tatara_b200 as tb
from tatara_b200 import synthetic as syn
from gpu_util import assert_close_bf16, bf16_ulp_distance, dev_bf16, dev_f32, host_f32, host_u16

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import cases  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    c = tb.Context(0)
    yield c
    c.close()


def bf(shape):
    return torch.zeros(shape, dtype=torch.bfloat16, device="cuda")


def gpu_prepare(ctx, proj, conv, conv_w):
    rows = proj.shape[0]
    qk, v, z, new_conv = bf((rows, 4096)), bf((rows, 4096)), bf((rows, 4096)), bf((3, 8192))
    ctx.gdn_prepare(dev_bf16(proj), dev_bf16(conv), dev_bf16(conv_w), qk, v, z, new_conv, rows)
    ctx.sync()
    return host_u16(qk), host_u16(v), host_u16(z), host_u16(new_conv)


def assert_bf16_steps(got, want, what, max_steps=1, max_frac=5e-3):
    dist = bf16_ulp_distance(got, want)
    assert dist.max() <= max_steps, f"{what}: {dist.max()} bf16 steps"
    assert (dist > 0).mean() <= max_frac, f"{what}: {(dist > 0).mean():.3%} elements differ"


@pytest.mark.parametrize("rows", [1, 2, 3, 4, 7, 31, 32, 33, 64, 200])
def test_prepare_matches_oracle(ctx, rows):
    rng = np.random.default_rng(rows)
    conv_w, *_ = syn.gdn_weights(rng)
    conv, _ = syn.gdn_state(rng)
    proj = syn.gdn_projection(rng, rows)
    qk, v, z, new_conv = gpu_prepare(ctx, proj, conv, conv_w)
    oqk, ov, oz, oconv = oracle.gdn_prepare(proj, conv, conv_w)
    assert np.array_equal(z, oz) and np.array_equal(new_conv, oconv)
    assert_bf16_steps(v, ov, "value")
    assert_bf16_steps(qk, oqk, "qk")
    assert_close_bf16(qk, oqk, "qk"); assert_close_bf16(v, ov, "value", max_abs=4e-2)


@pytest.mark.parametrize("rows", [32, 129, 2048 + 5])
def test_prepare_block_kernel_equals_row_kernel_bit_for_bit(ctx, rows):
    """A block of 32 rows or more runs gdn_prepare_block_kernel (a warp per group and run of rows); the same rows
    in calls of at most 31, the conv state carried from call to call, run the one-CTA-per-row kernel: same bits
    in q/k, v, z and the final conv state."""
    rng = np.random.default_rng(600 + rows)
    conv_w, *_ = syn.gdn_weights(rng)
    conv, _ = syn.gdn_state(rng)
    proj = dev_bf16(syn.gdn_projection(rng, rows))
    w = dev_bf16(conv_w)
    qk, v, z, new_conv = bf((rows, 4096)), bf((rows, 4096)), bf((rows, 4096)), bf((3, 8192))
    ctx.gdn_prepare(proj, dev_bf16(conv), w, qk, v, z, new_conv, rows)
    qk2, v2, z2 = bf((rows, 4096)), bf((rows, 4096)), bf((rows, 4096))
    state = [dev_bf16(conv), bf((3, 8192))]
    at = 0
    while at < rows:
        n = min(31, rows - at)
        ctx.gdn_prepare(proj[at:at + n], state[0], w, qk2[at:at + n], v2[at:at + n], z2[at:at + n], state[1], n)
        state.reverse()
        at += n
    ctx.sync()
    assert torch.equal(qk, qk2) and torch.equal(v, v2) and torch.equal(z, z2)
    assert torch.equal(new_conv, state[0])


def test_gates_match_oracle(ctx):
    rng = np.random.default_rng(21)
    _, a_log, dt_bias, _ = syn.gdn_weights(rng)
    proj = syn.gdn_projection(rng, 50)
    decay = torch.zeros((50, 32), device="cuda"); beta = torch.zeros((50, 32), device="cuda")
    ctx.gdn_gates(dev_bf16(proj), dev_bf16(a_log), dev_bf16(dt_bias), decay, beta, 50)
    ctx.sync()
    od, ob = oracle.gdn_gates(proj, a_log, dt_bias)
    np.testing.assert_allclose(host_f32(decay), od, rtol=2e-5, atol=1e-7)
    np.testing.assert_allclose(host_f32(beta), ob, rtol=0, atol=0.0079)  # one bf16 step below 1
    assert (host_f32(beta) != ob).mean() < 0.02


def test_step_and_gate_norm_match_oracle(ctx):
    rng = np.random.default_rng(22)
    conv_w, a_log, dt_bias, norm_w = syn.gdn_weights(rng)
    conv, state = syn.gdn_state(rng)
    proj = syn.gdn_projection(rng, 1)
    oqk, ov, oz, _ = oracle.gdn_prepare(proj, conv, conv_w)
    od, ob = oracle.gdn_gates(proj, a_log, dt_bias)
    oy, ostate = oracle.gdn_scan(oqk, ov, od, ob, state, threads=8)
    y = bf((1, 4096)); state_out = torch.zeros((32, 128, 128), device="cuda")
    ctx.gdn_step(dev_bf16(oqk), dev_bf16(ov), dev_bf16(proj), dev_bf16(a_log), dev_bf16(dt_bias),
                 dev_f32(state), y, state_out)
    ctx.sync()
    assert_close_bf16(host_u16(y), oy, "gdn step y")
    np.testing.assert_allclose(host_f32(state_out), ostate, rtol=1e-4, atol=1e-6)
    out = bf((1, 4096))
    ctx.gdn_gate_norm(dev_bf16(oy), dev_bf16(oz), dev_bf16(norm_w), out, 1)
    ctx.sync()
    want = oracle.gdn_gate_norm(oy, oz, norm_w)
    assert_bf16_steps(host_u16(out), want, "gate_norm")
    # in/out slot aliasing is rejected before anything is enqueued
    st = dev_f32(state)
    with pytest.raises(tb.TataraError) as e:
        ctx.gdn_step(dev_bf16(oqk), dev_bf16(ov), dev_bf16(proj), dev_bf16(a_log), dev_bf16(dt_bias), st, y, st)
    assert e.value.status == tb.STATUS_NAMES.index("StateSlotMismatch")


def make_pools(rng, n):
    convs, states = zip(*[syn.gdn_state(rng) for _ in range(n)])
    conv_pool = torch.zeros((n, 2, 3, 8192), dtype=torch.bfloat16, device="cuda")
    rec_pool = torch.zeros((n, 2, 32, 128, 128), dtype=torch.float32, device="cuda")
    for i in range(n):
        conv_pool[i, 0] = dev_bf16(convs[i]); rec_pool[i, 0] = dev_f32(states[i])
    return convs, states, conv_pool, rec_pool


def lane_table(n, swapped):
    cs, rs = 3 * 8192, 32 * 128 * 128
    a, b = (1, 0) if swapped else (0, 1)
    return tb.Context.gdn_lanes([((2 * i + a) * cs, (2 * i + b) * cs, (2 * i + a) * rs, (2 * i + b) * rs)
                                 for i in range(n)])


def test_fused_decode_batch_4_lanes(ctx):
    """Benchmark config 1: 4 lanes, two consecutive tokens (ping-pong), vs the oracle chain, and
    bit-identical to each lane run alone."""
    rng = np.random.default_rng(23)
    n = 4
    conv_w, a_log, dt_bias, norm_w = syn.gdn_weights(rng)
    convs, states, conv_pool, rec_pool = make_pools(rng, n)
    solo_conv, solo_rec = conv_pool.clone(), rec_pool.clone()
    w = [dev_bf16(x) for x in (conv_w, a_log, dt_bias, norm_w)]
    o_conv, o_state = list(convs), list(states)
    for token in range(2):
        proj = syn.gdn_projection(rng, n)
        y, gated = bf((n, 4096)), bf((n, 4096))
        ctx.gdn_decode_batch(dev_bf16(proj), w[0], w[1], w[2], w[3], conv_pool, rec_pool,
                             lane_table(n, token % 2 == 1), y, gated)
        ctx.sync()
        for i in range(n):
            oqk, ov, oz, o_conv[i] = oracle.gdn_prepare(proj[i:i + 1], o_conv[i], conv_w)
            od, ob = oracle.gdn_gates(proj[i:i + 1], a_log, dt_bias)
            oy, o_state[i] = oracle.gdn_scan(oqk, ov, od, ob, o_state[i], threads=8)
            og = oracle.gdn_gate_norm(oy, oz, norm_w)
            assert_close_bf16(host_u16(y[i]), oy[0], f"token {token} lane {i} y")
            assert_close_bf16(host_u16(gated[i]), og[0], f"token {token} lane {i} gated", max_abs=4e-2)
            slot = (token + 1) % 2
            np.testing.assert_allclose(host_f32(rec_pool[i, slot]), o_state[i], rtol=2e-4, atol=2e-6)
            assert np.array_equal(host_u16(conv_pool[i, slot]), o_conv[i])
            # solo run of the same lane: same bits
            ys, gs = bf((1, 4096)), bf((1, 4096))
            cs, rs = 3 * 8192, 32 * 128 * 128
            a, b = (1, 0) if token % 2 else (0, 1)
            lane = tb.Context.gdn_lanes([((2 * i + a) * cs, (2 * i + b) * cs, (2 * i + a) * rs, (2 * i + b) * rs)])
            ctx.gdn_decode_batch(dev_bf16(proj[i:i + 1]), w[0], w[1], w[2], w[3], solo_conv, solo_rec, lane, ys, gs)
            ctx.sync()
            assert torch.equal(ys[0], y[i]) and torch.equal(gs[0], gated[i])
            assert torch.equal(solo_rec[i, slot], rec_pool[i, slot])


def test_projection_chained_into_step_matches_synchronised_calls(ctx):
    """gdn_project -> fused step -> out projection as they run in a token: every kernel is a programmatic
    dependent of the one before it and starts before that one has finished.  Twelve chained tokens without a
    host synchronisation must leave the bits of the same calls with a synchronisation after each (a load of the
    projection row that slips ahead of the dependency wait reads rows the projection kernel is still writing)."""
    rng = np.random.default_rng(77)
    n, tokens = 3, 12
    conv_w, a_log, dt_bias, norm_w = syn.gdn_weights(rng)
    w = [dev_bf16(x) for x in (conv_w, a_log, dt_bias, norm_w)]
    convs, states, conv_pool, rec_pool = make_pools(rng, n)
    pools = [(conv_pool, rec_pool), (conv_pool.clone(), rec_pool.clone())]
    proj_sets = []
    for _ in range(3):   # rotate weight sets so that the projection kernel really streams from memory
        mats = [syn.q4_matrix(rng, m, 2048) for m in (8192, 4096, 32, 32)]
        held = [(torch.from_numpy(a.view(np.int32)).cuda(), dev_bf16(b), dev_bf16(c)) for a, b, c in mats]
        proj_sets.append((held, tb.Context.q4_matrices(held)))
    out_mat = syn.q4_matrix(rng, 2048, 4096)
    out_held = [(torch.from_numpy(out_mat[0].view(np.int32)).cuda(), dev_bf16(out_mat[1]), dev_bf16(out_mat[2]))]
    out_arr = tb.Context.q4_matrices(out_held)
    hidden0 = dev_bf16(syn.hidden_rows(rng, n, 2048))
    results = []
    for synchronise, (cp, rp) in zip((False, True), pools):
        hidden = hidden0.clone()
        slab, y, gated = bf((n, 12352)), bf((n, 4096)), bf((n, 4096))
        trace = []
        for token in range(tokens):
            ctx.q4_project(hidden, proj_sets[token % 3][1], 2048, slab)
            if synchronise:
                ctx.sync()
            ctx.gdn_decode_batch(slab, w[0], w[1], w[2], w[3], cp, rp, lane_table(n, token % 2 == 1), y, gated)
            if synchronise:
                ctx.sync()
            ctx.q4_project(gated, out_arr, 4096, hidden)
            if synchronise:
                ctx.sync()
                trace.append(hidden.clone())
        ctx.sync()
        results.append((hidden.clone(), cp.clone(), rp.clone()))
    for chained, stepped in zip(results[0], results[1]):
        assert torch.equal(chained, stepped)


def test_layer_walk_with_early_dependents_matches_synchronised_calls(ctx):
    """TATARA_POLICY_GDN_STEP_EARLY_DEPENDENTS: in a walk over TWO gated-delta layers (projection, step, out
    projection per layer, eight tokens, no host synchronisation) the step lets its successors be staged while
    it computes; the bits are those of the same calls with the policy off and a synchronisation after each."""
    rng = np.random.default_rng(78)
    n, tokens, n_layers = 2, 8, 2
    conv_w, a_log, dt_bias, norm_w = syn.gdn_weights(rng)
    w = [dev_bf16(x) for x in (conv_w, a_log, dt_bias, norm_w)]
    layer_pools = [make_pools(rng, n)[2:] for _ in range(n_layers)]
    proj_sets, out_sets = [], []
    for _ in range(n_layers):
        mats = [syn.q4_matrix(rng, m, 2048) for m in (8192, 4096, 32, 32)]
        held = [(torch.from_numpy(a.view(np.int32)).cuda(), dev_bf16(b), dev_bf16(c)) for a, b, c in mats]
        proj_sets.append((held, tb.Context.q4_matrices(held)))
        om = syn.q4_matrix(rng, 2048, 4096)
        oh = [(torch.from_numpy(om[0].view(np.int32)).cuda(), dev_bf16(om[1]), dev_bf16(om[2]))]
        out_sets.append((oh, tb.Context.q4_matrices(oh)))
    hidden0 = dev_bf16(syn.hidden_rows(rng, n, 2048))
    results = []
    for early in (1, 0):
        pools = [(c.clone(), r.clone()) for c, r in layer_pools]
        hidden = hidden0.clone()
        slab, y, gated = bf((n, 12352)), bf((n, 4096)), bf((n, 4096))
        ctx.set_policy(tb.POLICY_GDN_STEP_EARLY_DEPENDENTS, early)
        try:
            for token in range(tokens):
                for layer in range(n_layers):
                    ctx.q4_project(hidden, proj_sets[layer][1], 2048, slab)
                    if not early:
                        ctx.sync()
                    ctx.gdn_decode_batch(slab, w[0], w[1], w[2], w[3], pools[layer][0], pools[layer][1],
                                         lane_table(n, token % 2 == 1), y, gated)
                    if not early:
                        ctx.sync()
                    ctx.q4_project(gated, out_sets[layer][1], 4096, hidden)
                    if not early:
                        ctx.sync()
            ctx.sync()
        finally:
            ctx.set_policy(tb.POLICY_GDN_STEP_EARLY_DEPENDENTS, 0)
        results.append([hidden.clone()] + [t.clone() for pair in pools for t in pair])
    for chained, stepped in zip(results[0], results[1]):
        assert torch.equal(chained, stepped)


def test_fused_equals_unfused_ops(ctx):
    rng = np.random.default_rng(24)
    conv_w, a_log, dt_bias, norm_w = syn.gdn_weights(rng)
    convs, states, conv_pool, rec_pool = make_pools(rng, 1)
    proj = syn.gdn_projection(rng, 1)
    w = [dev_bf16(x) for x in (conv_w, a_log, dt_bias, norm_w)]
    y, gated = bf((1, 4096)), bf((1, 4096))
    ctx.gdn_decode_batch(dev_bf16(proj), w[0], w[1], w[2], w[3], conv_pool, rec_pool, lane_table(1, False), y, gated)
    qk, v, z, new_conv = bf((1, 4096)), bf((1, 4096)), bf((1, 4096)), bf((3, 8192))
    ctx.gdn_prepare(dev_bf16(proj), dev_bf16(convs[0]), w[0], qk, v, z, new_conv, 1)
    y2 = bf((1, 4096)); s2 = torch.zeros((32, 128, 128), device="cuda")
    ctx.gdn_step(qk, v, dev_bf16(proj), w[1], w[2], dev_f32(states[0]), y2, s2)
    g2 = bf((1, 4096))
    ctx.gdn_gate_norm(y2, z, w[3], g2, 1)
    ctx.sync()
    assert torch.equal(y, y2) and torch.equal(gated, g2)
    assert torch.equal(rec_pool[0, 1], s2) and torch.equal(conv_pool[0, 1], new_conv)


@pytest.mark.parametrize("n", [3, 12])
def test_fused_decode_forms_bit_identical(ctx, n):
    """TATARA_POLICY_GDN_DECODE_FORM: the copy-engine data path (default; with few lanes half of the state is
    requested after the projection entries, with many all of it first) and the per-lane register path give
    the same bits in y, gated, the recurrent state and the conv state over two tokens."""
    rng = np.random.default_rng(31 + n)
    conv_w, a_log, dt_bias, norm_w = syn.gdn_weights(rng)
    w = [dev_bf16(x) for x in (conv_w, a_log, dt_bias, norm_w)]
    _, _, conv_pool, rec_pool = make_pools(rng, n)
    projs = [dev_bf16(syn.gdn_projection(rng, n)) for _ in range(2)]
    results = []
    assert ctx.get_policy(tb.POLICY_GDN_DECODE_FORM) == 0
    for form in (0, 1):
        ctx.set_policy(tb.POLICY_GDN_DECODE_FORM, form)
        try:
            cp, rp = conv_pool.clone(), rec_pool.clone()
            outs = []
            for token in range(2):
                y, gated = bf((n, 4096)), bf((n, 4096))
                ctx.gdn_decode_batch(projs[token], w[0], w[1], w[2], w[3], cp, rp, lane_table(n, token % 2 == 1), y, gated)
                outs += [y, gated]
            ctx.sync()
        finally:
            ctx.set_policy(tb.POLICY_GDN_DECODE_FORM, 0)
        results.append(outs + [cp, rp])
    for a, b in zip(*results):
        assert torch.equal(a, b)


@pytest.mark.parametrize("rows", [1, 5, 200])
def test_sequential_scan_prefill_matches_oracle(ctx, rows):
    rng = np.random.default_rng(30 + rows)
    conv_w, a_log, dt_bias, _ = syn.gdn_weights(rng)
    conv, state = syn.gdn_state(rng)
    proj = syn.gdn_projection(rng, rows)
    oqk, ov, _, _ = oracle.gdn_prepare(proj, conv, conv_w)
    od, ob = oracle.gdn_gates(proj, a_log, dt_bias)
    oy, ostate = oracle.gdn_scan(oqk, ov, od, ob, state, threads=8)
    y = bf((rows, 4096)); s = torch.zeros((32, 128, 128), device="cuda")
    ctx.gdn_prefill(dev_bf16(oqk), dev_bf16(ov), dev_f32(od), dev_f32(ob), dev_f32(state), y, s, rows, chunk=1)
    ctx.sync()
    assert_close_bf16(host_u16(y), oy, f"scan rows={rows}")
    np.testing.assert_allclose(host_f32(s), ostate, rtol=5e-4, atol=5e-6)


def test_gdn_chain_matches_reference_golden(ctx):
    gold = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.npz"))
    weights, conv, state, projections = cases.gdn_chain()
    conv_w, a_log, dt_bias, norm_w = weights
    w = [dev_bf16(x) for x in (conv_w, a_log, dt_bias, norm_w)]
    conv_pool = torch.zeros((2, 3, 8192), dtype=torch.bfloat16, device="cuda")
    rec_pool = torch.zeros((2, 32, 128, 128), dtype=torch.float32, device="cuda")
    conv_pool[0] = dev_bf16(conv); rec_pool[0] = dev_f32(state)
    for step, proj in enumerate(projections):
        y, gated = bf((1, 4096)), bf((1, 4096))
        ctx.gdn_decode_batch(dev_bf16(proj[None]), w[0], w[1], w[2], w[3], conv_pool, rec_pool,
                             lane_table(1, step % 2 == 1), y, gated)
        ctx.sync()
        assert_close_bf16(host_u16(y[0]), gold[f"gdn/{step}/y"], f"golden y step {step}")
        assert_close_bf16(host_u16(gated[0]), gold[f"gdn/{step}/gated"], f"golden gated step {step}", max_abs=4e-2)
    final = host_f32(rec_pool[len(projections) % 2])
    np.testing.assert_allclose(final[3], gold["gdn/final_state_head3"], rtol=1e-3, atol=1e-5)
    assert np.array_equal(host_u16(conv_pool[len(projections) % 2]), gold["gdn/final_conv"])


def chunk_scratch(rows):
    return torch.empty(tb.gdn_prefill_scratch_bytes(rows), dtype=torch.uint8, device="cuda")


def state_close(got, want, what):
    from gpu_util import cosine
    err = float(np.max(np.abs(got - want)))
    assert np.isfinite(got).all(), f"{what}: non-finite state"
    assert err <= 2e-2, f"{what}: state max-abs {err:.4g}"
    assert cosine(got, want) >= 0.9999, f"{what}: state cosine {cosine(got, want):.6f}"


@pytest.mark.parametrize("rows,zero_state", [(1, False), (63, False), (64, True), (65, False), (200, False),
                                              (1000, True)])
def test_chunked_prefill_matches_sequential_oracle(ctx, rows, zero_state):
    """Chunk-64 WY form on the tensor cores against the oracle's sequential scan (the reference
    has only the sequential form, prefill_gdn.metal:137-196)."""
    rng = np.random.default_rng(50 + rows)
    conv_w, a_log, dt_bias, _ = syn.gdn_weights(rng)
    conv, state = syn.gdn_state(rng, zero=zero_state)
    proj = syn.gdn_projection(rng, rows)
    oqk, ov, _, _ = oracle.gdn_prepare(proj, conv, conv_w)
    od, ob = oracle.gdn_gates(proj, a_log, dt_bias)
    oy, ostate = oracle.gdn_scan(oqk, ov, od, ob, state, threads=8)
    y = torch.full((rows + 2, 4096), 3.0, dtype=torch.bfloat16, device="cuda")
    s = torch.zeros((32, 128, 128), device="cuda")
    ctx.gdn_prefill(dev_bf16(oqk), dev_bf16(ov), dev_f32(od), dev_f32(ob), dev_f32(state), y, s, rows, chunk=64,
                    scratch=chunk_scratch(rows))
    ctx.sync()
    assert torch.all(y[rows:] == 3.0), "rows past the block were written"
    assert_close_bf16(host_u16(y[:rows]), oy, f"chunked rows={rows}")
    state_close(host_f32(s), ostate, f"chunked rows={rows}")


def test_chunked_prefill_slow_decay_and_split_blocks(ctx):
    """Slowly forgetting heads (decay near 1) stress the intra-chunk solve; two consecutive
    blocks must equal one block (state hand-over), and the chunked form must agree with the
    device's own sequential scan."""
    rng = np.random.default_rng(61)
    rows = 384
    conv_w, _, _, _ = syn.gdn_weights(rng)
    conv, state = syn.gdn_state(rng)
    proj = syn.gdn_projection(rng, rows)
    oqk, ov, _, _ = oracle.gdn_prepare(proj, conv, conv_w)
    od = (1.0 - 0.02 * rng.random((rows, 32))).astype(np.float32)       # decay in [0.98, 1]
    ob = (0.2 + 0.8 * rng.random((rows, 32))).astype(np.float32)
    oy, ostate = oracle.gdn_scan(oqk, ov, od, ob, state, threads=8)
    dq, dv, dd, db = dev_bf16(oqk), dev_bf16(ov), dev_f32(od), dev_f32(ob)
    y = bf((rows, 4096)); s = torch.zeros((32, 128, 128), device="cuda")
    ctx.gdn_prefill(dq, dv, dd, db, dev_f32(state), y, s, rows, chunk=64, scratch=chunk_scratch(rows))
    ctx.sync()
    assert_close_bf16(host_u16(y), oy, "slow decay chunked")
    state_close(host_f32(s), ostate, "slow decay chunked")
    # two blocks of 200 + 184 rows
    y2 = bf((rows, 4096)); mid = torch.zeros_like(s); s2 = torch.zeros_like(s)
    ctx.gdn_prefill(dq, dv, dd, db, dev_f32(state), y2, mid, 200, chunk=64, scratch=chunk_scratch(200))
    ctx.gdn_prefill(dq[200:], dv[200:], dd[200:], db[200:], mid, y2[200:], s2, 184, chunk=64,
                    scratch=chunk_scratch(184))
    ctx.sync()
    assert_close_bf16(host_u16(y2), oy, "two blocks")
    state_close(host_f32(s2), ostate, "two blocks")
    # device sequential scan
    y3 = bf((rows, 4096)); s3 = torch.zeros_like(s)
    ctx.gdn_prefill(dq, dv, dd, db, dev_f32(state), y3, s3, rows, chunk=1)
    ctx.sync()
    assert_close_bf16(host_u16(y), host_u16(y3), "chunked vs device scan")
    with pytest.raises(tb.TataraError) as e:
        ctx.gdn_prefill(dq, dv, dd, db, dev_f32(state), y, s, rows, chunk=64, scratch=chunk_scratch(64))
    assert e.value.status == tb.STATUS_NAMES.index("ScratchTooSmall")
    with pytest.raises(tb.TataraError) as e:
        ctx.gdn_prefill(dq, dv, dd, db, dev_f32(state), y, s, rows, chunk=32, scratch=chunk_scratch(rows))
    assert e.value.status == tb.STATUS_NAMES.index("InvalidDispatchExtent")


def test_chunked_prefill_both_forms_agree_with_the_oracle(ctx):
    """The chunk-64 evaluation has two implementations behind one entry point -- the tensor-memory
    transition form, as one launch with roles (the default for blocks of eight chunks or more) or as two
    launches, and the register-resident mma.sync form: each against the CPU oracle's sequential scan on a
    block with a ragged tail, slowly forgetting heads and a non-zero initial state, the one-launch and
    two-launch forms bit for bit, and the two algebras against each other."""
    rng = np.random.default_rng(404)
    rows = 717
    conv_w, a_log, dt_bias, _ = syn.gdn_weights(rng)
    conv, state = syn.gdn_state(rng)
    proj = syn.gdn_projection(rng, rows)
    oqk, ov, _, _ = oracle.gdn_prepare(proj, conv, conv_w)
    od, ob = oracle.gdn_gates(proj, a_log, dt_bias)
    od = np.ascontiguousarray(od ** 0.02)          # decay close to 1: the state matters across many chunks
    oy, ostate = oracle.gdn_scan(oqk, ov, od, ob, state, threads=8)
    outs = []
    try:
        for form in (0, 2, 1):
            ctx.set_policy(tb.POLICY_GDN_CHUNK_FORM, form)
            y = torch.zeros((rows, 4096), dtype=torch.bfloat16, device="cuda")
            s = torch.zeros((32, 128, 128), dtype=torch.float32, device="cuda")
            ctx.gdn_prefill(dev_bf16(oqk), dev_bf16(ov), dev_f32(od), dev_f32(ob), dev_f32(state), y, s, rows, chunk=64,
                            scratch=chunk_scratch(rows))
            ctx.sync()
            assert_close_bf16(host_u16(y), oy, f"chunk form {form}")
            state_close(host_f32(s), ostate, f"chunk form {form}")
            outs.append(host_u16(y))
    finally:
        ctx.set_policy(tb.POLICY_GDN_CHUNK_FORM, 0)
    assert np.array_equal(outs[0], outs[1]), "one launch with roles and two launches run the same arithmetic"
    assert_close_bf16(outs[0], outs[2], "tensor-memory form vs register form")


def test_chunked_prefill_one_launch_hand_over_on_poisoned_scratch(ctx):
    """The one-launch form hands every unit's planes from the preparation groups to the scan through a ready
    word.  Run it repeatedly on scratch filled with 0xFF (a NaN wherever a plane is read before it was
    written) and require the bits of the two-launch form, where the planes are complete before the scan starts."""
    rows = 4096
    g = torch.Generator(device="cuda").manual_seed(77)
    x = torch.randn((rows, 32, 128), generator=g, device="cuda")
    x = x / x.norm(dim=-1, keepdim=True)
    qk = torch.cat([(x[:, :16] / 128 ** 0.5).reshape(rows, 2048), x[:, 16:].reshape(rows, 2048)], 1).to(torch.bfloat16).contiguous()
    v = torch.randn((rows, 4096), generator=g, device="cuda").to(torch.bfloat16)
    a = torch.randn((rows, 32), generator=g, device="cuda")
    a_log = torch.log(1 + 15 * torch.rand(32, generator=g, device="cuda"))
    decay = torch.exp(-torch.exp(a_log)[None, :] * torch.nn.functional.softplus(a)).contiguous()
    beta = torch.sigmoid(torch.randn((rows, 32), generator=g, device="cuda")).contiguous()
    s0 = torch.randn((32, 128, 128), generator=g, device="cuda") * 0.05
    want = None
    try:
        for it in range(13):
            ctx.set_policy(tb.POLICY_GDN_CHUNK_FORM, 2 if it == 0 else 0)
            scratch = torch.full((tb.gdn_prefill_scratch_bytes(rows),), 0xFF, dtype=torch.uint8, device="cuda")
            y = torch.zeros((rows, 4096), dtype=torch.bfloat16, device="cuda")
            s1 = torch.zeros_like(s0)
            ctx.gdn_prefill(qk, v, decay, beta, s0, y, s1, rows, chunk=64, scratch=scratch)
            ctx.sync()
            if want is None:
                assert torch.isfinite(y.float()).all() and torch.isfinite(s1).all()
                want = (y, s1)
            else:
                assert torch.equal(y, want[0]) and torch.equal(s1, want[1]), f"one-launch run {it} differs from the two-launch form"
    finally:
        ctx.set_policy(tb.POLICY_GDN_CHUNK_FORM, 0)


def test_chunked_prefill_config3_full_size(ctx):
    """Benchmark config 3: 16384 rows, chunk 64, initial state zero; per-token outputs and the
    final f32 state against the sequential oracle."""
    rng = np.random.default_rng(70)
    rows = 16384
    conv_w, a_log, dt_bias, _ = syn.gdn_weights(rng)
    conv, state = syn.gdn_state(rng, zero=True)
    proj = syn.gdn_projection(rng, rows)
    oqk, ov, _, _ = oracle.gdn_prepare(proj, conv, conv_w)
    od, ob = oracle.gdn_gates(proj, a_log, dt_bias)
    oy, ostate = oracle.gdn_scan(oqk, ov, od, ob, state, threads=16)
    y = bf((rows, 4096)); s = torch.zeros((32, 128, 128), device="cuda")
    ctx.gdn_prefill(dev_bf16(oqk), dev_bf16(ov), dev_f32(od), dev_f32(ob), dev_f32(state), y, s, rows, chunk=64,
                    scratch=chunk_scratch(rows))
    ctx.sync()
    assert_close_bf16(host_u16(y), oy, "config 3 outputs")
    state_close(host_f32(s), ostate, "config 3 final state")


# ---- speculative-decode support: tape of a verify band and its replay ------------------------
def _band(rng, rows):
    conv_w, a_log, dt_bias, _ = syn.gdn_weights(rng)
    conv, state = syn.gdn_state(rng)
    proj = syn.gdn_projection(rng, rows)
    qk, v, z, _ = oracle.gdn_prepare(proj, conv, conv_w)
    decay, beta = oracle.gdn_gates(proj, a_log, dt_bias)
    return proj, conv, conv_w, qk, v, decay, beta, state


@pytest.mark.parametrize("rows", [1, 7, 16])
def test_tape_scan_and_replay(ctx, rows):
    """The taped scan computes what the plain scan computes (same bits), its tape matches the oracle's, and
    replaying r rows onto the pre-band state gives the bits of the device scan after r rows."""
    rng = np.random.default_rng(40 + rows)
    proj, conv, conv_w, qk, v, decay, beta, state = _band(rng, rows)
    d_qk, d_v, d_dec, d_beta, d_state = dev_bf16(qk), dev_bf16(v), dev_f32(decay), dev_f32(beta), dev_f32(state)
    tape = torch.full((tb.gdn_tape_bytes() // 4,), 7.5, dtype=torch.float32, device="cuda")
    y, out = bf((rows, 4096)), torch.zeros_like(d_state)
    y0, out0 = bf((rows, 4096)), torch.zeros_like(d_state)
    layer = 17
    ctx.gdn_prefill_tape(d_qk, d_v, d_dec, d_beta, d_state, y, out, rows, tape, layer)
    ctx.gdn_prefill(d_qk, d_v, d_dec, d_beta, d_state, y0, out0, rows, chunk=1)
    ctx.sync()
    assert torch.equal(y.view(torch.int16), y0.view(torch.int16)) and torch.equal(out.view(torch.int32), out0.view(torch.int32))
    want = np.full(oracle.gdn_tape_floats(), np.float32(7.5))
    oracle.gdn_scan_tape(qk, v, decay, beta, state, want, layer, threads=oracle.hardware_threads())
    got = host_f32(tape)
    assert np.array_equal(got == np.float32(7.5), want == np.float32(7.5))          # same cells written
    key_off, gate_off = 40 * 16 * 32 * 128, 40 * 16 * 32 * 128 + 40 * 16 * 16 * 128
    assert np.array_equal(got[key_off:], want[key_off:])                              # keys and gates exactly
    np.testing.assert_allclose(got[:key_off], want[:key_off], rtol=2e-4, atol=2e-5)   # deltas: f32 reduction order
    for r in sorted({0, 1, rows // 2, rows}):
        replayed = torch.zeros_like(d_state)
        ctx.gdn_tape_replay(tape, d_state, replayed, r, layer)
        if r == 0:
            ref = d_state
        else:
            ref, yy = torch.zeros_like(d_state), bf((r, 4096))
            ctx.gdn_prefill(d_qk, d_v, d_dec, d_beta, d_state, yy, ref, r, chunk=1)
        ctx.sync()
        assert torch.equal(replayed.view(torch.int32), ref.view(torch.int32)), f"replay of {r} rows"
    np.testing.assert_allclose(host_f32(out), oracle.gdn_tape_replay(want, state, rows, layer, threads=4), rtol=1e-3, atol=1e-4)


def test_conv_tape_matches_oracle_and_block_prepare(ctx):
    rng = np.random.default_rng(50)
    rows = 11
    proj, conv, conv_w, *_ = _band(rng, rows)
    d_proj, d_conv, d_w = dev_bf16(proj), dev_bf16(conv), dev_bf16(conv_w)
    conv_tape = torch.zeros((40, 16, 3, 8192), dtype=torch.bfloat16, device="cuda")
    assert conv_tape.numel() * 2 == tb.gdn_conv_tape_bytes()
    qk, v, z, new_conv = bf((rows, 4096)), bf((rows, 4096)), bf((rows, 4096)), bf((3, 8192))
    ctx.gdn_prepare_tape(d_proj, d_conv, d_w, qk, v, z, new_conv, rows, conv_tape, 5)
    ctx.sync()
    want = np.zeros((40, 16, 3, 8192), np.uint16)
    oracle.gdn_conv_tape(proj, conv, want, 5)
    assert np.array_equal(host_u16(conv_tape), want)
    pqk, pv, pz, pconv = gpu_prepare(ctx, proj, conv, conv_w)
    assert np.array_equal(host_u16(qk), pqk) and np.array_equal(host_u16(v), pv) and np.array_equal(host_u16(new_conv), pconv)
    assert np.array_equal(host_u16(conv_tape)[5, rows - 1], pconv)


def test_tape_entry_points_reject_long_bands(ctx):
    t = torch.zeros(64, device="cuda")
    before = ctx.launches
    for call in (lambda: ctx.gdn_prefill_tape(t, t, t, t, t, t, torch.zeros(64, device="cuda"), 17, t, 0),
                 lambda: ctx.gdn_prefill_tape(t, t, t, t, t, t, torch.zeros(64, device="cuda"), 4, t, 40),
                 lambda: ctx.gdn_tape_replay(t, t, torch.zeros(64, device="cuda"), 17, 0),
                 lambda: ctx.gdn_prepare_tape(t, t, t, t, t, t, torch.zeros(64, device="cuda"), 17, t, 0)):
        with pytest.raises(tb.TataraError) as e:
            call()
        assert e.value.status == tb.STATUS_NAMES.index("InvalidDispatchExtent")
    assert ctx.launches == before

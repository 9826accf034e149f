"""GPU parity of the gated GQA attention operators against the CPU oracle, through the C ABI.

Gate (stated in the task): max-abs-error <= 2e-2 and cosine >= 0.9999 on bf16 outputs with fp32
accumulation; lane outputs bit-identical alone vs batched.  Intermediate bf16 tensors (rotated
q/k) are compared in bf16 steps: they match the oracle to the bit except where an f32 sin/cos
differs in its last place.
"""
import os
import sys

import numpy as np
import pytest
import torch

import oracle
import tatara_b200 as tb
from tatara_b200 import synthetic as syn
from gpu_util import (assert_close_bf16, bf16_ulp_distance, dev_bf16, host_f32, host_u16)

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import cases  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    c = tb.Context(0)
    yield c
    c.close()


def scratch_for(max_keys, lanes=1):
    return torch.empty(tb.decode_scratch_bytes(max_keys, lanes) // 4, dtype=torch.float32, device="cuda")


def run_decode(ctx, q, gate, keys, values, context, capacity):
    out = torch.full((16, 256), 7.0, dtype=torch.bfloat16, device="cuda")
    ctx.attn_decode(dev_bf16(q), dev_bf16(gate), dev_bf16(keys), dev_bf16(values), context, capacity,
                    out, scratch_for(context + 1))
    ctx.sync()
    return host_u16(out)


@pytest.mark.parametrize("position,rows", [(0, 1), (1, 13), (300, 17), (4096, 1), (262143, 1), (65000, 16),
                                           (0, 32), (7, 77), (261900, 200)])   # 32 rows and more: the block kernel
def test_qk_rope_matches_oracle(ctx, position, rows):
    rng = np.random.default_rng(position + rows)
    cap = position + rows
    qw, kw = syn.attn_weights(rng, unit=False)
    proj = syn.attn_projection(rng, rows)
    # Only the written rows of a (possibly huge) cache are compared; allocate a window.
    keys = torch.zeros((2, cap, 256), dtype=torch.bfloat16, device="cuda")
    values = torch.zeros_like(keys)
    q = torch.zeros((rows, 16, 256), dtype=torch.bfloat16, device="cuda")
    gate = torch.zeros_like(q)
    ctx.attn_qk_rope(dev_bf16(proj), dev_bf16(qw), dev_bf16(kw), q, gate, keys, values, position, cap, rows)
    ctx.sync()
    big_k = np.zeros((2, cap, 256), np.uint16); big_v = np.zeros_like(big_k)
    oq, og = oracle.attn_qk_rope(proj, qw, kw, big_k, big_v, position, cap)
    ok, ov = big_k[:, position:], big_v[:, position:]
    gq, gk = host_u16(q), host_u16(keys[:, position:])
    assert np.array_equal(host_u16(gate), og)
    assert np.array_equal(host_u16(values[:, position:]), ov)
    for got, want, name in ((gq, oq, "q"), (gk, ok, "k")):
        dist = bf16_ulp_distance(got, want)
        assert dist.max() <= 1, f"{name}: {dist.max()} bf16 steps"
        assert (dist > 0).mean() < 2e-3, f"{name}: {(dist > 0).mean():.4%} elements differ"
    # untouched cache rows stay zero (canary)
    if position > 0:
        assert not host_u16(keys[:, :min(position, 64)]).any()


@pytest.mark.parametrize("position,rows", [(0, 32), (1000, 129), (100000, 300)])
def test_qk_rope_block_kernel_equals_row_kernel_bit_for_bit(ctx, position, rows):
    """A block of 32 rows or more runs attn_qk_rope_block_kernel (a warp per row, the row's angles computed once);
    the same rows in calls of at most 31 run the 18-CTAs-per-row kernel: same bits in q, gate and the appended
    K/V rows."""
    rng = np.random.default_rng(4000 + position + rows)
    cap = position + rows + 2
    qw, kw = syn.attn_weights(rng, unit=False)
    proj = dev_bf16(syn.attn_projection(rng, rows))
    dq, dk = dev_bf16(qw), dev_bf16(kw)
    outs = []
    for chunk in (rows, 31):
        keys = torch.zeros((2, cap, 256), dtype=torch.bfloat16, device="cuda")
        values = torch.zeros_like(keys)
        q = torch.zeros((rows, 16, 256), dtype=torch.bfloat16, device="cuda")
        gate = torch.zeros_like(q)
        at = 0
        while at < rows:
            n = min(chunk, rows - at)
            ctx.attn_qk_rope(proj[at:at + n], dq, dk, q[at:at + n], gate[at:at + n], keys, values, position + at, cap, n)
            at += n
        ctx.sync()
        outs.append((q, gate, keys, values))
    for a, b in zip(*outs):
        assert torch.equal(a, b)


@pytest.mark.parametrize("context", [0, 1, 15, 16, 17, 63, 64, 65, 255, 256, 257, 1000, 4095, 4096,
                                     4735, 4736, 8192, 20000])
def test_decode_matches_oracle(ctx, context):
    rng = np.random.default_rng(context)
    cap = context + 3
    keys, values = syn.attn_cache(rng, context + 1, cap)
    q, gate = syn.attn_query(rng, np.array([context]))
    got = run_decode(ctx, q[0], gate[0], keys, values, context, cap)
    want = oracle.attn_decode(q[0], gate[0], keys, values, context, cap, threads=8)
    assert_close_bf16(got, want, f"decode ctx={context}")


@pytest.mark.parametrize("context", [32767, 65535, 131071, 262143])
def test_decode_matches_oracle_long_context(ctx, context):
    """The contexts the benchmark figures are quoted on, against the CPU oracle.  The cache is
    drawn on the device (the benchmark's generator) and copied to the host for the oracle, whose
    decode over 262 144 keys takes a fraction of a second on the host threads.  The reference's own
    long-context gate on bf16 outputs is max-abs <= 0.015625
    (tools/native/attention_fixture_probe.cpp:884, 963-968); this repo's is written in gpu_util."""
    from bench_workloads import device_cache, device_query
    n = cap = context + 1
    keys, values = device_cache(torch, n, cap, 400 + context % 7)
    q, gate = device_query(torch, [context], 401)
    out = torch.full((16, 256), 7.0, dtype=torch.bfloat16, device="cuda")
    ctx.attn_decode(q[0].contiguous(), gate[0].contiguous(), keys, values, context, cap, out, scratch_for(n))
    ctx.sync()
    want = oracle.attn_decode(host_u16(q[0]), host_u16(gate[0]), host_u16(keys), host_u16(values), context, cap,
                              threads=oracle.hardware_threads())
    err, _ = assert_close_bf16(host_u16(out), want, f"decode ctx={context}")
    assert err <= 0.015625, f"decode ctx={context}: max-abs {err} above the reference's long-context gate"


@pytest.mark.parametrize("context", [0, 16, 200, 4500, 32767, 100000])
def test_decode_merge_in_the_partition_launch_equals_the_two_kernel_form(ctx, context):
    """TATARA_POLICY_DECODE_FUSED_MERGE: a single-lane decode merges its records in a second kernel (default)
    or in the partition kernel's own launch; the bits are equal, call after call (the item counters of the
    fused form are put back to zero by the launch that used them), and nothing past the row is written."""
    rng = np.random.default_rng(977 + context)
    cap = context + 3
    keys, values = syn.attn_cache(rng, context + 1, cap)
    q, gate = syn.attn_query(rng, [context])
    dq, dg, dk, dv = dev_bf16(q), dev_bf16(gate), dev_bf16(keys), dev_bf16(values)
    scratch = scratch_for(context + 1)
    assert ctx.get_policy(tb.POLICY_DECODE_FUSED_MERGE) == 0
    launches = ctx.launches
    two = torch.full((2, 16, 256), 7.0, dtype=torch.bfloat16, device="cuda")
    ctx.attn_decode(dq, dg, dk, dv, context, cap, two, scratch)
    assert ctx.launches - launches == 2          # partition kernel + merge kernel
    fused = []
    ctx.set_policy(tb.POLICY_DECODE_FUSED_MERGE, 1)
    try:
        for _ in range(3):
            out = torch.full((2, 16, 256), 7.0, dtype=torch.bfloat16, device="cuda")
            ctx.attn_decode(dq, dg, dk, dv, context, cap, out, scratch)
            fused.append(out)
        assert ctx.launches - launches == 5      # one kernel per call
    finally:
        ctx.set_policy(tb.POLICY_DECODE_FUSED_MERGE, 0)
    ctx.sync()
    for out in fused:
        assert torch.equal(out, two)
    assert (two[1].float() == 7.0).all()


@pytest.mark.parametrize("name_inputs", list(cases.attention_cases()), ids=lambda c: c[0])
def test_decode_matches_reference_golden(ctx, name_inputs):
    """The committed outputs of the reference's own CPU model (tests/golden)."""
    gold = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.npz"))
    name, (q, gate, keys, values, context) = name_inputs
    got = run_decode(ctx, q, gate, keys, values, context, cases.CAP)
    assert_close_bf16(got, gold[f"{name}/decode"], name)
    assert_close_bf16(got, gold[f"{name}/split"], name + " (partitioned family)")


def test_partial_records_and_combine(ctx):
    """Split-KV building blocks: two key ranges -> records -> combine == one decode."""
    rng = np.random.default_rng(77)
    context, cap = 9000, 9100
    keys, values = syn.attn_cache(rng, context + 1, cap)
    q, gate = syn.attn_query(rng, np.array([context]))
    dq, dk, dv, dg = dev_bf16(q[0]), dev_bf16(keys), dev_bf16(values), dev_bf16(gate[0])
    cut = 5003
    recs = torch.zeros((2, 16, 258), dtype=torch.float32, device="cuda")
    ctx.attn_decode_partial(dq, dk, dv, 0, cut, cap, recs[0], scratch_for(cut))
    ctx.attn_decode_partial(dq, dk, dv, cut, context + 1, cap, recs[1], scratch_for(context + 1 - cut))
    out = torch.zeros((16, 256), dtype=torch.bfloat16, device="cuda")
    # all-gather layout [rank][head][258]: head stride 258, part stride 16*258
    ctx.attn_combine(recs, 2, 258, 16 * 258, dg, out)
    ctx.sync()
    want = oracle.attn_decode(q[0], gate[0], keys, values, context, cap, threads=8)
    assert_close_bf16(host_u16(out), want, "partial+combine")
    # each record against the oracle's record: compare o/l and the log-sum-exp
    r = host_f32(recs)
    for i, (b, e) in enumerate(((0, cut), (cut, context + 1))):
        o = oracle.attn_partial(q[0], keys, values, b, e, cap, threads=8)
        np.testing.assert_allclose(r[i, :, :256] / r[i, :, 257:258], o[:, :256] / o[:, 257:258], atol=5e-3)
        np.testing.assert_allclose(r[i, :, 256] + np.log(r[i, :, 257]), o[:, 256] + np.log(o[:, 257]),
                                   atol=2e-3)
    # oracle combine of the GPU's records
    rec_hpl = np.ascontiguousarray(r.transpose(1, 0, 2))
    assert_close_bf16(oracle.attn_combine(rec_hpl, gate[0]), want, "oracle combine of GPU records")


def test_batched_lanes_bit_identical_to_solo(ctx):
    """Lossless concurrency: each lane's output bits are the same alone and inside a batch."""
    rng = np.random.default_rng(5)
    contexts = [0, 37, 256, 4096, 4800, 9999, 20000, 777, 32767]   # up to the longest lane of benchmark config 4b
    cap = 32768
    n = len(contexts)
    kpool = torch.zeros((n, 2, cap, 256), dtype=torch.bfloat16, device="cuda")
    vpool = torch.zeros_like(kpool)
    q_all, g_all = [], []
    for i, c in enumerate(contexts):
        k, v = syn.attn_cache(rng, c + 1, c + 1)
        kpool[i, :, :c + 1] = dev_bf16(k); vpool[i, :, :c + 1] = dev_bf16(v)
        q, g = syn.attn_query(rng, np.array([c]))
        q_all.append(q[0]); g_all.append(g[0])
    dq, dg = dev_bf16(np.stack(q_all)), dev_bf16(np.stack(g_all))
    stripe = 2 * cap * 256
    lanes = tb.Context.attn_lanes([(i * stripe, c) for i, c in enumerate(contexts)])
    out = torch.zeros((n, 16, 256), dtype=torch.bfloat16, device="cuda")
    ctx.attn_decode_batch(dq, dg, kpool, vpool, lanes, cap, out, scratch_for(max(contexts) + 1, n))
    ctx.sync()
    batched = host_u16(out)
    for i, c in enumerate(contexts):
        solo = torch.zeros((16, 256), dtype=torch.bfloat16, device="cuda")
        ctx.attn_decode(dq[i], dg[i], kpool[i], vpool[i], c, cap, solo, scratch_for(c + 1))
        ctx.sync()
        assert np.array_equal(host_u16(solo), batched[i]), f"lane {i} (ctx {c}) differs from its solo run"
    # a different batch composition and order gives the same bits too
    order = [6, 2, 4]
    lanes2 = tb.Context.attn_lanes([(i * stripe, contexts[i]) for i in order])
    out2 = torch.zeros((len(order), 16, 256), dtype=torch.bfloat16, device="cuda")
    ctx.attn_decode_batch(dq[order].contiguous(), dg[order].contiguous(), kpool, vpool, lanes2, cap, out2,
                          scratch_for(max(contexts) + 1, len(order)))
    ctx.sync()
    assert np.array_equal(host_u16(out2), batched[order])
    # and the batch agrees with the oracle
    for i in (5, 8):
        want = oracle.attn_decode(q_all[i], g_all[i], host_u16(kpool[i]), host_u16(vpool[i]), contexts[i], cap,
                                  threads=8)
        assert_close_bf16(batched[i], want, f"batched lane {i} vs oracle")


def test_qk_rope_then_decode_step(ctx):
    """A full decode step: append the new token's K/V at `context`, then attend 0..context."""
    rng = np.random.default_rng(9)
    context, cap = 300, 512
    qw, kw = syn.attn_weights(rng, unit=False)
    keys = np.zeros((2, cap, 256), np.uint16); values = np.zeros_like(keys)
    hist = syn.attn_projection(rng, context)
    oracle.attn_qk_rope(hist, qw, kw, keys, values, 0, cap)
    step = syn.attn_projection(rng, 1)
    dk, dv = dev_bf16(keys), dev_bf16(values)
    q = torch.zeros((1, 16, 256), dtype=torch.bfloat16, device="cuda"); gate = torch.zeros_like(q)
    ctx.attn_qk_rope(dev_bf16(step), dev_bf16(qw), dev_bf16(kw), q, gate, dk, dv, context, cap, 1)
    out = torch.zeros((16, 256), dtype=torch.bfloat16, device="cuda")
    ctx.attn_decode(q, gate, dk, dv, context, cap, out, scratch_for(context + 1))
    ctx.sync()
    oq, og = oracle.attn_qk_rope(step, qw, kw, keys, values, context, cap)
    want = oracle.attn_decode(oq[0], og[0], keys, values, context, cap)
    assert_close_bf16(host_u16(out), want, "rope+decode step")


def test_attention_layer_chained_matches_synchronised_calls(ctx):
    """attn_project -> qk_rope -> decode (partition + merge) -> out projection for three lanes, sixteen tokens
    in a row without a host synchronisation: the kernels are programmatic dependents that start early (the
    partition kernel requests K/V rows of older partitions before its dependency wait, the projections their
    weights).  The bits must be those of the same calls with a synchronisation after each; the contexts
    cross a 128-key partition boundary on the way."""
    rng = np.random.default_rng(31)
    cap, tokens = 512, 16
    starts = [120, 250, 7]
    n = len(starts)
    qw, kw = (dev_bf16(w) for w in syn.attn_weights(rng, unit=False))
    in_sets = []
    for _ in range(3):
        mats = [syn.q4_matrix(rng, m, 2048) for m in (8192, 512, 512)]
        held = [(torch.from_numpy(a.view(np.int32)).cuda(), dev_bf16(b), dev_bf16(c)) for a, b, c in mats]
        in_sets.append((held, tb.Context.q4_matrices(held)))
    out_mat = syn.q4_matrix(rng, 2048, 4096)
    out_held = [(torch.from_numpy(out_mat[0].view(np.int32)).cuda(), dev_bf16(out_mat[1]), dev_bf16(out_mat[2]))]
    out_arr = tb.Context.q4_matrices(out_held)
    hidden0 = dev_bf16(syn.hidden_rows(rng, n, 2048))
    g = torch.Generator(device="cuda").manual_seed(5)
    kpool0 = torch.randn((n, 2, cap, 256), generator=g, device="cuda").to(torch.bfloat16)
    vpool0 = torch.randn((n, 2, cap, 256), generator=g, device="cuda").to(torch.bfloat16)
    results = []
    for synchronise in (False, True):
        kpool, vpool, hidden = kpool0.clone(), vpool0.clone(), hidden0.clone()
        slab = torch.zeros((n, 9216), dtype=torch.bfloat16, device="cuda")
        q = torch.zeros((n, 16, 256), dtype=torch.bfloat16, device="cuda"); gate = torch.zeros_like(q)
        attended = torch.zeros((n, 4096), dtype=torch.bfloat16, device="cuda")
        scratch = scratch_for(cap, n)
        for token in range(tokens):
            lanes = tb.Context.attn_lanes([(i * 2 * cap * 256, c + token) for i, c in enumerate(starts)])
            steps = (lambda: ctx.q4_project(hidden, in_sets[token % 3][1], 2048, slab),
                     lambda: ctx.attn_qk_rope_batch(slab, qw, kw, q, gate, kpool, vpool, cap, lanes),
                     lambda: ctx.attn_decode_batch(q, gate, kpool, vpool, lanes, cap, attended, scratch),
                     lambda: ctx.q4_project(attended, out_arr, 4096, hidden))
            for step in steps:
                step()
                if synchronise:
                    ctx.sync()
        ctx.sync()
        results.append((hidden.clone(), kpool, vpool))
    for chained, stepped in zip(results[0], results[1]):
        assert torch.equal(chained, stepped)


def test_batched_qk_rope_matches_solo(ctx):
    rng = np.random.default_rng(10)
    cap, contexts = 64, [0, 5, 63]
    qw, kw = syn.attn_weights(rng, unit=False)
    proj = syn.attn_projection(rng, len(contexts))
    kpool = torch.zeros((len(contexts), 2, cap, 256), dtype=torch.bfloat16, device="cuda"); vpool = torch.zeros_like(kpool)
    q = torch.zeros((len(contexts), 16, 256), dtype=torch.bfloat16, device="cuda"); gate = torch.zeros_like(q)
    lanes = tb.Context.attn_lanes([(i * 2 * cap * 256, c) for i, c in enumerate(contexts)])
    ctx.attn_qk_rope_batch(dev_bf16(proj), dev_bf16(qw), dev_bf16(kw), q, gate, kpool, vpool, cap, lanes)
    ctx.sync()
    for i, c in enumerate(contexts):
        k1 = torch.zeros((2, cap, 256), dtype=torch.bfloat16, device="cuda"); v1 = torch.zeros_like(k1)
        q1 = torch.zeros((1, 16, 256), dtype=torch.bfloat16, device="cuda"); g1 = torch.zeros_like(q1)
        ctx.attn_qk_rope(dev_bf16(proj[i:i + 1]), dev_bf16(qw), dev_bf16(kw), q1, g1, k1, v1, c, cap, 1)
        ctx.sync()
        assert torch.equal(q1[0], q[i]) and torch.equal(g1[0], gate[i])
        assert torch.equal(k1, kpool[i]) and torch.equal(v1, vpool[i])


def test_prefill_control_rows_match_oracle(ctx):
    rng = np.random.default_rng(11)
    base, rows, cap = 250, 300, 600
    keys, values = syn.attn_cache(rng, base + rows, cap)
    q, gate = syn.attn_query(rng, np.arange(base, base + rows))
    out = torch.zeros((rows, 16, 256), dtype=torch.bfloat16, device="cuda")
    ctx.attn_prefill_control(dev_bf16(q), dev_bf16(gate), dev_bf16(keys), dev_bf16(values), base, rows, cap,
                             out, scratch_for(base + rows, min(rows, 256)))
    ctx.sync()
    pick = [0, 1, 5, 6, 255, 256, 299]
    want = oracle.attn_prefill(q, gate, keys, values, base, cap, row_list=pick, threads=8)
    got = host_u16(out)
    for r in pick:
        assert_close_bf16(got[r], want[r], f"prefill control row {r}")


def test_full_size_decode_properties(ctx):
    """The headline size (context 262143, unit-variance unnormalised keys: a peaked softmax): the CPU
    oracle on the same inputs, plus size-independent properties.  (a) v constant => out =
    v * sigmoid(gate) whatever the scores; (b) split anywhere + combine equals the unsplit decode;
    (c) deterministic run to run."""
    context = 262143
    cap = context + 1
    g = torch.Generator(device="cuda").manual_seed(3)
    keys = torch.randn((2, cap, 256), generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    values = torch.randn((2, cap, 256), generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    q = torch.randn((16, 256), generator=g, device="cuda").to(torch.bfloat16)
    gate = torch.randn((16, 256), generator=g, device="cuda").to(torch.bfloat16)
    scratch = scratch_for(cap)
    out = torch.zeros((16, 256), dtype=torch.bfloat16, device="cuda")
    ctx.attn_decode(q, gate, keys, values, context, cap, out, scratch)
    again = torch.zeros_like(out)
    ctx.attn_decode(q, gate, keys, values, context, cap, again, scratch)
    ctx.sync()
    assert torch.equal(out, again)
    want = oracle.attn_decode(host_u16(q), host_u16(gate), host_u16(keys), host_u16(values), context, cap,
                              threads=oracle.hardware_threads())
    assert_close_bf16(host_u16(out), want, "decode ctx=262143 (peaked softmax) vs oracle")
    recs = torch.zeros((4, 16, 258), dtype=torch.float32, device="cuda")
    cuts = [0, 70001, 131072, 200017, cap]
    for i in range(4):
        ctx.attn_decode_partial(q, keys, values, cuts[i], cuts[i + 1], cap, recs[i], scratch)
    merged = torch.zeros_like(out)
    ctx.attn_combine(recs, 4, 258, 16 * 258, gate, merged)
    ctx.sync()
    assert_close_bf16(host_u16(merged), host_u16(out), "4-way split vs unsplit")
    const_v = torch.ones_like(values) * 0.75
    ctx.attn_decode(q, gate, keys, const_v, context, cap, out, scratch)
    ctx.sync()
    want = (0.75 * torch.sigmoid(gate.float())).to(torch.bfloat16)
    assert_close_bf16(host_u16(out), host_u16(want), "constant-v closed form", max_abs=8e-3)


def test_argument_validation_enqueues_nothing(ctx):
    q = torch.zeros((16, 256), dtype=torch.bfloat16, device="cuda")
    kv = torch.zeros((2, 8, 256), dtype=torch.bfloat16, device="cuda")
    out = torch.full((16, 256), 3.0, dtype=torch.bfloat16, device="cuda")
    sc = scratch_for(8)
    before = ctx.launches
    with pytest.raises(tb.TataraError) as e:
        ctx.attn_decode(q, q, kv, kv, 8, 8, out, sc)            # context == capacity
    assert e.value.status == tb.STATUS_NAMES.index("ContextOutOfRange")
    with pytest.raises(tb.TataraError) as e:
        ctx.attn_decode(q, q, None, kv, 3, 8, out, sc)
    assert e.value.status == tb.STATUS_NAMES.index("InvalidBuffer")
    with pytest.raises(tb.TataraError) as e:
        ctx.attn_decode(q, q, kv, kv, 3, 8, out, sc[:16])
    assert e.value.status == tb.STATUS_NAMES.index("ScratchTooSmall")
    with pytest.raises(tb.TataraError) as e:
        ctx.attn_decode_batch(q, q, kv, kv, tb.Context.attn_lanes([]), 8, out, sc)
    assert e.value.status == tb.STATUS_NAMES.index("InvalidStreamGroup")
    with pytest.raises(tb.TataraError) as e:
        ctx.attn_qk_rope(q, q, q, q, q, kv, kv, 7, 8, 2)
    assert e.value.status == tb.STATUS_NAMES.index("ContextOutOfRange")
    ctx.sync()
    assert ctx.launches == before
    assert torch.all(out == 3.0)

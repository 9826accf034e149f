"""GPU parity of the tcgen05 causal block prefill against the CPU oracle and against the
numerical-control family (every row through the decode kernels), through the C ABI.

The reference gates its fast prefill families against its partial+combine control with
max |d|/(1+|ref|) <= 0.02 and relative-L2 <= 0.02 (tools/native/attention_fixture_probe.cpp:982,
1237-1269); this repo's gate is tighter: max-abs <= 2e-2 and cosine >= 0.9999.
"""
import numpy as np
import pytest
import torch

import oracle
import tatara_b200 as tb
from tatara_b200 import synthetic as syn
from gpu_util import assert_close_bf16, dev_bf16, host_u16

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    c = tb.Context(0)
    yield c
    c.close()


def run_prefill(ctx, q, gate, keys, values, base, rows, cap, pad_rows=3):
    out = torch.full((rows + pad_rows, 16, 256), 5.0, dtype=torch.bfloat16, device="cuda")
    ctx.attn_prefill(dev_bf16(q), dev_bf16(gate), dev_bf16(keys), dev_bf16(values), base, rows, cap, out)
    ctx.sync()
    got = host_u16(out)
    assert (syn.from_bf16(got[rows:]) == 5.0).all(), "rows past the block were written"
    return got[:rows]


@pytest.mark.parametrize("base,rows", [(0, 1), (0, 64), (0, 128), (0, 129), (0, 200), (300, 77), (64, 256),
                                       (1000, 130), (5, 513),
                                       (2047, 16), (777, 5),    # the 16-row verify band of speculative decoding
                                       # the reference's own chunk shapes: a first chunk of 256 rows at position 0, then
                                       # chunks of at most 2048 rows at a large context_base (14336 = 256 + 6*2048 + 1792:
                                       # the last full chunk of a 16384-token prompt;
                                       # include/tatara/runtime/prefill_geometry.h:13-15, tools/native/tatara_serve.cpp:485-497)
                                       (0, 256), (256, 2048), (14336, 2048)])
def test_prefill_matches_oracle(ctx, base, rows):
    rng = np.random.default_rng(base * 7 + rows)
    cap = base + rows + 5
    keys, values = syn.attn_cache(rng, base + rows, cap)
    # stale data past the visible keys must not leak in (the reference zero-fills its buffers;
    # put a poison value there to prove the kernel never reads it into the result)
    keys[:, base + rows:] = 0x7F80
    values[:, base + rows:] = 0x7F80
    q, gate = syn.attn_query(rng, np.arange(base, base + rows))
    got = run_prefill(ctx, q, gate, keys, values, base, rows, cap)
    pick = sorted(set(int(r) for r in [0, min(1, rows - 1), rows // 2, rows - 1] + [r for r in (127, 128, 255, 256, 1023, 1024) if r < rows] +
                                   list(rng.integers(0, rows, size=12))))
    want = oracle.attn_prefill(q, gate, keys, values, base, cap, row_list=pick, threads=8)
    for r in pick:
        assert_close_bf16(got[r], want[r], f"prefill base={base} rows={rows} row {r}")


def test_prefill_matches_control_family_all_rows(ctx):
    rng = np.random.default_rng(99)
    base, rows, cap = 700, 1500, 2304
    keys, values = syn.attn_cache(rng, base + rows, cap)
    q, gate = syn.attn_query(rng, np.arange(base, base + rows))
    got = run_prefill(ctx, q, gate, keys, values, base, rows, cap)
    control = torch.zeros((rows, 16, 256), dtype=torch.bfloat16, device="cuda")
    scratch = torch.empty(tb.decode_scratch_bytes(base + rows, 256) // 4, dtype=torch.float32, device="cuda")
    ctx.attn_prefill_control(dev_bf16(q), dev_bf16(gate), dev_bf16(keys), dev_bf16(values), base, rows, cap,
                             control, scratch)
    ctx.sync()
    assert_close_bf16(got, host_u16(control), "tcgen05 prefill vs control family")
    again = run_prefill(ctx, q, gate, keys, values, base, rows, cap)
    assert np.array_equal(got, again), "prefill is not deterministic run to run"


@pytest.mark.parametrize("base,rows", [(0, 1), (0, 129), (300, 77), (5, 513), (256, 2048)])
def test_prefill_pair_form_equals_single_cta_form_bit_for_bit(ctx, base, rows):
    """TATARA_POLICY_ATTN_PREFILL_FORM: the CTA-pair kernel (default) and the one-CTA kernel accumulate every
    score and every output element over the same k-steps in the same order."""
    rng = np.random.default_rng(base * 11 + rows)
    cap = base + rows + 9
    keys, values = syn.attn_cache(rng, base + rows, cap)
    q, gate = syn.attn_query(rng, np.arange(base, base + rows))
    assert ctx.get_policy(tb.POLICY_ATTN_PREFILL_FORM) == 0
    pair = run_prefill(ctx, q, gate, keys, values, base, rows, cap)
    ctx.set_policy(tb.POLICY_ATTN_PREFILL_FORM, 1)
    try:
        single = run_prefill(ctx, q, gate, keys, values, base, rows, cap)
    finally:
        ctx.set_policy(tb.POLICY_ATTN_PREFILL_FORM, 0)
    assert np.array_equal(pair, single)
    with pytest.raises(tb.TataraError):
        ctx.set_policy(tb.POLICY_ATTN_PREFILL_FORM, 2)


def test_prefill_config2_full_size_sampled(ctx):
    """Benchmark config 2: 16384 rows from position 0.  Row-sampled oracle (tile-boundary rows
    included) plus the control family on a slice of rows."""
    from bench_workloads import device_cache, device_query
    rows = cap = 16384
    keys, values = device_cache(torch, rows, cap, 21)
    q, gate = device_query(torch, list(range(rows)), 22)
    out = torch.zeros((rows, 16, 256), dtype=torch.bfloat16, device="cuda")
    ctx.attn_prefill(q, gate, keys, values, 0, rows, cap, out)
    ctx.sync()
    got = host_u16(out)
    pick = [0, 1, 63, 64, 127, 128, 255, 256, 2047, 2048, 8191, 12345, 16383]
    hq, hg, hk, hv = host_u16(q), host_u16(gate), host_u16(keys), host_u16(values)
    want = oracle.attn_prefill(hq, hg, hk, hv, 0, cap, row_list=pick, threads=8)
    for r in pick:
        assert_close_bf16(got[r], want[r], f"config 2 row {r}")
    # control family on rows 16000..16255 (one launch of 256 decode lanes)
    sl = slice(16000, 16256)
    control = torch.zeros((256, 16, 256), dtype=torch.bfloat16, device="cuda")
    scratch = torch.empty(tb.decode_scratch_bytes(cap, 256) // 4, dtype=torch.float32, device="cuda")
    ctx.attn_prefill_control(q[sl], gate[sl], keys, values, 16000, 256, cap, control, scratch)
    ctx.sync()
    assert_close_bf16(got[sl], host_u16(control), "config 2 vs control rows 16000..16255")


def test_prefill_argument_validation(ctx):
    t = torch.zeros((4, 16, 256), dtype=torch.bfloat16, device="cuda")
    kv = torch.zeros((2, 8, 256), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(tb.TataraError) as e:
        ctx.attn_prefill(t, t, kv, kv, 6, 4, 8, t)
    assert e.value.status == tb.STATUS_NAMES.index("ContextOutOfRange")
    with pytest.raises(tb.TataraError) as e:
        ctx.attn_prefill(t, t, kv, kv, 0, 0, 8, t)
    assert e.value.status == tb.STATUS_NAMES.index("InvalidDispatchExtent")

"""GPU parity of the affine-Q4 projections (hidden -> projection row, gated row -> hidden) through the C ABI.

Exact-row policy: bit-identical to the oracle's fused chain (the reference's q4_dot sequence) for every
row count.  Tensor-unit policy: dequantised weights bit-identical to the oracle's; the GEMM within one bf16
step of the oracle's f32 accumulation (the order of a matrix unit's accumulation is not specified).
"""
import numpy as np
import pytest
import torch

import oracle
import tatara_b200 as tb
from tatara_b200 import synthetic as syn
from gpu_util import assert_close_bf16, bf16_ulp_distance, dev_bf16, host_u16

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    c = tb.Context(0)
    yield c
    c.close()


def dev_mats(mats):
    """[(words u32, scales u16, biases u16)] -> device tensors + the tatara_q4_matrix array."""
    held = [(torch.from_numpy(w.view(np.int32)).cuda(), dev_bf16(s), dev_bf16(b)) for w, s, b in mats]
    return held, tb.Context.q4_matrices(held)


def oracle_project(x, mats, threads):
    return np.concatenate([oracle.q4_project(x, w, s, b, fused=True, threads=threads) for w, s, b in mats], axis=1)


@pytest.mark.parametrize("rows", [1, 2, 3, 4, 5, 8, 9, 16, 19])
@pytest.mark.parametrize("k", [512, 1024, 1536, 2048, 4096])
def test_exact_row_bits_small(ctx, rows, k):
    rng = np.random.default_rng(rows * 10000 + k)
    mats = [syn.q4_matrix(rng, n, k) for n in (64, 32, 16)]
    x = syn.hidden_rows(rng, rows, k)
    held, arr = dev_mats(mats)
    out = torch.zeros((rows, 112), dtype=torch.bfloat16, device="cuda")
    ctx.q4_project(dev_bf16(x), arr, k, out)
    ctx.sync()
    assert np.array_equal(host_u16(out), oracle_project(x, mats, 4))


@pytest.mark.parametrize("rows", [1, 2, 4])
@pytest.mark.parametrize("k", [512, 2048, 4096])
def test_exact_row_bits_lane_load_form(ctx, rows, k):
    """TATARA_POLICY_Q4_ROW_FORM = 1: the per-lane loads two blocks ahead (the default for one to four rows is
    the bulk-copy form, which the other tests of this file run) give the oracle's bits too."""
    rng = np.random.default_rng(rows * 977 + k)
    mats = [syn.q4_matrix(rng, n, k) for n in (64, 32, 16)]
    x = syn.hidden_rows(rng, rows, k)
    held, arr = dev_mats(mats)
    out = torch.zeros((rows, 112), dtype=torch.bfloat16, device="cuda")
    assert ctx.get_policy(tb.POLICY_Q4_ROW_FORM) == 0
    ctx.set_policy(tb.POLICY_Q4_ROW_FORM, 1)
    try:
        ctx.q4_project(dev_bf16(x), arr, k, out)
        ctx.sync()
    finally:
        ctx.set_policy(tb.POLICY_Q4_ROW_FORM, 0)
    assert np.array_equal(host_u16(out), oracle_project(x, mats, 4))


@pytest.mark.parametrize("rows", [1, 4, 8])
def test_exact_row_bits_with_scales_off_the_16_byte_grid(ctx, rows):
    """The bulk-copy forms need 16-byte aligned rows of scales and biases; the ABI only asks for 2-byte alignment,
    and a matrix whose affine constants start 2 bytes off the grid runs the per-lane-load kernels: same bits."""
    rng = np.random.default_rng(4242 + rows)
    k = 2048
    w, sc, bi = syn.q4_matrix(rng, 64, k)
    x = syn.hidden_rows(rng, rows, k)
    words = torch.from_numpy(w.view(np.int32)).cuda()
    sbuf = torch.zeros(sc.size + 8, dtype=torch.bfloat16, device="cuda")
    bbuf = torch.zeros(bi.size + 8, dtype=torch.bfloat16, device="cuda")
    scales = sbuf[1:1 + sc.size].view(sc.shape)
    biases = bbuf[1:1 + bi.size].view(bi.shape)
    scales.copy_(dev_bf16(sc)); biases.copy_(dev_bf16(bi))
    assert scales.data_ptr() % 16 == 2
    held = [(words, scales, biases)]
    arr = tb.Context.q4_matrices(held)
    out = torch.zeros((rows, 64), dtype=torch.bfloat16, device="cuda")
    ctx.q4_project(dev_bf16(x), arr, k, out)
    ctx.sync()
    assert np.array_equal(host_u16(out), oracle_project(x, [(w, sc, bi)], 4))


@pytest.mark.parametrize("name,sizes,k", [("attn_project", (8192, 512, 512), 2048),
                                          ("gdn_project", (8192, 4096, 32, 32), 2048),
                                          ("out_projection", (2048,), 4096)])
def test_exact_row_bits_model_geometry(ctx, name, sizes, k):
    """The three call sites at the model's sizes, two rows; a row alone gives the same bits as in the pair."""
    rng = np.random.default_rng(len(sizes))
    mats = [syn.q4_matrix(rng, n, k) for n in sizes]
    x = syn.hidden_rows(rng, 2, k)
    held, arr = dev_mats(mats)
    n = sum(sizes)
    out = torch.zeros((2, n), dtype=torch.bfloat16, device="cuda")
    xd = dev_bf16(x)
    ctx.q4_project(xd, arr, k, out)
    alone = torch.zeros((1, n), dtype=torch.bfloat16, device="cuda")
    ctx.q4_project(xd[1:2], arr, k, alone)
    ctx.sync()
    want = oracle_project(x, mats, oracle.hardware_threads())
    assert np.array_equal(host_u16(out), want)
    assert np.array_equal(host_u16(alone)[0], want[1])
    assert 0.2 < syn.from_bf16(want).std() < 2.0


@pytest.mark.parametrize("name,sizes,k", [("attn_project", (8192, 512, 512), 2048),
                                          ("gdn_project", (8192, 4096, 32, 32), 2048),
                                          ("out_projection", (2048,), 4096)])
@pytest.mark.parametrize("rows", [5, 8])
def test_exact_row_bits_wave_of_eight_model_geometry(ctx, name, sizes, k, rows):
    """The three call sites at a decode wave's row counts (the row-pair kernel with bulk-copied weights: eight,
    four or two columns per warp and 7 to 12 warps per SM, chosen per site): the oracle's chain, bit for bit."""
    rng = np.random.default_rng(800 + rows + len(sizes))
    mats = [syn.q4_matrix(rng, n, k) for n in sizes]
    x = syn.hidden_rows(rng, rows, k)
    held, arr = dev_mats(mats)
    out = torch.zeros((rows, sum(sizes)), dtype=torch.bfloat16, device="cuda")
    ctx.q4_project(dev_bf16(x), arr, k, out)
    ctx.sync()
    assert np.array_equal(host_u16(out), oracle_project(x, mats, oracle.hardware_threads()))


def test_exact_row_batch_of_16_model_geometry(ctx):
    """gdn_project at the largest decode batch of the reference (16 rows: two passes of the row-pair kernel);
    every row has the bits of the oracle's chain, i.e. of the same row projected alone."""
    rng = np.random.default_rng(1616)
    sizes, k = (8192, 4096, 32, 32), 2048
    mats = [syn.q4_matrix(rng, n, k) for n in sizes]
    x = syn.hidden_rows(rng, 16, k)
    held, arr = dev_mats(mats)
    out = torch.zeros((16, sum(sizes)), dtype=torch.bfloat16, device="cuda")
    ctx.q4_project(dev_bf16(x), arr, k, out)
    ctx.sync()
    assert np.array_equal(host_u16(out), oracle_project(x, mats, oracle.hardware_threads()))


def test_exact_row_strides(ctx):
    """Input rows inside a wider buffer, output into a column window of a wider projection buffer."""
    rng = np.random.default_rng(77)
    k = 2048
    mats = [syn.q4_matrix(rng, 48, k)]
    x = syn.hidden_rows(rng, 3, k + 64)
    held, arr = dev_mats(mats)
    out = torch.full((3, 96), 7.0, dtype=torch.bfloat16, device="cuda")
    xd = dev_bf16(x)
    ctx.q4_project(xd, arr, k, out[:, 16:], n_rows=3, x_stride=k + 64, out_stride=96)
    ctx.sync()
    got = host_u16(out)
    assert np.array_equal(got[:, 16:64], oracle_project(np.ascontiguousarray(x[:, :k]), mats, 2))
    assert (syn.from_bf16(got[:, :16]) == 7.0).all() and (syn.from_bf16(got[:, 64:]) == 7.0).all()


def test_exact_row_rejects_bad_extents(ctx):
    rng = np.random.default_rng(3)
    held, arr = dev_mats([syn.q4_matrix(rng, 24, 512)])            # rows not a multiple of 16
    x = dev_bf16(syn.hidden_rows(rng, 1, 512))
    out = torch.zeros((1, 24), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(tb.TataraError) as e:
        ctx.q4_project(x, arr, 512, out)
    assert e.value.status == tb.STATUS_NAMES.index("InvalidDispatchExtent")
    held, arr = dev_mats([syn.q4_matrix(rng, 32, 512)])
    with pytest.raises(tb.TataraError):
        ctx.q4_project(x, arr, 256, out)                            # k not a multiple of 512


def test_dequantize_bits(ctx):
    rng = np.random.default_rng(8)
    k = 2048
    mats = [syn.q4_matrix(rng, n, k) for n in (96, 32)]
    held, arr = dev_mats(mats)
    w = torch.zeros((128, k), dtype=torch.bfloat16, device="cuda")
    ctx.q4_dequantize(arr, k, w)
    ctx.sync()
    want = np.concatenate([oracle.q4_dequantize(*m) for m in mats], axis=0)
    assert np.array_equal(host_u16(w), want)


@pytest.mark.parametrize("rows,n,k", [(1, 32, 64), (7, 544, 2048), (128, 256, 512), (300, 544, 2048),
                                      (129, 800, 4096), (1000, 96, 128),
                                      # 256 rows and 256 columns or more: the CTA-pair kernel (256 x 256 tiles)
                                      (256, 256, 64), (257, 288, 512), (700, 1280, 2048), (513, 544, 4096)])
def test_dense_matches_oracle(ctx, rows, n, k):
    rng = np.random.default_rng(rows + n + k)
    mat = syn.q4_matrix(rng, n, k)
    wq = oracle.q4_dequantize(*mat)
    x = syn.hidden_rows(rng, rows, k)
    out = torch.full((rows, n), 9.0, dtype=torch.bfloat16, device="cuda")
    ctx.project_dense(dev_bf16(x), dev_bf16(wq), out)
    ctx.sync()
    want = oracle.project_dense(x, wq, threads=oracle.hardware_threads())
    got = host_u16(out)
    # one bf16 step of the larger of |value| and the outputs' spread (values near zero have tiny steps)
    gf, wf = syn.from_bf16(got), syn.from_bf16(want)
    excess = np.abs(gf - wf) / np.maximum(np.abs(wf), wf.std())
    assert excess.max() <= 2.0 ** -7, f"relative error {excess.max():.3g}"
    differing = (bf16_ulp_distance(got, want) > 0).mean()
    assert differing <= 0.2, f"{differing:.2%} of the outputs differ from the k-ordered f32 sum"
    assert_close_bf16(got, want, "dense")
    # and against the exact-row policy on the same Q4 weights: the two policies agree within the gate
    if rows <= 8 and k % 512 == 0:
        assert_close_bf16(got, oracle.q4_project(x, *mat, threads=4), "dense vs exact row")


def test_dense_full_size_against_fp32_matmul(ctx):
    """attn_project at the prefill size (16384 rows x 9216 x 2048) against an fp32 matmul of the same bf16
    operands; tolerance one bf16 step of the fp32 result."""
    g = torch.Generator(device="cuda").manual_seed(5)
    rows, n, k = 16384, 9216, 2048
    x = torch.randn((rows, k), generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn((n, k), generator=g, device="cuda") * (0.5 / k ** 0.5)).to(torch.bfloat16)
    out = torch.zeros((rows, n), dtype=torch.bfloat16, device="cuda")
    ctx.project_dense(x, w, out)
    ctx.sync()
    for r0 in (0, 5000, 16384 - 1024):
        ref = x[r0:r0 + 1024].float() @ w.float().T
        got = out[r0:r0 + 1024].float()
        err = (got - ref).abs()
        assert float((err / (ref.abs() + 1.0)).max()) <= 2.0 ** -8
        assert float(torch.nn.functional.cosine_similarity(got.flatten(), ref.flatten(), dim=0)) >= 0.9999


def test_dense_rejects_bad_extents(ctx):
    x = torch.zeros((4, 64), dtype=torch.bfloat16, device="cuda")
    w = torch.zeros((40, 64), dtype=torch.bfloat16, device="cuda")   # n not a multiple of 32
    out = torch.zeros((4, 40), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(tb.TataraError):
        ctx.project_dense(x, w, out)

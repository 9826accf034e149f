"""Lane tables in device memory: the indirect entry points give the bits of the host-table ones, and one
captured CUDA graph of a decode token (qk_rope -> decode attention; fused gated-delta step) replays for
successive tokens with tatara_lanes_advance between them."""
import numpy as np
import pytest
import torch

import tatara_b200 as tb
from tatara_b200 import synthetic as syn
from gpu_util import dev_bf16, dev_f32, host_u16

pytestmark = pytest.mark.gpu

CAP = 640


@pytest.fixture(scope="module")
def ctx():
    c = tb.Context(0)
    yield c
    c.close()


def _attention_state(rng, contexts):
    lanes = len(contexts)
    per_lane = 2 * CAP * 256
    kpool = torch.zeros((lanes, per_lane), dtype=torch.bfloat16, device="cuda")
    vpool = torch.zeros_like(kpool)
    for i, c in enumerate(contexts):
        k, v = syn.attn_cache(rng, c, CAP)
        kpool[i] = dev_bf16(k).reshape(-1)
        vpool[i] = dev_bf16(v).reshape(-1)
    return kpool, vpool, per_lane


def test_indirect_calls_match_host_table_calls(ctx):
    rng = np.random.default_rng(61)
    contexts = [0, 5, 127, 128, 300, 511, 638]
    lanes = len(contexts)
    kpool, vpool, per_lane = _attention_state(rng, contexts)
    k2, v2 = kpool.clone(), vpool.clone()
    qw, kw = (dev_bf16(w) for w in syn.attn_weights(rng))
    proj = dev_bf16(syn.attn_projection(rng, lanes))
    table = tb.Context.attn_lanes([(i * per_lane, c) for i, c in enumerate(contexts)])
    dtable = tb.Context.device_lanes(table)
    scratch = torch.empty(tb.decode_scratch_bytes(CAP, lanes) // 4, dtype=torch.float32, device="cuda")
    outs = []
    for indirect, (kp, vp) in ((False, (kpool, vpool)), (True, (k2, v2))):
        q = torch.zeros((lanes, 4096), dtype=torch.bfloat16, device="cuda")
        gate, out = torch.zeros_like(q), torch.zeros_like(q)
        if indirect:
            ctx.attn_qk_rope_batch_indirect(proj, qw, kw, q, gate, kp, vp, CAP, dtable, lanes)
            ctx.attn_decode_batch_indirect(q, gate, kp, vp, dtable, lanes, CAP, out, scratch)
        else:
            ctx.attn_qk_rope_batch(proj, qw, kw, q, gate, kp, vp, CAP, table)
            ctx.attn_decode_batch(q, gate, kp, vp, table, CAP, out, scratch)
        ctx.sync()
        outs.append((host_u16(q), host_u16(out), host_u16(kp)))
    for a, b in zip(*outs):
        assert np.array_equal(a, b)
    # single lane: the 32-warp merge instantiation
    one = tb.Context.attn_lanes([(3 * per_lane, contexts[3])])
    out1 = torch.zeros((1, 4096), dtype=torch.bfloat16, device="cuda")
    q1 = torch.zeros((1, 4096), dtype=torch.bfloat16, device="cuda")
    g1 = torch.zeros_like(q1)
    ctx.attn_qk_rope_batch_indirect(proj[3:4], qw, kw, q1, g1, k2, v2, CAP, tb.Context.device_lanes(one), 1)
    ctx.attn_decode_batch_indirect(q1, g1, k2, v2, tb.Context.device_lanes(one), 1, CAP, out1, scratch)
    ctx.sync()
    assert np.array_equal(host_u16(out1)[0], outs[1][1][3])


def test_context_beyond_capacity_is_latched_on_the_device(ctx):
    rng = np.random.default_rng(62)
    kpool, vpool, per_lane = _attention_state(rng, [4, 4])
    dtable = tb.Context.device_lanes(tb.Context.attn_lanes([(0, 4), (per_lane, CAP)]))   # lane 1: context == capacity
    q = torch.zeros((2, 4096), dtype=torch.bfloat16, device="cuda")
    gate, out = torch.zeros_like(q), torch.full((2, 4096), 3.0, dtype=torch.bfloat16, device="cuda")
    scratch = torch.empty(tb.decode_scratch_bytes(CAP, 2) // 4, dtype=torch.float32, device="cuda")
    ctx.attn_decode_batch_indirect(q, gate, kpool, vpool, dtable, 2, CAP, out, scratch)
    with pytest.raises(tb.TataraError) as e:
        ctx.sync()
    assert e.value.status == tb.STATUS_NAMES.index("ContextOutOfRange")
    assert (out[1].float() == 3.0).all()      # nothing written for the rejected lane
    ctx.sync()                                # the status was cleared by the failing sync


def test_one_graph_serves_successive_tokens(ctx):
    """Three tokens: eager host-table calls with contexts c, c+1, c+2 (and flipped gated-delta slots) against
    three replays of ONE graph captured with device tables."""
    rng = np.random.default_rng(63)
    contexts = [10, 200, 400]
    lanes, tokens = len(contexts), 3
    kpool, vpool, per_lane = _attention_state(rng, contexts)
    k2, v2 = kpool.clone(), vpool.clone()
    qw, kw = (dev_bf16(w) for w in syn.attn_weights(rng))
    conv_w, a_log, dt_bias, norm_w = (dev_bf16(w) for w in syn.gdn_weights(rng))
    conv_pool = torch.randn((lanes, 2, 3, 8192), device="cuda").to(torch.bfloat16)
    rec_pool = 0.02 * torch.randn((lanes, 2, 32, 128, 128), device="cuda")
    conv2, rec2 = conv_pool.clone(), rec_pool.clone()
    projs = [dev_bf16(syn.attn_projection(rng, lanes)) for _ in range(tokens)]
    gprojs = [dev_bf16(syn.gdn_projection(rng, lanes)) for _ in range(tokens)]
    scratch = torch.empty(tb.decode_scratch_bytes(CAP, lanes) // 4, dtype=torch.float32, device="cuda")
    cs, rs = 3 * 8192, 32 * 128 * 128

    def gdn_table(parity):
        a, b = (0, 1) if parity == 0 else (1, 0)
        return tb.Context.gdn_lanes([((2 * i + a) * cs, (2 * i + b) * cs, (2 * i + a) * rs, (2 * i + b) * rs) for i in range(lanes)])

    # eager reference
    want = []
    for t in range(tokens):
        table = tb.Context.attn_lanes([(i * per_lane, c + t) for i, c in enumerate(contexts)])
        q = torch.zeros((lanes, 4096), dtype=torch.bfloat16, device="cuda")
        gate, out, y, gated = torch.zeros_like(q), torch.zeros_like(q), torch.zeros_like(q), torch.zeros_like(q)
        ctx.attn_qk_rope_batch(projs[t], qw, kw, q, gate, kpool, vpool, CAP, table)
        ctx.attn_decode_batch(q, gate, kpool, vpool, table, CAP, out, scratch)
        ctx.gdn_decode_batch(gprojs[t], conv_w, a_log, dt_bias, norm_w, conv_pool, rec_pool, gdn_table(t & 1), y, gated)
        ctx.sync()
        want.append((host_u16(out), host_u16(gated)))

    # one captured graph, device tables, static input / output buffers
    d_attn = tb.Context.device_lanes(tb.Context.attn_lanes([(i * per_lane, c) for i, c in enumerate(contexts)]))
    d_gdn = tb.Context.device_lanes(gdn_table(0))
    proj_in, gproj_in = torch.zeros_like(projs[0]), torch.zeros_like(gprojs[0])
    q = torch.zeros((lanes, 4096), dtype=torch.bfloat16, device="cuda")
    gate, out, y, gated = torch.zeros_like(q), torch.zeros_like(q), torch.zeros_like(q), torch.zeros_like(q)
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        # the attribute setup of the first launches happens outside the capture
        tmp_k, tmp_v = k2.clone(), v2.clone()
        ctx.attn_qk_rope_batch_indirect(proj_in, qw, kw, q, gate, tmp_k, tmp_v, CAP, d_attn, lanes)
        ctx.attn_decode_batch_indirect(q, gate, tmp_k, tmp_v, d_attn, lanes, CAP, out, scratch)
        stream.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            ctx.attn_qk_rope_batch_indirect(proj_in, qw, kw, q, gate, k2, v2, CAP, d_attn, lanes)
            ctx.attn_decode_batch_indirect(q, gate, k2, v2, d_attn, lanes, CAP, out, scratch)
            ctx.gdn_decode_batch_indirect(gproj_in, conv_w, a_log, dt_bias, norm_w, conv2, rec2, d_gdn, lanes, y, gated)
            ctx.lanes_advance(d_attn, lanes, d_gdn, lanes)
    for t in range(tokens):
        proj_in.copy_(projs[t])
        gproj_in.copy_(gprojs[t])
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        assert np.array_equal(host_u16(out), want[t][0]), f"attention token {t}"
        assert np.array_equal(host_u16(gated), want[t][1]), f"gated delta token {t}"
    ctx.sync()

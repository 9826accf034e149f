"""Split-KV merge over peer memory (push + bounded wait) on one GPU.

Two ranks are emulated on one device by running both ranks' push kernels one after the other on
one stream before the waiting combine is launched, so no kernel ever waits for a kernel that has
not finished (the real multi-GPU run is exercised by `bench.py --gpus N`).  The time-out path
is tested with a flag that nothing sets and a 0.2 s limit: the kernel returns, the context stays
usable, and tatara_ctx_sync reports DeviceWaitTimeout.
"""
import numpy as np
import pytest
import torch

import oracle
import tatara_b200 as tb
from tatara_b200 import sharding, synthetic as syn
from gpu_util import assert_close_bf16, dev_bf16, host_u16

pytestmark = pytest.mark.gpu


def test_push_and_wait_merge_two_emulated_ranks():
    ctx = tb.Context(0)
    rng = np.random.default_rng(81)
    n, world = 6000, 2
    keys, values = syn.attn_cache(rng, n, n)
    q, gate = syn.attn_query(rng, np.array([n - 1]))
    dq, dg, dk, dv = dev_bf16(q[0]), dev_bf16(gate[0]), dev_bf16(keys), dev_bf16(values)
    want = oracle.attn_decode(q[0], gate[0], keys, values, n - 1, n, threads=8)
    ranges = sharding.split_kv_ranges(n, world)
    rec_bytes = sharding.PeerExchange.RECORD_BYTES
    buf, _ = ctx.peer_buffer_create(2 * world * rec_bytes + 2 * world * 4)
    scratch = torch.empty(tb.decode_scratch_bytes(n) // 4, dtype=torch.float32, device="cuda")
    out = torch.zeros((16, 256), dtype=torch.bfloat16, device="cuda")
    for epoch in (1, 2, 3):                        # alternating parities, reused buffers
        parity = epoch & 1
        gather = buf + parity * world * rec_bytes
        flags = buf + 2 * world * rec_bytes + parity * world * 4
        for rank, (b, e) in enumerate(ranges):     # both "ranks" write into the one buffer
            ctx.attn_decode_partial_push(dq, dk, dv, b, e, n, [gather] * world, [flags] * world, rank, epoch, scratch)
        out.zero_()
        ctx.attn_combine_wait(gather, flags, world, epoch, dg, out)
        ctx.sync()
        assert_close_bf16(host_u16(out), want, f"p2p merge epoch {epoch}")
    # the same through the unsplit kernel
    solo = torch.zeros_like(out)
    ctx.attn_decode(dq, dg, dk, dv, n - 1, n, solo, scratch)
    ctx.sync()
    assert_close_bf16(host_u16(out), host_u16(solo), "p2p merge vs unsplit")
    ctx.peer_buffer_close(buf, owned=True)
    ctx.close()


def test_single_submission_step_counts_on_the_device_and_replays_as_a_graph():
    """tatara_attn_decode_split with a world of one rank (a second rank cannot run beside it on one
    GPU: its waiting kernel would wait for a kernel queued behind it): the whole step is one call, the
    step counter and the parity live on the device, so five eager steps and three replays of a captured
    step all give the unsplit decode's result and leave the counter at eight."""
    ctx = tb.Context(0)
    rng = np.random.default_rng(82)
    n = 5000
    keys, values = syn.attn_cache(rng, n, n)
    q, gate = syn.attn_query(rng, np.array([n - 1]))
    dq, dg, dk, dv = dev_bf16(q[0]), dev_bf16(gate[0]), dev_bf16(keys), dev_bf16(values)
    want = oracle.attn_decode(q[0], gate[0], keys, values, n - 1, n, threads=8)
    nbytes = tb.split_buffer_bytes(1)
    buf, _ = ctx.peer_buffer_create(nbytes)
    peers = tb.Context.pointer_array([buf])
    scratch = torch.empty(tb.decode_scratch_bytes(n) // 4, dtype=torch.float32, device="cuda")
    out = torch.zeros((16, 256), dtype=torch.bfloat16, device="cuda")
    solo = torch.zeros_like(out)
    ctx.attn_decode(dq, dg, dk, dv, n - 1, n, solo, scratch)
    for step in range(5):
        out.zero_()
        ctx.attn_decode_split(dq, dg, dk, dv, 0, n, n, peers, 0, out, scratch)
        ctx.sync()
        assert_close_bf16(host_u16(out), want, f"single-submission step {step}")
        assert_close_bf16(host_u16(out), host_u16(solo), f"single-submission step {step} vs unsplit")
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            ctx.attn_decode_split(dq, dg, dk, dv, 0, n, n, peers, 0, out, scratch, stream=stream.cuda_stream)
    for replay in range(3):
        out.zero_()
        graph.replay()
        ctx.sync()
        assert_close_bf16(host_u16(out), want, f"replayed step {replay}")
    words = torch.zeros(nbytes // 4, dtype=torch.int32, device="cuda")
    ctx.state_copy(tb.Context.copy_segments([(buf, words.data_ptr(), nbytes)]))
    ctx.sync()
    step_word = (nbytes - 16) // 4
    assert int(words[step_word]) == 8, "the device step counter counts every step, eager or replayed"
    ctx.peer_buffer_close(buf, owned=True)
    ctx.close()


def test_single_submission_step_gives_up_when_a_rank_never_stores():
    """A world of two whose second rank never runs: the merge kernel's bounded wait (0.2 s) runs out,
    nothing is written, the status is DeviceWaitTimeout and the context stays usable."""
    ctx = tb.Context(0)
    n = 2000
    g = torch.Generator(device="cuda").manual_seed(83)
    kv = torch.randn((2, n, 256), generator=g, device="cuda").to(torch.bfloat16)
    q = torch.randn((16, 256), generator=g, device="cuda").to(torch.bfloat16)
    bufs = [ctx.peer_buffer_create(tb.split_buffer_bytes(2))[0] for _ in range(2)]
    scratch = torch.empty(tb.decode_scratch_bytes(n) // 4, dtype=torch.float32, device="cuda")
    out = torch.full((16, 256), 4.0, dtype=torch.bfloat16, device="cuda")
    ctx.attn_decode_split(q, q, kv, kv, 0, n // 2, n, tb.Context.pointer_array(bufs), 0, out, scratch, wait_limit_us=200000)
    with pytest.raises(tb.TataraError) as e:
        ctx.sync()
    assert e.value.status == tb.STATUS_NAMES.index("DeviceWaitTimeout")
    assert torch.all(out == 4.0), "a step that gave up must not write its output"
    ctx.sync()
    solo = torch.zeros_like(out)
    ctx.attn_decode(q, q, kv, kv, n - 1, n, solo, scratch)
    ctx.sync()
    for b in bufs:
        ctx.peer_buffer_close(b, owned=True)
    ctx.close()


def test_wait_runs_out_and_reports_timeout():
    ctx = tb.Context(0)
    world = 2
    rec_bytes = sharding.PeerExchange.RECORD_BYTES
    buf, _ = ctx.peer_buffer_create(2 * world * rec_bytes + 2 * world * 4)
    gate = torch.zeros((16, 256), dtype=torch.bfloat16, device="cuda")
    out = torch.full((16, 256), 4.0, dtype=torch.bfloat16, device="cuda")
    ctx.attn_combine_wait(buf, buf + 2 * world * rec_bytes, world, 7, gate, out, wait_limit_us=200000)
    with pytest.raises(tb.TataraError) as e:
        ctx.sync()
    assert e.value.status == tb.STATUS_NAMES.index("DeviceWaitTimeout")
    assert torch.all(out == 4.0), "a timed-out combine must not write its output"
    ctx.sync()                                     # status was cleared; the context is still usable
    solo = torch.zeros((16, 256), dtype=torch.bfloat16, device="cuda")
    kv = torch.randn((2, 64, 256), device="cuda").to(torch.bfloat16)
    scratch = torch.empty(tb.decode_scratch_bytes(64) // 4, dtype=torch.float32, device="cuda")
    ctx.attn_decode(gate, gate, kv, kv, 63, 64, solo, scratch)
    ctx.sync()
    with pytest.raises(tb.TataraError) as e:
        ctx.attn_combine_wait(buf, buf, 9, 1, gate, out)
    assert e.value.status == tb.STATUS_NAMES.index("InvalidStreamGroup")
    ctx.peer_buffer_close(buf, owned=True)
    ctx.close()

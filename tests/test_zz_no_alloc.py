"""The allocation-free decode entry point against the ordinary one.

tatara_attn_decode_static serves callers that cannot allocate device memory (a serving loop
with a frozen memory plan, a plug-in that may not touch its host's allocator): its record
scratch is an array inside the library instead of a caller buffer.  The test calls it through
the C ABI twice in a row -- the second call starts from the first call's leftover records --
and requires the bits of tatara_attn_decode on the same inputs each time, and the CPU oracle's
result within the repository's tolerance.  It runs last so a stop-at-first-failure run has
already covered every other test.
"""
import numpy as np
import pytest
import torch

import oracle
import tatara_b200 as tb
from gpu_util import assert_close_bf16, host_u16

pytestmark = pytest.mark.gpu


def test_static_scratch_decode_matches_caller_scratch_decode_twice():
    ctx = tb.Context(0)
    g = torch.Generator(device="cuda").manual_seed(41)
    cap = 40000
    keys = torch.randn((2, cap, 256), generator=g, device="cuda").to(torch.bfloat16)
    values = torch.randn((2, cap, 256), generator=g, device="cuda").to(torch.bfloat16)
    for call, context in enumerate((37123, 5000)):        # second call reuses dirty records
        q = torch.randn((16, 256), generator=g, device="cuda").to(torch.bfloat16)
        gate = torch.randn((16, 256), generator=g, device="cuda").to(torch.bfloat16)
        want = torch.zeros((16, 256), dtype=torch.bfloat16, device="cuda")
        scratch = torch.empty(tb.decode_scratch_bytes(context + 1) // 4, dtype=torch.float32, device="cuda")
        ctx.attn_decode(q, gate, keys, values, context, cap, want, scratch)
        got = torch.full((16, 256), 9.0, dtype=torch.bfloat16, device="cuda")
        ctx.sync()
        free_before = torch.cuda.mem_get_info()[0]
        ctx.attn_decode_static(q, gate, keys, values, context, cap, got)
        ctx.sync()
        if call == 1:   # the driver's free-memory figure does not move: nothing was allocated
            assert torch.cuda.mem_get_info()[0] == free_before
        assert_close_bf16(host_u16(got), host_u16(want), f"static decode call {call}")
        assert torch.equal(got, want), f"call {call}: same kernels, same partitions, so the same bits"
        cpu = oracle.attn_decode(host_u16(q), host_u16(gate), host_u16(keys), host_u16(values), context, cap,
                                 threads=oracle.hardware_threads())
        assert_close_bf16(host_u16(got), cpu, f"static decode call {call} vs the CPU oracle")
    # beyond the built-in maximum the call refuses, clearly, and enqueues nothing
    big = torch.zeros((2, 8, 256), dtype=torch.bfloat16, device="cuda")
    launches = ctx.launches
    with pytest.raises(tb.TataraError) as e:
        ctx.attn_decode_static(q, gate, big, big, 262144, 262145, got)
    assert e.value.status == tb.STATUS_NAMES.index("ScratchTooSmall")
    assert "262144" in str(e.value)
    assert ctx.launches == launches
    ctx.close()

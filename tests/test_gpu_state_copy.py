"""GPU tests of the segment copy behind state snapshots (tatara_state_copy): byte-exact against torch slices."""
import numpy as np
import pytest
import torch

import tatara_b200 as tb

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    c = tb.Context(0)
    yield c
    c.close()


def test_segments_of_mixed_length(ctx):
    """Snapshot-shaped list: short and long segments, strided sources, packed destination; 130 segments
    exercise the split into more than one launch."""
    g = torch.Generator(device="cuda").manual_seed(3)
    src = torch.randint(0, 256, (64 << 20,), generator=g, device="cuda", dtype=torch.uint8)
    dst = torch.zeros(48 << 20, dtype=torch.uint8, device="cuda")
    rng = np.random.default_rng(0)
    lengths = [16, 48, 49152, 20480, 2097152, 32768, 32784] + [int(rng.integers(1, 20000)) * 16 for _ in range(123)]
    entries, want, at, cursor = [], [], 0, 0
    for n in lengths:
        cursor = (cursor + int(rng.integers(0, 64)) * 16) % (src.numel() - n)
        cursor -= cursor % 16
        entries.append((src.data_ptr() + cursor, dst.data_ptr() + at, n))
        want.append((at, cursor, n))
        at += n
    assert at <= dst.numel()
    ctx.state_copy(tb.Context.copy_segments(entries))
    ctx.sync()
    for a, c, n in want:
        assert torch.equal(dst[a:a + n], src[c:c + n])
    assert int(dst[at:].max()) == 0


def test_rejects_bad_segments(ctx):
    a = torch.zeros(1024, dtype=torch.uint8, device="cuda")
    b = torch.zeros(1024, dtype=torch.uint8, device="cuda")
    before = ctx.launches
    for entry in [(a.data_ptr() + 8, b.data_ptr(), 64), (a.data_ptr(), b.data_ptr(), 24), (a.data_ptr(), b.data_ptr(), 0),
                  (0, b.data_ptr(), 64)]:
        with pytest.raises(tb.TataraError):
            ctx.state_copy(tb.Context.copy_segments([(a.data_ptr(), b.data_ptr(), 64), entry]))
    assert ctx.launches == before   # the list is validated before anything is enqueued

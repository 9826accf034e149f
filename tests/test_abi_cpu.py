"""Host-only checks of the C-ABI library: it loads, exports every declared symbol, and its pure
geometry functions behave (the reference pins its geometry the same way,
tests/native/decode_geometry_test.cpp:30-110).  No compute call is made."""
import ctypes
import re

import pytest

import tatara_b200 as tb


def declared_symbols():
    text = open(tb.HEADER_PATH).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tatara_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = tb.lib()
    names = declared_symbols()
    assert len(names) >= 20
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/tatara_b200.h but not exported"


def test_status_names_mirror_reference_enum():
    lib = tb.lib()
    got = [lib.tatara_status_name(i).decode() for i in range(len(tb.STATUS_NAMES))]
    assert got == tb.STATUS_NAMES
    assert lib.tatara_abi_version() == 1


def test_ctx_create_without_device_is_invalid_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    handle = ctypes.c_void_p()
    assert tb.lib().tatara_ctx_create(0, ctypes.byref(handle)) == tb.STATUS_NAMES.index("InvalidDevice")
    assert not handle.value
    with pytest.raises(tb.TataraError):
        tb.Context(0)


def test_partition_function_is_sound():
    """Partitions tile [0, n) exactly, in 16-key multiples, for every probed n."""
    probes = list(range(1, 600)) + [4095, 4096, 4097, 4736, 4737, 8193, 16385, 32769, 65537,
                                    98303, 98304, 131073, 262144, 262145]
    for n in probes:
        p, c = tb.partition_keys(n), tb.partitions(n)
        assert p % 16 == 0 and p >= 16
        assert (c - 1) * p < n <= c * p
    # beyond 9472 keys a lane is cut into 74 partitions: with 2 kv heads, exactly one work item per SM
    for n in (32769, 65537, 131073, 262145):
        assert 73 <= tb.partitions(n) <= 74
    assert max(tb.partitions(n) for n in range(1, 300000, 97)) == 74


def test_scratch_bound_covers_every_shorter_context():
    for max_keys in (1, 64, 4097, 32769, 262145):
        bound = tb.decode_scratch_bytes(max_keys, 1)
        step = max(1, max_keys // 3000)
        worst = max(tb.partitions(n) for n in range(1, max_keys + 1, step))
        worst = max(worst, tb.partitions(max_keys))
        assert bound >= worst * 16 * 258 * 4
    assert tb.decode_scratch_bytes(4097, 4) == 4 * tb.decode_scratch_bytes(4097, 1)

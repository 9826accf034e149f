"""Builds and runs the native (C++) tests of the host layer that mirrors the reference's layer
encoders and owner loop over the C ABI (tests/native/hybrid_layers_test.cpp, wave_loop_test.cpp)."""
import os
import subprocess

import pytest

HERE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "native")


def _build(name="hybrid_layers_test"):
    import oracle
    import tatara_b200
    oracle.lib()
    tatara_b200.lib()
    subprocess.check_call(["make", "-s", "-C", HERE, name])
    return os.path.join(HERE, name)


def test_native_host_checks_without_device():
    import torch
    exe = _build()
    res = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    if not torch.cuda.is_available():
        assert "device checks skipped" in res.stdout


@pytest.mark.gpu
def test_native_host_and_device_checks():
    exe = _build()
    res = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "host and device checks passed" in res.stdout


def test_wave_loop_checks_without_device():
    import torch
    exe = _build("wave_loop_test")
    res = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    if not torch.cuda.is_available():
        assert "device checks skipped" in res.stdout


@pytest.mark.gpu
def test_wave_loop_host_and_device_checks():
    exe = _build("wave_loop_test")
    res = subprocess.run([exe], capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "host and device checks passed" in res.stdout

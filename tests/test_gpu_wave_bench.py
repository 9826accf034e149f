"""The wave-loop timing program (bench_wave_loop.cpp, beside bench.py) on a small stack: it must join every stream
through the owner loop, reach full waves and report one graph per wave size."""
import json
import os
import subprocess

import pytest

import tatara_b200 as tb

pytestmark = pytest.mark.gpu


def test_wave_bench_small_stack():
    exe = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench_wave_loop")
    assert os.path.exists(exe), "bench_wave_loop is not built (__graft_entry__.build())"
    res = subprocess.run([exe, "--lanes", "3", "--context", "700", "--tokens", "12", "--layers", "8", "--unit", "256"],
                         capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["workload"] == "wave_loop" and line["lanes"] == 3 and line["layers"] == 8
    assert 1 <= line["graphs_captured"] <= 3            # one graph per wave size seen (1, 2, 3 rows)
    assert line["wave_ms_graph"] > 0 and line["wave_ms_eager_host_tables"] > 0
    assert line["join_rows_per_s"] > 0

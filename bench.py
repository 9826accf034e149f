#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

Headline (one JSON line): decode attention of one lane at context 262144 -- the HBM GB/s the
split-KV decode achieves over that lane's KV cache (K+V = 512 MiB, larger than the 126 MB L2),
with the microseconds per layer beside it.  A "step" is one decode-attention call over the
lane's cache.  The same line carries the context sweep 4k..262k, the prefill-attention TFLOP/s
at 16k, the GDN decode step and GDN prefill, the roofline of the dominant kernel, the CPU
oracle timing and the end-to-end number measured through the C ABI from host buffers.

    python bench.py                          # N=1, defaults
    python bench.py --gpus 1 --steps 50 --warmup 5
    torchrun --nproc-per-node N bench.py --gpus N ...   # lanes spread over N GPUs (weak scaling)
    python bench.py --impl reference         # the CPU oracle on the host cores, same metric
    python bench.py --only decode --context 32768        # one small case (profiling under ncu)
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HEADLINE_CONTEXT = 262144          # keys attended by the headline step
SWEEP = [4096, 8192, 16384, 32768, 65536, 131072, 262144]
PREFILL_ROWS = 16384
L2_BYTES = 126 * 1000 * 1000


from bench_workloads import decode_bytes, measured_peaks, prefill_flops  # noqa: E402,F401


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, flag in zip(names, r[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


# --------------------------------------------------------------------------------------------
# reference arm / cpu baseline: the scalar fp32 oracle on the host cores
def cpu_decode_sample(n_keys: int, threads: int, repeats: int):
    """Times the oracle's decode attention over one lane of n_keys keys (all 16 heads)."""
    import oracle
    from tatara_b200 import synthetic as syn
    rng = np.random.default_rng(0)
    keys, values = syn.attn_cache(rng, n_keys, n_keys)
    q, gate = syn.attn_query(rng, np.array([n_keys - 1]))
    best, total = None, 0.0
    for _ in range(repeats):
        t0 = time.perf_counter()
        oracle.attn_decode(q[0], gate[0], keys, values, n_keys - 1, n_keys, threads=threads)
        dt = time.perf_counter() - t0
        total += dt
        best = dt if best is None else min(best, dt)
    return best, total


def run_reference(args):
    import oracle
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    oracle.lib()
    threads = oracle.hardware_threads()
    n = HEADLINE_CONTEXT
    import oracle as _o
    from tatara_b200 import synthetic as syn
    rng = np.random.default_rng(0)
    keys, values = syn.attn_cache(rng, n, n)
    q, gate = syn.attn_query(rng, np.array([n - 1]))
    for _ in range(max(1, min(args.warmup, 1))):
        _o.attn_decode(q[0], gate[0], keys, values, n - 1, n, threads=threads)
    steps = max(1, min(args.steps, 8))      # each step ~1 s of host time: bounded sample
    t0 = time.perf_counter()
    for _ in range(steps):
        _o.attn_decode(q[0], gate[0], keys, values, n - 1, n, threads=threads)
    dt = (time.perf_counter() - t0) / steps
    gbs = decode_bytes(n) / dt / 1e9
    line = {
        "impl": "reference", "metric": "decode_attn_hbm_gbs", "value": gbs, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": 1, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"decode_attn_ctx{n}", "lanes": 1, "context": n,
                   "note": "scalar fp32 CPU restatement of the reference kernels (its Metal path cannot run here)"},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": f"{steps} full decode steps at context {n}, all 16 heads"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))
    return 0


# --------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--only", default=None, choices=[None, "decode", "prefill", "gdn_step", "gdn_prefill", "lanes32", "project", "state_copy", "layers", "wave"],
                    help="run one workload only (small profiling runs)")
    ap.add_argument("--context", type=int, default=HEADLINE_CONTEXT)
    ap.add_argument("--rows", type=int, default=PREFILL_ROWS)
    ap.add_argument("--lanes", type=int, default=4, help="lanes of --only gdn_step")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist
    import tatara_b200 as tb
    from bench_workloads import Workloads

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path)")
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = tb.Context(local)
    wl = Workloads(ctx, torch, rank=rank, world=world)
    peaks = measured_peaks()
    steps, warmup = args.steps, max(args.warmup, 3)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def capture(fn, k, first):
        """Captures k back-to-back steps fn(first), fn(first+1), ... into one CUDA graph, so the
        timed region holds GPU work only (one graph launch instead of k host-side call sequences)."""
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(k):
                fn(first + i)
        return graph

    def replay_ms(graph, k):
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        graph.replay()
        stop.record()
        barrier()
        ms = start.elapsed_time(stop) / k
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def timed(fn, k, w, eager=False, hold_s=0.0):
        """w untimed warm-up steps, then exactly k timed steps, bracketed by a barrier + synchronize
        on both sides; per-step ms from CUDA events on the launching stream, max over ranks.
        Default: the k steps are one CUDA-graph replay.  eager=True times k host-issued calls
        (used for the end-to-end number, which includes the host side of every call).
        hold_s keeps the same graph running before and after the timed replay so that the
        clock sampler sees the GPU under this load."""
        for i in range(w):
            fn(i)
        barrier()
        if eager:
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for i in range(k):
                fn(w + i)
            stop.record()
            barrier()
            ms = start.elapsed_time(stop) / k
            if world > 1:
                t = torch.tensor([ms], device="cuda")
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            return ms
        graph = capture(fn, k, w)
        graph.replay()          # one untimed replay (graph upload)
        t_end = time.perf_counter() + hold_s
        while time.perf_counter() < t_end:
            graph.replay()
            torch.cuda.synchronize()
        ms = replay_ms(graph, k)
        t_end = time.perf_counter() + hold_s / 2
        while time.perf_counter() < t_end:
            graph.replay()
            torch.cuda.synchronize()
        return ms

    if args.only is not None:
        # small single-workload runs for profiling; prints a short JSON line
        res = wl.run_only(args.only, args, timed, steps, warmup)
        if rank == 0:
            print(json.dumps(res))
        return 0

    n = HEADLINE_CONTEXT
    decode = wl.decode_setup(n)
    launches0 = ctx.launches
    with ClockSampler(local) as clocks:
        ms = timed(decode.step, steps, warmup, hold_s=1.0)
    launches = ctx.launches - launches0 - 2 * warmup   # launches captured for the k timed steps
    bytes_step = decode_bytes(n)
    gbs = world * bytes_step / (ms * 1e-3) / 1e9

    # end to end through the C ABI from host buffers: H2D the token's projection row,
    # qk_rope (appends K/V), decode attention, D2H the attended row.
    e2e_ms = timed(decode.step_e2e, steps, warmup, eager=True)
    e2e_gbs = world * bytes_step / (e2e_ms * 1e-3) / 1e9
    e2e_direct_mapped_ms = timed(decode.step_e2e_mapped, steps, warmup, eager=True)
    # the same token as one captured CUDA graph (lane tables in device memory), one graph launch per token
    try:
        e2e_graph_ms = timed(decode.token_graph(), steps, warmup, eager=True)
        e2e_mapped_ms = timed(decode.token_graph(mapped_host=True), steps, warmup, eager=True)
    except tb.TataraError as e:   # pragma: no cover
        e2e_graph_ms = e2e_mapped_ms = None

    extra = {}
    if world == 1:
        sweep = []
        for c in SWEEP:
            d = decode if c == n else wl.decode_setup(c)
            t = timed(d.step, max(2 * d.replicas, steps), max(warmup, d.replicas))
            sweep.append({"context": c, "us_per_layer": t * 1e3, "gbs": decode_bytes(c) / (t * 1e-3) / 1e9,
                          "frac_of_measured_hbm": decode_bytes(c) / (t * 1e-3) / 1e9 / peaks["hbm_gbs"],
                          "l2": f"{d.replicas} rotating caches (> 2x L2 between reuse)"})
            if c != n:
                d.free()
        extra["decode_sweep"] = sweep
        extra["lanes32"] = wl.lanes32(timed, steps, warmup)
        extra["gdn_step"] = wl.gdn_step(timed, steps, warmup)
        extra["gdn_step_lanes32"] = wl.gdn_step(timed, steps, warmup, n=32)
        extra["gdn_prefill"] = wl.gdn_prefill(timed)
        extra["projections"] = wl.project(timed, peaks, steps, warmup)
        extra["state_snapshot"] = wl.state_copy(timed, peaks)
        extra["decode_layer_slices"] = wl.layer_slices(timed, steps, warmup)
        extra["prefill_attn"] = wl.prefill(timed, peaks, sampler=ClockSampler(local))
        try:   # the owner's wave loop over a 40-layer stack (a native program; its failure never costs the headline)
            extra["wave_loop"] = wl.wave_loop(lanes=8, context=4096, tokens=24)
        except Exception as e:   # pragma: no cover
            extra["wave_loop"] = {"error": str(e)[-300:]}
    else:
        extra["split_kv"] = wl.split_kv(dist, n, timed, steps, warmup)
        extra["lanes32"] = wl.lanes32(timed, steps, warmup)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        import oracle
        threads = oracle.hardware_threads()
        best, total = cpu_decode_sample(n, threads, repeats=8)
        cpu = {"value": decode_bytes(n) / best / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
               "sample": f"best of 8 full decode steps at context {n} ({total:.1f} s of host time)"}

    if rank == 0:
        line = {
            "metric": "decode_attn_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": ms, "us_per_layer": ms * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": f"decode_attn_ctx{n}", "lanes_per_gpu": 1, "context": n,
                       "kv_bytes": n * 2048, "l2": "inputs larger than L2 (512 MiB of K+V streamed per step, steps back to back)",
                       "timing": "k steps captured in one CUDA graph, timed with CUDA events around its replay",
                       "parallelism": "one lane per GPU, no collective" if world > 1 else "single GPU"},
            "roofline": {"bound": "hbm", "achieved": gbs / world, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / world / peaks["hbm_gbs"], "traffic": wl.traffic_hint(),
                         "peak_source": peaks["source"],
                         "kernel": "attn_decode_partition_kernel (+ attn_combine_kernel in the timed step)"},
            "e2e": {"value": e2e_gbs, "unit": "GB/s", "ms_per_step": e2e_ms,
                    "mapped_host_ms_per_step": e2e_direct_mapped_ms,
                    "graph_replay_ms_per_step": e2e_graph_ms,
                    "graph_replay_mapped_host_ms_per_step": e2e_mapped_ms,
                    "path": "host-issued C-ABI calls from Python: pinned H2D of the token projection, qk_rope, decode, D2H",
                    "h2d_bytes_per_step": 9216 * 2, "d2h_bytes_per_step": 4096 * 2},
            "gpu_launches": int(launches),
            "clocks": clocks.summary(),
            "cpu_baseline": cpu,
        }
        line.update(extra)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())

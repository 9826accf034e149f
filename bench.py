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
def headline_config(n_gpus: int) -> dict:
    """The `config` object of the JSON line: one dict for both arms, so the two lines can be compared
    key by key.  The workload is ONE lane at 262144 attended keys at every N."""
    n = HEADLINE_CONTEXT
    return {"workload": f"decode_attn_ctx{n}", "lanes": 1, "context": n, "kv_bytes": n * 2048, "n_gpus": n_gpus,
            "l2": "inputs larger than L2 (512 MiB of K+V streamed per step, steps back to back)",
            "parallelism": "single GPU" if n_gpus == 1 else
                           f"split-KV: the lane's key axis cut into {n_gpus} contiguous ranges, one per GPU; "
                           "records merged over NVLink peer memory"}


def cpu_decode_sample(q, gate, keys, values, n_keys: int, threads: int, repeats: int):
    """Times the oracle's decode attention over one lane of n_keys keys (all 16 heads); host arrays
    are bf16 bit patterns.  Returns (best seconds, total seconds, the oracle's output)."""
    import oracle
    best, total, out = None, 0.0, None
    for _ in range(repeats):
        t0 = time.perf_counter()
        out = oracle.attn_decode(q, gate, keys, values, n_keys - 1, n_keys, threads=threads)
        dt = time.perf_counter() - t0
        total += dt
        best = dt if best is None else min(best, dt)
    return best, total, out


def run_reference(args):
    """The reference arm: the reference's algorithm for this path on the host cores (the CPU oracle,
    kind "port": the reference's own kernels are Metal and cannot run here), all host threads, the
    repo arm's workload, config, steps and warm-up.  Under torchrun rank 0 alone runs and prints."""
    import oracle
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    oracle.lib()
    threads = oracle.hardware_threads()
    n = HEADLINE_CONTEXT
    from tatara_b200 import synthetic as syn
    rng = np.random.default_rng(0)
    keys, values = syn.attn_cache(rng, n, n)
    q, gate = syn.attn_query(rng, np.array([n - 1]))
    steps, warmup = args.steps, max(args.warmup, 3)
    for _ in range(warmup):
        oracle.attn_decode(q[0], gate[0], keys, values, n - 1, n, threads=threads)
    t0 = time.perf_counter()
    for _ in range(steps):          # each step: one full decode over the lane, ~0.2 s of host time
        oracle.attn_decode(q[0], gate[0], keys, values, n - 1, n, threads=threads)
    dt = (time.perf_counter() - t0) / steps
    gbs = decode_bytes(n) / dt / 1e9
    line = {
        "impl": "reference", "metric": "decode_attn_hbm_gbs", "value": gbs, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak" if args.gpus == 1 else "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": headline_config(args.gpus),
        "note": "scalar fp32 CPU restatement of the reference kernels (its Metal path cannot run here), timed on "
                f"rank 0's {threads} host threads only; no GPU is used by this arm at any --gpus",
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
    ap.add_argument("--policy", action="append", default=[], metavar="ID=VALUE",
                    help="tatara_ctx_set_policy(ID, VALUE) on the bench's context before anything runs "
                         "(e.g. 5=1: the per-lane-load form of the exact-row projections); may be repeated")
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
    for item in args.policy:
        pid, _, value = item.partition("=")
        ctx.set_policy(int(pid), int(value))
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
        torch.cuda.synchronize()
        if world > 1:
            # The ranks of a split-KV step wait for one another inside the kernels, so every rank must
            # replay the same number of times: rank 0 turns the hold time into a replay count.
            t0 = time.perf_counter()
            graph.replay()
            torch.cuda.synchronize()
            count = torch.tensor([max(1, int(hold_s / max(time.perf_counter() - t0, 1e-5)))], device="cuda")
            dist.broadcast(count, 0)
            holds = int(count.item()) if hold_s > 0 else 0
            for _ in range(holds):
                graph.replay()
            torch.cuda.synchronize()
            ms = replay_ms(graph, k)
            for _ in range(holds // 2):
                graph.replay()
            torch.cuda.synchronize()
            return ms
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
    bytes_step = decode_bytes(n)
    extra = {}
    parity = None
    if world == 1:
        decode = wl.decode_setup(n)
        launches0 = ctx.launches
        with ClockSampler(local) as clocks:
            ms = timed(decode.step, steps, warmup, hold_s=1.0)
        launches = ctx.launches - launches0 - 2 * warmup   # launches captured for the k timed steps
        kernel_note = "attn_decode_partition_kernel (+ attn_combine_kernel in the timed step)"
        # end to end through the C ABI from host buffers: H2D the token's projection row,
        # qk_rope (appends K/V), decode attention, D2H the attended row.
        e2e_ms = timed(decode.step_e2e, steps, warmup, eager=True)
        e2e = {"ms_per_step": e2e_ms,
               "mapped_host_ms_per_step": timed(decode.step_e2e_mapped, steps, warmup, eager=True),
               "path": "host-issued C-ABI calls from Python: pinned H2D of the token projection, qk_rope, decode, D2H"}
        # the same token as one captured CUDA graph (lane tables in device memory), one graph launch per token
        try:
            e2e["graph_replay_ms_per_step"] = timed(decode.token_graph(), steps, warmup, eager=True)
            e2e["graph_replay_mapped_host_ms_per_step"] = timed(decode.token_graph(mapped_host=True), steps, warmup, eager=True)
        except tb.TataraError:   # pragma: no cover
            pass
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
        # N > 1: the SAME lane, its key axis split over the ranks (strong scaling).  One submission per
        # rank and step (tatara_attn_decode_split), k steps captured in one graph per rank.
        split = wl.split_setup(dist, n)
        parity = split.check()
        launches0 = ctx.launches
        with ClockSampler(local) as clocks:
            ms = timed(split.step, steps, warmup, hold_s=1.0)
        ctx.sync()          # a bounded device wait that ran out raises here instead of reporting a fast time
        launches = ctx.launches - launches0 - 3 * warmup
        kernel_note = ("attn_decode_partition_kernel over this rank's key range (+ the two attn_combine_kernel "
                       "launches of the step: merge + peer stores, bounded wait + merge)")
        e2e_ms = timed(split.step_e2e, steps, warmup, eager=True)
        ctx.sync()
        e2e = {"ms_per_step": e2e_ms,
               "path": "host-issued C-ABI calls from Python on every rank: pinned H2D of the token projection, qk_rope, "
                       "tatara_attn_decode_split, D2H"}
        k_ms = timed(split.step_kernel_only, steps, warmup)
        c_ms = timed(split.step_collective_only, steps, warmup, eager=True)
        f_ms = timed(split.step_nccl, steps, warmup, eager=True)
        p_ms = timed(split.step, steps, warmup, eager=True)
        ctx.sync()
        local_keys = split.end - split.begin
        extra["split_kv"] = {
            "context": n, "gpus": world, "keys_per_gpu": local_keys, "kernel_us": k_ms * 1e3,
            "kernel_gbs_per_gpu": local_keys * 2048 / (k_ms * 1e-3) / 1e9,
            "one_submission_graph_us": ms * 1e3, "one_submission_host_issued_us": p_ms * 1e3,
            "nccl_form": {"collective_us": c_ms * 1e3, "end_to_end_us": f_ms * 1e3,
                          "aggregate_gbs": bytes_step / (f_ms * 1e-3) / 1e9,
                          "path": "partial records -> ncclAllGather (16512 B per rank) -> combine, host-issued"},
            "message_bytes_per_rank": 16 * 258 * 4, "parity": parity,
            "timing": "kernel and one_submission_graph: CUDA graph of k steps; the others: host-issued; CUDA events, max over ranks"}
        split.close()
        del split
        torch.cuda.empty_cache()
        # weak scaling beside it: one whole 262144-key lane per GPU, no collective
        decode = wl.decode_setup(n)
        w_ms = timed(decode.step, steps, warmup)
        extra["weak_lane_per_gpu"] = {"lanes": world, "ms_per_step": w_ms, "aggregate_gbs": world * bytes_step / (w_ms * 1e-3) / 1e9,
                                      "parallelism": "one lane per GPU, no collective"}
        decode.free()
        extra["lanes32"] = wl.lanes32(timed, steps, warmup)
    gbs = bytes_step / (ms * 1e-3) / 1e9           # the ONE lane's bytes over the step, whatever N
    e2e_gbs = bytes_step / (e2e_ms * 1e-3) / 1e9

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        import oracle

        def host_bits(t):   # bf16 device tensor -> uint16 bit patterns on the host
            return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
        threads = oracle.hardware_threads()
        keys, values = decode.caches[0]
        hq, hg, hk, hv = (host_bits(t) for t in (decode.q, decode.gate, keys, values))
        best, total, want = cpu_decode_sample(hq, hg, hk, hv, n, threads, repeats=8)
        cpu = {"value": decode_bytes(n) / best / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
               "sample": f"best of 8 full decode steps at context {n} ({total:.1f} s of host time)"}
        # parity of the GPU headline step against that oracle output (same inputs)
        decode.step(0)
        ctx.sync()
        got = host_bits(decode.out).astype(np.uint32) << 16
        got, ref = got.view(np.float32).astype(np.float64).ravel(), (want.astype(np.uint32) << 16).view(np.float32).astype(np.float64).ravel()
        parity = {"max_abs": float(np.abs(got - ref).max()),
                  "cosine": float(got @ ref / (np.linalg.norm(got) * np.linalg.norm(ref))),
                  "against": "the CPU oracle's decode of the headline step's own inputs", "gate": "max_abs <= 2e-2, cosine >= 0.9999"}

    if rank == 0:
        cfg = headline_config(world)
        line = {
            "metric": "decode_attn_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": ms, "us_per_layer": ms * 1e3,
            "higher_is_better": True, "scaling": "weak" if world == 1 else "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": cfg,
            "timing": "k steps captured in one CUDA graph per rank, timed with CUDA events around its replay, max over ranks",
            "roofline": {"bound": "hbm", "achieved": gbs / world, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / world / peaks["hbm_gbs"], "traffic": wl.traffic_hint() // world,
                         "peak_source": peaks["source"], "per": "GPU",
                         "kernel": kernel_note},
            "e2e": dict({"value": e2e_gbs, "unit": "GB/s", "h2d_bytes_per_step": 9216 * 2, "d2h_bytes_per_step": 4096 * 2}, **e2e),
            "gpu_launches": int(launches),
            "clocks": clocks.summary(),
            "cpu_baseline": cpu,
            "parity": parity,
        }
        line.update(extra)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())

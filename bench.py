#!/usr/bin/env python
"""Benchmark of the frame->action forward path: the 2-D frame encoder configuration (BGRA 256x144
frames -> conv/ResConv encoder -> mask attention -> pool -> FC heads) at 256 frames per GPU.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch 256] [--impl ours|reference]

One process per GPU (torchrun for N > 1).  Frames are independent, so ranks shard the batch
(weak scaling: 256 frames per GPU), the checkpoint is broadcast once with NCCL and there is no
collective in the step loop.  Prints ONE JSON line on rank 0.

`value`     frames/s with the frames already resident in HBM (CUDA events, max over ranks).
`e2e`       the same metric through the host-buffer entry point (aig_cnn_infer_host): pinned host
            frames -> H2D copy -> forward -> D2H copy of the fp32 outputs, every step.
`roofline`  the heaviest kernel launch of the step: algorithmic FLOP / its mean duration measured
            with CUDA events between launches inside the timed steps, against the measured peak.
`cpu_baseline` / `--impl reference`: the CPU oracle (a port of the reference's layer math; the
            reference has no CPU path and its Windows/cuDNN-7 program cannot run here) timed on the
            host cores on a bounded sample of the same workload.
"""
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

WIDTHS = (32, 64, 128, 256, 256)
HEIGHT, WIDTH = 144, 256
N_OUT, N_SIG = 18, 16
FLOP_PER_FRAME = 2 * 620.9e6  # 2 * MAC of the convolutions of one frame


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(hbm=d["hbm_gbs"], tensor=d["bf16_tflops_sustained"], tensor_burst=d["bf16_tflops"], source="measured")
    return dict(hbm=6650.0, tensor=1400.0, tensor_burst=1590.0, source="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs (read-only)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for nm, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_oracle_rate(frames_per_sample, repeats):
    """frames/s of the CPU oracle on a bounded sample of the workload (all host threads)."""
    from oracle import oracle as O
    from oracle import pipelines as PL

    O.build()
    O.set_threads(os.cpu_count() or 1)  # launchers export OMP_NUM_THREADS=1 for their ranks; this leg wants every core
    params = PL.make_cnn_params(0, widths=WIDTHS)
    frames = PL.make_frames(0, frames_per_sample, HEIGHT, WIDTH)
    PL.cnn_forward(params, frames[:1])  # warm
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        PL.cnn_forward(params, frames)
        times.append(time.perf_counter() - t0)
    return frames_per_sample / float(np.median(times)), times


def streaming_latency(pkg, ctx, SY, n_frames):
    """p50/p99 frame->action latency of the full streaming agent at batch 1: pinned host frame in,
    fp32 outputs on the host out (aig_agent_step_host), one frame at a time, carried LSTM state and
    a 64-slot attention ring cache."""
    import torch
    from ai_gamer_b200 import runners as R

    agent = R.Agent(ctx, 1, HEIGHT, WIDTH, widths=WIDTHS, d=512, layers=2, heads=8, n_out=N_OUT, n_sigmoid=N_SIG, window=64)
    agent.load_bytes(SY.serialize_agent_params(SY.make_agent_params(0, widths=WIDTHS), WIDTH, HEIGHT))
    rng = np.random.default_rng(7)
    frames = [torch.from_numpy(rng.integers(0, 256, (1, HEIGHT, WIDTH, 4), dtype=np.uint8)).pin_memory() for _ in range(8)]
    out = torch.empty((1, N_OUT), dtype=torch.float32).pin_memory()
    for i in range(20):
        agent.step_host(frames[i % 8], out)
    agent.reset()
    lat = []
    for i in range(n_frames):
        t0 = time.perf_counter()
        agent.step_host(frames[i % 8], out)
        lat.append((time.perf_counter() - t0) * 1e3)
    agent.close()
    lat = np.array(lat)
    return {"workload": "streaming agent (cnn + fc + 2xLSTM512 + MHA8x64 ring-64 + LN + FC), batch 1, %d frames" % n_frames,
            "p50_ms": float(np.percentile(lat, 50)), "p99_ms": float(np.percentile(lat, 99)), "mean_ms": float(lat.mean())}


def run_reference(args, rank):
    """--impl reference: the reference's layer math on the host cores (oracle port)."""
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    sample = 16
    for _ in range(max(args.warmup, 0)):
        cpu_oracle_rate(2, 1)
    t0 = time.perf_counter()
    per_step = []
    for _ in range(args.steps):
        rate, times = cpu_oracle_rate(sample, 1)
        per_step.append(times[0])
    total = time.perf_counter() - t0
    value = sample * args.steps / sum(per_step)
    line = {
        "impl": "reference", "metric": "frames/s per B200 (batch 256)", "value": value, "unit": "frames/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * sum(per_step) / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16 storage, f64 accumulate", "data": "synthetic",
        "config": {"workload": "cnn2d_encoder_144x256_b256", "note": "each step is a %d-frame sample of the workload" % sample},
        "cpu_baseline": {"value": value, "unit": "frames/s", "cores": cores, "kind": "port",
                         "sample": "%d frames per step, %d steps, OpenMP over all host threads" % (sample, args.steps)},
        "e2e": {"value": value, "unit": "frames/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": total,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=256, help="frames per GPU per step")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (used for short profiler captures)")
    ap.add_argument("--no-latency", action="store_true", help="skip the batch-1 streaming latency leg")
    ap.add_argument("--latency-frames", type=int, default=1000)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry

    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    pkg = entry.load_package()
    from ai_gamer_b200 import synth as SY  # seeded parameter / frame generators (numpy only)

    ctx = pkg.Context(local_rank)
    B = args.batch
    enc = pkg.CnnEncoder(ctx, B, HEIGHT, WIDTH, widths=WIDTHS, n_out=N_OUT, n_sigmoid=N_SIG)

    # checkpoint: rank 0 builds it, one NCCL broadcast, every rank loads its own copy
    from ai_gamer_b200 import sharding as SH

    nbytes = enc.checkpoint_bytes()
    blob = SY.serialize_cnn_checkpoint(SY.make_cnn_params(0, widths=WIDTHS), WIDTH, HEIGHT) if rank == 0 else None
    enc.load_bytes(SH.broadcast_bytes(blob, nbytes, 0, "cuda"))

    # inputs: rotate over enough frame batches to exceed the 126 MB L2
    n_rot = max(2, -(-150_000_000 // (B * HEIGHT * WIDTH * 4)))
    rng = np.random.default_rng(1000 + rank)
    host_frames = [torch.from_numpy(rng.integers(0, 256, (B, HEIGHT, WIDTH, 4), dtype=np.uint8)).pin_memory() for _ in range(n_rot)]
    dev_frames = [f.cuda() for f in host_frames]
    host_out = torch.empty((B, N_OUT), dtype=torch.float32).pin_memory()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        enc.forward(dev_frames[i % n_rot])
    ctx.sync()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # ---- device-resident throughput: exactly K forwards between two CUDA events
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        enc.forward(dev_frames[i % n_rot])
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    # ---- the same forwards again with one CUDA event between consecutive launches (per-kernel durations for
    # the roofline; the extra event records cost ~4 % of a step, which is why they are not in the region above)
    prof_n = min(args.steps, 200)
    enc.profile_begin(prof_n)
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record()
    for i in range(prof_n):
        enc.forward(dev_frames[i % n_rot])
    p1.record()
    barrier()
    prof_ms = p0.elapsed_time(p1) / prof_n
    sites, prof_steps = enc.profile_end()
    ctx.sync()
    # ---- end to end through the host-buffer entry point
    # every step: H2D copy of that step's 256 frames from pinned memory, forward, D2H of the fp32 outputs into
    # pinned memory; two slots alternate so the copy of step i+1 overlaps the forward of step i, and each
    # step's outputs are waited for (aig_cnn_wait) before its slot is reused
    e2e_steps = 0 if args.no_e2e else args.steps
    host_outs = [torch.empty((B, N_OUT), dtype=torch.float32).pin_memory() for _ in range(2)]
    for i in range(4 if e2e_steps else 0):
        enc.submit_host(i & 1, host_frames[i % n_rot], host_outs[i & 1])
        enc.wait(i & 1)
    barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        if i >= 2:
            enc.wait(i & 1)
        enc.submit_host(i & 1, host_frames[i % n_rot], host_outs[i & 1])
    for i in range(max(e2e_steps - 2, 0), e2e_steps):
        enc.wait(i & 1)
    torch.cuda.synchronize()
    e2e_s = max(time.perf_counter() - t0, 1e-9)
    barrier()
    # a short run gives the 50 ms sampler too few readings: keep the same forwards going (outside every timed
    # region) until there are enough samples of the clocks under this load
    extra_load_s = 0.0
    if rank == 0 and len(sampler.lines) < 8:
        t_load = time.perf_counter()
        while len(sampler.lines) < 8 and time.perf_counter() - t_load < 2.0:
            for i in range(50):
                enc.forward(dev_frames[i % n_rot])
            ctx.sync()
        extra_load_s = time.perf_counter() - t_load
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    if clocks is not None and extra_load_s > 0:
        clocks["note"] = "timed regions too short for the sampler: %.2f s of the same forwards added after them" % extra_load_s

    ms, e2e_ms = SH.max_over_ranks([ms, e2e_s * 1e3], "cuda")

    latency = None
    if rank == 0 and not args.no_latency:
        latency = streaming_latency(pkg, ctx, SY, args.latency_frames)

    if rank == 0:
        peaks = measured_peaks()
        value = world * B * args.steps / (ms * 1e-3)
        e2e_value = world * B * args.steps / (e2e_ms * 1e-3) if not args.no_e2e else None
        layers = []
        for name, lms, flops, nbytes_ in sites:
            layers.append({"site": name, "ms": round(lms, 5), "tflops": round(flops / (lms * 1e-3) / 1e12, 2) if lms > 0 and flops else None,
                           "gbs": round(nbytes_ / (lms * 1e-3) / 1e9, 1) if lms > 0 else None})
        # dominant kernel = the convolution GEMM kernel (every residual-block launch of a step); its roofline
        # figure is the sum of their algorithmic FLOPs over the sum of their CUDA-event durations
        gemm = [(n, m_, f, b_) for n, m_, f, b_ in sites if n.startswith("res") and m_ > 0]
        g_ms = sum(r[1] for r in gemm)
        g_flops = sum(r[2] for r in gemm)
        g_bytes = sum(r[3] for r in gemm)
        achieved = g_flops / (g_ms * 1e-3) / 1e12
        traffic = None
        tpath = os.path.join(ROOT, "profiles", "traffic.json")
        if os.path.exists(tpath):
            with open(tpath) as f:
                tj = json.load(f)
            if all(r[0] in tj for r in gemm):
                traffic = sum(tj[r[0]] for r in gemm)
        top_kernel = "pconv_kernel / igemm_kernel (tcgen05 convolution GEMM), %d launches per step, %.0f%% of the step" % (
            len(gemm), 100.0 * g_ms / sum(r[1] for r in sites))
        line = {
            "metric": "frames/s per B200 (batch 256)", "value": value, "unit": "frames/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16 (fp32 accumulate)", "data": "synthetic",
            "config": {"workload": "cnn2d_encoder_144x256_b%d" % B, "frames_per_gpu": B, "global_batch": world * B,
                       "sharding": "batch of independent frames, no step-loop collective",
                       "l2": "inputs rotate over %d batches (%.0f MB > 126 MB L2); activations written ~%.2f GB per step" % (
                           n_rot, n_rot * B * HEIGHT * WIDTH * 4 / 1e6, B * 2.19e6 / 1e9)},
            "e2e": {"value": e2e_value, "unit": "frames/s", "h2d_bytes_per_step": B * HEIGHT * WIDTH * 4,
                    "d2h_bytes_per_step": B * N_OUT * 4, "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": args.steps * enc.kernel_launches,
            "latency": latency,
            "roofline": {"bound": "tensor", "kernel": top_kernel, "achieved": achieved, "peak": peaks["tensor"],
                         "unit": "TFLOP/s", "frac": achieved / peaks["tensor"], "traffic": traffic, "peak_source": peaks["source"] + " (sustained bf16)",
                         "timed_with": "one CUDA event between launches over %d further steps of the same loop (%.4f ms/step with the events)" % (
                             prof_steps, prof_ms),
                         "algorithmic_gbs": g_bytes / (g_ms * 1e-3) / 1e9, "hbm_frac": g_bytes / (g_ms * 1e-3) / 1e9 / peaks["hbm"],
                         "whole_step_tflops": FLOP_PER_FRAME * B / (ms / args.steps * 1e-3) / 1e12,
                         "whole_step_frac": FLOP_PER_FRAME * B / (ms / args.steps * 1e-3) / 1e12 / peaks["tensor"]},
            "layers": layers,
            "clocks": clocks,
        }
        if not args.no_cpu_baseline and world == 1:
            cores = os.cpu_count() or 1
            sample = 16
            rate, times = cpu_oracle_rate(sample, 5)
            line["cpu_baseline"] = {"value": rate, "unit": "frames/s", "cores": cores, "kind": "port",
                                    "sample": "%d frames, median of 5 runs (%.2f s each), OpenMP over all host threads" % (
                                        sample, float(np.median(times)))}
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line), flush=True)
    enc.close()
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

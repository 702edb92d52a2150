#!/usr/bin/env python
"""Benchmark of the frame->action forward path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cnn2d|conv3d|seqhead|agent_batched]
                    [--impl ours|reference] [--legs all|none|conv3d,seqhead,agent_batched]

Headline workload (`cnn2d`): the 2-D frame encoder configuration (BGRA 256x144 frames -> conv/ResConv
encoder -> mask attention -> pool -> FC heads) at 256 frames per GPU.  The other configurations ride on the
same JSON line under `workloads` (or become the headline with --workload): `conv3d` = the temporal clip
encoder on 16 clips of 8x144x256, `seqhead` = 2xLSTM-512 -> 8x64 attention -> LayerNorm -> FC on 128
sequences x 64 steps, `agent_batched` = the full streaming agent on 128 sequences per GPU, one frame per
sequence per step.

One process per GPU (torchrun for N > 1).  Units (frames, clips, sequences) are independent, so every rank
runs the per-GPU batch (weak scaling), the parameters are broadcast once with NCCL and there is no collective
in the step loop.  Rank 0 prints ONE JSON line.

Timing: a region is exactly K steps between two CUDA events with a barrier + synchronize on both sides;
R >= 25 regions run back to back (at least ~2 s in all) and the MEDIAN region gives `ms_per_step` and `value`
(min/max beside it); clocks are sampled with nvidia-smi (read only) around exactly those regions.

`value`     units/s with the inputs already resident in HBM (max over ranks per region).
`e2e`       the same metric through the host-buffer entry points: pinned host frames -> H2D copy ->
            forward -> D2H copy of the fp32 outputs, every step, two slots in flight.
`roofline`  the dominant kernel class: algorithmic FLOP / CUDA-event duration against the measured peaks
            (`frac` = of the sustained figure, `frac_burst` = of the burst figure).
`cpu_baseline` / `--impl reference`: the CPU oracle (a port of the reference's layer math; the reference
            has no CPU path and its Windows/cuDNN-7 program cannot run here) on a bounded sample.
"""
import argparse
import json
import math
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
FLOP_PER_FRAME = 2 * 620.9e6           # 2 * MAC of the convolutions of one frame (encoder)
FLOP_PER_CLIP = 2 * 2229.5e6           # clip encoder: 191.1 + 1019.2 + 1019.2 MMAC
FLOP_CLIP_LAYER = 2 * 1019.2e6         # each of its two channel-rich layers
SEQ_B, SEQ_T, SEQ_D = 128, 64, 512
FLOP_PER_SEQ_BATCH = 86.6e9            # 128 x 64 steps: LSTM 34.36, projections 8.59, attention 0.27, FC 0.08 GMAC
FLOP_PER_AGENT_FRAME = 1.253e9         # encoder + bridge FC + sequence-head step
MIN_REGIONS, MIN_TOTAL_S, MAX_REGIONS = 25, 2.0, 400


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(hbm=d["hbm_gbs"], tensor=d["bf16_tflops_sustained"], tensor_burst=d["bf16_tflops"], source="measured")
    return dict(hbm=6650.0, tensor=1400.0, tensor_burst=1590.0, source="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while a timed region runs (read-only)."""
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
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def stop(self, t_lo=None, t_hi=None):
        """Summary of the samples taken between t_lo and t_hi (perf_counter times; default: all)."""
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ts, ln in self.lines:
            if (t_lo is not None and ts < t_lo) or (t_hi is not None and ts > t_hi + 0.06):
                continue
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                pw.append(float(f[3]))
            except ValueError:
                continue
            for nm, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w": float(np.median(pw)) if pw else None, "samples": len(sm), "reasons": sorted(reasons)}


class Timer:
    """R regions of exactly K steps each, CUDA events on the launching stream, barrier + synchronize on both
    sides of every region, max over ranks per region; the median region is the result."""

    def __init__(self, world, device):
        import torch
        import torch.distributed as dist

        self.torch, self.dist, self.world, self.device = torch, dist, world, device

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, values):
        from ai_gamer_b200 import sharding as SH

        return SH.max_over_ranks(values, self.device)

    def region(self, step, k, i0=0):
        self.barrier()
        e0, e1 = self.torch.cuda.Event(enable_timing=True), self.torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(k):
            step(i0 + i)
        e1.record()
        self.barrier()
        return e0.elapsed_time(e1)

    def regions(self, step, k, warmup, sample_clocks_on=None):
        """-> dict(ms_per_step median/min/max, repeats, clocks).  The number of regions is agreed between the
        ranks from one untimed trial region."""
        for i in range(warmup):
            step(i)
        trial = self.max_over_ranks([self.region(step, k)])[0]
        reps = int(min(MAX_REGIONS, max(MIN_REGIONS, math.ceil(MIN_TOTAL_S * 1e3 / max(trial, 1e-3)))))
        sampler = ClockSampler(sample_clocks_on).start() if sample_clocks_on is not None else None
        time.sleep(0.06 if sampler else 0.0)
        t_lo = time.perf_counter()
        ms = [self.region(step, k, r * k) for r in range(reps)]
        t_hi = time.perf_counter()
        clocks = sampler.stop(t_lo, t_hi) if sampler else None
        ms = np.array(self.max_over_ranks(ms))
        return {"ms_per_step": float(np.median(ms)) / k, "ms_per_step_min": float(ms.min()) / k, "ms_per_step_max": float(ms.max()) / k,
                "repeats": reps, "timed_s": float(ms.sum()) * 1e-3, "clocks": clocks}


def fracs(achieved_tflops, peaks):
    return {"achieved": achieved_tflops, "peak": peaks["tensor"], "unit": "TFLOP/s", "frac": achieved_tflops / peaks["tensor"],
            "peak_burst": peaks["tensor_burst"], "frac_burst": achieved_tflops / peaks["tensor_burst"],
            "peak_source": peaks["source"] + " (bf16 GEMM: sustained = frac, burst = frac_burst)"}


# --------------------------------------------------------------------------------------------- CPU oracle legs
def oracle_modules():
    from oracle import oracle as O
    from oracle import pipelines as PL

    O.build()
    O.set_threads(os.cpu_count() or 1)  # launchers export OMP_NUM_THREADS=1 for their ranks; this leg wants every core
    return O, PL


def cpu_sample(workload, repeats):
    """(units/s, unit, seconds per run, description of the sample) of the CPU oracle on a bounded sample."""
    O, PL = oracle_modules()
    if workload == "cnn2d":
        n = 16
        params, frames = PL.make_cnn_params(0, widths=WIDTHS), PL.make_frames(0, n, HEIGHT, WIDTH)
        PL.cnn_forward(params, frames[:1])
        run, unit, what = (lambda: PL.cnn_forward(params, frames)), "frames/s", "%d frames of 144x256" % n
    elif workload == "conv3d":
        n = 1
        params, clips = PL.make_conv3d_params(0), PL.make_clips(0, n)
        run, unit, what = (lambda: PL.conv3d_forward(params, clips)), "clips/s", "%d clip of 8x144x256" % n
    elif workload == "seqhead":
        nseq = 2
        params, emb = PL.make_seq_params(0), PL.make_embeddings(0, SEQ_T, nseq, SEQ_D)
        n = nseq * SEQ_T
        run, unit, what = (lambda: PL.seq_forward(params, emb)), "frame-steps/s", "%d sequences x %d steps" % (nseq, SEQ_T)
    elif workload == "agent_batched":
        n = 8
        p = PL.make_agent_params(0, widths=WIDTHS)
        frames = PL.make_frames(0, n, HEIGHT, WIDTH)

        def run():
            emb = O.fc(PL.cnn_forward(p["cnn"], frames)[0], p["bw"], p["bb"])[:, None]   # 8 steps of one sequence
            return PL.seq_forward(p["seq"], emb, window=64)
        unit, what = "frames/s", "%d frames of one sequence (encoder + sequence-head steps)" % n
    else:
        raise ValueError(workload)
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        run()
        times.append(time.perf_counter() - t0)
    return n / float(np.median(times)), unit, times, what


def cpu_baseline_block(workload, repeats=3):
    rate, unit, times, what = cpu_sample(workload, repeats)
    return {"value": rate, "unit": unit, "cores": os.cpu_count() or 1, "kind": "port",
            "sample": "%s, median of %d runs (%.2f s each), OpenMP over all host threads" % (what, len(times), float(np.median(times)))}


METRICS = {"agent_stream": ("frames/s of one sequence, one frame per step (device-resident frames)", "frames/s", "streaming_agent_b1_window64"),
           "cnn2d": ("frames/s per GPU-batch of 256, summed over the GPUs", "frames/s", "cnn2d_encoder_144x256_b256"),
           "conv3d": ("clips/s (16 clips of 8x144x256 per GPU), summed over the GPUs", "clips/s", "conv3d_clip_encoder_8x144x256_b16"),
           "seqhead": ("frame-steps/s (128 sequences x 64 steps per GPU), summed over the GPUs", "frame-steps/s", "seqhead_lstm2x512_mha8x64_b128_t64"),
           "agent_batched": ("frames/s (128 sequences per GPU, one frame each per step), summed over the GPUs", "frames/s",
                             "streaming_agent_b128_window64")}


def run_reference(args, rank):
    """--impl reference: the reference's layer math on the host cores (oracle port), each step a bounded sample."""
    if rank != 0:
        return
    wl = args.workload
    for _ in range(max(args.warmup, 0)):
        cpu_sample(wl, 1)
    t0 = time.perf_counter()
    per_step, rate, unit, what = [], 0.0, "", ""
    for _ in range(args.steps):
        rate, unit, times, what = cpu_sample(wl, 1)
        per_step.append(times[0])
    n = rate * per_step[-1]
    value = n * args.steps / sum(per_step)
    cores = os.cpu_count() or 1
    line = {
        "impl": "reference", "metric": METRICS[wl][0], "value": value, "unit": METRICS[wl][1], "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * sum(per_step) / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16 storage, f64 accumulate", "data": "synthetic",
        "config": {"workload": METRICS[wl][2], "note": "each step is a sample of the workload: " + what},
        "cpu_baseline": {"value": value, "unit": METRICS[wl][1], "cores": cores, "kind": "port",
                         "sample": "%s per step, %d steps, OpenMP over all host threads" % (what, args.steps)},
        "e2e": {"value": value, "unit": METRICS[wl][1], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------- GPU legs
class Env:
    def __init__(self, args):
        import torch
        import torch.distributed as dist
        import __graft_entry__ as entry

        self.torch, self.dist = torch, dist
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local_rank)
        if self.world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local_rank))
        self.pkg = entry.load_package()
        from ai_gamer_b200 import runners, sharding, synth

        self.R, self.SH, self.SY = runners, sharding, synth
        self.ctx = self.pkg.Context(self.local_rank)
        self.timer = Timer(self.world, "cuda")
        self.peaks = measured_peaks()
        self.args = args
        self.profile = False   # profiler captures: a few untimed steps only

    def broadcast(self, make_blob, nbytes):
        """Rank 0 builds the parameter bytes, one NCCL broadcast, every rank loads its own copy."""
        blob = make_blob() if self.rank == 0 else None
        return self.SH.broadcast_bytes(blob, nbytes, 0, "cuda")

    def close(self):
        self.ctx.close()
        if self.world > 1:
            self.dist.destroy_process_group()


def leg_cnn2d(env, full):
    """The headline: 256 frames per GPU through the 2-D encoder."""
    torch, pkg, SY, args = env.torch, env.pkg, env.SY, env.args
    B = args.batch
    enc = pkg.CnnEncoder(env.ctx, B, HEIGHT, WIDTH, widths=WIDTHS, n_out=N_OUT, n_sigmoid=N_SIG)
    enc.load_bytes(env.broadcast(lambda: SY.serialize_cnn_checkpoint(SY.make_cnn_params(0, widths=WIDTHS), WIDTH, HEIGHT), enc.checkpoint_bytes()))
    # inputs: rotate over enough frame batches to exceed the 126 MB L2
    n_rot = max(2, -(-150_000_000 // (B * HEIGHT * WIDTH * 4)))
    rng = np.random.default_rng(1000 + env.rank)
    host_frames = [torch.from_numpy(rng.integers(0, 256, (B, HEIGHT, WIDTH, 4), dtype=np.uint8)).pin_memory() for _ in range(n_rot)]
    dev_frames = [f.cuda() for f in host_frames]
    # the same frames as planar R, G, B planes (what the reference's recorder stores and GrabFrameInt8(planar) delivers)
    host_planar = [f[..., [2, 1, 0]].permute(0, 3, 1, 2).contiguous().pin_memory() for f in host_frames]
    K = args.steps
    res = env.timer.regions(lambda i: enc.forward(dev_frames[i % n_rot]), K, args.warmup, env.local_rank if env.rank == 0 else None)
    ms = res["ms_per_step"]
    out = {"value": env.world * B / (ms * 1e-3), "unit": "frames/s", **{k: res[k] for k in ("ms_per_step", "ms_per_step_min", "ms_per_step_max", "repeats", "timed_s")},
           "clocks": res["clocks"], "gpu_launches": K * enc.kernel_launches, "launches_per_step": enc.kernel_launches,
           "l2": "inputs rotate over %d batches (%.0f MB > 126 MB L2); activations written ~%.2f GB per step" % (
               n_rot, n_rot * B * HEIGHT * WIDTH * 4 / 1e6, B * 2.19e6 / 1e9)}
    if env.profile:
        enc.close()
        return out
    # ---- per-launch durations: the same forwards with one CUDA event between consecutive launches (the event
    # records cost a few % of a step, which is why they are not in the regions above), clocks sampled around it
    prof_n = max(50, min(400, int(1.0 / max(ms * 1e-3, 1e-6))))
    sampler = ClockSampler(env.local_rank).start() if env.rank == 0 else None
    time.sleep(0.06 if sampler else 0.0)
    enc.profile_begin(prof_n)
    env.timer.barrier()
    t_lo = time.perf_counter()
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record()
    for i in range(prof_n):
        enc.forward(dev_frames[i % n_rot])
    p1.record()
    env.timer.barrier()
    t_hi = time.perf_counter()
    prof_ms = p0.elapsed_time(p1) / prof_n
    sites, prof_steps = enc.profile_end()
    prof_clocks = sampler.stop(t_lo, t_hi) if sampler else None
    env.ctx.sync()
    # ---- end to end through the host-buffer entry point: every step copies its 256 frames H2D from pinned
    # memory, runs the forward and copies the fp32 outputs D2H into pinned memory; two slots alternate so the
    # copy of step i+1 overlaps the forward of step i; each step's outputs are waited for before its slot is reused
    e2e = None
    if not args.no_e2e:
        host_outs = [torch.empty((B, N_OUT), dtype=torch.float32).pin_memory() for _ in range(2)]

        def e2e_leg(submit, frames, bytes_per_px, entry):
            def e2e_region(k, i0):
                env.timer.barrier()
                t0 = time.perf_counter()
                for i in range(k):
                    if i >= 2:
                        enc.wait(i & 1)
                    submit(i & 1, frames[(i0 + i) % n_rot], host_outs[i & 1])
                for i in range(max(k - 2, 0), k):
                    enc.wait(i & 1)
                torch.cuda.synchronize()
                dt = time.perf_counter() - t0
                env.timer.barrier()
                return dt * 1e3

            e2e_region(4, 0)
            trial = env.timer.max_over_ranks([e2e_region(K, 0)])[0]
            reps = int(min(MAX_REGIONS, max(MIN_REGIONS, math.ceil(MIN_TOTAL_S * 1e3 / max(trial, 1e-3)))))
            ems = np.array(env.timer.max_over_ranks([e2e_region(K, r * K) for r in range(reps)]))
            e_ms = float(np.median(ems)) / K
            h2d = B * HEIGHT * WIDTH * bytes_per_px
            return {"value": env.world * B / (e_ms * 1e-3), "unit": "frames/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": B * N_OUT * 4,
                    "ms_per_step": e_ms, "ms_per_step_min": float(ems.min()) / K, "ms_per_step_max": float(ems.max()) / K, "repeats": reps,
                    "h2d_gbs_per_gpu": h2d / (e_ms * 1e-3) / 1e9, "entry_point": entry}

        # headline: planar RGB host frames, 3 bytes per pixel; beside it the BGRA form of the same frames
        e2e = e2e_leg(enc.submit_host_rgb, host_planar, 3, "aig_cnn_submit_host_rgb / aig_cnn_wait (planar R,G,B uint8 frames, 3 bytes per pixel)")
        e2e["bgra"] = e2e_leg(enc.submit_host, host_frames, 4, "aig_cnn_submit_host / aig_cnn_wait (BGRA frames, 4 bytes per pixel)")
    # ---- roofline of the convolution-GEMM kernel class (every residual-block launch of a step)
    layers = [{"site": n, "ms": round(m_, 5), "tflops": round(f / (m_ * 1e-3) / 1e12, 2) if m_ > 0 and f else None,
               "gbs": round(b_ / (m_ * 1e-3) / 1e9, 1) if m_ > 0 else None} for n, m_, f, b_ in sites]
    gemm = [r for r in sites if r[0].startswith("res") and r[1] > 0]
    g_ms, g_flops, g_bytes = sum(r[1] for r in gemm), sum(r[2] for r in gemm), sum(r[3] for r in gemm)
    achieved = g_flops / (g_ms * 1e-3) / 1e12
    traffic = None
    tpath = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(tpath):
        with open(tpath) as f:
            tj = json.load(f)
        if all(r[0] in tj for r in gemm):
            traffic = sum(tj[r[0]] for r in gemm)
    whole = FLOP_PER_FRAME * B / (ms * 1e-3) / 1e12
    roof = {"bound": "tensor", "kernel": "pconv_kernel (tcgen05 convolution GEMM), %d launches per step, %.0f%% of the step" % (
                len(gemm), 100.0 * g_ms / sum(r[1] for r in sites)),
            **fracs(achieved, env.peaks), "traffic": traffic,
            "timed_with": "one CUDA event between launches over %d steps of the same loop (%.4f ms/step with the events)" % (prof_steps, prof_ms),
            "sm_mhz": prof_clocks["sm_mhz"] if prof_clocks else None, "clocks": prof_clocks,
            "algorithmic_gbs": g_bytes / (g_ms * 1e-3) / 1e9, "hbm_frac": g_bytes / (g_ms * 1e-3) / 1e9 / env.peaks["hbm"],
            "whole_step_tflops": whole, "whole_step_frac": whole / env.peaks["tensor"], "whole_step_frac_burst": whole / env.peaks["tensor_burst"]}
    out.update({"e2e": e2e, "roofline": roof, "layers": layers})
    enc.close()
    return out


def leg_conv3d(env, full):
    """Temporal clip encoder: 16 clips of 8 x 144 x 256 per GPU."""
    torch, pkg, SY, R, args = env.torch, env.pkg, env.SY, env.R, env.args
    B, D = 16, 8
    enc = R.ClipEncoder(env.ctx, B, D, HEIGHT, WIDTH)
    enc.load_bytes(env.broadcast(lambda: SY.serialize_conv3d_params(SY.make_conv3d_params(0)), enc.param_bytes()))
    n_rot = 6                                                                   # 6 x 28.3 MB of clips > 126 MB L2
    clips = [torch.rand((B, 3, D, HEIGHT, WIDTH), device="cuda", generator=torch.Generator("cuda").manual_seed(7 + i + 100 * env.rank)).half() for i in range(n_rot)]
    K = args.steps if env.profile else max(args.steps, 10)
    res = env.timer.regions(lambda i: enc.forward(clips[i % n_rot]), K, args.warmup, env.local_rank if env.rank == 0 else None)
    ms = res["ms_per_step"]
    enc.close()
    out = {"value": env.world * B / (ms * 1e-3), "unit": "clips/s", "frames_per_s": env.world * B * D / (ms * 1e-3), "steps": K,
           **{k: res[k] for k in ("ms_per_step", "ms_per_step_min", "ms_per_step_max", "repeats", "timed_s")}, "clocks": res["clocks"],
           "gpu_launches": K * 8, "l2": "inputs rotate over %d clip batches (%.0f MB > 126 MB L2)" % (n_rot, n_rot * B * 3 * D * HEIGHT * WIDTH * 2 / 1e6)}
    whole = FLOP_PER_CLIP * B / (ms * 1e-3) / 1e12
    roof = {"bound": "tensor", "kernel": "whole forward (3 convolution launches + pool + FC head)", **fracs(whole, env.peaks)}
    if full:
        # the two channel-rich layers alone (the igemm kernel class of this workload), each on rotating buffers > L2
        lay = []
        for (ci, co, h, w) in ((32, 64, 72, 128), (64, 128, 36, 64)):
            plan = pkg.ConvPlan(env.ctx, B, ci, h, w, co, 3, 2, 1, act=pkg.ACT_LEAKY, in_d=D, kd=3, sd=1, pd=1)
            wt = (torch.randn(co * ci * 27, device="cuda") * 0.05).half()
            bs = torch.zeros(co, device="cuda").half()
            torch.cuda.synchronize()   # (torch fills these on its own stream; the library's context has another)
            plan.set_weights(wt, bs)
            n_in, n_out = B * D * h * w * ci, B * D * (h // 2) * (w // 2) * co
            rot = max(2, -(-140_000_000 // (n_in * 2)))
            xs = [torch.randn(n_in, device="cuda").half() for _ in range(rot)]
            ys = [torch.empty(n_out, device="cuda", dtype=torch.float16) for _ in range(2)]
            r = env.timer.regions(lambda i: plan.forward(xs[i % rot], ys[i & 1]), 20, 3)
            plan.close()
            tf = FLOP_CLIP_LAYER * B / (r["ms_per_step"] * 1e-3) / 1e12
            lay.append({"site": "conv3d %d->%d on %dx%dx%d" % (ci, co, D, h, w), "ms": r["ms_per_step"], "tflops": tf,
                        "frac": tf / env.peaks["tensor"], "frac_burst": tf / env.peaks["tensor_burst"],
                        "gbs": (n_in + n_out) * 2 / (r["ms_per_step"] * 1e-3) / 1e9})
        g_ms = sum(x["ms"] for x in lay)
        roof = {"bound": "tensor", "kernel": "convolution GEMM of the two channel-rich Conv3D layers (timed alone, inputs rotating > L2)",
                **fracs(2 * FLOP_CLIP_LAYER * B / (g_ms * 1e-3) / 1e12, env.peaks), "layers": lay,
                "whole_step_tflops": whole, "whole_step_frac": whole / env.peaks["tensor"], "whole_step_frac_burst": whole / env.peaks["tensor_burst"]}
    out["roofline"] = roof
    return out


def leg_seqhead(env, full):
    """Sequence head: 128 sequences x 64 steps x 512 per GPU (2 x LSTM-512 -> MHA 8x64 causal + RoPE -> LN -> FC)."""
    torch, pkg, SY, R, args = env.torch, env.pkg, env.SY, env.R, env.args
    B, T, d = SEQ_B, SEQ_T, SEQ_D
    head = R.SeqHead(env.ctx, B, T, in_c=d, hidden=d, layers=2, heads=8, rope_base=10000.0, window=0)
    head.load_bytes(env.broadcast(lambda: SY.serialize_seq_params(SY.make_seq_params(0)), head.param_bytes()))
    n_rot = 16                                                                  # 16 x 8.4 MB of embeddings > 126 MB L2
    embs = [torch.randn(B * T * d, device="cuda", generator=torch.Generator("cuda").manual_seed(11 + i + 100 * env.rank)).half() for i in range(n_rot)]
    K = args.steps if env.profile else max(args.steps, 10)
    res = env.timer.regions(lambda i: head.forward(embs[i % n_rot]), K, args.warmup, env.local_rank if env.rank == 0 else None)
    ms = res["ms_per_step"]
    head.close()
    whole = FLOP_PER_SEQ_BATCH / (ms * 1e-3) / 1e12
    out = {"value": env.world * B * T / (ms * 1e-3), "unit": "frame-steps/s", "sequences_per_s": env.world * B / (ms * 1e-3), "steps": K,
           **{k: res[k] for k in ("ms_per_step", "ms_per_step_min", "ms_per_step_max", "repeats", "timed_s")}, "clocks": res["clocks"],
           "l2": "inputs rotate over %d embedding batches (%.0f MB > 126 MB L2)" % (n_rot, n_rot * B * T * d * 2 / 1e6)}
    roof = {"bound": "tensor", "kernel": "whole forward", **fracs(whole, env.peaks)}
    if full:
        # the parts alone: the two-layer LSTM (hoisted projections + persistent recurrence) and the attention layer
        sp = SY.make_seq_params(0)
        lp = pkg.LstmPlan(env.ctx, T, 2, d, B, d, batch_major=True)
        blob = torch.from_numpy(sp["lstm"]).cuda()
        torch.cuda.synchronize()
        lp.set_weights(blob)
        yy = torch.empty(B * T * d, device="cuda", dtype=torch.float16)
        r_l = env.timer.regions(lambda i: lp.forward(embs[i % n_rot], yy), 10, 3)
        lp.close()
        fp = pkg.FcPlan(env.ctx, B * T, d, 4 * d)
        pkg.lib().aig_fc_plan_set_output_f32(fp.handle, 1)
        wfc, bfc = torch.randn(4 * d * d, device="cuda").half(), torch.zeros(4 * d, device="cuda").half()
        torch.cuda.synchronize()
        fp.set_weights_out_in(wfc, bfc)
        gx = torch.empty(B * T * 4 * d, device="cuda", dtype=torch.float32)
        r_p = env.timer.regions(lambda i: fp.forward(embs[i % n_rot], gx), 10, 3)
        fp.close()
        mp = pkg.MhaPlan(env.ctx, B, T, d, 8, rope_base=10000.0)
        ws = [torch.from_numpy(sp[k]).cuda() for k in ("wq", "wk", "wv", "wo")]
        torch.cuda.synchronize()
        mp.set_weights(*ws)
        r_m = env.timer.regions(lambda i: mp.forward(embs[i % n_rot], yy), 10, 3)
        mp.close()
        rec_ms = (r_l["ms_per_step"] - 2 * r_p["ms_per_step"]) / 2             # one layer's recurrence
        # bytes one layer's recurrence moves: fp32 projections read once, h written once, and every CTA re-reads
        # the 128 x 512 previous h each step
        rec_bytes = B * T * 4 * d * 4 + B * T * d * 2
        roof.update({"lstm": {"ms_two_layers": r_l["ms_per_step"], "projection_ms_per_layer": r_p["ms_per_step"],
                              "projection_tflops": 2 * B * T * d * 4 * d / (r_p["ms_per_step"] * 1e-3) / 1e12,
                              "recurrence_ms_per_layer": rec_ms, "recurrence_us_per_step": rec_ms * 1e3 / T,
                              "recurrence_steps_per_s": T / (rec_ms * 1e-3), "recurrence_tflops": 2 * B * T * d * 4 * d / (rec_ms * 1e-3) / 1e12,
                              "recurrence_hbm_gbs": rec_bytes / (rec_ms * 1e-3) / 1e9, "recurrence_hbm_frac": rec_bytes / (rec_ms * 1e-3) / 1e9 / env.peaks["hbm"]},
                     "mha": {"ms": r_m["ms_per_step"], "tflops": 2 * (4 * B * T * d * d + B * 8 * T * T * 64) / (r_m["ms_per_step"] * 1e-3) / 1e12}})
    out["roofline"] = roof
    return out


def leg_agent_batched(env, full):
    """Full streaming agent, 128 sequences per GPU: every step feeds one new frame per sequence through the
    encoder, the bridge FC and the sequence-head step (carried LSTM state, 64-slot ring cache)."""
    torch, SY, R, args = env.torch, env.SY, env.R, env.args
    B = 128
    agent = R.Agent(env.ctx, B, HEIGHT, WIDTH, widths=WIDTHS, d=512, layers=2, heads=8, n_out=N_OUT, n_sigmoid=N_SIG, window=64)
    agent.load_bytes(env.broadcast(lambda: SY.serialize_agent_params(SY.make_agent_params(0, widths=WIDTHS), WIDTH, HEIGHT), agent.param_bytes()))
    n_rot = 8                                                                   # 8 x 18.9 MB of frames > 126 MB L2
    gen = torch.Generator("cuda").manual_seed(23 + 100 * env.rank)
    frames = [torch.randint(0, 256, (B, HEIGHT, WIDTH, 4), dtype=torch.uint8, device="cuda", generator=gen) for _ in range(n_rot)]
    K = args.steps if env.profile else 64                                       # one region = 64 frames of every sequence
    res = env.timer.regions(lambda i: agent.step(frames[i % n_rot]), K, max(args.warmup, n_rot), env.local_rank if env.rank == 0 else None)
    ms = res["ms_per_step"]
    agent.close()
    whole = FLOP_PER_AGENT_FRAME * B / (ms * 1e-3) / 1e12
    return {"value": env.world * B / (ms * 1e-3), "unit": "frames/s", "sequences_per_gpu": B, "steps": K,
            **{k: res[k] for k in ("ms_per_step", "ms_per_step_min", "ms_per_step_max", "repeats", "timed_s")}, "clocks": res["clocks"],
            "l2": "inputs rotate over %d frame batches (%.0f MB > 126 MB L2)" % (n_rot, n_rot * B * HEIGHT * WIDTH * 4 / 1e6),
            "roofline": {"bound": "tensor", "kernel": "whole step (encoder graph + bridge FC + sequence-head step launches)", **fracs(whole, env.peaks)}}


def streaming_latency(env, n_frames):
    """p50/p99 frame->action latency of the full streaming agent at batch 1: pinned host frame in, fp32 outputs
    on the host out (aig_agent_step_host), one frame at a time, carried LSTM state and a 64-slot ring cache."""
    torch, SY, R = env.torch, env.SY, env.R
    agent = R.Agent(env.ctx, 1, HEIGHT, WIDTH, widths=WIDTHS, d=512, layers=2, heads=8, n_out=N_OUT, n_sigmoid=N_SIG, window=64)
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


def reference_call_pattern(env):
    """The reference's own layer classes (oracle/_ref/libaig_reflayers.so: its sources compiled unchanged, calling
    cuDNN / cuBLAS as it does) run layer by layer on the encoder trunk of the headline workload at 256 frames:
    ConvLayer(3->32, k5 s2 p2) + BatchNorm + Swish, then four ResConvLayer blocks 32->64->128->256->256 -- the
    launch pattern of NN::Forward (NN.cpp:93-100) on this GPU.  A reported baseline beside the CPU one; it is a
    comparator built only where the reference tree was present, and nothing of it is part of the product."""
    import ctypes

    path = os.path.join(ROOT, "oracle", "_ref", "libaig_reflayers.so")
    if not os.path.exists(path):
        return {"unavailable": "oracle/_ref/libaig_reflayers.so was not built (reference tree absent at build time)"}
    torch = env.torch
    ref = ctypes.CDLL(path)
    P = ctypes.c_void_p
    ref.ref_layer_create.restype, ref.ref_layer_create.argtypes = P, [ctypes.c_char_p, ctypes.POINTER(ctypes.c_int), ctypes.c_int]
    ref.ref_layer_forward.restype, ref.ref_layer_forward.argtypes = P, [P, P]
    ref.ref_layer_destroy.argtypes = [P]
    ref.ref_last_error.restype = ctypes.c_char_p
    if ref.ref_init() != 0:
        return {"unavailable": ref.ref_last_error().decode()}
    B = 256
    torch.cuda.synchronize()

    def make(kind, *a):
        arr = (ctypes.c_int * len(a))(*a)
        h = ref.ref_layer_create(kind.encode(), arr, len(a))
        if not h:
            raise RuntimeError(ref.ref_last_error().decode())
        return h

    try:
        chain = [("conv0 k5s2", make("ConvLayer", B, 3, WIDTHS[0], 5, 2, 2, HEIGHT, WIDTH)), ("conv0 BatchNorm", make("BatchNorm", 1, B, WIDTHS[0], 72, 128)),
                 ("conv0 Swish", make("Swish", B * WIDTHS[0] * 72 * 128))]
        h, w = 72, 128
        for i in range(4):
            chain.append(("ResConv%d %d->%d" % (i, WIDTHS[i], WIDTHS[i + 1]), make("ResConvLayer", B, WIDTHS[i], WIDTHS[i + 1], h, w)))
            h, w = (h + 2 - 4) // 2 + 1, (w + 2 - 4) // 2 + 1
    except RuntimeError as e:
        return {"unavailable": str(e)}
    legacy = torch.cuda.default_stream()
    with torch.cuda.stream(legacy):
        xs = [torch.rand((B, 3, HEIGHT, WIDTH), device="cuda").half() for _ in range(3)]      # 3 x 56.6 MB > 126 MB L2
    torch.cuda.synchronize()

    def forward(i, events=None):
        data = ctypes.c_void_p(xs[i % 3].data_ptr())
        for j, (_, layer) in enumerate(chain):
            if events is not None:
                events[j].record(legacy)
            out = ref.ref_layer_forward(layer, data)
            if not out:
                raise RuntimeError(ref.ref_last_error().decode())
            data = ctypes.c_void_p(out)
        if events is not None:
            events[len(chain)].record(legacy)

    try:
        for i in range(3):
            forward(i)
        torch.cuda.synchronize()
        steps = 20
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(legacy)
        for i in range(steps):
            forward(i)
        e1.record(legacy)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(len(chain) + 1)] for _ in range(5)]
        for i in range(5):
            forward(i, ev[i])
        torch.cuda.synchronize()
        layers = [{"site": chain[j][0], "ms": float(np.mean([ev[i][j].elapsed_time(ev[i][j + 1]) for i in range(5)]))} for j in range(len(chain))]
    except RuntimeError as e:
        return {"unavailable": str(e)}
    finally:
        for _, layer in chain:
            ref.ref_layer_destroy(layer)
    tf = FLOP_PER_FRAME * B / (ms * 1e-3) / 1e12
    return {"value": B / (ms * 1e-3), "unit": "frames/s", "ms_per_step": ms, "frames": B, "tflops": tf, "frac": tf / env.peaks["tensor"],
            "what": "the reference's ConvLayer/BatchNorm/Swish/ResConvLayer classes (cuDNN, NCHW fp16, compute type HALF) on the encoder trunk, "
                    "46 library launches per step, planar fp16 input already on the device, no head", "layers": layers}


def fc_training_step(env):
    """One Forward / Backward / UpdateParameters step of FCLayer in training mode (FCLayer.cpp:48-70) on the
    reference's own CPU-runnable shape, 64 x 1024 -> 1024: this library's class (`aig_layer_*` hooks, kind
    "FCLayerTrain": tcgen05 GEMMs for the three products, AdamW on fp16 parameters) and, where it was built, the
    reference's class on cuBLAS beside it.  The 2 MB of weights live in L2 in both; the step is launch-bound."""
    import ctypes

    torch, lib, ctx = env.torch, env.pkg.lib(), env.ctx
    B, I, N, steps = 64, 1024, 1024, 200
    P = ctypes.c_void_p
    arr = (ctypes.c_int * 3)(B, I, N)
    gen = torch.Generator("cuda").manual_seed(5)
    xs = [torch.randn((B, I), device="cuda", generator=gen).half() for _ in range(4)]
    gs = [(0.1 * torch.randn((B, N), device="cuda", generator=gen)).half() for _ in range(4)]
    torch.cuda.synchronize()
    layer = P()
    env.ctx.check(lib.aig_layer_create(ctx.handle, b"FCLayerTrain", arr, 3, ctypes.byref(layer)))
    out, gx = P(), P()

    def ours(i):
        lib.aig_layer_forward(layer, P(xs[i % 4].data_ptr()), ctypes.byref(out))
        lib.aig_layer_backward(layer, P(gs[i % 4].data_ptr()), ctypes.byref(gx))
        env.ctx.check(lib.aig_layer_update(layer, 1e-3))

    res = env.timer.regions(ours, steps, 10)
    lib.aig_layer_destroy(layer)
    flop = 3 * 2.0 * B * I * N
    block = {"shape": "batch %d, %d -> %d" % (B, I, N), "value": 1.0 / (res["ms_per_step"] * 1e-3), "unit": "steps/s", "us_per_step": res["ms_per_step"] * 1e3,
             "repeats": res["repeats"], "steps": steps, "tflops": flop / (res["ms_per_step"] * 1e-3) / 1e12}
    path = os.path.join(ROOT, "oracle", "_ref", "libaig_reflayers.so")
    if not os.path.exists(path):
        block["reference_class"] = {"unavailable": "oracle/_ref/libaig_reflayers.so was not built (reference tree absent at build time)"}
        return block
    ref = ctypes.CDLL(path)
    ref.ref_layer_create.restype, ref.ref_layer_create.argtypes = P, [ctypes.c_char_p, ctypes.POINTER(ctypes.c_int), ctypes.c_int]
    ref.ref_layer_forward.restype, ref.ref_layer_forward.argtypes = P, [P, P]
    ref.ref_fc_backward.restype, ref.ref_fc_backward.argtypes = P, [P, P, P, P]
    ref.ref_layer_update.argtypes = [P, ctypes.c_float]
    ref.ref_layer_destroy.argtypes = [P]
    ref.ref_last_error.restype = ctypes.c_char_p
    torch.cuda.synchronize()
    rl = ref.ref_layer_create(b"FCLayerTrain", arr, 3) if ref.ref_init() == 0 else None
    if not rl:
        block["reference_class"] = {"unavailable": ref.ref_last_error().decode()}
        return block
    legacy = torch.cuda.default_stream()

    def theirs(i):
        ref.ref_layer_forward(rl, P(xs[i % 4].data_ptr()))
        ref.ref_fc_backward(rl, P(gs[i % 4].data_ptr()), None, None)
        ref.ref_layer_update(rl, 1e-3)

    for i in range(10):
        theirs(i)
    torch.cuda.synchronize()
    times = []
    for r in range(25):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(legacy)
        for i in range(steps):
            theirs(i)
        e1.record(legacy)
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) / steps)
    ref.ref_layer_destroy(rl)
    ms = float(np.median(times))
    block["reference_class"] = {"value": 1.0 / (ms * 1e-3), "unit": "steps/s", "us_per_step": ms * 1e3,
                                "what": "the reference's FCLayer (cublasGemmEx x3, cudnnAddTensor, BiasGradient, AdamWHalf x2) on the legacy default stream"}
    return block


def leg_agent_stream(env, full):
    """Profiler captures only: the batch-1 streaming agent on device-resident frames (encoder graph, bridge FC, the
    one-kernel sequence-head step); the timed form of this workload is the `latency` block."""
    torch, SY, R, args = env.torch, env.SY, env.R, env.args
    agent = R.Agent(env.ctx, 1, HEIGHT, WIDTH, widths=WIDTHS, d=512, layers=2, heads=8, n_out=N_OUT, n_sigmoid=N_SIG, window=64)
    agent.load_bytes(SY.serialize_agent_params(SY.make_agent_params(0, widths=WIDTHS), WIDTH, HEIGHT))
    frames = [torch.randint(0, 256, (1, HEIGHT, WIDTH, 4), dtype=torch.uint8, device="cuda") for _ in range(4)]
    res = env.timer.regions(lambda i: agent.step(frames[i % 4]), args.steps, args.warmup)
    agent.close()
    return {"value": 1.0 / (res["ms_per_step"] * 1e-3), "unit": "frames/s", **res, "l2": "batch 1: weights stay in L2 by design",
            "roofline": {"bound": "hbm", "kernel": "seq_step_kernel", "achieved": None}}


LEGS = {"agent_stream": leg_agent_stream, "cnn2d": leg_cnn2d, "conv3d": leg_conv3d, "seqhead": leg_seqhead, "agent_batched": leg_agent_batched}
GLOBAL_BATCH = {"agent_stream": 1, "cnn2d": None, "conv3d": 16, "seqhead": SEQ_B, "agent_batched": 128}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50, help="steps per timed region")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=256, help="frames per GPU per step (cnn2d)")
    ap.add_argument("--workload", default="cnn2d", choices=sorted(LEGS))
    ap.add_argument("--legs", default="all", help="other workloads reported under `workloads`: all, none or a comma list")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (used for short profiler captures)")
    ap.add_argument("--no-latency", action="store_true", help="skip the batch-1 streaming latency leg")
    ap.add_argument("--latency-frames", type=int, default=1000)
    ap.add_argument("--profile-iters", type=int, default=0,
                    help="profiler captures: run only this many untimed steps of --workload (no regions, no other legs) and exit")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    env = Env(args)
    wl = args.workload
    if args.profile_iters > 0:
        MIN_REGIONS_SAVED = globals()["MIN_REGIONS"], globals()["MIN_TOTAL_S"]
        globals()["MIN_REGIONS"], globals()["MIN_TOTAL_S"] = 1, 0.0      # one region of --profile-iters steps
        args.steps, args.warmup, args.no_e2e = args.profile_iters, 3, True
        env.profile = True
        LEGS[wl](env, False)
        globals()["MIN_REGIONS"], globals()["MIN_TOTAL_S"] = MIN_REGIONS_SAVED
        env.close()
        return
    head = LEGS[wl](env, True)
    extra = {}
    others = [w for w in LEGS if w != wl and w != "agent_stream"] if args.legs == "all" else ([] if args.legs == "none" else [w for w in args.legs.split(",") if w in LEGS and w != wl])
    for w in others:
        extra[w] = LEGS[w](env, env.world == 1)
    latency = streaming_latency(env, args.latency_frames) if env.rank == 0 and not args.no_latency else None

    if env.rank == 0:
        B = args.batch if wl == "cnn2d" else GLOBAL_BATCH[wl]
        line = {
            "metric": METRICS[wl][0], "value": head["value"], "unit": METRICS[wl][1], "n_gpus": env.world, "steps": head.get("steps", args.steps),
            "warmup": args.warmup, "ms_per_step": head["ms_per_step"], "ms_per_step_min": head["ms_per_step_min"],
            "ms_per_step_max": head["ms_per_step_max"], "repeats": head["repeats"], "timed_s": head["timed_s"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16 (fp32 accumulate)", "data": "synthetic",
            "config": {"workload": METRICS[wl][2] if wl != "cnn2d" else "cnn2d_encoder_144x256_b%d" % B, "units_per_gpu": B, "global_batch": env.world * B,
                       "sharding": "batch of independent units, no step-loop collective", "l2": head["l2"],
                       "timing": "median of `repeats` regions of `steps` steps each, CUDA events, barrier + synchronize around every region"},
            "e2e": head.get("e2e"), "gpu_launches": head.get("gpu_launches"), "latency": latency, "roofline": head["roofline"],
            "layers": head.get("layers"), "clocks": head["clocks"],
        }
        for w, r in extra.items():
            r["metric"] = METRICS[w][0]
            r["config"] = {"workload": METRICS[w][2]}
        line["workloads"] = extra
        if env.world == 1 and wl == "cnn2d" and args.legs == "all":
            line["reference_call_pattern"] = reference_call_pattern(env)
            line["fc_training_step"] = fc_training_step(env)
        if not args.no_cpu_baseline and env.world == 1:
            line["cpu_baseline"] = cpu_baseline_block(wl, 5 if wl == "cnn2d" else 3)
            for w in extra:
                extra[w]["cpu_baseline"] = cpu_baseline_block(w, 3)
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line), flush=True)
    env.close()


if __name__ == "__main__":
    main()

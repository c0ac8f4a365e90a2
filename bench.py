"""Benchmark of the Kokoro iSTFTNet generator path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--t T]

Metric: audio-seconds per second of the generator alone (24 kHz, f32), whole job over N GPUs. One step = one
generator forward of one utterance per GPU (default T = 2080 input frames = the 26 s paragraph case: 624000
samples, 1.279 TFLOP of conv work). N > 1 (torchrun, one rank per GPU): independent utterances, one per rank, no
data-path collective -> weak scaling; time = max over ranks.

`value`   : inputs already resident in HBM, one CUDA-graph replay per step, timed with CUDA events.
`e2e`     : the same metric through the host-buffer API (Generator.pipeline: SynthesisPipeline with two utterances in
            flight): every step's pinned host -> device copies of x / har / s, the replay, and the device -> host copy
            of the waveform are inside the timed region; the copies of one utterance overlap the compute of the next.
            `e2e_serial` is Generator.synthesize(), one utterance at a time (copy in, replay, copy out, synchronise).
`roofline`: the fused conv kernels (the dominant kernels), timed live per launch with CUDA events in an extra
            eager pass; achieved = algorithmic conv FLOPs (2 Co Ci K Lo per launch) / summed launch time, against
            the split-operand tensor roofline = measured dense bf16 peak / 3 (the kernel spends three f16 MMA products,
            which run at the bf16 rate, per f32 multiply-add: hi*hi, lo*hi, hi*lo).
`cpu_baseline` / --impl reference: the CPU oracle (torch f32, the basic-op graph the reference's eager PyTorch
            modules run) on all host cores, one utterance of the same T per step.
Extra keys on the same line (the other BASELINE configs): `cfg0` one AdaINResBlock1 per kernel size at C = 128,
L = 19200 / 19201; `cfg1` the 4 s sentence case (T = 320); `sweep` the conv / ConvTranspose kernel sweep of config 4;
`batch64` config 3 (64 utterances of 120..800 frames, sharded by utterance over the ranks: strong scaling);
`time_sharded` (N > 1) config 2 with one utterance cut along time over the ranks.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from lokinfer_b200 import synth  # noqa: E402

# DRAM traffic of one launch of the dominant conv shape (ncu capture, summary under profiles/); algorithmic bytes =
# x + residual read, out written = 3 * 4 * C * L.
TRAFFIC = {"bytes": 129688576 + 29296384, "algorithmic": 3 * 4 * 128 * 124801,
           "kernel": "convTcKernel, conv1d_snake_res, Ci = Co = 128, L = 124801, K = 11, dilation 5 (one launch)",
           "source": "profiles/conv_tc_c128_k11_L124801.md"}

BATCH_STREAMS = 3  # utterance graphs of one GPU are replayed round-robin on this many streams (config 3)
METRIC = "kokoro_generator_audio_seconds_per_second"
UNIT = "audio-s/s"
SAMPLE_RATE = 24000.0


def conv_flops_per_t() -> float:
    """Algorithmic conv FLOPs per unit of T (2 * MACs): ups + noise convs + resblocks + conv_post."""
    macs = 0
    macs += 512 * 256 * 20 * 1  # ups.0: 2 Ci Co K Lin / 2 per input column
    macs += 22 * 256 * 12 * 10  # noise_convs.0 over L0 = 10 T
    macs += 6 * 256 * 256 * 7 * 10  # noise_res.0
    macs += 6 * 256 * 256 * (3 + 7 + 11) * 10  # resblocks.0-2
    macs += 256 * 128 * 12 * 10  # ups.1 over Lin = 10 T
    macs += 22 * 128 * 1 * 60  # noise_convs.1 over L1 = 60 T (+1)
    macs += 6 * 128 * 128 * 11 * 60  # noise_res.1
    macs += 6 * 128 * 128 * (3 + 7 + 11) * 60  # resblocks.3-5
    macs += 128 * 22 * 7 * 60  # conv_post
    return 2.0 * macs


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons of one GPU every 50 ms while the timed regions run (the `value`
    loop and the `e2e` loops that follow it)."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        pw = [float(r[2]) for r in self.rows if len(r) > 2 and r[2].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for j, n in enumerate(names) if any(len(r) > 3 + j and r[3 + j].lower() == "active" for r in self.rows)]
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "sm_min_mhz": min(sm) if sm else None, "power_w_median": float(np.median(pw)) if pw else None,
                "reasons": reasons, "samples": len(sm), "covers": "the value loop and the e2e loops after it"}


def cpu_generator_rate(t_sample: int, reps: int, warmup: int, threads: int | None):
    """audio-s/s of the CPU oracle (f32, basic-op graph) for an utterance of t_sample frames."""
    from oracle import kokoro_oracle as O

    # all host cores of this process (torchrun exports OMP_NUM_THREADS=1, which would otherwise pin torch to one)
    torch.set_num_threads(threads or len(os.sched_getaffinity(0)))
    cores = torch.get_num_threads()
    sd = synth.generator_weights(0)
    sd_t = {k: O.T(v) for k, v in sd.items()}
    inp = synth.generator_inputs(t_sample, 1)
    a = [O.T(inp[k]) for k in ("x", "har", "s")]
    times = []
    for i in range(warmup + reps):
        t0 = time.perf_counter()
        O.generator(sd_t, *a, fused=False)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    sec = float(np.median(times))
    return 300.0 * t_sample / SAMPLE_RATE / sec, sec, cores


def _event_ms(fn, reps: int, warmup: int) -> float:
    """Average milliseconds of fn() over reps calls after warmup calls (CUDA events on the current stream)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps


def _graph_ms(fn, reps: int, warmup: int) -> float:
    """Average milliseconds of one fn() launch: `reps` calls captured back to back into one CUDA graph (after `warmup`
    eager calls), the graph replayed once untimed and then three times between two events. Keeps the host's launch
    path (Python, ctypes, tensor-map encoding: tens of microseconds per call) out of the number, which matters for
    kernels that run shorter than that."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            keep = [fn() for _ in range(reps)]
    graph.replay()
    ms = _event_ms(graph.replay, 3, 0) / reps
    del keep, graph
    return ms


def measure_cfg1(gen, dev, steps: int) -> dict:
    """BASELINE config 1: the 4 s sentence case (T = 320), one CUDA-graph replay per step, inputs resident."""
    t = 320
    inp = synth.generator_inputs(t, 7)
    bufs = gen.capture(t)
    for k in ("x", "har", "s"):
        bufs[k].copy_(torch.from_numpy(inp[k]))
    ms = _event_ms(lambda: bufs["graph"].replay(), max(steps, 10), 3)
    audio_s = synth.shapes(t)["S"] / SAMPLE_RATE
    return {"workload": "kokoro_generator_T320", "ms_per_step": ms, "value": audio_s / (ms * 1e-3), "unit": UNIT,
            "conv_gflop": conv_flops_per_t() * t / 1e9,
            "conv_tflops_step_bound": conv_flops_per_t() * t / (ms * 1e-3) / 1e12}


def measure_cfg0(dev, peak: float) -> dict:
    """BASELINE config 0: one AdaINResBlock1 (six fused convs + their AdaIN affines) per kernel size at C = 128,
    L = 19200 and L = 19201 (the generator's stage-1 length for T = 320), rows padded to 16 bytes as in the generator;
    FLOPs = 6 * 2 * C^2 * k * L per block. Each kernel size alone (`blocks`, `sum_L*`) and the three side by side on
    three streams (`concurrent_L*`)."""
    from lokinfer_b200 import Generator, ops

    out = {"workload": "adain_resblock1 C=128 k in (3, 7, 11), dilations (1, 3, 5)", "blocks": []}
    for l in (19200, 19201):
        tot_ms, tot_fl = 0.0, 0.0
        for k in (3, 7, 11):
            sd, x, s = synth.resblock_case(128, l, k, 300 + k)
            g = Generator(sd, dev)
            with ops.padded_rows():
                dx = ops.to_cuda(x, dev, rows=True)
                gb = g.style(ops.to_cuda(s, dev))
                for _ in range(2):  # warm-up outside the capture
                    g.adain_resblock1_fused(dx, gb, "rb", k)
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()  # one replay per block: the 13 launches are not host-bound
                with torch.cuda.graph(graph):
                    keep = g.adain_resblock1_fused(dx, gb, "rb", k)
                ms = _event_ms(graph.replay, 20, 3)
                del keep
            fl = 6 * 2.0 * 128 * 128 * k * l
            tf = fl / (ms * 1e-3) / 1e12
            out["blocks"].append({"L": l, "k": k, "ms": ms, "tflops": tf, "frac": tf / peak})
            tot_ms += ms
            tot_fl += fl
        out[f"sum_L{l}"] = {"ms": tot_ms, "tflops": tot_fl / (tot_ms * 1e-3) / 1e12,
                            "frac": tot_fl / (tot_ms * 1e-3) / 1e12 / peak}
        # The three branches of the config side by side, as the generator runs the resblocks of a stage: one captured
        # graph, each kernel size on its own stream (75-76 tiles per conv leave half of the 148 SMs to the others).
        gens, xs, gbs = [], [], []
        with ops.padded_rows():
            for k in (3, 7, 11):
                sd, x, s = synth.resblock_case(128, l, k, 300 + k)
                g = Generator(sd, dev)
                gens.append(g), xs.append(ops.to_cuda(x, dev, rows=True)), gbs.append(g.style(ops.to_cuda(s, dev)))
            lanes = [torch.cuda.Stream(device=dev) for _ in range(3)]

            def three():
                cur = torch.cuda.current_stream(dev)
                keep = []
                for ln, g, x, gb, k in zip(lanes, gens, xs, gbs, (3, 7, 11)):
                    ln.wait_stream(cur)
                    with torch.cuda.stream(ln):
                        keep.append(g.adain_resblock1_fused(x, gb, "rb", k))
                for ln in lanes:
                    cur.wait_stream(ln)
                return keep

            for _ in range(2):
                three()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                keep = three()
            ms = _event_ms(graph.replay, 20, 3)
            del keep
        out[f"concurrent_L{l}"] = {"ms": ms, "tflops": tot_fl / (ms * 1e-3) / 1e12,
                                   "frac": tot_fl / (ms * 1e-3) / 1e12 / peak}
    return out


def measure_sweep(dev, peak: float) -> dict:
    """BASELINE config 4: fused conv1d_snake_res at Cin = Cout in {128, 256, 512}, K in {3, 7, 11}, dilation in
    {1, 3, 5}, L in {320, 3200, 19200, 124800} (rows 16-byte aligned: every L is a multiple of 4), and the two
    ConvTranspose upsamplers at Lin in {320, 2080} (x10) / {3200, 20800} (x6). Inputs are seeded normal draws made on
    the device; per point 5 launches captured into one CUDA graph after 2 warm-ups, the graph replayed three times
    between two events (the host's launch path is longer than the kernels of the short rows). Rows: [C, L, K,
    dilation, ms, TFLOP/s, fraction of the split-operand tensor roofline]."""
    from lokinfer_b200 import ops

    g = torch.Generator(device=dev)
    g.manual_seed(4)
    rows = []
    for c in (128, 256, 512):
        affine = torch.stack([torch.zeros(c, device=dev), torch.ones(c, device=dev), torch.zeros(c, device=dev)])
        alpha = torch.rand(c, device=dev, generator=g) + 0.5
        bias = torch.randn(c, device=dev, generator=g) * 0.01
        for k in (3, 7, 11):
            w = torch.randn(c, c, k, device=dev, generator=g) / math.sqrt(c * k)
            st = ops.conv1d_prepare_f32_cuda(w)
            for l in (320, 3200, 19200, 124800):
                x = torch.randn(c, l, device=dev, generator=g)
                res = torch.randn(c, l, device=dev, generator=g)
                for d in (1, 3, 5):
                    pad = d * (k - 1) // 2
                    ms = _graph_ms(lambda: ops.conv1d_snake_f32_cuda(x, w, bias, affine, alpha, residual=res,
                                                                     padding=pad, dilation=d, state=st), 5, 2)
                    tf = 2.0 * c * c * k * l / (ms * 1e-3) / 1e12
                    rows.append([c, l, k, d, round(ms, 5), round(tf, 2), round(tf / peak, 4)])
                del x, res
    convt = []
    for ci, co, k, s, p, pl, lins in ((512, 256, 20, 10, 5, 0, (320, 2080)), (256, 128, 12, 6, 3, 1, (3200, 20800))):
        w = torch.randn(ci, co, k, device=dev, generator=g) * math.sqrt(s / (ci * k))
        bias = torch.randn(co, device=dev, generator=g) * 0.1
        wp = ops.convt_poly_weights_cuda(w, s, p)
        st = ops.conv_transpose1d_prepare_f32_cuda(w, s, p)
        for lin in lins:
            x = torch.randn(ci, lin, device=dev, generator=g)
            with ops.padded_rows():
                res = ops.to_cuda(torch.randn(co, lin * s + pl, device=dev, generator=g), dev, rows=True)
                ms = _graph_ms(lambda: ops.conv_transpose1d_poly_f32_cuda(x, wp, bias, res, stride=s, padding=p,
                                                                          taps=k // s, slope=0.1, pad_left=pl,
                                                                          state=st), 5, 2)
            tf = 2.0 * ci * co * k * lin / (ms * 1e-3) / 1e12
            convt.append([ci, co, k, s, lin, round(ms, 5), round(tf, 2), round(tf / peak, 4)])
    status = ops.conv_tc_status()
    by_l = {}
    for c, l, k, d, ms, tf, fr in rows:
        by_l.setdefault(l, []).append(fr)
    return {"conv1d_snake_res": {"columns": ["C", "L", "K", "dilation", "ms", "tflops", "frac"], "rows": rows,
                                 "mean_frac_by_L": {str(l): round(float(np.mean(v)), 4) for l, v in by_l.items()}},
            "conv_transpose1d_poly": {"columns": ["Ci", "Co", "K", "stride", "Lin", "ms", "tflops", "frac"],
                                      "rows": convt},
            "peak_tflops": peak, "tc_status": status}


def measure_batch64(gen, dev, rank: int, world: int, steps: int, warmup: int) -> dict | None:
    """BASELINE config 3: 64 independent utterances with T ~ U{120..800} (seeded), sharded by utterance across the
    ranks (longest-processing-time-first on T, lokinfer_b200/sharding.py), no inter-GPU communication. One step =
    every utterance once (each rank replays the CUDA graphs of its own utterances back to back); strong scaling:
    the total work is fixed as N grows. Aggregate audio-seconds/sec = all audio seconds / max-over-ranks time.
    Returns the record on rank 0, None elsewhere."""
    import torch.distributed as dist

    from lokinfer_b200 import sharding

    lengths = np.random.default_rng(64).integers(120, 801, 64).tolist()
    plan = sharding.assign(lengths, world)
    graphs = []
    for i in plan[rank]:  # one graph per distinct length; inputs are resident in HBM
        t = lengths[i]
        inp = synth.generator_inputs(t, 100 + i)
        bufs = gen.capture(t)
        for k in ("x", "har", "s"):
            bufs[k].copy_(torch.from_numpy(inp[k]))
        graphs.append(bufs["graph"])
    torch.cuda.synchronize()
    # Utterances are independent (own static buffers, own arena): their graphs are replayed round-robin on a few
    # streams, so that the convs of a short utterance (a 1.5 s utterance has 10-30 tiles per conv for 148 SMs) share
    # the GPU with those of another one instead of leaving most SMs idle.
    main = torch.cuda.current_stream(dev)
    lanes = [torch.cuda.Stream(device=dev) for _ in range(BATCH_STREAMS)]

    def step():
        for ln in lanes:
            ln.wait_stream(main)
        for i, g in enumerate(graphs):
            with torch.cuda.stream(lanes[i % BATCH_STREAMS]):
                g.replay()
        for ln in lanes:
            main.wait_stream(ln)

    for _ in range(max(warmup, 3)):
        step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        step()
    b.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if rank != 0:
        return None
    total_audio = sharding.audio_seconds(lengths)
    return {"workload": "kokoro_generator_batch64", "value": total_audio * steps / (float(ms.item()) * 1e-3),
            "unit": UNIT, "ms_per_step": float(ms.item()) / steps, "scaling": "strong", "utterances": 64,
            "T_range": [120, 800], "audio_seconds_per_step": total_audio,
            "sharding": "by utterance, longest first, no communication",
            "streams_per_gpu": BATCH_STREAMS, "rank_loads_T": sharding.loads(lengths, plan)}


def measure_time_sharded(gen, dev, rank: int, world: int, t: int, steps: int, single_ms: float) -> dict | None:
    """BASELINE config 2 on N GPUs: ONE utterance of t frames cut along time over the ranks (lokinfer_b200/timeshard.py:
    halo columns by plain peer stores + release flags, chunk statistics gathered into every rank's row, bounded
    waits), one captured graph replay per step on every rank, time = max over ranks. Strong scaling of a single
    utterance: about 53 exchanges per forward, each one kernel (push, peer round trip, wait), so the step is bound by
    exchange latency; the record says how far. Returns the record on rank 0."""
    import torch.distributed as dist

    from lokinfer_b200 import ops, timeshard as ts

    inp = synth.generator_inputs(t, 1)  # the same utterance on every rank
    x, har, s = [ops.to_cuda(inp[k], dev) for k in ("x", "har", "s")]
    single = gen.forward(x, har, s)
    fabric = ts.IpcFabric(ts.TimeShardedGenerator.arena_bytes(t, world), dev)
    tsg = ts.TimeShardedGenerator(gen, t, rank, world, fabric)
    lo, hi = tsg.part.bs[rank], tsg.part.bs[rank + 1]
    dist.barrier()
    graph = tsg.capture(x, har, s)
    for _ in range(3):
        dist.barrier()
        graph.replay()
    torch.cuda.synchronize()
    dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        graph.replay()
    b.record()
    torch.cuda.synchronize()
    dist.barrier()
    vals = torch.tensor([a.elapsed_time(b), (tsg.audio - single[lo:hi]).abs().max().item(), float(tsg.status())],
                        dtype=torch.float64, device=dev)
    dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    if rank != 0:
        return None
    ms = float(vals[0].item()) / steps
    audio_s = synth.shapes(t)["S"] / SAMPLE_RATE
    return {"workload": f"kokoro_generator_T{t} time-sharded over {world} GPUs", "ms_per_step": ms,
            "value": audio_s / (ms * 1e-3), "unit": UNIT, "scaling": "strong",
            "single_gpu_ms_per_step": single_ms, "speedup_vs_single_gpu": single_ms / ms,
            "frames_per_rank": [y - x_ for x_, y in zip(tsg.part.bx, tsg.part.bx[1:])],
            "exchanges_per_forward": 53, "us_per_exchange_over_ideal": (ms - single_ms / world) * 1e3 / 53,
            "max_abs_diff_vs_single_gpu": float(vals[1].item()), "wait_status": int(vals[2].item()),
            "limiter": "exchange latency: every conv output is followed by one exchange kernel (peer stores of the "
                       "boundary columns and the statistics slice, release flags, then a bounded wait for the "
                       "neighbours' flags) before the next conv may start; NCCL is not on this path"}


def init_nccl(dev):
    """Process group over NCCL (rank / world size / master address from the torchrun environment). NCCL prints its
    version banner on stdout when the communicator is created: stdout is pointed at stderr until the first
    collective is done, so that rank 0's stdout carries exactly one JSON line."""
    import torch.distributed as dist

    sys.stdout.flush()
    saved = os.dup(1)
    os.dup2(2, 1)
    try:
        dist.init_process_group("nccl", device_id=dev)
        dist.barrier()
        torch.cuda.synchronize()
    finally:
        sys.stdout.flush()
        os.dup2(saved, 1)
        os.close(saved)


def run_reference(args, rank: int):
    if rank != 0:
        return
    t_sample = args.t
    rate, sec, cores = cpu_generator_rate(t_sample, args.steps, args.warmup, None)
    sample = (f"CPU oracle (torch f32, basic-op graph = what the reference's eager PyTorch modules run), one "
              f"utterance of T={t_sample} ({300 * t_sample / SAMPLE_RATE:.1f} s audio) per step, median of {args.steps}")
    line = {
        "impl": "reference", "metric": METRIC, "value": rate, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"kokoro_generator_T{args.t}", "sample_T": t_sample},
        "cpu_baseline": {"value": rate, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": rate, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference's NEON/Accelerate kernels do not build on this host; the oracle port stands in",
    }
    print(json.dumps(line), flush=True)


def run_ours(args, rank: int, local_rank: int, world: int):
    import torch.distributed as dist

    from lokinfer_b200 import Generator, ops

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    dev = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(dev)
    if world > 1:
        init_nccl(dev)
    t = args.t
    sh = synth.shapes(t)
    audio_s = sh["S"] / SAMPLE_RATE
    gen = Generator(synth.generator_weights(0), dev)
    inp = synth.generator_inputs(t, 1 + rank)  # each rank synthesises its own utterance
    host = [torch.from_numpy(inp[k]).pin_memory() for k in ("x", "har", "s")]
    audio_host = torch.empty(sh["S"], dtype=torch.float32).pin_memory()

    # count launches of one forward and capture the graph
    with ops.Profile(time_kernels=False) as cnt:
        gen.forward(*[h.to(dev) for h in host])
    launches_per_step = cnt.count
    bufs = gen.capture(t)
    for k, h in zip(("x", "har", "s"), host):
        bufs[k].copy_(h)
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(step_fn, steps, warmup):
        for _ in range(warmup):
            step_fn()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            step_fn()
        b.record()
        barrier()
        ms = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    ms_dev = timed(lambda: bufs["graph"].replay(), args.steps, args.warmup)
    ms_e2e_serial = timed(lambda: gen.synthesize(host[0], host[1], host[2], audio_host), args.steps,
                          max(1, args.warmup // 2))
    # throughput form: two utterances in flight, each step still copies its inputs in and its waveform out
    pipe = gen.pipeline(t, depth=2)
    outs = [audio_host, torch.empty_like(audio_host).pin_memory()]
    submitted = [0]

    def pipe_steps(n):
        first = submitted[0]
        for i in range(first, first + n):
            pipe.submit(host[0], host[1], host[2], outs[i % 2])
        submitted[0] += n
        for i in range(max(first, first + n - 2), first + n):
            pipe.wait(i)

    pipe_steps(max(2, args.warmup // 2))
    barrier()
    ea, eb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ea.record()
    pipe_steps(args.steps)  # returns after the last waveform has reached the host
    eb.record()
    barrier()
    ms_pipe = torch.tensor([ea.elapsed_time(eb)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ms_pipe, op=dist.ReduceOp.MAX)
    ms_e2e = float(ms_pipe.item())
    pipe_ok = bool(np.array_equal(outs[0].numpy(), outs[1].numpy()))  # same inputs -> same waveform in both slots
    clocks = sampler.stop() if sampler else None

    # input option B: the `har` input computed on the device from the F0 curve (harmonic source with in-kernel noise +
    # STFT, the step before the generator in the reference graph); h2d carries x, f0 and s only
    f0_host = torch.from_numpy(synth.f0_curve(t, 1 + rank)).pin_memory()
    ms_e2e_f0 = timed(lambda: gen.synthesize_f0(host[0], f0_host, 1234 + rank, host[2], audio_host), args.steps,
                      max(1, args.warmup // 2))
    value = world * audio_s * args.steps / (ms_dev * 1e-3)
    e2e = world * audio_s * args.steps / (ms_e2e * 1e-3)
    h2d = sum(h.numel() * 4 for h in host)
    d2h = audio_host.numel() * 4

    # config 3 on every rank (strong scaling), before the single-rank extras
    batch64 = None if args.no_extras else measure_batch64(gen, dev, rank, world, 3, 3)
    time_sharded = None
    if world > 1 and not args.no_extras:
        time_sharded = measure_time_sharded(gen, dev, rank, world, t, args.steps, ms_dev / args.steps)
    roofline, cpu_base, kernels = None, None, None
    if rank == 0:
        # per-launch timing of the fused conv kernels (eager pass, CUDA event pair around every launch)
        # one stream; every launch is followed by a small captured graph of 4 repeats of itself, replayed once untimed
        # and once inside its event pair: no host launch path inside the timed region, as in the captured forward
        with ops.Profile(repeat=4, graph=True) as prof:
            gen.forward(bufs["x"], bufs["har"], bufs["s"], concurrent=False)
        rows = prof.rows()
        agg = {}
        conv_ms, conv_flops = 0.0, 0.0
        for name, ints, ms in rows:
            a = agg.setdefault(name, [0, 0.0])
            a[0] += 1
            a[1] += ms
            # the fused convs of the resblocks and conv_post; the two noise convs (conv1d_affine over the polyphase
            # view of har, 0.2 % of the FLOPs, channels padded to 16) stay out, as they did as CUDA-core launches
            if name.startswith("conv1d_snake") or name.startswith("conv1d_leaky"):
                ci, l, co, _, k = ints[0], ints[1], ints[2], ints[3], ints[4]
                if name == "conv1d_leaky_mean3_f32_cuda":
                    co, k = ints[6], ints[8]
                conv_ms += ms
                conv_flops += 2.0 * co * ci * k * l  # "same" padding: Lo = L
        pk = peaks()
        peak = pk["bf16_tflops"] / 3.0  # three f16-rate MMA products per f32 product
        achieved = conv_flops / (conv_ms * 1e-3) / 1e12
        total_ms = sum(v[1] for v in agg.values())
        kernels = {n: {"launches": v[0], "ms": round(v[1], 4), "share": round(v[1] / total_ms, 4)}
                   for n, v in sorted(agg.items(), key=lambda kv: -kv[1][1])}
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                    # DRAM bytes (read + written) of ONE launch of ONE shape, from its ncu capture: not an aggregate
                    "traffic": TRAFFIC["bytes"], "traffic_kernel": TRAFFIC["kernel"],
                    "traffic_source": TRAFFIC["source"], "traffic_algorithmic": TRAFFIC["algorithmic"],
                    "kernel": "conv1d_{snake,leaky}[_res]_f32_cuda (all fused conv launches of one "
                    "forward)", "peak_source": f"{pk['source']}: bf16 {pk['bf16_tflops']} TF/s / 3 (f16 hi/lo split: 3 MMA products per f32 "
                    "product)",
                    "conv_ms_per_step": conv_ms, "conv_flops_per_step": conv_flops,
                    "note": "conv_ms_per_step sums the launches timed one at a time on one stream (each alone on the "
                            "GPU, 4 graph-captured repeats per launch inside its event pair); ms_per_step is the "
                            "captured forward, where independent branches run on side streams and the tail of one "
                            "persistent conv overlaps the start of another, so it can be smaller than conv_ms_per_step",
                    # the same FLOPs over the whole captured step (all kernels of the forward, not only the convs): a
                    # lower bound of what the convs reach inside the step
                    "achieved_step_bound": conv_flops / (ms_dev / args.steps * 1e-3) / 1e12,
                    "frac_step_bound": conv_flops / (ms_dev / args.steps * 1e-3) / 1e12 / peak}
        if world == 1 and not args.no_cpu:
            t_sample = t
            rate, sec, cores = cpu_generator_rate(t_sample, 3, 1, None)
            cpu_base = {"value": rate, "unit": UNIT, "cores": cores, "kind": "port",
                        "sample": f"CPU oracle (torch f32, basic-op graph), one utterance of T={t_sample} "
                                  f"({300 * t_sample / SAMPLE_RATE:.1f} s audio), median of 3 after 1 warm-up, "
                                  f"{sec * 1e3:.0f} ms each"}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_dev / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"kokoro_generator_T{t}", "audio_seconds_per_utterance": audio_s,
                       "utterances_per_step": world, "L0": sh["L0"], "L1": sh["L1"], "samples": sh["S"],
                       "sharding": "one utterance per GPU, no communication" if world > 1 else "single GPU",
                       "l2": "working set per step is larger than the 126 MB L2",
                       "arena_bytes": bufs.get("arena_bytes"), "unplanned_bytes": bufs.get("unplanned_bytes"),
                       "conv_gflop_per_utterance": conv_flops_per_t() * t / 1e9},
            "e2e": {"value": e2e, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": ms_e2e / args.steps, "api": "Generator.pipeline(t, depth=2): submit / wait",
                    "in_flight": 2, "slots_agree": pipe_ok},
            "e2e_serial": {"value": world * audio_s * args.steps / (ms_e2e_serial * 1e-3), "unit": UNIT,
                           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                           "ms_per_step": ms_e2e_serial / args.steps, "api": "Generator.synthesize"},
            "e2e_from_f0": {"value": world * audio_s * args.steps / (ms_e2e_f0 * 1e-3), "unit": UNIT,
                            "h2d_bytes_per_step": host[0].numel() * 4 + f0_host.numel() * 4 + host[2].numel() * 4,
                            "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e_f0 / args.steps,
                            "note": "har = STFT(harmonic_source_rng(F0, seed)) computed on the device inside the "
                                    "timed region (Generator.synthesize_f0)"},
            "gpu_launches": launches_per_step * args.steps,
            "roofline": roofline, "clocks": clocks, "kernels": kernels,
        }
        if cpu_base:
            line["cpu_baseline"] = cpu_base
        if not args.no_extras:
            line["batch64"] = batch64
            if time_sharded is not None:
                line["time_sharded"] = time_sharded
            line["cfg1"] = measure_cfg1(gen, dev, args.steps)
            line["cfg0"] = measure_cfg0(dev, peak)
            line["sweep"] = measure_sweep(dev, peak)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_batch(args, rank: int, local_rank: int, world: int):
    """Config 3 alone (see measure_batch64): prints one JSON line with the batch as the workload."""
    import torch.distributed as dist

    from lokinfer_b200 import Generator

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    dev = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(dev)
    if world > 1:
        init_nccl(dev)
    gen = Generator(synth.generator_weights(0), dev)
    rec = measure_batch64(gen, dev, rank, world, args.steps, args.warmup)
    if rank == 0:
        line = {
            "metric": METRIC, "value": rec["value"], "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": rec["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "kokoro_generator_batch64", "utterances": 64, "T_range": [120, 800],
                       "audio_seconds_per_step": rec["audio_seconds_per_step"], "sharding": rec["sharding"],
                       "rank_loads_T": rec["rank_loads_T"]},
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_sweep(args):
    """Conv kernel sweep (f32, batch 1): one fused conv1d_snake_res launch per step at each point, timed with CUDA
    events; prints one JSON line per point with achieved TFLOP/s (2 Co Ci K L / time) and the fraction of the
    split-operand tensor roofline (measured bf16 peak / 3). --point Ci,Co,L,K,d runs a single point (used for ncu captures)."""
    from lokinfer_b200 import ops

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    dev = torch.device("cuda:0")
    pk = peaks()
    peak = pk["bf16_tflops"] / 3.0
    if args.point:
        points = [tuple(int(v) for v in args.point.split(","))]
    else:
        points = [(c, c, l, k, d) for c in (128, 256, 512) for k in (3, 7, 11) for d in (1, 3, 5)
                  for l in (320, 3200, 19200, 124800)]
    for ci, co, l, k, d in points:
        x, w, b, affine, alpha, res = synth.conv_case(ci, co, l, k, 7, big=False)
        dw, db, daf, dal = [ops.to_cuda(v, dev) for v in (w, b, affine, alpha)]
        padded = not args.plain_rows  # rows padded to 16 bytes, as the generator keeps its intermediates
        with ops.padded_rows(padded):
            dx, dres = ops.to_cuda(x, dev, rows=True), ops.to_cuda(res, dev, rows=True)
        st = ops.conv1d_prepare_f32_cuda(dw)
        pad = d * (k - 1) // 2

        def step():
            with ops.padded_rows(padded):
                return ops.conv1d_snake_f32_cuda(dx, dw, db, daf, dal, residual=dres, padding=pad, dilation=d,
                                                 state=st)

        for _ in range(args.warmup):
            step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        flops = 2.0 * co * ci * k * l
        tf = flops / (ms * 1e-3) / 1e12
        print(json.dumps({"sweep": "conv1d_snake_res_f32_cuda", "ci": ci, "co": co, "L": l, "K": k, "dilation": d,
                          "ms": ms, "tflops": tf, "frac_split_roofline": tf / peak, "peak_tflops": peak,
                          "peak_source": pk["source"], "path": "tcgen05" if st is not None else "cuda-core",
                          "rows": "padded to 16 bytes (TMA route)" if padded else "contiguous (4-byte route when L is odd)",
                          "tc_status": ops.conv_tc_status()}), flush=True)


def run_sweep_hbm(args):
    """The HBM-bound kernels of the path at the shapes of the 26 s case, one JSON line each: channel_stats over
    [128, 124801] and [256, 20800] (reads 4 C L bytes), adain_affine (reads the chunk statistics), add3_scale
    (3 reads + 1 write), istft_logits over [22, 124801] (reads 4 * 22 * L bytes, writes 4 * 5 (L - 1)). Achieved GB/s =
    algorithmic bytes / event time, against the measured HBM copy bandwidth. Rows are padded to 16 bytes, as the
    generator keeps them."""
    from lokinfer_b200 import ops

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    dev = torch.device("cuda:0")
    pk = peaks()
    g = torch.Generator(device=dev)
    g.manual_seed(9)
    flush = torch.empty(64 * 1024 * 1024, dtype=torch.float32, device=dev)  # 256 MB: larger than the L2

    def timed(fn):
        ms = []
        for i in range(args.warmup + args.steps):
            flush.zero_()  # evicts the operands from the L2 between launches
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            if i >= args.warmup:
                ms.append(a.elapsed_time(b))
        return float(np.median(ms))

    with ops.padded_rows():
        for c, l in ((128, 124801), (256, 20800)):
            x = ops.to_cuda(torch.randn(c, l, device=dev, generator=g), dev, rows=True)
            ms = timed(lambda: ops.channel_stats_f32_cuda(x))
            st = ops.channel_stats_f32_cuda(x)
            gbs = 4.0 * c * l / (ms * 1e-3) / 1e9
            print(json.dumps({"sweep": "channel_stats_f32_cuda", "C": c, "L": l, "ms": ms, "gbs": gbs,
                              "frac_hbm": gbs / pk["hbm_gbs"], "peak_gbs": pk["hbm_gbs"], "l2": "flushed"}), flush=True)
            gb = torch.randn(2 * c, device=dev, generator=g)
            ms = timed(lambda: ops.adain_affine_f32_cuda(st, gb, length=l))
            gbs = 4.0 * st.numel() / (ms * 1e-3) / 1e9
            print(json.dumps({"sweep": "adain_affine_f32_cuda", "C": c, "L": l, "ms": ms, "gbs": gbs,
                              "frac_hbm": gbs / pk["hbm_gbs"], "note": "latency-bound: C blocks, one row of chunk "
                              "statistics each"}), flush=True)
            y, z = (ops.to_cuda(torch.randn(c, l, device=dev, generator=g), dev, rows=True) for _ in range(2))
            ms = timed(lambda: ops.add3_scale_f32_cuda(x, y, z, 1.0 / 3.0))
            gbs = 16.0 * c * x.stride(0) / (ms * 1e-3) / 1e9
            print(json.dumps({"sweep": "add3_scale_f32_cuda", "C": c, "L": l, "ms": ms, "gbs": gbs,
                              "frac_hbm": gbs / pk["hbm_gbs"]}), flush=True)
        l = 124801
        post = ops.to_cuda(torch.randn(22, l, device=dev, generator=g) * 0.5, dev, rows=True)
        ms = timed(lambda: ops.istft_logits_f32_cuda(post))
        gbs = (4.0 * 22 * l + 4.0 * 5 * (l - 1)) / (ms * 1e-3) / 1e9
        print(json.dumps({"sweep": "istft_logits_f32_cuda", "L": l, "ms": ms, "gbs": gbs,
                          "frac_hbm": gbs / pk["hbm_gbs"],
                          "note": "13.5 MB per launch: too small to fill the HBM pipes (launch + one wave of blocks)"}),
              flush=True)


def run_sweep_convt(args):
    """ConvTranspose sweep: the generator's two upsamplers (512 -> 256, k 20, s 10, p 5) and (256 -> 128, k 12, s 6,
    p 3) at Lin = 320 and 2080, one conv_transpose1d_poly launch (leaky prologue, residual, pad_left as in the
    generator) per step on the tensor-core path; one JSON line per point, FLOPs = 2 Ci Co K Lin."""
    from lokinfer_b200 import ops

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    dev = torch.device("cuda:0")
    pk = peaks()
    peak = pk["bf16_tflops"] / 3.0
    r = np.random.default_rng(11)
    for ci, co, k, s, p, pl in ((512, 256, 20, 10, 5, 0), (256, 128, 12, 6, 3, 1)):
        for lin in (320, 2080) if ci == 512 else (3200, 20800):
            x = r.standard_normal((ci, lin)).astype(np.float32)
            w = (r.standard_normal((ci, co, k)) * math.sqrt(s / (ci * k))).astype(np.float32)
            bias = (r.standard_normal(co) * 0.1).astype(np.float32)
            res = r.standard_normal((co, lin * s + pl)).astype(np.float32)
            dx, dw, db, dres = [ops.to_cuda(v, dev) for v in (x, w, bias, res)]
            wp = ops.convt_poly_weights_cuda(dw, s, p)
            st = ops.conv_transpose1d_prepare_f32_cuda(dw, s, p)

            def step():
                return ops.conv_transpose1d_poly_f32_cuda(dx, wp, db, dres, stride=s, padding=p, taps=k // s, slope=0.1,
                                                          pad_left=pl, state=st)

            for _ in range(args.warmup):
                step()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.steps):
                step()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / args.steps
            tf = 2.0 * ci * co * k * lin / (ms * 1e-3) / 1e12
            print(json.dumps({"sweep": "conv_transpose1d_poly_f32_cuda", "ci": ci, "co": co, "K": k, "stride": s,
                              "Lin": lin, "ms": ms, "tflops": tf, "frac_split_roofline": tf / peak,
                              "peak_tflops": peak, "peak_source": pk["source"],
                              "path": "tcgen05" if st is not None else "cuda-core",
                              "tc_status": ops.conv_tc_status()}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--t", type=int, default=2080, help="generator input frames per utterance (2080 = 26 s, 320 = 4 s)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the other BASELINE configs (cfg0, cfg1, sweep, batch64) carried as extra keys")
    ap.add_argument("--sweep", default=None, choices=["conv", "convt", "hbm"],
                    help="run the conv / ConvTranspose kernel sweep instead of the generator")
    ap.add_argument("--workload", default="single", choices=["single", "batch64"],
                    help="single: one utterance of --t frames per GPU (default, weak scaling); batch64: 64 utterances of "
                         "120..800 frames sharded across the GPUs (strong scaling)")
    ap.add_argument("--point", default=None, help="single sweep point Ci,Co,L,K,dilation")
    ap.add_argument("--plain-rows", action="store_true",
                    help="conv sweep: contiguous rows instead of rows padded to 16 bytes")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.sweep == "convt":
        if rank == 0:
            run_sweep_convt(args)
        return
    if args.sweep == "hbm":
        if rank == 0:
            run_sweep_hbm(args)
        return
    if args.sweep:
        if rank == 0:
            run_sweep(args)
        return
    if args.workload == "batch64":
        run_batch(args, rank, local_rank, world)
        return
    if world != args.gpus and world == 1 and args.gpus > 1:
        print(f"bench.py: --gpus {args.gpus} needs torchrun with {args.gpus} ranks; running 1 rank", file=sys.stderr)
    run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()

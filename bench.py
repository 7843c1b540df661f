#!/usr/bin/env python
"""Benchmark of the convolution-layer hot path: the 13 conv layers of VGG-16 (3x3, stride 1, pad 1).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--mode fp32|3xtf32|tf32] [--batch B]
    python bench.py --impl reference ...      # the reference's own CPU algorithm on the host cores

A step is one Forward() of every layer of the stack on this rank's own images (each layer has its
own seeded synthetic input and weights: the reference benchmarks single layers, it does not chain
them).  With N GPUs every rank runs the same stack on different images, no collective in the data
path (weak scaling).  The metric is direct-convolution-equivalent GFLOP/s,
sum(2*N*K*C*9*OH*OW) / time, whole job.  One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# C, K, H(=W) of the 13 VGG-16 conv layers at 224x224 input
VGG16 = [(3, 64, 224), (64, 64, 224), (64, 128, 112), (128, 128, 112), (128, 256, 56), (256, 256, 56), (256, 256, 56),
         (256, 512, 28), (512, 512, 28), (512, 512, 28), (512, 512, 14), (512, 512, 14), (512, 512, 14)]

HBM_FALLBACK_GBS = 6650.0

# Arithmetic peaks the per-layer roofline divides by, in TFLOP/s.  TF32 and FP32 are not in MEASURED_PEAKS.json;
# they were measured on this pool's B200 the same way as its bf16 figure (torch.matmul 8192^3, best of 10, CUDA
# events): TF32 759.9, FP32 (FFMA) 63.7.  3xTF32 issues three TF32 MMAs per product, so its peak is a third.
TF32_TFLOPS = 759.9
FP32_TFLOPS = 63.7
MODE_PEAK_TFLOPS = {"tf32": TF32_TFLOPS, "3xtf32": TF32_TFLOPS / 3.0, "fp32": FP32_TFLOPS}

# DRAM bytes (read + write) per TensorGEMM launch, averaged over the 13 launches of one step of the default
# workload (VGG-16, batch 1), from one ncu capture of `dram__bytes_read.sum + dram__bytes_write.sum`
# (profiles/tensorgemm_dram_traffic_vgg16_batch1.md).  None for any other workload.
NCU_GEMM_TRAFFIC_BYTES = {"fp32": 43.20e6, "tf32": 44.01e6, "3xtf32": 44.01e6}


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 1590.0)), "measured"
    return HBM_FALLBACK_GBS, 1590.0, "fallback"


def layer_flops(n, c, k, h):
    return 2.0 * n * k * c * 9 * h * h


def wino_geometry(n, c, k, h):
    t = n * ((h + 5) // 6) ** 2
    return t, (t + 7) // 8 * 8, (c + 7) // 8 * 8


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.lines, self.marks = gpu_index, None, [], []
        self.topped_up = False

    def mark(self):
        """Remembers how many samples had arrived: the first two marks bracket the device-timed region."""
        self.marks.append(len(self.lines))

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def wait_first(self, timeout: float = 4.0) -> None:
        """Blocks until nvidia-smi has delivered its first sample (its start-up can take longer than the whole run)."""
        t_end = time.time() + timeout
        while self.proc is not None and not self.lines and time.time() < t_end:
            time.sleep(0.01)

    def samples_since_first_mark(self) -> int:
        return len(self.lines) - (self.marks[0] if self.marks else 0)

    def top_up(self, step, sync, seconds: float = 0.4, want: int = 4) -> None:
        """The timed region is a few milliseconds, shorter than one sampling period.  When too few samples fell
        under load, the same steps are repeated, untimed, right after it until a handful of samples exists."""
        if self.proc is None or self.samples_since_first_mark() >= want:
            return
        self.topped_up = True
        t_end = time.time() + seconds
        while time.time() < t_end and self.samples_since_first_mark() < want:
            for _ in range(20):
                step()
            sync()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        window = "device-timed region"
        lines = self.lines[self.marks[0]:self.marks[1]] if len(self.marks) >= 2 else []
        if len(lines) < 2:  # region shorter than the sampling period: use every sample taken under load
            lines, window = self.lines[self.marks[0] if self.marks else 0:], "timed + end-to-end regions"
            if self.topped_up:
                window += " + the same steps repeated untimed right after (the timed region is shorter than a sampling period)"
        for line in lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "window": window}


def reference_cpu_pass(layers, batch, threads, seeds_base=0):
    """One pass of the reference's own Winograd driver (oracle/_ref, compiled from the reference sources
    through the NEON stand-in header) over the layer stack, all host threads.  Returns seconds."""
    sys.path.insert(0, str(ROOT / "tests"))
    from _oracle import Reference
    from fastconv_b200 import synth

    ref = Reference.try_load()
    if ref is None:
        return None, "oracle/_ref/libfastconv_ref.so is not built"
    total = 0.0
    for idx, (c, k, h) in enumerate(layers):
        x = synth.conv_input(1, c, h, h, 1000 + idx + seeds_base)
        w = synth.conv_weights(k, c, 3, 3, 2000 + idx)
        t0 = time.perf_counter()
        for _ in range(batch):
            ref.wino_forward(x, w, 1, threads=threads)
        total += time.perf_counter() - t0
    return total, None


def run_reference_arm(args, rank, world):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    layers = VGG16
    flops = sum(layer_flops(args.batch, c, k, h) for c, k, h in layers)
    for _ in range(min(args.warmup, 1)):
        reference_cpu_pass(layers, args.batch, threads)
    times = []
    for _ in range(args.steps):
        t, err = reference_cpu_pass(layers, args.batch, threads)
        if t is None:
            print(json.dumps({"impl": "reference", "unavailable": err}))
            return
        times.append(t)
    sec = sum(times) / len(times)
    value = flops / sec / 1e9
    line = {
        "impl": "reference", "metric": "conv GFLOP/s (direct-equiv), VGG-16 conv stack", "value": value,
        "unit": "GFLOP/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": f"VGG-16 13 conv layers, batch {args.batch}, 224x224, 3x3 s1 p1, fp32 NCHW",
                   "algorithm": "reference winoF63_v1_multi (tileReg 5), online filter transform"},
        "cpu_baseline": {"value": value, "unit": "GFLOP/s", "cores": threads, "kind": "reference",
                         "sample": "all 13 layers, every step; NEON emulated through a vector-type stand-in header"},
        "e2e": {"value": value, "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


WIDE = [(c, c, h) for c in (512, 1024, 2048) for h in (14, 28, 56)]


def run_k_sharded(args, rank, world, local_rank, dist):
    """Single-image wide layers (C = K in {512,1024,2048} at 14/28/56), output channels split over the ranks:
    each rank keeps only its slice of the transformed weights, computes its channel slab and one NCCL
    all-gather per layer reassembles the NCHW output on every rank.  Total work is fixed: strong scaling."""
    import torch

    import fastconv_b200 as fc
    from fastconv_b200 import parallel, synth

    if dist is None:  # single rank: a one-member group keeps the code path identical
        import torch.distributed as dist_mod
        torch.cuda.set_device(local_rank)
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29577")
        dist_mod.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", local_rank))
        dist = dist_mod
    layers = WIDE if args.layers == "vgg16" else VGG16
    need = sum(4 * (64 * (k // world + 8) * c + 2 * 64 * 128 * (c + k) + k * c * 9 + 2 * (c + k) * h * h) for c, k, h in layers)
    ctx = fc.Context(local_rank, arena_bytes=int(need * 1.1) + (256 << 20))
    convs, flops = [], 0.0
    for idx, (c, k, h) in enumerate(layers):
        w = synth.conv_weights(k, c, 3, 3, 2000 + idx)
        x = synth.conv_input(1, c, h, h, 1000 + idx)
        if args.gather == "peer":
            conv = parallel.PeerKShardedConv(ctx, w, h, h, 1, args.mode)
            conv.upload(x)
            conv.forward()
        else:
            conv = parallel.KShardedConv.gpu(ctx, w, h, h, 1, args.mode)
            conv.forward(x)  # plans the slice, uploads the input once
        convs.append(conv)
        flops += layer_flops(1, c, k, h)
        del w

    def step():
        for conv in convs:
            if args.gather == "peer":
                conv.forward()
            else:
                conv.forward(None)

    for _ in range(args.warmup):
        step()
    sampler = ClockSampler(local_rank)
    sampler.start()
    sampler.wait_first()
    ctx.synchronize(); torch.cuda.synchronize(); dist.barrier()
    sampler.mark()
    ctx.timer_record(0)
    for _ in range(args.steps):
        step()
    ctx.timer_record(1)
    ms = ctx.timer_elapsed_ms(0, 1)
    torch.cuda.synchronize(); dist.barrier()
    sampler.mark()
    # the timed region is shorter than a sampling period: the same steps once more, untimed, the same count on every
    # rank (the ranks exchange step flags), so that the clock record has samples under this load
    for _ in range(10 * args.steps):
        step()
    ctx.synchronize(); torch.cuda.synchronize(); dist.barrier()
    sampler.topped_up = True
    clocks = sampler.stop()
    t = torch.tensor([ms], dtype=torch.float64, device=f"cuda:{local_rank}")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps
    if rank == 0:
        print(json.dumps({
            "metric": "conv GFLOP/s (direct-equiv), wide single-image layers, K-sharded", "value": round(flops / ms_step / 1e6, 1),
            "unit": "GFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 4),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": args.mode, "data": "synthetic",
            "config": {"workload": "3x3 s1 p1, batch 1, " + ";".join(f"{c}->{k}@{h}" for c, k, h in layers),
                       "parallelism": f"output channels split over {world} GPU(s), " + (
                           "slabs stored into every rank's output by the output transform (peer stores over NVLink)"
                           if args.gather == "peer" else "one NCCL all-gather per layer"),
                       "math_mode": args.mode},
            "gpu_launches": (5 if args.gather == "peer" else 3) * len(layers) * args.steps, "clocks": clocks}))
    ctx.synchronize()
    ctx.close_peer_mappings()
    dist.barrier()
    ctx.close()
    dist.barrier()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="fastconv", choices=["fastconv", "reference"])
    ap.add_argument("--mode", default="fp32", choices=["fp32", "3xtf32", "tf32", "tf32-strict"],
                    help="tf32-strict (with --algo auto): TF32 only where it stays within 3e-3 of fp32 -- per layer the direct "
                         "tensor-core kernel or the bit-exact fp32 Winograd path")
    ap.add_argument("--batch", type=int, default=1, help="images per GPU")
    ap.add_argument("--layers", default="vgg16",
                    help="'vgg16' (the 13-layer stack) or a list 'C,K,H;C,K,H;...' of 3x3 s1 p1 layers")
    ap.add_argument("--shard", default="batch", choices=["batch", "k"],
                    help="'batch': every rank runs the stack on its own images (no collective, the default); "
                         "'k': single-image wide layers with output channels split over the ranks + NCCL all-gather")
    ap.add_argument("--gather", default="peer", choices=["peer", "nccl"],
                    help="with --shard k: 'peer' = slabs stored into every rank's output by the output transform itself "
                         "(peer pointers over NVLink, flags); 'nccl' = separate all-gather after the layer")
    ap.add_argument("--chain", action="store_true",
                    help="not the reference's per-layer benchmark: layers of one VGG block feed each other on the device "
                         "(bias + ReLU in the epilogue), only block inputs and outputs cross PCIe in the end-to-end number")
    ap.add_argument("--algo", default="winograd", choices=["winograd", "auto", "direct"],
                    help="winograd: every layer through F(6x6,3x3) (the reference's path, the default); auto: the "
                         "library's choice per layer (in --mode tf32 the direct tensor-core kernel where it is faster); "
                         "direct: the direct tensor-core kernel for every layer (--mode tf32; rel-L2 <= 1e-3)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "fastconv":
        args.warmup = 3

    global VGG16
    workload_name = "VGG-16 13 conv layers"
    if args.layers != "vgg16":
        VGG16 = [tuple(int(v) for v in item.split(",")) for item in args.layers.split(";") if item]
        workload_name = "layers " + args.layers
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import fastconv_b200 as fc
    from fastconv_b200 import _lib, synth

    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist_mod

        torch.cuda.set_device(local_rank)
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist = dist_mod

    if args.shard == "k":
        run_k_sharded(args, rank, world, local_rank, dist)
        return

    lib = fc.load()
    mode = _lib.MODE_NAMES[args.mode]
    n = args.batch
    layers = VGG16
    # arena: weights (U is 64/9 of the raw filter), Winograd-domain V and M, activations
    need = 0
    for c, k, h in layers:
        t, tp, icp = wino_geometry(n, c, k, h)
        need += 4 * (64 * k * icp + 64 * tp * icp + 64 * k * tp + k * c * 9 + n * c * h * h + n * k * h * h) + 8 * 4096
        if args.algo != "winograd":  # the direct kernel's NHWC copy of the input and its re-laid-out weights
            c32 = (c + 31) // 32 * 32
            need += 4 * (n * c32 * h * h + 9 * k * c32) + 2 * 4096
    ctx = fc.Context(local_rank, arena_bytes=int(need * 1.05) + (64 << 20))

    convs, flops, h2d, d2h, footprint = [], 0.0, 0, 0, 0
    host_in, host_out = [], []
    for idx, (c, k, h) in enumerate(layers):
        desc = fc.make_desc(n, c, h, h, k)
        w = synth.conv_weights(k, c, 3, 3, 2000 + idx)
        x = synth.conv_input(n, c, h, h, 1000 + idx + 100 * rank)
        hdl = C.c_void_p()
        _lib.check(lib.fc_conv_create(ctx.handle, C.byref(desc), _lib.ALGO_NAMES[args.algo], mode,
                                      C.c_void_p(w.ctypes.data), C.byref(hdl)), "fc_conv_create")
        d_in, d_out = C.c_void_p(), C.c_void_p()
        _lib.check(lib.fc_conv_device_buffers(hdl, C.byref(d_in), C.byref(d_out)), "fc_conv_device_buffers")
        ctx.upload(x, d_in.value)
        px = ctx.pinned(x.shape)
        px[...] = x
        po = ctx.pinned((n, k, h, h))
        host_in.append(px)
        host_out.append(po)
        convs.append((hdl, d_in, d_out, desc))
        flops += layer_flops(n, c, k, h)
        h2d += x.nbytes
        d2h += po.nbytes
        t, tp, icp = wino_geometry(n, c, k, h)
        footprint += 4 * (64 * k * icp + 64 * tp * icp + 64 * k * tp + n * c * h * h + n * k * h * h)

    d_ins, d_outs = [c[1].value for c in convs], [c[2].value for c in convs]
    if args.chain:
        # layer i+1 of a block (same H, its C == the K before it) reads layer i's output where it lies on the device
        for i in range(1, len(layers)):
            if layers[i][0] == layers[i - 1][1] and layers[i][2] == layers[i - 1][2]:
                d_ins[i] = d_outs[i - 1]
                h2d -= host_in[i].nbytes
                d2h -= host_out[i - 1].nbytes
                host_in[i] = None
                host_out[i - 1] = None
        for i, (hdl, _, _, _) in enumerate(convs):
            bias = (synth.conv_input(1, 1, 1, layers[i][1], 3000 + i).reshape(-1) * np.float32(0.1)).astype(np.float32)
            _lib.check(lib.fc_conv_set_epilogue(hdl, C.c_void_p(bias.ctypes.data), 1), "fc_conv_set_epilogue")
    # the whole stack as one CUDA graph: a step is one graph launch
    stack = fc.LayerList(ctx, [c[0] for c in convs], d_ins, d_outs)

    def step_device():
        stack.forward()

    def step_host():
        stack.forward_host(host_in, host_out)  # pinned host buffers in, pinned host buffers out

    def barrier():
        ctx.synchronize()
        if dist is not None:
            dist.barrier()

    def reduce_max(v: float) -> float:
        if dist is None:
            return v
        import torch
        t = torch.tensor([v], dtype=torch.float64, device=f"cuda:{local_rank}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident throughput (`value`) -----------------------------------------------------
    sampler = ClockSampler(local_rank)
    sampler.start()
    sampler.wait_first()
    for _ in range(args.warmup):
        step_device()
    barrier()
    sampler.mark()
    ctx.timer_record(0)
    for _ in range(args.steps):
        step_device()
    ctx.timer_record(1)
    ms_total = ctx.timer_elapsed_ms(0, 1)
    barrier()
    sampler.mark()
    ms_step = reduce_max(ms_total) / args.steps

    # ---- end to end through the host-pointer entry point (pinned host buffers) ----------------------
    for _ in range(3):
        step_host()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step_host()
    ctx.synchronize()
    e2e_ms = reduce_max((time.perf_counter() - t0) * 1e3) / args.steps
    barrier()
    sampler.top_up(step_device, ctx.synchronize)
    clocks = sampler.stop()

    # ---- per-layer and per-kernel device times (CUDA events around each stage, same inputs) ----------
    per_layer, stage_tot = [], [0.0] * 5
    roof_sum_ms = 0.0
    launches_per_step = 0
    gemm_bytes = gemm_ms = gemm_flops = 0.0
    direct_ms = direct_flops = 0.0
    n_wino = n_direct = 0
    hbm_peak, bf16_peak, peak_kind = measured_peaks()
    for (hdl, d_in, d_out, desc), (c, k, h) in zip(convs, layers):
        ms = (C.c_float * 5)()
        _lib.check(lib.fc_conv_profile(hdl, d_in, d_out, max(3, args.steps), ms), "fc_conv_profile")
        one = C.c_float()
        _lib.check(lib.fc_conv_time_device(hdl, d_in, d_out, 3, max(3, args.steps), C.byref(one)), "fc_conv_time_device")
        nl = C.c_int()
        lib.fc_conv_launches_per_forward(hdl, C.byref(nl))
        launches_per_step += nl.value
        algo, resolved = C.c_int(), C.c_int()
        lib.fc_conv_algorithm(hdl, C.byref(algo))
        lib.fc_conv_math_mode(hdl, C.byref(resolved))
        layer_mode = {0: "fp32", 1: "3xtf32", 2: "tf32"}[resolved.value]  # tf32-strict resolves per layer
        is_wino = algo.value == _lib.ALGO_WINOGRAD
        t, tp, icp = wino_geometry(n, c, k, h)
        # roofline of a layer: the slower of its flops (Winograd-domain for a Winograd layer, direct otherwise) at the
        # mode's arithmetic peak and its HBM bytes (input, filter as the kernel reads it, output) at the measured
        # copy bandwidth
        bytes_min = 4.0 * (n * c * h * h + 9 * c * k + n * k * h * h)
        bytes_wino = 4.0 * (n * c * h * h + 64 * c * k + n * k * h * h) if is_wino else bytes_min
        wino_flops = 2.0 * 64 * t * c * k if is_wino else layer_flops(n, c, k, h)
        t_hbm_ms = bytes_wino / hbm_peak / 1e6
        t_flop_ms = wino_flops / (MODE_PEAK_TFLOPS[layer_mode] * 1e12) * 1e3
        roof_ms = max(t_hbm_ms, t_flop_ms)
        roof_sum_ms += roof_ms
        per_layer.append({
            "layer": f"{c}->{k}@{h}", "algo": {v: kk for kk, v in _lib.ALGO_NAMES.items()}[algo.value], "math": layer_mode,
            "ms": round(one.value, 5),
            "gflops_direct_equiv": round(layer_flops(n, c, k, h) / one.value / 1e6, 1),
            "stage_ms": [round(float(v), 5) for v in ms],
            "t_hbm_ms": round(t_hbm_ms, 5), "t_flop_ms": round(t_flop_ms, 5),
            "bound": "hbm" if t_hbm_ms >= t_flop_ms else "math",
            "frac_of_roofline": round(roof_ms / one.value, 4),
            "frac_of_min_bytes_roofline": round(max(bytes_min / hbm_peak / 1e6, t_flop_ms) / one.value, 4),
        })
        for i in range(5):
            stage_tot[i] += ms[i]
        if is_wino:
            gemm_bytes += 4.0 * (64 * k * icp + 64 * tp * icp + 64 * k * tp)
            gemm_ms += ms[2]
            gemm_flops += wino_flops
            n_wino += 1
        else:  # stage 2 of a direct layer = the layout pass + direct_tc_kernel
            direct_ms += ms[2]
            direct_flops += wino_flops
            n_direct += 1

    nl = max(n_wino, 1)
    achieved_gbs = gemm_bytes / (gemm_ms / 1e3) / 1e9 if gemm_ms > 0 else 0.0
    roofline = {
        "kernel": "TensorGEMM (64 batched U*V products, one launch per layer)",
        "bound": "hbm", "achieved": round(achieved_gbs, 1), "peak": hbm_peak, "unit": "GB/s",
        "frac": round(achieved_gbs / hbm_peak, 4), "peak_source": f"of {peak_kind}",
        "traffic": NCU_GEMM_TRAFFIC_BYTES.get(args.mode) if (args.layers == "vgg16" and n == 1 and args.algo == "winograd") else None,
        "algorithmic_bytes_per_launch": gemm_bytes / nl, "avg_launch_ms": gemm_ms / nl,
        "stack_roofline_ms": round(roof_sum_ms, 5), "stack_frac_of_roofline": round(roof_sum_ms / ms_step, 4),
        "arithmetic_peak_tflops": round(MODE_PEAK_TFLOPS.get(args.mode, TF32_TFLOPS), 1),
        "winograd_domain_tflops": round(gemm_flops / (gemm_ms / 1e3) / 1e12, 2) if gemm_ms > 0 else None,
        "share_of_step": {"InputTran": round(stage_tot[0] / stage_tot[4], 3), "TensorGEMM": round(stage_tot[2] / stage_tot[4], 3),
                          "OutputTran": round(stage_tot[3] / stage_tot[4], 3)},
    }
    if direct_ms > gemm_ms:
        # the direct tensor-core kernel dominates the step: bound by the tensor pipe
        ach = direct_flops / (direct_ms / 1e3) / 1e12
        roofline = {
            "kernel": "direct_tc_kernel (+ its layout pass), one launch pair per layer",
            "bound": "tensor", "achieved": round(ach, 1), "peak": MODE_PEAK_TFLOPS["tf32"], "unit": "TFLOP/s",
            "frac": round(ach / MODE_PEAK_TFLOPS["tf32"], 4),
            "peak_source": "TF32 library GEMM (8192^3) measured on a B200 of this pool",
            "traffic": None, "algorithmic_flops_per_launch": direct_flops / n_direct, "avg_launch_ms": direct_ms / n_direct,
            "stack_roofline_ms": round(roof_sum_ms, 5), "stack_frac_of_roofline": round(roof_sum_ms / ms_step, 4),
            "layers_direct": n_direct, "layers_winograd": n_wino,
        }

    line = None
    if rank == 0:
        value = world * flops / (ms_step / 1e3) / 1e9
        e2e_value = world * flops / (e2e_ms / 1e3) / 1e9
        line = {
            "metric": "conv GFLOP/s (direct-equiv), VGG-16 conv stack", "value": round(value, 1), "unit": "GFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": {"fp32": "f32", "3xtf32": "3xtf32", "tf32": "tf32", "tf32-strict": "tf32/f32 per layer"}[args.mode],
            "data": "synthetic",
            "config": {"workload": f"{workload_name}, batch {n} per GPU, 224x224, 3x3 s1 p1, fp32 NCHW",
                       "algorithm": {"winograd": "winograd F(6x6,3x3)", "direct": "direct convolution on the tensor cores",
                                     "auto": "per layer: winograd F(6x6,3x3) or direct convolution on the tensor cores"}[args.algo],
                       "math_mode": args.mode,
                       "launch": "all layers of a step replayed as one CUDA graph",
                       "chain": bool(args.chain),
                       "parallelism": f"images sharded over {world} GPU(s), no collective",
                       "l2": f"inputs larger than L2: the stack touches {footprint / 1e6:.0f} MB per step"},
            "e2e": {"value": round(e2e_value, 1), "unit": "GFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": round(e2e_ms, 4)},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
            "roofline": roofline,
            "layers": per_layer,
        }
        if not args.no_cpu_baseline and world == 1:
            threads = os.cpu_count() or 1
            sec, err = reference_cpu_pass(layers, n, threads)
            if sec is not None:
                line["cpu_baseline"] = {"value": round(flops / sec / 1e9, 2), "unit": "GFLOP/s", "cores": threads,
                                        "kind": "reference",
                                        "sample": "one pass over all 13 layers with the reference's winoF63_v1_multi "
                                                  "(NEON emulated via a vector-type stand-in header), all host threads"}
            else:
                line["cpu_baseline"] = {"value": None, "unit": "GFLOP/s", "cores": threads, "kind": "reference",
                                        "sample": err}
    stack.close()
    for hdl, _, _, _ in convs:
        lib.fc_conv_destroy(hdl)
    ctx.close()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if line is not None:
        print(json.dumps(line))


if __name__ == "__main__":
    main()

#!/usr/bin/env python
"""Benchmark of the convolution-layer hot path: the 13 conv layers of VGG-16 (3x3, stride 1, pad 1).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--mode fp32|3xtf32|tf32] [--batch B] [--algo A]
    python bench.py --impl reference ...      # the reference's own CPU algorithm on the host cores
    python bench.py --shard k ...             # single-image wide layers, output channels split over the GPUs

Default workload: the batched VGG-16 stack, 64 images IN ALL, split by image over the N GPUs (no collective in the
data path; total work is fixed, so the scaling is strong).  A step is one Forward() of every layer of the stack on this
rank's images (each layer has its own seeded synthetic input and weights: the reference benchmarks single layers, it
does not chain them); all layers of a step are replayed as one CUDA graph.  The metric is direct-convolution-equivalent
GFLOP/s, sum(2*N*K*C*9*OH*OW) / time, whole job.  `value` is measured in the bit-exact fp32 mode; the same workload
in the TF32 mode and the batch-1 stack are carried as sub-records of the same JSON line, which rank 0 prints.

With N > 1 the launcher starts one process per GPU (RANK / LOCAL_RANK / WORLD_SIZE in the environment); process
group, barrier and max-over-ranks all go through the library's communicator (fc_comm_*), not through torch.
"""
from __future__ import annotations

import argparse
import atexit
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# C, K, H(=W) of the 13 VGG-16 conv layers at 224x224 input
VGG16 = [(3, 64, 224), (64, 64, 224), (64, 128, 112), (128, 128, 112), (128, 256, 56), (256, 256, 56), (256, 256, 56),
         (256, 512, 28), (512, 512, 28), (512, 512, 28), (512, 512, 14), (512, 512, 14), (512, 512, 14)]
WIDE = [(c, c, h) for c in (512, 1024, 2048) for h in (14, 28, 56)]

HBM_FALLBACK_GBS = 6650.0
# TF32 dense throughput of a library GEMM (torch.matmul 8192^3, best of 10, CUDA events) on a B200: the arithmetic
# peak the TF32 fractions divide by; 3xTF32 issues three MMAs per product.  Half of the bf16 figure of
# MEASURED_PEAKS.json is reported beside it.  The same measurement in fp32 gives 63.7 TFLOP/s; the fp32 fractions
# divide by the pipe's own peak instead: SMs x 128 lanes x 2 flop x the SM clock sampled while the kernels ran.
TF32_LIBRARY_TFLOPS = 759.9
FP32_LIBRARY_TFLOPS = 63.7

# DRAM bytes (read + write) per TensorGEMM launch, averaged over the 12 launches of one step of the default workload
# (VGG-16, 64 images, fp32 mode, one GPU; the first layer has no TensorGEMM launch), from one ncu capture of
# `dram__bytes_read.sum + dram__bytes_write.sum` (profiles/tensorgemm_dram_traffic_vgg16_batch64.md).  None for any other
# workload.
NCU_GEMM_TRAFFIC_BYTES_DEFAULT = 841.89e6


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


def shard_range(total, world, rank):
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed regions run."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.lines, self.marks = gpu_index, None, [], []

    def mark(self):
        """Remembers how many samples had arrived: the first two marks bracket the device-timed regions."""
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
        """Blocks until nvidia-smi has delivered its first sample (its start-up can take longer than a short run)."""
        t_end = time.time() + timeout
        while self.proc is not None and not self.lines and time.time() < t_end:
            time.sleep(0.01)

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
        window = "device-timed regions (the K timed steps and their repeats)"
        lines = self.lines[self.marks[0]:self.marks[1]] if len(self.marks) >= 2 else []
        if len(lines) < 2:  # regions shorter than the sampling period: use every sample taken under load
            lines, window = self.lines[self.marks[0] if self.marks else 0:], "all samples after the warm-up"
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


def make_batch(one_image: np.ndarray, n: int, first: int = 0) -> np.ndarray:
    """n distinct images from one generated image: image i (global index first + i) is the image scaled by
    1 - i/256, an exact fp32 factor.  Generating 64 independent images per layer would take longer than the benchmark."""
    scale = (1.0 - (np.arange(first, first + n, dtype=np.float32) % 128) / 256.0).reshape(n, 1, 1, 1)
    return np.ascontiguousarray(one_image * scale)


# ---- the reference's own CPU implementation ---------------------------------------------------------

def reference_cpu_pass(layers, images, threads):
    """`images` images through the reference's own Winograd driver (oracle/_ref, compiled from the reference sources
    through the NEON stand-in header) over the layer stack, all host threads.  Returns seconds."""
    sys.path.insert(0, str(ROOT / "tests"))
    from _oracle import Reference
    from fastconv_b200 import synth

    ref = Reference.try_load()
    if ref is None:
        return None, "oracle/_ref/libfastconv_ref.so is not built"
    total = 0.0
    for idx, (c, k, h) in enumerate(layers):
        x = synth.conv_input(1, c, h, h, 1000 + idx)
        w = synth.conv_weights(k, c, 3, 3, 2000 + idx)
        t0 = time.perf_counter()
        for _ in range(images):  # the reference has no batch dimension: one Forward per image
            ref.wino_forward(x, w, 1, threads=threads)
        total += time.perf_counter() - t0
    return total, None


def run_reference_arm(args, rank, layers, workload):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    images = max(1, min(args.batch, args.ref_images))  # a bounded sample of the batch per step
    flops = sum(layer_flops(images, c, k, h) for c, k, h in layers)
    for _ in range(min(args.warmup, 1)):
        reference_cpu_pass(layers, images, threads)
    times = []
    for _ in range(args.steps):
        t, err = reference_cpu_pass(layers, images, threads)
        if t is None:
            print(json.dumps({"impl": "reference", "unavailable": err}))
            return
        times.append(t)
    sec = sum(times) / len(times)
    value = flops / sec / 1e9
    sample = (f"{images} of the {args.batch} images through all {len(layers)} layers per step (the reference runs one "
              f"image per Forward, so GFLOP/s does not depend on the sample); NEON emulated through a vector-type "
              f"stand-in header")
    print(json.dumps({
        "impl": "reference", "metric": "conv GFLOP/s (direct-equiv), VGG-16 conv stack", "value": value,
        "unit": "GFLOP/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": sec * 1e3 * args.batch / images, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload,
                   "algorithm": "reference winoF63_v1_multi (tileReg 5), online filter transform",
                   "note": "ms_per_step is the sample's time scaled to the whole batch"},
        "cpu_baseline": {"value": value, "unit": "GFLOP/s", "cores": threads, "kind": "reference", "sample": sample},
        "e2e": {"value": value, "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ---- one planned stack on one GPU -------------------------------------------------------------------

class Stack:
    """The layer stack planned for `n` images on one context, with device-resident inputs and (optionally) pinned
    host buffers for the end-to-end path."""

    def __init__(self, fc, ctx, layers, n, first_image, mode, algo, chain=False, host=True, tune=False):
        from fastconv_b200 import _lib, synth
        self.fc, self.ctx, self.lib, self._lib = fc, ctx, fc.load(), _lib
        self.layers, self.n = layers, n
        self.convs, self.host_in, self.host_out = [], [], []
        self.flops = self.h2d = self.d2h = self.footprint = 0
        for idx, (c, k, h) in enumerate(layers):
            desc = fc.make_desc(n, c, h, h, k)
            w = synth.conv_weights(k, c, 3, 3, 2000 + idx)
            x = make_batch(synth.conv_input(1, c, h, h, 1000 + idx), n, first_image)
            hdl = C.c_void_p()
            _lib.check(self.lib.fc_conv_create(ctx.handle, C.byref(desc), _lib.ALGO_NAMES[algo], _lib.MODE_NAMES[mode],
                                               C.c_void_p(w.ctypes.data), C.byref(hdl)), "fc_conv_create")
            d_in, d_out = C.c_void_p(), C.c_void_p()
            _lib.check(self.lib.fc_conv_device_buffers(hdl, C.byref(d_in), C.byref(d_out)), "fc_conv_device_buffers")
            ctx.upload(x, d_in.value)
            if tune:  # Tuning(): the layer's kernel configuration by measured device time, before anything is timed
                _lib.check(self.lib.fc_conv_tune(hdl, 3, 0), "fc_conv_tune")
            if host:
                px = ctx.pinned(x.shape)
                px[...] = x
                self.host_in.append(px)
                self.host_out.append(ctx.pinned((n, k, h, h)))
                self.h2d += x.nbytes
                self.d2h += self.host_out[-1].nbytes
            self.convs.append((hdl, d_in, d_out, desc))
            self.flops += layer_flops(n, c, k, h)
            t, tp, icp = wino_geometry(n, c, k, h)
            self.footprint += 4 * (64 * k * icp + 64 * tp * icp + 64 * k * tp + n * c * h * h + n * k * h * h)
            del x, w
        d_ins, d_outs = [c[1].value for c in self.convs], [c[2].value for c in self.convs]
        if chain:
            # layer i+1 of a block (same H, its C == the K before it) reads layer i's output where it lies on the device
            for i in range(1, len(layers)):
                if layers[i][0] == layers[i - 1][1] and layers[i][2] == layers[i - 1][2]:
                    d_ins[i] = d_outs[i - 1]
                    if host:
                        self.h2d -= self.host_in[i].nbytes
                        self.d2h -= self.host_out[i - 1].nbytes
                        self.host_in[i] = None
                        self.host_out[i - 1] = None
            for i, (hdl, _, _, _) in enumerate(self.convs):
                bias = (synth.conv_input(1, 1, 1, layers[i][1], 3000 + i).reshape(-1) * np.float32(0.1)).astype(np.float32)
                _lib.check(self.lib.fc_conv_set_epilogue(hdl, C.c_void_p(bias.ctypes.data), 1), "fc_conv_set_epilogue")
        # the whole stack as one CUDA graph: a step is one graph launch
        self.graph = fc.LayerList(ctx, [c[0] for c in self.convs], d_ins, d_outs)

    @staticmethod
    def arena_need(layers, n, algo):
        need = 0
        for c, k, h in layers:
            t, tp, icp = wino_geometry(n, c, k, h)
            need += 4 * (64 * k * icp + 64 * tp * icp + 64 * k * tp + k * c * 9 + n * c * h * h + n * k * h * h) + 8 * 4096
            if algo != "winograd":  # the direct kernel's NHWC copy of the input and its re-laid-out weights
                c32 = (c + 31) // 32 * 32
                need += 4 * (n * c32 * h * h + 9 * k * c32) + 2 * 4096
        return int(need * 1.05) + (64 << 20)

    def step_device(self):
        self.graph.forward()

    def step_host(self):
        self.graph.forward_host(self.host_in, self.host_out)  # pinned host buffers in, pinned host buffers out

    def launches_per_step(self):
        total = 0
        for hdl, _, _, _ in self.convs:
            nl = C.c_int()
            self.lib.fc_conv_launches_per_forward(hdl, C.byref(nl))
            total += nl.value
        return total

    def per_layer(self, iters, hbm_peak, peak_tflops):
        """Per-layer and per-kernel device times (CUDA events around each stage, same inputs) and the roofline of
        each layer: the slower of its flops (Winograd-domain for a Winograd layer, direct otherwise) at the mode's
        arithmetic peak and its HBM bytes (input, filter as the kernel reads it, output) at the measured copy bandwidth."""
        rows, agg = [], {"stage": [0.0] * 5, "gemm_ms": 0.0, "gemm_flops": 0.0, "gemm_bytes": 0.0, "n_wino": 0,
                         "direct_ms": 0.0, "direct_flops": 0.0, "n_direct": 0, "roof_ms": 0.0}
        n = self.n
        for (hdl, d_in, d_out, desc), (c, k, h) in zip(self.convs, self.layers):
            ms = (C.c_float * 5)()
            self._lib.check(self.lib.fc_conv_profile(hdl, d_in, d_out, iters, ms), "fc_conv_profile")
            one = C.c_float()
            self._lib.check(self.lib.fc_conv_time_device(hdl, d_in, d_out, 3, iters, C.byref(one)), "fc_conv_time_device")
            algo, resolved = C.c_int(), C.c_int()
            self.lib.fc_conv_algorithm(hdl, C.byref(algo))
            self.lib.fc_conv_math_mode(hdl, C.byref(resolved))
            layer_mode = {0: "fp32", 1: "3xtf32", 2: "tf32", 4: "tf32"}[resolved.value]  # "tf32" resolves per layer
            work = [C.c_double() for _ in range(4)]
            self._lib.check(self.lib.fc_conv_work(hdl, *[C.byref(v) for v in work]), "fc_conv_work")
            direct, algo_flops, algo_bytes, min_bytes = (v.value for v in work)
            is_wino = algo.value == self._lib.ALGO_WINOGRAD
            t, tp, icp = wino_geometry(n, c, k, h)
            t_hbm_ms = algo_bytes / hbm_peak / 1e6
            t_flop_ms = algo_flops / (peak_tflops[layer_mode] * 1e12) * 1e3
            roof_ms = max(t_hbm_ms, t_flop_ms)
            agg["roof_ms"] += roof_ms
            rows.append({
                "layer": f"{c}->{k}@{h}", "algo": {v: kk for kk, v in self._lib.ALGO_NAMES.items()}[algo.value],
                "math": layer_mode, "ms": round(one.value, 5), "gflops_direct_equiv": round(direct / one.value / 1e6, 1),
                "stage_ms": [round(float(v), 5) for v in ms],
                "t_hbm_ms": round(t_hbm_ms, 5), "t_flop_ms": round(t_flop_ms, 5),
                "bound": "hbm" if t_hbm_ms >= t_flop_ms else "math",
                "frac_of_roofline": round(roof_ms / one.value, 4),
                "frac_of_min_bytes_roofline": round(max(min_bytes / hbm_peak / 1e6, t_flop_ms) / one.value, 4),
            })
            for i in range(5):
                agg["stage"][i] += ms[i]
            nl = C.c_int()
            self.lib.fc_conv_launches_per_forward(hdl, C.byref(nl))
            if is_wino and nl.value == 2:
                # a layer of at most 4 input channels: its multiply-accumulate runs inside the output transform, there
                # is no TensorGEMM launch to count
                rows[-1]["tensor_gemm"] = "inside the output transform"
            elif is_wino:
                agg["gemm_bytes"] += 4.0 * (64 * k * icp + 64 * tp * icp + 64 * k * tp)
                agg["gemm_ms"] += ms[2]
                agg["gemm_flops"] += algo_flops
                agg["n_wino"] += 1
            else:  # stage 2 of a direct layer = the layout pass + direct_tc_kernel
                agg["direct_ms"] += ms[2]
                agg["direct_flops"] += algo_flops
                agg["n_direct"] += 1
        return rows, agg

    def close(self):
        self.graph.close()
        for hdl, _, _, _ in self.convs:
            self.lib.fc_conv_destroy(hdl)
        self.convs = []
        self.host_in = self.host_out = []


def timed_region(comm, ctx, step, steps):
    """EXACTLY `steps` steps between a barrier + synchronize on both sides, CUDA events on the launching stream,
    maximum over the ranks; returns milliseconds per step."""
    comm.barrier()
    ctx.timer_record(0)
    for _ in range(steps):
        step()
    ctx.timer_record(1)
    ms = ctx.timer_elapsed_ms(0, 1)
    comm.barrier()
    return comm.max(ms) / steps


def measure_stack(comm, ctx, stack, args, repeats):
    for _ in range(args.warmup):
        stack.step_device()
    first = timed_region(comm, ctx, stack.step_device, args.steps)
    more = [timed_region(comm, ctx, stack.step_device, args.steps) for _ in range(repeats)]
    return first, [first] + more


def measure_e2e(comm, ctx, stack, steps):
    for _ in range(2):
        stack.step_host()
    comm.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        stack.step_host()
    ctx.synchronize()
    ms = (time.perf_counter() - t0) * 1e3
    comm.barrier()
    return comm.max(ms) / steps


def copy_bandwidths(ctx, stack, reps=3):
    """Plain pinned-memory copies of this rank's per-step byte counts, all ranks at once: what the host's PCIe path
    gives each rank while the others use it too (GB/s up, GB/s down)."""
    pairs = [(a, b) for a, b in zip(stack.host_in, stack.host_out) if a is not None and b is not None]
    if not pairs:
        return 0.0, 0.0
    lib = stack.lib
    t0 = time.perf_counter()
    for _ in range(reps):
        for (hdl, d_in, _, _), px in zip(stack.convs, stack.host_in):
            if px is not None:
                lib.fc_memcpy_h2d(ctx.handle, d_in, C.c_void_p(px.ctypes.data), px.nbytes)
    up = stack.h2d * reps / (time.perf_counter() - t0) / 1e9
    t0 = time.perf_counter()
    for _ in range(reps):
        for (hdl, _, d_out, _), po in zip(stack.convs, stack.host_out):
            if po is not None:
                lib.fc_memcpy_d2h(ctx.handle, C.c_void_p(po.ctypes.data), d_out, po.nbytes)
    down = stack.d2h * reps / (time.perf_counter() - t0) / 1e9
    return up, down


# ---- K-sharded wide sweep ---------------------------------------------------------------------------

def run_k_sharded(args, comm, ctx, rank, world, local_rank):
    """Single-image wide layers (C = K in {512,1024,2048} at 14/28/56), output channels split over the ranks:
    each rank keeps only its slice of the transformed weights and computes its channel slab; the slabs reach every
    rank through the stores of the output transform (peer memory over NVLink) or one NCCL all-gather per layer.
    Total work is fixed: strong scaling."""
    from fastconv_b200 import parallel, synth

    layers = WIDE if args.layers == "vgg16" else parse_layers(args.layers)
    convs, flops = [], 0.0
    for idx, (c, k, h) in enumerate(layers):
        w = synth.conv_weights(k, c, 3, 3, 2000 + idx)
        x = synth.conv_input(1, c, h, h, 1000 + idx)
        sc = parallel.ShardedConv(comm, w, 1, h, h, shard="k", gather=args.gather, algorithm="winograd", mode=args.mode)
        sc.upload(x)
        convs.append(sc)
        flops += layer_flops(1, c, k, h)
        del w

    def step():  # every layer's forward, then the waits for the other ranks' slabs of all of them
        for sc in convs:
            sc.forward()
        for sc in convs:
            sc.wait()

    for _ in range(args.warmup):
        step()
    sampler = ClockSampler(local_rank)
    sampler.start()
    sampler.wait_first()
    sampler.mark()
    first = timed_region(comm, ctx, step, args.steps)
    times = [first] + [timed_region(comm, ctx, step, args.steps) for _ in range(args.repeats)]
    sampler.mark()
    clocks = sampler.stop()
    per_layer = [{"layer": f"{c}->{k}@{h}", "ms": round(sc.time_device(2, max(3, args.steps)), 5)}
                 for sc, (c, k, h) in zip(convs, layers)]
    if rank == 0:
        launches = (3 if args.gather == "peer" else 4) * len(layers) + (len(layers) if args.gather == "peer" else 0)
        print(json.dumps({
            "metric": "conv GFLOP/s (direct-equiv), wide single-image layers, K-sharded", "value": round(flops / first / 1e6, 1),
            "unit": "GFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(first, 4),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": args.mode, "data": "synthetic",
            "config": {"workload": "3x3 s1 p1, batch 1, " + ";".join(f"{c}->{k}@{h}" for c, k, h in layers),
                       "parallelism": f"output channels split over {world} GPU(s), " + (
                           "slabs stored into every rank's output by the output transform, which also publishes the "
                           "step (peer stores over NVLink); one bounded wait per layer at the end of the step"
                           if args.gather == "peer" else "one NCCL all-gather per layer"),
                       "math_mode": args.mode},
            "repeat_stats": repeat_stats(times, args.steps),
            "gpu_launches": launches * args.steps * world, "clocks": clocks, "layers": per_layer}))
    for sc in convs:
        sc.release()


def repeat_stats(times, steps):
    return {"regions": len(times), "steps_per_region": steps, "median_ms_per_step": round(statistics.median(times), 5),
            "min_ms_per_step": round(min(times), 5), "max_ms_per_step": round(max(times), 5)}


def parse_layers(text):
    return [tuple(int(v) for v in item.split(",")) for item in text.split(";") if item]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="fastconv", choices=["fastconv", "reference"])
    ap.add_argument("--mode", default="fp32", choices=["fp32", "3xtf32", "tf32", "tf32-unbounded", "tf32-u16"],
                    help="arithmetic of `value`: fp32 = bit-identical to the reference (default); tf32 keeps rel-L2 <= 3e-3 "
                         "on every layer; tf32-unbounded also runs one TF32 pass through Winograd (6.4e-3)")
    ap.add_argument("--batch", type=int, default=64, help="images IN ALL, split by image over the GPUs")
    ap.add_argument("--layers", default="vgg16",
                    help="'vgg16' (the 13-layer stack) or a list 'C,K,H;C,K,H;...' of 3x3 s1 p1 layers")
    ap.add_argument("--shard", default="batch", choices=["batch", "k"],
                    help="'batch': every rank runs the stack on its share of the images (no collective, the default); "
                         "'k': single-image wide layers with the output channels split over the ranks")
    ap.add_argument("--gather", default="peer", choices=["peer", "nccl"],
                    help="with --shard k: 'peer' = slabs stored into every rank's output by the output transform itself "
                         "(peer pointers over NVLink, flags); 'nccl' = one all-gather after the layer")
    ap.add_argument("--chain", action="store_true",
                    help="not the reference's per-layer benchmark: layers of one VGG block feed each other on the device "
                         "(bias + ReLU in the epilogue), only block inputs and outputs cross PCIe in the end-to-end number")
    ap.add_argument("--algo", default=None, choices=["winograd", "auto", "direct"],
                    help="winograd: every layer through F(6x6,3x3) (the reference's path; default in the fp32 and 3xtf32 "
                         "modes); auto: the library's choice per layer (default in the tf32 modes); direct: the direct "
                         "tensor-core kernel for every layer (tf32 modes)")
    ap.add_argument("--repeats", type=int, default=25, help="further timed regions of K steps, for median/min/max")
    ap.add_argument("--ref-images", type=int, default=4, help="--impl reference: images of the batch run per step")
    ap.add_argument("--no-tuning", dest="tuning", action="store_false",
                    help="keep the launchers' heuristics instead of running Tuning() on every layer first")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-subrecords", action="store_true", help="skip the TF32 and batch-1 sub-records")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "fastconv":
        args.warmup = 3
    if args.algo is None:
        args.algo = "auto" if args.mode.startswith("tf32") else "winograd"

    layers, workload_name = VGG16, "VGG-16 13 conv layers"
    if args.layers != "vgg16":
        layers, workload_name = parse_layers(args.layers), "layers " + args.layers
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    workload = (f"{workload_name}, {args.batch} images in all split by image over {world} GPU(s), 224x224, 3x3 s1 p1, "
                f"fp32 NCHW")

    if args.impl == "reference":
        run_reference_arm(args, rank, layers, workload)
        return

    import fastconv_b200 as fc
    from fastconv_b200 import parallel

    if args.tuning and "FASTCONV_TUNING_LOG" not in os.environ:
        # a log of this run only: an entry left by another GPU, clock state or library build must not decide a layer
        fd, log_path = tempfile.mkstemp(prefix=f"fastconv_tuning_r{rank}_", suffix=".log")
        os.close(fd)
        os.environ["FASTCONV_TUNING_LOG"] = log_path
        atexit.register(lambda: os.path.exists(log_path) and os.remove(log_path))

    n0, n1 = shard_range(args.batch, world, rank)
    n = n1 - n0
    if n < 1:
        raise SystemExit(f"rank {rank}: {args.batch} images do not cover {world} GPUs")
    if args.shard == "k":
        need = sum(4 * (64 * (k // world + 8) * c + 2 * 64 * 128 * (c + k) + k * c * 9 + 4 * (c + k) * h * h)
                   for c, k, h in (WIDE if args.layers == "vgg16" else layers))
        arena = int(need * 1.1) + (256 << 20)
    else:
        arena = max(Stack.arena_need(layers, n, args.algo), Stack.arena_need(layers, n, "auto")) + (64 << 20)
    comm = parallel.Comm.from_env(local_rank, arena_bytes=arena)  # one rank per process; world 1 needs no NCCL
    ctx = comm.contexts[0]
    if args.shard == "k":
        run_k_sharded(args, comm, ctx, rank, world, local_rank)
        comm.close()
        return

    hbm_peak, bf16_peak, peak_kind = measured_peaks()
    sampler = ClockSampler(local_rank)
    sampler.start()
    sampler.wait_first()

    # ---- `value`: device-resident throughput of the whole job --------------------------------------------
    stack = Stack(fc, ctx, layers, n, n0, args.mode, args.algo, chain=args.chain, tune=args.tuning)
    for _ in range(args.warmup):
        stack.step_device()
    sampler.mark()
    ms_step = timed_region(comm, ctx, stack.step_device, args.steps)
    times = [ms_step] + [timed_region(comm, ctx, stack.step_device, args.steps) for _ in range(args.repeats)]
    sampler.mark()
    # ---- end to end through the host-pointer entry point (pinned host buffers, copies inside the timed region) ---
    e2e_ms = measure_e2e(comm, ctx, stack, args.steps)
    copy_bw = comm.allgather(list(copy_bandwidths(ctx, stack))) if world > 1 else None
    clocks = sampler.stop()

    sm_mhz = clocks.get("sm_mhz") or clocks.get("sm_max_mhz") or 1965.0
    sms, _mhz = C.c_int(), C.c_int()
    fc.load().fc_context_info(ctx.handle, C.byref(sms), C.byref(_mhz))
    fp32_peak = sms.value * 128 * 2 * sm_mhz * 1e-6  # TFLOP/s of the FP32 pipes at the clock the kernels ran at
    peak_tflops = {"fp32": fp32_peak, "tf32": TF32_LIBRARY_TFLOPS, "3xtf32": TF32_LIBRARY_TFLOPS / 3.0}
    per_layer, agg = stack.per_layer(max(3, args.steps), hbm_peak, peak_tflops)
    launches = stack.launches_per_step()
    total_flops = sum(layer_flops(args.batch, c, k, h) for c, k, h in layers)

    # ---- roofline entry of the dominant kernel ---------------------------------------------------------------
    stage = agg["stage"]
    share = {"InputTran": round(stage[0] / stage[4], 3), "TensorGEMM": round(stage[2] / stage[4], 3),
             "OutputTran": round(stage[3] / stage[4], 3)}
    common = {"stack_roofline_ms": round(agg["roof_ms"], 5), "stack_frac_of_roofline": round(agg["roof_ms"] / ms_step, 4),
              "share_of_step": share}
    if agg["direct_ms"] > agg["gemm_ms"]:
        ach = agg["direct_flops"] / (agg["direct_ms"] / 1e3) / 1e12
        roofline = {
            "kernel": "direct_tc_kernel (+ its layout pass), one launch pair per layer",
            "bound": "tensor", "achieved": round(ach, 1), "peak": TF32_LIBRARY_TFLOPS, "unit": "TFLOP/s",
            "frac": round(ach / TF32_LIBRARY_TFLOPS, 4),
            "peak_source": "TF32 library GEMM (8192^3) measured on a B200",
            "frac_of_half_bf16_peak": round(ach / (bf16_peak / 2.0), 4), "half_bf16_peak": round(bf16_peak / 2.0, 1),
            "traffic": None, "algorithmic_flops_per_launch": agg["direct_flops"] / agg["n_direct"],
            "avg_launch_ms": agg["direct_ms"] / agg["n_direct"],
            "layers_direct": agg["n_direct"], "layers_winograd": agg["n_wino"], **common}
    else:
        nl = max(agg["n_wino"], 1)
        gemm_tflops = agg["gemm_flops"] / (agg["gemm_ms"] / 1e3) / 1e12
        gemm_gbs = agg["gemm_bytes"] / (agg["gemm_ms"] / 1e3) / 1e9
        # the arithmetic the Winograd layers of this run use ("tf32" runs them in the split arithmetic)
        gemm_mode = {"fp32": "fp32", "3xtf32": "3xtf32", "tf32": "3xtf32", "tf32-unbounded": "tf32", "tf32-u16": "tf32"}[args.mode]
        mode_peak = peak_tflops[gemm_mode]
        t_math = agg["gemm_flops"] / (mode_peak * 1e12)
        t_hbm = agg["gemm_bytes"] / (hbm_peak * 1e9)
        math_bound = t_math >= t_hbm  # which of the two bounds binds the TensorGEMM launches of this workload
        roofline = {
            "kernel": "TensorGEMM (64 batched U*V products, one launch per layer)",
            "bound": ("math" if gemm_mode == "fp32" else "tensor") if math_bound else "hbm",
            "achieved": round(gemm_tflops if math_bound else gemm_gbs, 2),
            "peak": round(mode_peak, 2) if math_bound else hbm_peak,
            "unit": "TFLOP/s" if math_bound else "GB/s",
            "frac": round((gemm_tflops / mode_peak) if math_bound else (gemm_gbs / hbm_peak), 4),
            "peak_source": (f"{sms.value} SMs x 128 FP32 lanes x 2 x {sm_mhz:.0f} MHz (median SM clock sampled while the "
                            f"kernels ran); a library SGEMM of 8192^3 reaches {FP32_LIBRARY_TFLOPS} TFLOP/s"
                            if math_bound and gemm_mode == "fp32" else
                            "TF32 library GEMM (8192^3) measured on a B200" + (" / 3 passes" if gemm_mode == "3xtf32" else "")
                            if math_bound else f"copy bandwidth of MEASURED_PEAKS.json, of {peak_kind}"),
            "traffic": NCU_GEMM_TRAFFIC_BYTES_DEFAULT if (args.layers == "vgg16" and args.batch == 64 and world == 1 and
                                                          args.mode == "fp32" and args.algo == "winograd" and not args.chain) else None,
            "algorithmic_flops_per_launch": agg["gemm_flops"] / nl, "algorithmic_bytes_per_launch": agg["gemm_bytes"] / nl,
            "avg_launch_ms": agg["gemm_ms"] / nl,
            "winograd_domain_tflops": round(gemm_tflops, 2), "operand_gbs": round(gemm_gbs, 1),
            "the_other_bound": {"hbm_frac": round(gemm_gbs / hbm_peak, 4), "math_frac": round(gemm_tflops / mode_peak, 4)},
            **common}
        if gemm_mode != "fp32":  # the same fraction against half of the measured bf16 GEMM throughput
            roofline["frac_of_half_bf16_peak"] = round(gemm_tflops / (bf16_peak / 2.0 / (3 if gemm_mode == "3xtf32" else 1)), 4)

    line = None
    if rank == 0:
        value = total_flops / (ms_step / 1e3) / 1e9
        line = {
            "metric": "conv GFLOP/s (direct-equiv), VGG-16 conv stack", "value": round(value, 1), "unit": "GFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 4),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": {"fp32": "f32", "3xtf32": "3xtf32", "tf32": "tf32 (3xtf32 where one pass misses 3e-3)",
                      "tf32-unbounded": "tf32", "tf32-u16": "tf32 (fp16 filter)"}[args.mode],
            "data": "synthetic",
            "config": {"workload": workload,
                       "images_per_gpu": n,
                       "algorithm": {"winograd": "winograd F(6x6,3x3)", "direct": "direct convolution on the tensor cores",
                                     "auto": "per layer: winograd F(6x6,3x3) or direct convolution on the tensor cores"}[args.algo],
                       "math_mode": args.mode,
                       "launch": "all layers of a step replayed as one CUDA graph",
                       "chain": bool(args.chain),
                       "tuning": ("Tuning() per layer before the timed region (block shapes by measured device time, the "
                                  "reference's -tn tuning)" if args.tuning else "no_tuning (launcher heuristics)"),
                       "parallelism": f"images sharded over {world} GPU(s), no collective in the data path; barrier and "
                                      f"max-over-ranks through the library's communicator",
                       "l2": f"inputs larger than L2: the stack touches {stack.footprint / 1e6:.0f} MB per step and GPU"},
            "repeat_stats": repeat_stats(times, args.steps),
            "e2e": {"value": round(total_flops / (e2e_ms / 1e3) / 1e9, 1), "unit": "GFLOP/s",
                    "h2d_bytes_per_step": stack.h2d * world, "d2h_bytes_per_step": stack.d2h * world,
                    "ms_per_step": round(e2e_ms, 4)},
            "gpu_launches": launches * args.steps * world,
            "clocks": clocks,
            "roofline": roofline,
            "layers": per_layer,
        }
        if copy_bw is not None:
            line["e2e"]["plain_copy_gbs_per_rank"] = [{"rank": r, "h2d": round(float(u), 1), "d2h": round(float(d), 1)}
                                                      for r, (u, d) in enumerate(copy_bw)]
    stack.close()

    # ---- sub-records: the same images in the TF32 mode; the batch-1 stack (one GPU) -----------------------------
    subs = {}
    if not args.no_subrecords and args.mode == "fp32" and not args.chain:
        for name, mode, algo in (("tf32", "tf32", "auto"), ("3xtf32", "3xtf32", "winograd")):
            s = Stack(fc, ctx, layers, n, n0, mode, algo, host=False, tune=args.tuning)
            first, many = measure_stack(comm, ctx, s, args, 4)
            rows, _ = s.per_layer(max(3, args.steps), hbm_peak, peak_tflops)
            subs[name] = {"math_mode": mode, "algorithm": algo, "value": round(total_flops / first / 1e6, 1),
                          "unit": "GFLOP/s", "ms_per_step": round(first, 4), "repeat_stats": repeat_stats(many, args.steps),
                          "tolerance": "rel-L2 <= 3e-3 on every layer" if mode == "tf32" else
                                       "rel-L2 <= 1e-5 (see tests); the `math` of a layer says whether it ran the split "
                                       "tensor-core arithmetic or, with at most 64 input channels, the fp32 kernels",
                          "layers": [{k: r[k] for k in ("layer", "algo", "math", "ms", "frac_of_roofline", "bound")} for r in rows]}
            s.close()
        if world == 1:
            s = Stack(fc, ctx, layers, 1, 0, "fp32", "winograd", tune=args.tuning)
            first, many = measure_stack(comm, ctx, s, args, 24)
            e2e1 = measure_e2e(comm, ctx, s, args.steps)
            rows, agg1 = s.per_layer(max(3, args.steps), hbm_peak, peak_tflops)
            f1 = sum(layer_flops(1, c, k, h) for c, k, h in layers)
            subs["batch1"] = {"workload": f"{workload_name}, batch 1, one GPU", "math_mode": "fp32", "algorithm": "winograd",
                              "value": round(f1 / first / 1e6, 1), "unit": "GFLOP/s", "ms_per_step": round(first, 5),
                              "repeat_stats": repeat_stats(many, args.steps),
                              "e2e": {"value": round(f1 / e2e1 / 1e6, 1), "unit": "GFLOP/s", "h2d_bytes_per_step": s.h2d,
                                      "d2h_bytes_per_step": s.d2h, "ms_per_step": round(e2e1, 4)},
                              "stack_frac_of_roofline": round(agg1["roof_ms"] / first, 4),
                              "layers": [{k: r[k] for k in ("layer", "ms", "frac_of_roofline", "bound")} for r in rows]}
            s.close()
    if line is not None:
        if subs:
            line["sub_records"] = subs
        if not args.no_cpu_baseline and world == 1:
            threads = os.cpu_count() or 1
            images = max(1, min(args.batch, args.ref_images))
            sec, err = reference_cpu_pass(layers, images, threads)
            base = {"unit": "GFLOP/s", "cores": threads, "kind": "reference"}
            if sec is not None:
                f = sum(layer_flops(images, c, k, h) for c, k, h in layers)
                line["cpu_baseline"] = {"value": round(f / sec / 1e9, 2), **base,
                                        "sample": f"{images} of the {args.batch} images through all {len(layers)} layers with "
                                                  f"the reference's winoF63_v1_multi (NEON emulated via a vector-type "
                                                  f"stand-in header), all host threads"}
            else:
                line["cpu_baseline"] = {"value": None, **base, "sample": err}
    comm.barrier()
    comm.close()
    if line is not None:
        print(json.dumps(line))


if __name__ == "__main__":
    main()

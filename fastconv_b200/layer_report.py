"""Per-layer report over the benchmark configurations: VGG-16, ResNet-50 v1.5 and the wide single-image sweep.

    python -m fastconv_b200.layer_report --set resnet50 --mode fp32 [--batch N] [--tune] [--iters 50] [--only I]
                                         [--algo auto|winograd|im2col|direct]

Every layer is planned with `-a auto` unless --algo says otherwise (select_algorithm of ConvTest.cpp:318-331,
1x1 stride 1 routed to the implicit GEMM), run `iters` times back to back on device-resident data and timed with CUDA events; one
JSON line per layer carries the algorithm, milliseconds, direct-equivalent GFLOP/s and the fraction of
the layer's roofline  max(flops / peak, bytes / HBM bandwidth)  with
    Winograd:  flops = 2*64*T*C*K,  bytes = 4*(N*C*H*W + 64*C*K + N*K*OH*OW)
    im2col:    flops = 2*N*K*C*R*S*OH*OW,  bytes = 4*(N*C*H*W + K*C*R*S + N*K*OH*OW)
Peaks: HBM from MEASURED_PEAKS.json (copy bandwidth); FP32 = SMs x 128 lanes x 2 flop x the maximum SM clock
(74.5 TFLOP/s on a B200; a library SGEMM of 8192^3 reaches 63.7); TF32 759.9 TFLOP/s measured with an 8192^3
library GEMM on a B200, 3xTF32 a third of it.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
from pathlib import Path

import numpy as np

from . import _lib, synth
from .layers import Context, make_desc

ROOT = Path(__file__).resolve().parents[1]

# ic, oc, hw, k, stride, pad
VGG16 = [(3, 64, 224, 3, 1, 1), (64, 64, 224, 3, 1, 1), (64, 128, 112, 3, 1, 1), (128, 128, 112, 3, 1, 1),
         (128, 256, 56, 3, 1, 1), (256, 256, 56, 3, 1, 1), (256, 256, 56, 3, 1, 1), (256, 512, 28, 3, 1, 1),
         (512, 512, 28, 3, 1, 1), (512, 512, 28, 3, 1, 1), (512, 512, 14, 3, 1, 1), (512, 512, 14, 3, 1, 1),
         (512, 512, 14, 3, 1, 1)]
RESNET50 = [(3, 64, 224, 7, 2, 3),
            (64, 64, 56, 1, 1, 0), (64, 64, 56, 3, 1, 1), (64, 256, 56, 1, 1, 0), (256, 64, 56, 1, 1, 0),
            (256, 128, 56, 1, 1, 0), (128, 128, 56, 3, 2, 1), (256, 512, 56, 1, 2, 0),
            (128, 128, 28, 3, 1, 1), (128, 512, 28, 1, 1, 0), (512, 128, 28, 1, 1, 0),
            (512, 256, 28, 1, 1, 0), (256, 256, 28, 3, 2, 1), (512, 1024, 28, 1, 2, 0),
            (256, 256, 14, 3, 1, 1), (256, 1024, 14, 1, 1, 0), (1024, 256, 14, 1, 1, 0),
            (1024, 512, 14, 1, 1, 0), (512, 512, 14, 3, 2, 1), (1024, 2048, 14, 1, 2, 0),
            (512, 512, 7, 3, 1, 1), (512, 2048, 7, 1, 1, 0), (2048, 512, 7, 1, 1, 0)]
WIDE = [(c, c, h, 3, 1, 1) for c in (512, 1024, 2048) for h in (14, 28, 56)]
SETS = {"vgg16": VGG16, "resnet50": RESNET50, "wide": WIDE}


FP32_PEAK_TFLOPS = 148 * 128 * 2 * 1965e-6  # replaced by the context's own SM count and clock in main()


def peaks(mode: str):
    """HBM GB/s (measured copy bandwidth when the file is there) and the arithmetic peak of the mode in TFLOP/s:
    FP32 from the SM count and maximum clock, TF32 759.9 measured with an 8192^3 library GEMM on a B200, 3xTF32 a
    third of TF32."""
    hbm = 6650.0
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        hbm = float(json.loads(p.read_text())["hbm_gbs"])
    flops = {"fp32": FP32_PEAK_TFLOPS, "tf32": 759.9, "3xtf32": 759.9 / 3, "tf32-unbounded": 759.9, "tf32-u16": 759.9}[mode]
    return hbm, flops


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--set", default="resnet50", choices=sorted(SETS))
    ap.add_argument("--mode", default="fp32", choices=["fp32", "3xtf32", "tf32", "tf32-unbounded", "tf32-u16"],
                    help="tf32 keeps rel-L2 <= 3e-3 on every layer (direct kernel, or Winograd in the split arithmetic); "
                         "tf32-unbounded also runs one TF32 pass through Winograd (6.4e-3); tf32-u16 does the same "
                         "over a filter stored as fp16")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--tune", action="store_true", help="run Tuning() (timed configuration search) before measuring")
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--only", type=int, default=None, help="index of the one layer of the set to run")
    ap.add_argument("--algo", default="auto", choices=["auto", "winograd", "im2col", "direct"],
                    help="-a of ConvTest: force one path for every layer that it can run")
    args = ap.parse_args()

    lib = _lib.load()
    hbm, peak_tf = peaks(args.mode)
    n = args.batch
    total_ms = total_flops = 0.0
    with Context(args.device, arena_bytes=12 << 30) as ctx:
        global FP32_PEAK_TFLOPS
        sms, mhz = C.c_int(), C.c_int()
        _lib.check(lib.fc_context_info(ctx.handle, C.byref(sms), C.byref(mhz)), "fc_context_info")
        FP32_PEAK_TFLOPS = sms.value * 128 * 2 * mhz.value * 1e-6
        for idx, (ic, oc, hw, k, s, p) in enumerate(SETS[args.set]):
            if args.only is not None and idx != args.only:
                continue
            desc = make_desc(n, ic, hw, hw, oc, k, k, s, s, p, p, p, p)
            w = synth.conv_weights(oc, ic, k, k, 2000 + idx)
            x = synth.conv_input(n, ic, hw, hw, 1000 + idx)
            h = C.c_void_p()
            want = _lib.ALGO_NAMES[args.algo]
            _lib.check(lib.fc_conv_create(ctx.handle, C.byref(desc), want, _lib.MODE_NAMES[args.mode],
                                          C.c_void_p(w.ctypes.data), C.byref(h)), "fc_conv_create")
            if args.tune:
                _lib.check(lib.fc_conv_tune(h, 10, 0), "fc_conv_tune")
            d_in, d_out = C.c_void_p(), C.c_void_p()
            _lib.check(lib.fc_conv_device_buffers(h, C.byref(d_in), C.byref(d_out)), "fc_conv_device_buffers")
            ctx.upload(x, d_in.value)
            ms = C.c_float()
            _lib.check(lib.fc_conv_time_device(h, d_in, d_out, 5, args.iters, C.byref(ms)), "fc_conv_time_device")
            algo, resolved = C.c_int(), C.c_int()
            lib.fc_conv_algorithm(h, C.byref(algo))
            lib.fc_conv_math_mode(h, C.byref(resolved))  # what "tf32" turned into for this layer
            mode_name = _lib.MODE_LABELS[resolved.value]
            hbm, peak_tf = peaks(mode_name)
            oh = (hw + 2 * p - k) // s + 1
            direct = 2.0 * n * oc * ic * k * k * oh * oh
            if algo.value == _lib.ALGO_WINOGRAD:
                tiles = n * ((oh + 5) // 6) ** 2
                u_bytes = 2.0 if mode_name == "tf32-u16" else 4.0  # the filter as the kernel reads it
                flops, nbytes = 2.0 * 64 * tiles * ic * oc, 4.0 * (n * ic * hw * hw + n * oc * oh * oh) + u_bytes * 64 * ic * oc
            else:
                flops, nbytes = direct, 4.0 * (n * ic * hw * hw + oc * ic * k * k + n * oc * oh * oh)
            roof_ms = max(flops / (peak_tf * 1e12), nbytes / (hbm * 1e9)) * 1e3
            print(json.dumps({
                "layer": f"{ic}->{oc}@{hw} {k}x{k}s{s}", "batch": n, "mode": mode_name,
                "algo": {v: k for k, v in _lib.ALGO_NAMES.items()}[algo.value], "ms": round(ms.value, 5),
                "gflops_direct_equiv": round(direct / ms.value / 1e6, 1), "roofline_ms": round(roof_ms, 5),
                "frac_of_roofline": round(roof_ms / ms.value, 4),
                "bound": "hbm" if nbytes / (hbm * 1e9) >= flops / (peak_tf * 1e12) else "math"}), flush=True)
            total_ms += ms.value
            total_flops += direct
            lib.fc_conv_destroy(h)
    print(json.dumps({"set": args.set, "mode": args.mode, "batch": n, "total_ms": round(total_ms, 4),
                      "gflops_direct_equiv": round(total_flops / total_ms / 1e6, 1)}))


if __name__ == "__main__":
    main()

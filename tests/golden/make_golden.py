"""Generates tests/golden/fastconv_golden.npz from the FastConv reference itself.

Run where the reference tree is present (its location is the REF variable of oracle/Makefile):

    make -C oracle ref [REF=...] && python tests/golden/make_golden.py

It loads oracle/_ref/libfastconv_ref.so -- the reference's own sources compiled through the NEON
stand-in header (oracle/Makefile) -- and records, for seeded inputs from fastconv_b200.synth:

  * the output of the reference Winograd driver winoF63_v1_multi (1 OpenMP thread: with more
    threads than output-channel register blocks the reference's OpenMP driver mis-computes, e.g.
    oc <= 4 at 8 threads, so the pins are taken single-threaded),
  * the output of the reference's naive layers (ConvNaiveLayer, both variants),
  * SHA-256 digests of the matrices gathered by ConvIm2colLayer::im2col() and im2col_v1(),
  * the output of the reference's im2col layer -- im2col_v1() then sgemm() -- with the constructor's default
    blocking on one thread: GEMM_v2 with the 8x8 register kernel and its corner kernels, across several kc and
    nc blocks, and the scalar GEMM that the reference switches to when M, N and K are all at most 32.

Small cases are stored whole; the two full-size layers are stored as digests plus a strided sample.
The reference ships no golden vectors of its own, so these files are the pins.
"""
from __future__ import annotations

import ctypes as C
import hashlib
import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from fastconv_b200 import synth  # noqa: E402

WINO_SMALL = [  # ic, oc, ih, iw, pad
    (1, 1, 6, 6, 1), (3, 5, 7, 9, 1), (4, 4, 1, 1, 1), (8, 8, 12, 12, 1), (5, 3, 6, 6, 0), (17, 6, 23, 20, 1),
    (6, 7, 13, 8, 2), (32, 30, 23, 23, 1), (64, 64, 14, 14, 1), (3, 64, 20, 20, 1), (9, 2, 5, 31, 1),
]
WINO_LARGE = [(256, 256, 56, 56, 1), (512, 512, 14, 14, 1), (64, 64, 112, 112, 1)]
GENERAL = [  # ic, oc, ih, iw, kh, kw, sh, sw, pad
    (3, 8, 30, 30, 7, 7, 2, 2, 3), (16, 12, 14, 14, 1, 1, 1, 1, 0), (8, 8, 15, 15, 3, 3, 2, 2, 1),
    (12, 6, 14, 14, 1, 1, 2, 2, 0), (5, 7, 9, 11, 3, 3, 1, 1, 1), (4, 4, 8, 8, 5, 3, 1, 2, 2),
]


SGEMM = [  # ic, oc, ih, iw, kh, kw, sh, sw, pad -- M % 8 corners, N % 8 tails, K > kc = 384, N > nc = 256, tiny
    (3, 8, 30, 30, 7, 7, 2, 2, 3), (16, 12, 14, 14, 1, 1, 1, 1, 0), (8, 8, 15, 15, 3, 3, 2, 2, 1),
    (12, 6, 14, 14, 1, 1, 2, 2, 0), (5, 7, 9, 11, 3, 3, 1, 1, 1), (4, 4, 8, 8, 5, 3, 1, 2, 2),
    (100, 37, 13, 13, 3, 3, 1, 1, 1), (130, 9, 10, 10, 5, 5, 1, 1, 2), (64, 19, 23, 17, 1, 1, 1, 1, 0),
    (2, 3, 4, 4, 3, 3, 1, 1, 1), (3, 32, 6, 5, 3, 3, 1, 1, 1), (32, 5, 4, 8, 1, 1, 1, 1, 0), (33, 5, 4, 8, 1, 1, 1, 1, 0),
]
SGEMM_LARGE = [(3, 64, 224, 224, 7, 7, 2, 2, 3), (256, 128, 28, 28, 3, 3, 2, 2, 1), (512, 128, 28, 28, 1, 1, 1, 1, 0)]


def P(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main() -> None:
    ref = C.CDLL(str(ROOT / "oracle" / "_ref" / "libfastconv_ref.so"))
    arrays, meta = {}, {"wino": [], "wino_large": [], "general": []}
    for idx, (ic, oc, ih, iw, pad) in enumerate(WINO_SMALL + WINO_LARGE):
        x = synth.conv_input(1, ic, ih, iw, 1000 + idx)
        w = synth.conv_weights(oc, ic, 3, 3, 2000 + idx)
        oh, ow = ih + 2 * pad - 2, iw + 2 * pad - 2
        out = np.zeros((oc, oh, ow), np.float32)
        naive = np.zeros_like(out)
        assert ref.ref_wino_f63_forward(P(out), P(x), P(w), ic, oc, ih, iw, pad, 1, 50, 140, 64, None) == 0
        assert ref.ref_naive_conv3x3(P(naive), P(x), P(w), ic, oc, ih, iw, pad) == 0
        rec = {"idx": idx, "ic": ic, "oc": oc, "ih": ih, "iw": iw, "pad": pad, "seed_in": 1000 + idx,
               "seed_w": 2000 + idx, "sha_in": sha(x), "sha_w": sha(w), "sha_wino": sha(out), "sha_naive": sha(naive)}
        if idx < len(WINO_SMALL):
            arrays[f"wino_{idx}"] = out
            arrays[f"naive_{idx}"] = naive
            meta["wino"].append(rec)
        else:
            arrays[f"wino_sample_{idx}"] = out.ravel()[::997].copy()
            meta["wino_large"].append(rec)
    for j, (ic, oc, ih, iw, kh, kw, sh, sw, pad) in enumerate(GENERAL):
        idx = 100 + j
        x = synth.conv_input(1, ic, ih, iw, 1000 + idx)
        w = synth.conv_weights(oc, ic, kh, kw, 2000 + idx)
        oh, ow = (ih + 2 * pad - kh) // sh + 1, (iw + 2 * pad - kw) // sw + 1
        naive = np.zeros((oc, oh, ow), np.float32)
        assert ref.ref_naive_conv_general(P(naive), P(x), P(w), ic, oc, ih, iw, kh, kw, sh, sw, pad, pad, pad, pad) == 0
        g0 = np.zeros((ic * kh * kw, oh * ow), np.float32)
        g1 = np.zeros_like(g0)
        assert ref.ref_im2col(P(g0), P(x), ic, ih, iw, kh, kw, sh, sw, pad, pad, pad, pad, 0) == 0
        assert ref.ref_im2col(P(g1), P(x), ic, ih, iw, kh, kw, sh, sw, pad, pad, pad, pad, 1) == 0
        assert np.array_equal(g0, g1), "im2col() and im2col_v1() of the reference disagree"
        arrays[f"general_naive_{idx}"] = naive
        meta["general"].append({"idx": idx, "ic": ic, "oc": oc, "ih": ih, "iw": iw, "kh": kh, "kw": kw, "sh": sh,
                                "sw": sw, "pad": pad, "seed_in": 1000 + idx, "seed_w": 2000 + idx, "sha_in": sha(x),
                                "sha_w": sha(w), "sha_gather": sha(g0), "sha_naive": sha(naive)})
    meta["sgemm"], meta["sgemm_large"] = [], []
    for j, (ic, oc, ih, iw, kh, kw, sh, sw, pad) in enumerate(SGEMM + SGEMM_LARGE):
        idx = 200 + j
        x = synth.conv_input(1, ic, ih, iw, 1000 + idx)
        w = synth.conv_weights(oc, ic, kh, kw, 2000 + idx)
        oh, ow = (ih + 2 * pad - kh) // sh + 1, (iw + 2 * pad - kw) // sw + 1
        out = np.zeros((oc, oh, ow), np.float32)
        assert ref.ref_im2col_sgemm(P(out), P(x), P(w), ic, oc, ih, iw, kh, kw, sh, sw, pad, pad, pad, pad, 1) == 0
        rec = {"idx": idx, "ic": ic, "oc": oc, "ih": ih, "iw": iw, "kh": kh, "kw": kw, "sh": sh, "sw": sw, "pad": pad,
               "seed_in": 1000 + idx, "seed_w": 2000 + idx, "sha_in": sha(x), "sha_w": sha(w), "sha_sgemm": sha(out)}
        if j < len(SGEMM):
            arrays[f"sgemm_{idx}"] = out
            meta["sgemm"].append(rec)
        else:
            arrays[f"sgemm_sample_{idx}"] = out.ravel()[::997].copy()
            meta["sgemm_large"].append(rec)
    out_path = Path(__file__).with_name("fastconv_golden.npz")
    np.savez_compressed(out_path, meta=np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8), **arrays)
    print(out_path, out_path.stat().st_size, "bytes")


if __name__ == "__main__":
    main()

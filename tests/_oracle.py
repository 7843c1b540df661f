"""Test-side access to the CPU oracle (oracle/liboracle.so) and, when built, the reference library."""
from __future__ import annotations

import ctypes as C
import json
import subprocess
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[1]
_fp = C.POINTER(C.c_float)
_dp = C.POINTER(C.c_double)


def P(a):
    return a.ctypes.data_as(_fp)


def f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class Oracle:
    def __init__(self):
        path = ROOT / "oracle" / "liboracle.so"
        if not path.exists():
            subprocess.run(["make", "-C", str(ROOT / "oracle"), "oracle"], check=True, capture_output=True)
        self.lib = C.CDLL(str(path))

    @staticmethod
    def out_hw(ih, iw, kh, kw, sh, sw, pl, pr, pt, pb):
        return (ih + pt + pb - kh) // sh + 1, (iw + pl + pr - kw) // sw + 1

    def wino_forward(self, x, w, pad=1):
        x, w = f32(x), f32(w)
        n, ic, ih, iw = x.shape
        oc = w.shape[0]
        out = np.zeros((n, oc, ih + 2 * pad - 2, iw + 2 * pad - 2), np.float32)
        assert self.lib.oracle_wino_forward(P(out), P(x), P(w), n, ic, oc, ih, iw, pad) == 0
        return out

    def filter_transform(self, w, icp=None):
        w = f32(w)
        oc, ic = w.shape[:2]
        icp = icp or ic
        U = np.zeros((64, oc, icp), np.float32)
        self.lib.oracle_wino_filter_transform(P(U), P(w), oc, ic, icp)
        return U

    def input_transform(self, x, pad, tp=None, icp=None):
        x = f32(x)
        n, ic, ih, iw = x.shape
        th, tw = (ih + 2 * pad - 2 + 5) // 6, (iw + 2 * pad - 2 + 5) // 6
        tiles = n * th * tw
        tp, icp = tp or tiles, icp or ic
        V = np.zeros((64, tp, icp), np.float32)
        self.lib.oracle_wino_input_transform(P(V), P(x), n, ic, ih, iw, pad, tp, icp)
        return V

    def wino_gemm(self, U, V, oc, ic, tiles):
        U, V = f32(U), f32(V)
        M = np.zeros((64, oc, V.shape[1]), np.float32)
        self.lib.oracle_wino_gemm(P(M), P(U), P(V), oc, ic, tiles, U.shape[2], V.shape[1], M.shape[2])
        return M

    def output_transform(self, M, n, oc, oh, ow):
        M = f32(M)
        out = np.zeros((n, oc, oh, ow), np.float32)
        self.lib.oracle_wino_output_transform(P(out), P(M), n, oc, oh, ow, M.shape[2])
        return out

    def im2col(self, x, kh, kw, sh, sw, pl, pr, pt, pb):
        x = f32(x)
        ic, ih, iw = x.shape[-3:]
        oh, ow = self.out_hw(ih, iw, kh, kw, sh, sw, pl, pr, pt, pb)
        B = np.zeros((ic * kh * kw, oh * ow), np.float32)
        self.lib.oracle_im2col(P(B), P(x), ic, ih, iw, kh, kw, sh, sw, pl, pr, pt, pb, None, None)
        return B

    def _conv(self, fn, x, w, sh, sw, pl, pr, pt, pb, dtype=np.float32):
        x, w = f32(x), f32(w)
        n, ic, ih, iw = x.shape
        oc, _, kh, kw = w.shape
        oh, ow = self.out_hw(ih, iw, kh, kw, sh, sw, pl, pr, pt, pb)
        out = np.zeros((n, oc, oh, ow), dtype)
        ptr = out.ctypes.data_as(_dp if dtype == np.float64 else _fp)
        assert fn(ptr, P(x), P(w), n, ic, oc, ih, iw, kh, kw, sh, sw, pl, pr, pt, pb) == 0
        return out

    def im2col_gemm_forward(self, x, w, sh=1, sw=1, pl=0, pr=0, pt=0, pb=0):
        return self._conv(self.lib.oracle_im2col_gemm_forward, x, w, sh, sw, pl, pr, pt, pb)

    def naive_conv(self, x, w, sh=1, sw=1, pl=0, pr=0, pt=0, pb=0):
        return self._conv(self.lib.oracle_naive_conv, x, w, sh, sw, pl, pr, pt, pb)

    def direct_f64(self, x, w, sh=1, sw=1, pl=0, pr=0, pt=0, pb=0):
        return self._conv(self.lib.oracle_direct_conv_f64, x, w, sh, sw, pl, pr, pt, pb, dtype=np.float64)

    def diff(self, a, b):
        a, b = f32(a).ravel(), f32(b).ravel()
        self.lib.oracle_diff.restype = C.c_float
        return float(self.lib.oracle_diff(P(a), P(b), a.size))


class Reference:
    """oracle/_ref/libfastconv_ref.so: the unmodified reference sources (see oracle/Makefile)."""

    def __init__(self, lib):
        self.lib = lib

    @classmethod
    def try_load(cls):
        path = ROOT / "oracle" / "_ref" / "libfastconv_ref.so"
        if not path.exists():
            return None
        return cls(C.CDLL(str(path)))

    def wino_forward(self, x, w, pad=1, threads=1):
        x, w = f32(x), f32(w)
        ic, ih, iw = x.shape[-3:]
        oc = w.shape[0]
        out = np.zeros((oc, ih + 2 * pad - 2, iw + 2 * pad - 2), np.float32)
        assert self.lib.ref_wino_f63_forward(P(out), P(x), P(w), ic, oc, ih, iw, pad, threads, 50, 140, 64, None) == 0
        return out

    def naive3x3(self, x, w, pad=1):
        x, w = f32(x), f32(w)
        ic, ih, iw = x.shape[-3:]
        oc = w.shape[0]
        out = np.zeros((oc, ih + 2 * pad - 2, iw + 2 * pad - 2), np.float32)
        assert self.lib.ref_naive_conv3x3(P(out), P(x), P(w), ic, oc, ih, iw, pad) == 0
        return out

    def im2col_sgemm(self, x, w, sh, sw, pad):
        """im2col_v1() + sgemm() of the reference's im2col layer on one thread, C cleared first."""
        x, w = f32(x), f32(w)
        ic, ih, iw = x.shape[-3:]
        oc, _, kh, kw = w.shape
        oh, ow = (ih + 2 * pad - kh) // sh + 1, (iw + 2 * pad - kw) // sw + 1
        out = np.zeros((oc, oh, ow), np.float32)
        assert self.lib.ref_im2col_sgemm(P(out), P(x), P(w), ic, oc, ih, iw, kh, kw, sh, sw, pad, pad, pad, pad, 1) == 0
        return out

    def im2col(self, x, kh, kw, sh, sw, pad, which=0):
        x = f32(x)
        ic, ih, iw = x.shape[-3:]
        oh, ow = (ih + 2 * pad - kh) // sh + 1, (iw + 2 * pad - kw) // sw + 1
        B = np.zeros((ic * kh * kw, oh * ow), np.float32)
        assert self.lib.ref_im2col(P(B), P(x), ic, ih, iw, kh, kw, sh, sw, pad, pad, pad, pad, which) == 0
        return B


def order_noise(oracle, x, w, want, pad=1):
    """How far the reference's own Winograd output moves when only the ORDER of its input channels changes: rel-L2
    between `want` = oracle(x, w) and the oracle run on the same layer with its channels permuted (same products,
    same exact sum, another fp32 accumulation order).  No implementation with a summation order of its own can be
    closer to the reference than this; tests of the 3xTF32 mode use max(1e-5, 1.25 * order_noise) as their bound."""
    perm = np.random.default_rng(5).permutation(x.shape[1])
    moved = oracle.wino_forward(np.ascontiguousarray(x[:, perm]), np.ascontiguousarray(w[:, perm]), pad)
    return rel_l2(moved, want)


def unpack_filter(packed, oc, ic):
    """The library keeps the transformed filter in contiguous boxes of 128 output channels x 32 input
    channels: box (p, ocb, kb) at ((p*n_ocb + ocb)*n_kb + kb)*4096 floats, element (oc%128)*32 + ic%32.
    Returns the plain [64][oc][ic] view the oracle uses."""
    n_ocb, n_kb = (oc + 127) // 128, (ic + 31) // 32
    boxes = np.asarray(packed, np.float32).reshape(64, n_ocb, n_kb, 128, 32)
    plain = boxes.transpose(0, 1, 3, 2, 4).reshape(64, n_ocb * 128, n_kb * 32)
    assert not plain[:, oc:, :].any() and not plain[:, :, ic:].any(), "padding of the packed filter must be zero"
    return np.ascontiguousarray(plain[:, :oc, :ic])


def load_golden():
    z = np.load(ROOT / "tests" / "golden" / "fastconv_golden.npz")
    meta = json.loads(bytes(z["meta"]).decode())
    return meta, z


def rel_l2(a, b):
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-300))


def max_abs_rel(a, b):
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    return float(np.max(np.abs(a - b)) / max(np.max(np.abs(b)), 1e-300))

"""The CPU oracle against the pins taken from the reference (tests/golden) and, when the reference
library is built in this checkout, against the reference itself -- bit for bit."""
import hashlib

import numpy as np
import pytest

from _oracle import rel_l2
from fastconv_b200 import synth


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def _inputs(rec, kh=3, kw=3):
    x = synth.conv_input(1, rec["ic"], rec["ih"], rec["iw"], rec["seed_in"])
    w = synth.conv_weights(rec["oc"], rec["ic"], kh, kw, rec["seed_w"])
    assert sha(x) == rec["sha_in"] and sha(w) == rec["sha_w"], "synthetic generator drifted from the fixture"
    return x, w


def test_wino_oracle_matches_golden_small(oracle, golden):
    meta, z = golden
    assert len(meta["wino"]) >= 10
    for rec in meta["wino"]:
        x, w = _inputs(rec)
        got = oracle.wino_forward(x, w, rec["pad"])[0]
        want = z[f"wino_{rec['idx']}"]
        assert got.shape == want.shape
        assert np.array_equal(got, want), f"winograd oracle differs from the reference output for {rec}"
        assert sha(got) == rec["sha_wino"]


def test_naive_oracle_matches_golden_small(oracle, golden):
    meta, z = golden
    for rec in meta["wino"]:
        x, w = _inputs(rec)
        p = rec["pad"]
        got = oracle.naive_conv(x, w, 1, 1, p, p, p, p)[0]
        assert np.array_equal(got, z[f"naive_{rec['idx']}"])


def test_wino_oracle_matches_golden_full_size(oracle, golden):
    meta, z = golden
    for rec in meta["wino_large"]:
        x, w = _inputs(rec)
        got = oracle.wino_forward(x, w, rec["pad"])[0]
        assert sha(got) == rec["sha_wino"], f"full-size layer {rec['ic']}->{rec['oc']}@{rec['ih']}"
        assert np.array_equal(got.ravel()[::997], z[f"wino_sample_{rec['idx']}"])


def test_general_paths_match_golden(oracle, golden):
    meta, z = golden
    for rec in meta["general"]:
        x, w = _inputs(rec, rec["kh"], rec["kw"])
        p = rec["pad"]
        g = oracle.im2col(x[0], rec["kh"], rec["kw"], rec["sh"], rec["sw"], p, p, p, p)
        assert sha(g) == rec["sha_gather"], f"im2col index map differs from the reference for {rec}"
        naive = oracle.naive_conv(x, w, rec["sh"], rec["sw"], p, p, p, p)[0]
        assert np.array_equal(naive, z[f"general_naive_{rec['idx']}"])
        # the mirrored GEMM chain (one FMA per k) is a different rounding order than the naive
        # layer's (9-term partial sums), so the two agree to fp32 accuracy, not bitwise
        gemm = oracle.im2col_gemm_forward(x, w, rec["sh"], rec["sw"], p, p, p, p)[0]
        assert rel_l2(gemm, naive) < 2e-6


def test_sgemm_oracle_matches_golden(oracle, golden):
    """The one-FMA-per-k chain of the oracle (and the unfused chain of the M, N, K <= 32 case) against the output of
    the reference's own im2col_v1() + sgemm(): GEMM_v2 with its 8x8 register and corner kernels over several kc and
    nc blocks, and the scalar GEMM."""
    meta, z = golden
    assert len(meta["sgemm"]) >= 12 and len(meta["sgemm_large"]) >= 3
    for rec in meta["sgemm"] + meta["sgemm_large"]:
        x, w = _inputs(rec, rec["kh"], rec["kw"])
        p = rec["pad"]
        got = oracle.im2col_gemm_forward(x, w, rec["sh"], rec["sw"], p, p, p, p)[0]
        assert sha(got) == rec["sha_sgemm"], f"SGEMM chain differs from the reference for {rec}"
        key = f"sgemm_{rec['idx']}"
        if key in z:
            assert np.array_equal(got, z[key])
        else:
            assert np.array_equal(got.ravel()[::997], z[f"sgemm_sample_{rec['idx']}"])


@pytest.mark.parametrize("g", [(3, 8, 30, 7, 2, 3), (16, 12, 14, 1, 1, 0), (100, 37, 13, 3, 1, 1), (130, 9, 10, 5, 1, 2),
                               (64, 64, 56, 1, 1, 0), (2, 3, 4, 3, 1, 1), (3, 32, 6, 3, 1, 1), (33, 5, 5, 1, 1, 0),
                               (40, 50, 20, 3, 1, 1)])
def test_sgemm_oracle_bit_equal_to_reference_build(oracle, reference, g):
    if reference is None:
        pytest.skip("oracle/_ref is not built in this checkout (needs the reference tree)")
    ic, oc, hw, k, s, pad = g
    x = synth.conv_input(1, ic, hw, hw, 13)
    w = synth.conv_weights(oc, ic, k, k, 14)
    assert np.array_equal(oracle.im2col_gemm_forward(x, w, s, s, pad, pad, pad, pad)[0],
                          reference.im2col_sgemm(x[0], w, s, s, pad))


@pytest.mark.parametrize("shape", [(3, 5, 7, 9, 1), (8, 8, 12, 12, 1), (17, 6, 23, 20, 1), (5, 3, 6, 6, 0),
                                   (6, 7, 13, 8, 2), (4, 4, 1, 1, 1), (64, 48, 28, 28, 1), (128, 128, 14, 14, 1)])
def test_oracle_bit_equal_to_reference_build(oracle, reference, shape):
    if reference is None:
        pytest.skip("oracle/_ref is not built in this checkout (needs the reference tree)")
    ic, oc, ih, iw, pad = shape
    x = synth.conv_input(1, ic, ih, iw, 7)
    w = synth.conv_weights(oc, ic, 3, 3, 8)
    assert np.array_equal(oracle.wino_forward(x, w, pad)[0], reference.wino_forward(x, w, pad, threads=1))
    assert np.array_equal(oracle.naive_conv(x, w, 1, 1, pad, pad, pad, pad)[0], reference.naive3x3(x, w, pad))


@pytest.mark.parametrize("g", [(3, 30, 30, 7, 7, 2, 2, 3), (16, 14, 14, 1, 1, 1, 1, 0), (8, 15, 15, 3, 3, 2, 2, 1),
                               (5, 9, 11, 3, 3, 1, 1, 1), (2, 6, 5, 3, 3, 1, 1, 2)])
def test_im2col_oracle_bit_equal_to_reference_build(oracle, reference, g):
    if reference is None:
        pytest.skip("oracle/_ref is not built in this checkout (needs the reference tree)")
    ic, ih, iw, kh, kw, sh, sw, pad = g
    x = synth.conv_input(1, ic, ih, iw, 11)[0]
    mine = oracle.im2col(x, kh, kw, sh, sw, pad, pad, pad, pad)
    assert np.array_equal(mine, reference.im2col(x, kh, kw, sh, sw, pad, 0))
    assert np.array_equal(mine, reference.im2col(x, kh, kw, sh, sw, pad, 1))


def test_winograd_identity_against_fp64(oracle):
    """A^T[(G g G^T) . (B^T d B)]A equals the direct 3x3 convolution (checked in fp64 terms)."""
    for (ic, oc, ih, iw, pad) in [(1, 1, 6, 6, 1), (4, 3, 8, 8, 0), (16, 16, 20, 17, 1), (64, 32, 28, 28, 1)]:
        x = synth.conv_input(2, ic, ih, iw, 21)
        w = synth.conv_weights(oc, ic, 3, 3, 22)
        truth = oracle.direct_f64(x, w, 1, 1, pad, pad, pad, pad)
        assert rel_l2(oracle.wino_forward(x, w, pad), truth) < 5e-6


def test_oracle_stages_compose(oracle):
    ic, oc, ih, iw, pad, n = 5, 7, 13, 9, 1, 2
    x = synth.conv_input(n, ic, ih, iw, 31)
    w = synth.conv_weights(oc, ic, 3, 3, 32)
    U = oracle.filter_transform(w)
    V = oracle.input_transform(x, pad)
    M = oracle.wino_gemm(U, V, oc, ic, V.shape[1])
    out = oracle.output_transform(M, n, oc, ih, iw)
    assert np.array_equal(out, oracle.wino_forward(x, w, pad))
    # padding the reduction and tile axes with zeros does not change a single bit
    Up = oracle.filter_transform(w, icp=8)
    Vp = oracle.input_transform(x, pad, tp=16, icp=8)
    Mp = oracle.wino_gemm(Up, Vp, oc, 8, 16)
    assert np.array_equal(oracle.output_transform(Mp, n, oc, ih, iw), out)


def test_diff_matches_reference_definition(oracle):
    a = np.array([0.0, 1.0, 2.0, 3.0], np.float32)
    b = np.array([0.0, 1.000001, 2.5, 2.0], np.float32)
    assert abs(oracle.diff(a, b) - 0.75) < 1e-6
    assert oracle.diff(a, a) == 0.0

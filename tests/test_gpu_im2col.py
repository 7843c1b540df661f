"""Parity of the im2col / implicit-GEMM path: the gathered matrix is bit-exact with the reference's
index map -- as dumped by the inspection entry point AND as the forward kernels' own operand producers gather it
(identity weights turn a layer's output into its gathered matrix); the mirrored fp32 GEMM is bit-exact with the
oracle's one-FMA-per-k chain, which is pinned to the reference's sgemm() by the golden vectors."""
import hashlib

import numpy as np
import pytest

import fastconv_b200 as fc
from _oracle import max_abs_rel, rel_l2
from fastconv_b200 import synth

pytestmark = pytest.mark.gpu

CASES = [  # n, ic, oc, ih, iw, kh, kw, sh, sw, pad
    (1, 3, 8, 30, 30, 7, 7, 2, 2, 3), (1, 16, 12, 14, 14, 1, 1, 1, 1, 0), (1, 8, 8, 15, 15, 3, 3, 2, 2, 1),
    (1, 12, 6, 14, 14, 1, 1, 2, 2, 0), (2, 5, 7, 9, 11, 3, 3, 1, 1, 1), (1, 4, 4, 8, 8, 5, 3, 1, 2, 2),
    (3, 64, 130, 7, 7, 1, 1, 1, 1, 0), (1, 70, 65, 9, 9, 3, 3, 1, 1, 1), (1, 1, 1, 1, 1, 1, 1, 1, 1, 0),
    (2, 33, 17, 12, 10, 3, 3, 2, 2, 1), (1, 256, 64, 14, 14, 1, 1, 1, 1, 0),
]


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def make(ctx, x, w, sh, sw, pad, mode="fp32", ref=None, iters=1):
    n, ic, ih, iw = x.shape
    oc, _, kh, kw = w.shape
    return fc.ConvIm2colLayer(x, w, None, ref, ic, ih, iw, oc, kh, kw, sh, sw, pad, pad, pad, pad, 1, False, 1, iters,
                              batch=n, mode=mode, ctx=ctx)


@pytest.mark.parametrize("case", CASES)
def test_gather_bit_exact(ctx, oracle, case):
    n, ic, oc, ih, iw, kh, kw, sh, sw, pad = case
    x = synth.conv_input(n, ic, ih, iw, 5)
    w = synth.conv_weights(oc, ic, kh, kw, 6)
    layer = make(ctx, x, w, sh, sw, pad)
    for img in range(n):
        want = oracle.im2col(x[img], kh, kw, sh, sw, pad, pad, pad, pad)
        assert np.array_equal(layer.im2col(img), want)


def test_gather_matches_reference_digests(ctx, golden):
    meta, _ = golden
    for rec in meta["general"]:
        x = synth.conv_input(1, rec["ic"], rec["ih"], rec["iw"], rec["seed_in"])
        w = synth.conv_weights(rec["oc"], rec["ic"], rec["kh"], rec["kw"], rec["seed_w"])
        layer = make(ctx, x, w, rec["sh"], rec["sw"], rec["pad"])
        assert sha(layer.im2col(0)) == rec["sha_gather"], rec


@pytest.mark.parametrize("case", CASES)
def test_mirrored_gemm_bit_exact(ctx, oracle, case):
    n, ic, oc, ih, iw, kh, kw, sh, sw, pad = case
    x = synth.conv_input(n, ic, ih, iw, 15)
    w = synth.conv_weights(oc, ic, kh, kw, 16)
    layer = make(ctx, x, w, sh, sw, pad)
    assert layer.Init() == 1 and layer.Forward() == 1  # return values of im2colConv.cpp:234, :258
    want = oracle.im2col_gemm_forward(x, w, sh, sw, pad, pad, pad, pad)
    assert np.array_equal(layer.output_data, want)
    layer.release()


def test_mirrored_gemm_matches_reference_sgemm_vectors(ctx, golden):
    """Outputs of the reference's own im2col_v1() + sgemm() (GEMM_v2 with its 8x8 register kernels, and the scalar
    GEMM of the M, N, K <= 32 case), recorded in tests/golden: the CUDA layer reproduces them bit for bit."""
    meta, z = golden
    for rec in meta["sgemm"] + meta["sgemm_large"]:
        x = synth.conv_input(1, rec["ic"], rec["ih"], rec["iw"], rec["seed_in"])
        w = synth.conv_weights(rec["oc"], rec["ic"], rec["kh"], rec["kw"], rec["seed_w"])
        layer = make(ctx, x, w, rec["sh"], rec["sw"], rec["pad"])
        layer.Init()
        layer.Forward()
        assert sha(layer.output_data[0]) == rec["sha_sgemm"], rec
        layer.release()


def _tf32_exact(a):
    """Values with 10 explicit mantissa bits: a tensor-core product of such a value with 1.0 is exact."""
    return (np.ascontiguousarray(a, np.float32).view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32)


# n, ic, ih, iw, kh, kw, sh, sw, (left, right, top, bottom)
IDENTITY_SHAPES = {
    "3x3": (2, 8, 13, 11, 3, 3, 1, 1, (1, 1, 1, 1)),
    "5x3s2": (1, 6, 17, 14, 5, 3, 2, 2, (2, 1, 0, 2)),
    "7x7s2": (1, 3, 40, 36, 7, 7, 2, 2, (3, 3, 3, 3)),
    "few-pixels": (1, 64, 14, 14, 3, 3, 2, 2, (1, 1, 1, 1)),  # 49 pixels, K = 576: the gathered matrix is written once
}
# mode, bm, bn, variant (see fc_conv_set_kernel_config)
IDENTITY_KERNELS = (
    [("fp32", bm, bn, 1) for bm, bn in [(128, 128), (128, 64), (64, 128), (64, 64), (32, 64), (32, 32), (16, 32), (8, 32)]]
    + [("fp32", 0, 0, 0), ("fp32", 64, 64, 2), ("fp32", 128, 128, 2)]
    + [(m, 0, bn, 2) for m in ("3xtf32", "tf32") for bn in (0, 32, 64, 128)])


@pytest.mark.parametrize("kernel", IDENTITY_KERNELS, ids=lambda k: "%s-%dx%d-v%d" % k)
@pytest.mark.parametrize("shape", sorted(IDENTITY_SHAPES))
def test_forward_kernels_gather_what_im2col_gathers(ctx, oracle, shape, kernel):
    """The gather that RUNS in a forward -- the table-driven cp.async producer of every FFMA block shape, the
    materialised-matrix route of few-pixel layers, the 16x16-thread kernel, the gather warps of the tcgen05 kernel --
    checked element by element: with oc = K and the identity as weight matrix, output row k IS row k of the gathered
    matrix (1*x + 0 is exact; in the tensor-core modes the inputs are TF32-representable so that it stays exact)."""
    n, ic, ih, iw, kh, kw, sh, sw, (pl, pr, pt, pb) = IDENTITY_SHAPES[shape]
    mode, bm, bn, variant = kernel
    K = ic * kh * kw
    x = _tf32_exact(synth.conv_input(n, ic, ih, iw, 23))
    w = np.eye(K, dtype=np.float32).reshape(K, ic, kh, kw)
    layer = fc.ConvIm2colLayer(x, w, None, None, ic, ih, iw, K, kh, kw, sh, sw, pl, pr, pt, pb, 1, False, 1, 1,
                               batch=n, mode=mode, ctx=ctx)
    layer.Init()
    layer.set_kernel_config(bm, bn, variant, 0)
    layer.Forward()
    for img in range(n):
        want = oracle.im2col(x[img], kh, kw, sh, sw, pl, pr, pt, pb)
        assert np.array_equal(layer.output_data[img].reshape(K, -1), want), (shape, kernel, img)
    layer.release()


def test_against_reference_naive_layer(ctx, golden):
    meta, z = golden
    for rec in meta["general"]:
        x = synth.conv_input(1, rec["ic"], rec["ih"], rec["iw"], rec["seed_in"])
        w = synth.conv_weights(rec["oc"], rec["ic"], rec["kh"], rec["kw"], rec["seed_w"])
        layer = make(ctx, x, w, rec["sh"], rec["sw"], rec["pad"])
        layer.Init()
        layer.Forward()
        assert rel_l2(layer.output_data[0], z[f"general_naive_{rec['idx']}"]) < 2e-6
        layer.release()


def test_auto_dispatch_and_labels(ctx, oracle, capsys):
    x = synth.conv_input(1, 16, 14, 14, 25)
    w = synth.conv_weights(32, 16, 1, 1, 26)
    layer = fc.make_layer("auto", x, w, None, None, 16, 14, 14, 32, 1, 1, 1, 1, 0, 0, 0, 0, ctx=ctx)
    assert isinstance(layer, fc.ConvIm2colLayer)  # 1x1 s1: "direct" in the reference, which runs nothing
    layer.Init()
    layer.Forward()
    text = capsys.readouterr().out
    for label in ("Algorithm: im2col", "Im2colTran time:", "Gemm time:", "Total time:"):
        assert label in text
    assert np.array_equal(layer.output_data, oracle.im2col_gemm_forward(x, w))
    w3 = synth.conv_weights(32, 16, 3, 3, 27)
    assert isinstance(fc.make_layer("auto", x, w3, None, None, 16, 14, 14, 32, ctx=ctx), fc.ConvWinoF63ZCLayer)


@pytest.mark.parametrize("mode, tol_l2, tol_max", [("3xtf32", 1e-5, 1e-4), ("tf32", 3e-3, 3e-2)])
@pytest.mark.parametrize("case", [(1, 3, 64, 64, 64, 7, 7, 2, 2, 3), (1, 64, 256, 56, 56, 1, 1, 1, 1, 0),
                                  (2, 128, 128, 28, 28, 3, 3, 2, 2, 1), (1, 1024, 256, 14, 14, 1, 1, 1, 1, 0),
                                  (1, 20, 36, 9, 9, 3, 3, 1, 1, 1)])
def test_tensor_core_modes_within_tolerance(ctx, oracle, mode, tol_l2, tol_max, case):
    n, ic, oc, ih, iw, kh, kw, sh, sw, pad = case
    x = synth.conv_input(n, ic, ih, iw, 35)
    w = synth.conv_weights(oc, ic, kh, kw, 36)
    want = oracle.im2col_gemm_forward(x, w, sh, sw, pad, pad, pad, pad)
    layer = make(ctx, x, w, sh, sw, pad, mode=mode)
    layer.Init()
    layer.Forward()
    assert rel_l2(layer.output_data, want) <= tol_l2, f"{mode} rel-L2 {rel_l2(layer.output_data, want):.3e}"
    assert max_abs_rel(layer.output_data, want) <= tol_max
    layer.release()


@pytest.mark.parametrize("mode", ["fp32", "3xtf32"])
@pytest.mark.parametrize("pads", [(0, 2, 1, 0), (3, 0, 0, 2), (1, 2, 2, 1)])  # left, right, top, bottom
def test_four_separate_paddings_and_a_non_square_kernel(ctx, oracle, mode, pads):
    """The operator interface carries one padding per side and kh != kw (conv_layer.h:51-58); the reference's own
    paths only ever use one value for all four.  The implicit GEMM computes the general case."""
    pl, pr, pt, pb = pads
    n, ic, oc, ih, iw, kh, kw, sh, sw = 2, 12, 20, 13, 17, 3, 5, 2, 1
    x = synth.conv_input(n, ic, ih, iw, 15)
    w = synth.conv_weights(oc, ic, kh, kw, 16)
    layer = fc.ConvIm2colLayer(x, w, None, None, ic, ih, iw, oc, kh, kw, sh, sw, pl, pr, pt, pb, 1, False, 1, 1,
                               batch=n, mode=mode, ctx=ctx)
    layer.Init(); layer.Forward()
    want = oracle.im2col_gemm_forward(x, w, sh, sw, pl, pr, pt, pb)
    assert layer.output_data.shape == want.shape
    if mode == "fp32":
        assert np.array_equal(layer.output_data, want)
    else:
        assert rel_l2(layer.output_data, want) <= 1e-5
    for img in range(n):
        assert np.array_equal(layer.im2col(img), oracle.im2col(x[img], kh, kw, sh, sw, pl, pr, pt, pb))
    layer.release()


def _random_cases(seed, count):
    rng = np.random.default_rng(seed)
    cases = []
    for _ in range(count):
        kh, kw = int(rng.choice([1, 3, 5, 7])), int(rng.choice([1, 3, 5, 7]))
        n, ic, oc = int(rng.integers(1, 3)), int(rng.integers(1, 97)), int(rng.integers(1, 97))
        ih, iw = int(rng.integers(kh, 25)), int(rng.integers(kw, 25))
        sh, sw = int(rng.integers(1, 3)), int(rng.integers(1, 3))
        pad = int(rng.integers(0, min(kh, kw) // 2 + 1))
        cases.append((n, ic, oc, ih, iw, kh, kw, sh, sw, pad))
    # few pixels and a long reduction: the layers that write the gathered matrix once and stream it
    cases += [(1, 128, 40, 14, 14, 3, 3, 2, 2, 1), (1, 600, 24, 7, 7, 1, 1, 1, 1, 0), (2, 64, 72, 9, 9, 3, 3, 1, 1, 1)]
    return cases


@pytest.mark.parametrize("case", _random_cases(77, 24))
def test_random_cases_mirrored_gemm_bit_exact(ctx, oracle, case):
    n, ic, oc, ih, iw, kh, kw, sh, sw, pad = case
    x = synth.conv_input(n, ic, ih, iw, 17)
    w = synth.conv_weights(oc, ic, kh, kw, 18)
    layer = fc.ConvIm2colLayer(x, w, None, None, ic, ih, iw, oc, kh, kw, sh, sw, pad, pad, pad, pad, 1, False, 1, 1,
                               batch=n, ctx=ctx)
    layer.Init(); layer.Forward()
    assert np.array_equal(layer.output_data, oracle.im2col_gemm_forward(x, w, sh, sw, pad, pad, pad, pad))
    layer.release()


# enough pixels x channels for the 128x128, 128x64 and 64x128 block shapes: whole blocks, a ragged channel block, a
# ragged pixel block, an odd plane size (which takes the scalar stores instead of the 128-bit ones), 64 channels
# (64x128) and a grid that only fills the machine in 128x64 blocks
LARGE_CASES = [(16, 64, 128, 56, 56, 1, 1, 1, 1, 0), (8, 32, 200, 112, 112, 3, 3, 2, 2, 1),
               (10, 24, 128, 63, 63, 1, 1, 1, 1, 0), (5, 16, 250, 100, 100, 3, 3, 1, 1, 1),
               (4, 3, 64, 224, 224, 7, 7, 2, 2, 3), (4, 32, 256, 56, 56, 3, 3, 1, 1, 1)]


@pytest.mark.parametrize("case", LARGE_CASES)
def test_large_problems_mirrored_gemm_bit_exact(ctx, oracle, case):
    n, ic, oc, ih, iw, kh, kw, sh, sw, pad = case
    x = synth.conv_input(n, ic, ih, iw, 19)
    w = synth.conv_weights(oc, ic, kh, kw, 20)
    layer = fc.ConvIm2colLayer(x, w, None, None, ic, ih, iw, oc, kh, kw, sh, sw, pad, pad, pad, pad, 1, False, 1, 1,
                               batch=n, ctx=ctx)
    layer.Init(); layer.Forward()
    assert np.array_equal(layer.output_data, oracle.im2col_gemm_forward(x, w, sh, sw, pad, pad, pad, pad))
    layer.release()


@pytest.mark.parametrize("mode,tol", [("3xtf32", 1e-5), ("tf32", 3e-3)])
@pytest.mark.parametrize("case", _random_cases(78, 10))
def test_random_cases_tensor_core_modes(ctx, oracle, case, mode, tol):
    n, ic, oc, ih, iw, kh, kw, sh, sw, pad = case
    x = synth.conv_input(n, ic, ih, iw, 19)
    w = synth.conv_weights(oc, ic, kh, kw, 20)
    layer = fc.ConvIm2colLayer(x, w, None, None, ic, ih, iw, oc, kh, kw, sh, sw, pad, pad, pad, pad, 1, False, 1, 1,
                               batch=n, mode=mode, ctx=ctx)
    layer.Init(); layer.Forward()
    want = oracle.im2col_gemm_forward(x, w, sh, sw, pad, pad, pad, pad)
    assert rel_l2(layer.output_data, want) <= tol
    layer.release()

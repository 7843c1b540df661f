"""`-a direct`: direct convolution on the tensor cores (stride 1 or 2, TF32) against the oracle's convolution.

The reference has no code behind the name (ConvTest.cpp:369-371), so the expected values are those of its im2col
layer restated by the oracle (im2colConv.cpp:285-309 + the sequential GEMM).  Tolerance: relative L2 <= 3e-3, the
figure stated for the TF32 mode; the kernel has no Winograd transform to amplify the operand rounding, so the tests
also pin the much smaller error it really has (<= 1e-3)."""
import numpy as np
import pytest

import fastconv_b200 as fc
from _oracle import rel_l2
from fastconv_b200 import _lib, synth

pytestmark = pytest.mark.gpu

CASES = [  # n, ic, oc, ih, iw, kh, kw, pad_l, pad_r, pad_t, pad_b
    (1, 3, 8, 30, 30, 3, 3, 1, 1, 1, 1),        # 3 channels padded to 32, one ragged patch row
    (2, 64, 64, 56, 56, 3, 3, 1, 1, 1, 1),      # two images, two 32-channel blocks per tap
    (1, 70, 130, 14, 14, 3, 3, 1, 1, 1, 1),     # ragged channel blocks on both sides, 14x14 in 8x16 patches
    (1, 16, 12, 14, 14, 1, 1, 0, 0, 0, 0),      # 1x1: a plain GEMM
    (1, 4, 4, 9, 11, 5, 3, 1, 1, 2, 2),         # non-square kernel
    (3, 33, 17, 7, 7, 3, 3, 1, 1, 1, 1),        # 7x7 maps
    (1, 8, 200, 28, 28, 3, 3, 0, 2, 1, 0),      # four different paddings, two channel blocks of 112
    (1, 1, 1, 1, 1, 1, 1, 0, 0, 0, 0),          # one pixel
    (1, 32, 16, 20, 20, 7, 7, 3, 3, 3, 3),      # 49 taps
    (1, 24, 40, 5, 130, 3, 3, 1, 1, 1, 1),      # a wide, flat image: 1x128 patches
    (1, 24, 40, 130, 5, 3, 3, 1, 1, 1, 1),      # a tall, narrow one: 32x4 patches
    (1, 16, 16, 12, 12, 3, 3, 0, 0, 0, 0),      # no padding: the output is smaller than the input
    (2, 2, 20, 17, 19, 3, 5, 1, 2, 0, 1),       # ic*kh*kw = 30 <= 32: taps folded into one k-block, four paddings
    (1, 1, 16, 12, 12, 5, 5, 2, 2, 2, 2),       # one channel, 25 taps folded
    (3, 3, 64, 64, 64, 3, 3, 1, 1, 1, 1),       # the first layer of VGG-16 in small: 27 folded taps, three images
    (12, 32, 300, 56, 56, 3, 3, 1, 1, 1, 1),    # enough work items for channel blocks wider than 128: two of 160
]


def _layer(ctx, x, w, case, mode="tf32"):
    n, ic, oc, ih, iw, kh, kw, pl, pr, pt, pb = case
    return fc.ConvDirectLayer(x, w, None, None, ic, ih, iw, oc, kh, kw, 1, 1, pl, pr, pt, pb, 1, False, 1, 1, batch=n,
                              mode=mode, ctx=ctx)


@pytest.mark.parametrize("case", CASES)
def test_direct_tf32_within_tolerance(ctx, oracle, case):
    n, ic, oc, ih, iw, kh, kw, pl, pr, pt, pb = case
    x = synth.conv_input(n, ic, ih, iw, 91)
    w = synth.conv_weights(oc, ic, kh, kw, 92)
    layer = _layer(ctx, x, w, case)
    assert layer.Init() == 1 and layer.Forward() == 1
    assert layer.algorithm == _lib.ALGO_DIRECT
    want = oracle.im2col_gemm_forward(x, w, 1, 1, pl, pr, pt, pb)
    assert layer.output_data.shape == want.shape
    err = rel_l2(layer.output_data, want)
    assert err <= 3e-3, err   # the tolerance stated for the TF32 mode
    assert err <= 1e-3, err   # what single-pass TF32 gives without a Winograd transform in the way
    assert np.abs(layer.output_data - want).max() <= 3e-2 * np.abs(want).max()
    layer.Forward()  # a second forward reuses the NHWC buffer
    assert rel_l2(layer.output_data, want) <= 1e-3
    layer.release()


STRIDED = [  # n, ic, oc, ih, iw, kh, kw, sh, sw, pad
    (1, 8, 8, 15, 15, 3, 3, 2, 2, 1), (2, 64, 48, 28, 28, 1, 1, 2, 2, 0), (1, 32, 16, 20, 21, 3, 3, 2, 2, 1),
    (4, 128, 128, 56, 56, 3, 3, 2, 2, 1), (1, 40, 24, 30, 30, 5, 5, 2, 2, 2), (1, 3, 16, 64, 64, 7, 7, 2, 2, 3),
    (1, 16, 16, 21, 18, 3, 3, 2, 1, 1), (1, 16, 16, 18, 21, 3, 3, 1, 2, 1),  # a stride along one axis only
]


@pytest.mark.parametrize("case", STRIDED)
def test_direct_strided_layers(ctx, oracle, case):
    """Stride 2 is the element stride of the input's tensor map: same kernel, every second pixel of a twice larger box."""
    n, ic, oc, ih, iw, kh, kw, sh, sw, pad = case
    x = synth.conv_input(n, ic, ih, iw, 101)
    w = synth.conv_weights(oc, ic, kh, kw, 102)
    layer = fc.ConvDirectLayer(x, w, None, None, ic, ih, iw, oc, kh, kw, sh, sw, pad, pad, pad, pad, 1, False, 1, 1,
                               batch=n, mode="tf32", ctx=ctx)
    layer.Init(); layer.Forward()
    assert layer.algorithm == _lib.ALGO_DIRECT
    want = oracle.im2col_gemm_forward(x, w, sh, sw, pad, pad, pad, pad)
    assert layer.output_data.shape == want.shape
    assert rel_l2(layer.output_data, want) <= 1e-3
    layer.release()


# a small layer (28 output blocks: its reduction is shared by several work items, bias and ReLU follow in a pass of
# their own: 3 launches) and one with more output blocks than SMs (one accumulator per output, epilogue in the kernel)
@pytest.mark.parametrize("case, launches", [((2, 48, 72, 28, 28, 3, 3, 1, 1, 1, 1), 3),
                                            ((6, 48, 72, 56, 56, 3, 3, 1, 1, 1, 1), 2)])
def test_direct_epilogue_and_repeatability(ctx, oracle, case, launches):
    n, ic, oc, ih, iw, kh, kw, pl, pr, pt, pb = case
    x = synth.conv_input(n, ic, ih, iw, 93)
    w = synth.conv_weights(oc, ic, kh, kw, 94)
    b = (synth.conv_input(1, 1, 1, oc, 95).reshape(oc) * np.float32(0.5)).astype(np.float32)
    layer = _layer(ctx, x, w, case)
    layer.set_epilogue(b, True)
    layer.Init(); layer.Forward()
    assert layer.kernel_launches == launches
    first = layer.output_data.copy()
    want = np.maximum(oracle.im2col_gemm_forward(x, w, 1, 1, pl, pr, pt, pb) + b[None, :, None, None], 0).astype(np.float32)
    assert rel_l2(first, want) <= 1e-3
    assert (first >= 0).all()
    layer.Forward()
    if launches == 2:
        assert np.array_equal(layer.output_data, first)  # one accumulator per output, fixed order: no run-to-run noise
    else:
        assert rel_l2(layer.output_data, first) <= 1e-6  # partial sums are added in whatever order they arrive
    layer.set_epilogue(None, False)
    layer.Forward()
    assert rel_l2(layer.output_data, oracle.im2col_gemm_forward(x, w, 1, 1, pl, pr, pt, pb)) <= 1e-3
    layer.release()


def test_direct_falls_back_to_the_implicit_gemm(ctx, oracle, capsys):
    """Strides above 2 and the other math modes have no direct kernel: they run as the im2col layer, bit-exact in fp32."""
    x = synth.conv_input(1, 8, 15, 15, 96)
    w = synth.conv_weights(8, 8, 3, 3, 97)
    strided = fc.ConvDirectLayer(x, w, None, None, 8, 15, 15, 8, 3, 3, 3, 3, 1, 1, 1, 1, 1, False, 1, 1, mode="tf32", ctx=ctx)
    strided.Init(); strided.Forward()
    assert strided.algorithm == _lib.ALGO_IM2COL
    assert rel_l2(strided.output_data, oracle.im2col_gemm_forward(x, w, 3, 3, 1, 1, 1, 1)) <= 3e-3
    strided.release()
    exact = fc.make_layer("direct", x, w, None, None, 8, 15, 15, 8, 3, 3, 1, 1, 1, 1, 1, 1, ctx=ctx)  # mode fp32
    assert isinstance(exact, fc.ConvDirectLayer)
    exact.Init(); exact.Forward()
    assert "Algorithm: direct" in capsys.readouterr().out
    assert exact.algorithm == _lib.ALGO_IM2COL
    assert np.array_equal(exact.output_data, oracle.im2col_gemm_forward(x, w, 1, 1, 1, 1, 1, 1))
    exact.release()


def test_direct_vgg_layer_and_tuner(ctx, oracle, tmp_path, monkeypatch):
    """conv3_2 of VGG-16 (256 -> 256 at 56x56): the TF32 figure that the Winograd path misses (6.4e-3) is met here."""
    monkeypatch.setenv("FASTCONV_TUNING_LOG", str(tmp_path / "tuning_log"))
    x = synth.conv_input(1, 256, 56, 56, 98)
    w = synth.conv_weights(256, 256, 3, 3, 99)
    layer = fc.ConvDirectLayer(x, w, None, None, 256, 56, 56, 256, iter=3, mode="tf32", ctx=ctx)
    layer.Tuning()
    layer.Init(); layer.Forward()
    assert layer.algorithm == _lib.ALGO_DIRECT
    err = rel_l2(layer.output_data, oracle.im2col_gemm_forward(x, w, 1, 1, 1, 1, 1, 1))
    assert err <= 1e-3, err
    assert layer.kernel_launches == 2
    layer.release()


def _create(ctx, desc, algo, mode, w):
    import ctypes as C
    lib = fc.load()
    h = C.c_void_p()
    _lib.check(lib.fc_conv_create(ctx.handle, C.byref(desc), algo, mode, C.c_void_p(w.ctypes.data), C.byref(h)), "create")
    a, m = C.c_int(), C.c_int()
    lib.fc_conv_algorithm(h, C.byref(a))
    lib.fc_conv_math_mode(h, C.byref(m))
    return lib, h, a.value, m.value


@pytest.mark.parametrize("shape, algo_in, want_algo, want_mode", [
    # n, ic, oc, hw, k, pad
    ((1, 64, 64, 56, 3, 1), "auto", "direct", "tf32"),          # few channels: the direct kernel
    ((1, 512, 512, 14, 3, 1), "auto", "direct", "tf32"),         # a small layer: its reduction is shared by the SMs
    ((8, 512, 512, 14, 3, 1), "auto", "direct", "tf32"),
    ((1, 64, 64, 56, 3, 1), "winograd", "winograd", "3xtf32"),   # Winograd by name: the split arithmetic complies
    ((4, 256, 128, 28, 1, 0), "auto", "direct", "tf32"),         # not a Winograd layer: as in the TF32 mode
    ((1, 16, 12, 14, 1, 0), "auto", "im2col", "tf32"),
])
def test_tf32_mode_never_runs_one_pass_through_winograd(ctx, oracle, shape, algo_in, want_algo, want_mode):
    import ctypes as C
    n, ic, oc, hw, k, pad = shape
    x = synth.conv_input(n, ic, hw, hw, 111)
    w = synth.conv_weights(oc, ic, k, k, 112)
    d = fc.make_desc(n, ic, hw, hw, oc, k, k, 1, 1, pad, pad, pad, pad)
    lib, h, algo, mode = _create(ctx, d, _lib.ALGO_NAMES[algo_in], _lib.MATH_TF32, w)
    assert algo == _lib.ALGO_NAMES[want_algo] and mode == _lib.MODE_NAMES[want_mode]
    y = np.empty((n, oc, hw, hw), np.float32)
    _lib.check(lib.fc_conv_forward_host(h, C.c_void_p(x.ctypes.data), C.c_void_p(y.ctypes.data)), "forward")
    if want_algo == "winograd":
        assert rel_l2(y, oracle.wino_forward(x, w, 1)) <= 1e-5
    else:
        assert rel_l2(y, oracle.im2col_gemm_forward(x, w, 1, 1, pad, pad, pad, pad)) <= 3e-3
    lib.fc_conv_destroy(h)

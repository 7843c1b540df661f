"""Per-channel bias + ReLU applied inside the layer's last kernel, and layers chained device to device.

The reference's Winograd and im2col layers have no bias and no activation (only its general naive layer adds a
per-element bias), so the expected values are the oracle's convolution followed by the same two elementwise
steps in numpy: one rounded fp32 addition, then max(., 0).  In the fp32 mirrored mode that is bit-exact."""
import ctypes as C

import numpy as np
import pytest

import fastconv_b200 as fc
from _oracle import rel_l2
from fastconv_b200 import _lib, synth
from fastconv_b200.layers import make_desc

pytestmark = pytest.mark.gpu


def _expect(y, bias, relu):
    if bias is not None:
        y = (y + bias.astype(np.float32)[None, :, None, None]).astype(np.float32)
    return np.maximum(y, np.float32(0)) if relu else y


def _bias(oc, seed):
    return (synth.conv_input(1, 1, 1, oc, seed).reshape(oc) * np.float32(0.5)).astype(np.float32)


# n, ic, oc, hw: 4 / 25 / 100 / 400 tiles -> the three latency-oriented shapes and the wide output transform;
# 3 input channels -> the output transform that holds the multiply-accumulate
WINO = [(1, 8, 12, 7), (1, 16, 20, 30), (1, 24, 40, 56), (4, 16, 24, 56), (2, 3, 18, 56)]


@pytest.mark.parametrize("shape", WINO)
@pytest.mark.parametrize("bias,relu", [(True, True), (True, False), (False, True)])
def test_winograd_epilogue_bit_exact(ctx, oracle, shape, bias, relu):
    n, ic, oc, hw = shape
    x = synth.conv_input(n, ic, hw, hw, 71)
    w = synth.conv_weights(oc, ic, 3, 3, 72)
    b = _bias(oc, 73) if bias else None
    layer = fc.ConvWinoF63ZCLayer(x, w, None, None, ic, hw, hw, oc, batch=n, iter=1, ctx=ctx)
    layer.set_epilogue(b, relu)
    layer.Init(); layer.Forward()
    assert np.array_equal(layer.output_data, _expect(oracle.wino_forward(x, w, 1), b, relu))
    layer.set_epilogue(None, False)  # and off again
    layer.Forward()
    assert np.array_equal(layer.output_data, oracle.wino_forward(x, w, 1))
    layer.release()


# n, ic, oc, ih, kh, stride, pad: table-driven kernel in small and large block shapes, and the 16x16-thread kernel
IGEMM = [(1, 16, 12, 14, 1, 1, 0), (1, 8, 40, 15, 3, 2, 1), (1, 3, 64, 64, 7, 2, 3), (8, 32, 128, 56, 3, 1, 1)]


@pytest.mark.parametrize("case", IGEMM)
def test_implicit_gemm_epilogue_bit_exact(ctx, oracle, case):
    n, ic, oc, ih, k, s, pad = case
    x = synth.conv_input(n, ic, ih, ih, 74)
    w = synth.conv_weights(oc, ic, k, k, 75)
    b = _bias(oc, 76)
    layer = fc.ConvIm2colLayer(x, w, None, None, ic, ih, ih, oc, k, k, s, s, pad, pad, pad, pad, 1, False, 1, 1,
                               batch=n, ctx=ctx)
    layer.set_epilogue(b, True)
    layer.Init(); layer.Forward()
    want = _expect(oracle.im2col_gemm_forward(x, w, s, s, pad, pad, pad, pad), b, True)
    assert np.array_equal(layer.output_data, want)
    layer.release()


@pytest.mark.parametrize("mode", ["3xtf32", "tf32"])
def test_tensor_core_modes_apply_the_epilogue(ctx, oracle, mode):
    tol = 2e-5 if mode == "3xtf32" else 3e-3
    x = synth.conv_input(1, 64, 28, 28, 77)
    b = _bias(96, 78)
    w3 = synth.conv_weights(96, 64, 3, 3, 79)
    layer = fc.ConvWinoF63ZCLayer(x, w3, None, None, 64, 28, 28, 96, iter=1, mode=mode, ctx=ctx)
    layer.set_epilogue(b, True)
    layer.Init(); layer.Forward()
    assert rel_l2(layer.output_data, _expect(oracle.wino_forward(x, w3, 1), b, True)) <= tol
    layer.release()
    # a small strided 3x3 layer (K = 576: long enough for the tcgen05 implicit GEMM), which would otherwise split K
    # and add partial sums: the epilogue must see complete sums
    w2 = synth.conv_weights(96, 64, 3, 3, 80)
    layer = fc.ConvIm2colLayer(x, w2, None, None, 64, 28, 28, 96, 3, 3, 2, 2, 1, 1, 1, 1, 1, False, 1, 1, mode=mode, ctx=ctx)
    layer.set_epilogue(b, True)
    layer.Init(); layer.Forward()
    want = _expect(oracle.im2col_gemm_forward(x, w2, 2, 2, 1, 1, 1, 1), b, True)
    assert rel_l2(layer.output_data, want) <= (1e-5 if mode == "3xtf32" else 3e-3)
    assert not np.array_equal(layer.output_data, want)  # i.e. it really ran on the tensor cores
    layer.release()


def test_three_layers_chained_on_the_device(ctx, oracle):
    """conv -> ReLU -> conv -> ReLU -> conv (a VGG block in miniature plus a 1x1 head): layer i writes where layer
    i+1 reads, one CUDA graph, nothing crosses PCIe in between; bit-equal to the oracle applied three times."""
    lib = fc.load()
    hw = 28
    specs = [(16, 32, 3, 1), (32, 32, 3, 1), (32, 8, 1, 0)]  # ic, oc, k, pad
    x = synth.conv_input(1, 16, hw, hw, 81)
    ws = [synth.conv_weights(oc, ic, k, k, 82 + i) for i, (ic, oc, k, _) in enumerate(specs)]
    bs = [_bias(oc, 90 + i) for i, (_, oc, _, _) in enumerate(specs)]
    convs, d_ins, d_outs = [], [], []
    for (ic, oc, k, pad), w, b in zip(specs, ws, bs):
        desc = make_desc(1, ic, hw, hw, oc, k, k, 1, 1, pad, pad, pad, pad)
        h = C.c_void_p()
        _lib.check(lib.fc_conv_create(ctx.handle, C.byref(desc), _lib.ALGO_AUTO, _lib.MODE_NAMES["fp32"],
                                      C.c_void_p(w.ctypes.data), C.byref(h)), "fc_conv_create")
        _lib.check(lib.fc_conv_set_epilogue(h, C.c_void_p(b.ctypes.data), 1), "fc_conv_set_epilogue")
        d_in, d_out = C.c_void_p(), C.c_void_p()
        _lib.check(lib.fc_conv_device_buffers(h, C.byref(d_in), C.byref(d_out)), "fc_conv_device_buffers")
        convs.append(h)
        d_ins.append(d_in.value if not d_outs else d_outs[-1])  # read what the previous layer wrote
        d_outs.append(d_out.value)
    ctx.upload(x, d_ins[0])
    chain = fc.LayerList(ctx, convs, d_ins, d_outs)
    for _ in range(2):
        chain.forward()
    ctx.synchronize()
    got = ctx.download(d_outs[-1], (1, specs[-1][1], hw, hw))
    y = x
    for (ic, oc, k, pad), w, b in zip(specs, ws, bs):
        y = oracle.wino_forward(y, w, pad) if k == 3 else oracle.im2col_gemm_forward(y, w, 1, 1, 0, 0, 0, 0)
        y = _expect(y, b, True)
    assert np.array_equal(got, y)
    chain.close()
    for h in convs:
        lib.fc_conv_destroy(h)

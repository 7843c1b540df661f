"""Grouped and depthwise convolution through the implicit-GEMM path.  The reference's operator interface carries
`group` (conv_layer.h:27) but none of its paths reads it; a grouped layer here is `group` independent convolutions
over channel slices, so the expected values are the oracle applied to each slice and concatenated -- bit-exact in
the fp32 mode, within the usual tolerances in the tensor-core modes."""
import numpy as np
import pytest

import fastconv_b200 as fc
from _oracle import rel_l2
from fastconv_b200 import synth

pytestmark = pytest.mark.gpu


def _expect(oracle, x, w, g, s, pad):
    icg, ocg = x.shape[1] // g, w.shape[0] // g
    parts = [oracle.im2col_gemm_forward(np.ascontiguousarray(x[:, i * icg:(i + 1) * icg]),
                                        np.ascontiguousarray(w[i * ocg:(i + 1) * ocg]), s, s, pad, pad, pad, pad)
             for i in range(g)]
    return np.concatenate(parts, axis=1)


def _run(ctx, x, w, g, k, s, pad, mode, bias=None, relu=False):
    n, ic, ih, iw = x.shape
    conv = fc.make_layer("auto", x, w, None, None, ic, ih, iw, w.shape[0], k, k, s, s, pad, pad, pad, pad, g, False, 1, 1,
                 batch=n, mode=mode, ctx=ctx)
    if bias is not None or relu:
        conv.set_epilogue(bias, relu)
    conv.Init(); conv.Forward()
    out = conv.output_data.copy()
    launches = conv.kernel_launches
    conv.release()
    return out, launches


# n, ic, oc, hw, k, stride, pad, group
GROUPED = [(1, 16, 24, 14, 3, 1, 1, 2), (2, 32, 32, 15, 3, 2, 1, 4), (1, 12, 18, 9, 1, 1, 0, 3), (1, 64, 128, 28, 3, 1, 1, 8)]


@pytest.mark.parametrize("case", GROUPED)
@pytest.mark.parametrize("mode", ["fp32", "3xtf32", "tf32"])
def test_grouped_layers(ctx, oracle, case, mode):
    n, ic, oc, hw, k, s, pad, g = case
    x = synth.conv_input(n, ic, hw, hw, 31)
    w = synth.conv_weights(oc, ic // g, k, k, 32)
    got, launches = _run(ctx, x, w, g, k, s, pad, mode)
    want = _expect(oracle, x, w, g, s, pad)
    assert launches == g
    if mode == "fp32":
        assert np.array_equal(got, want)
    else:
        assert rel_l2(got, want) <= (1e-5 if mode == "3xtf32" else 3e-3)


# n, channels, multiplier, hw, k, stride, pad
DEPTHWISE = [(1, 32, 1, 28, 3, 1, 1), (2, 48, 1, 15, 3, 2, 1), (1, 16, 2, 12, 5, 1, 2), (4, 96, 1, 56, 3, 1, 1)]


@pytest.mark.parametrize("case", DEPTHWISE)
@pytest.mark.parametrize("mode", ["fp32", "tf32"])
def test_depthwise_layers_bit_exact_in_every_mode(ctx, oracle, case, mode):
    n, c, mult, hw, k, s, pad = case
    x = synth.conv_input(n, c, hw, hw, 33)
    w = synth.conv_weights(c * mult, 1, k, k, 34)
    b = (synth.conv_input(1, 1, 1, c * mult, 35).reshape(-1) * np.float32(0.25)).astype(np.float32)
    got, launches = _run(ctx, x, w, c, k, s, pad, mode, bias=b, relu=True)
    want = _expect(oracle, x, w, c, s, pad)
    want = np.maximum((want + b[None, :, None, None]).astype(np.float32), np.float32(0))
    assert launches == 1
    assert np.array_equal(got, want)  # the depthwise kernel is plain fp32 in every mode


def test_grouped_layer_with_epilogue_and_winograd_refusal(ctx, oracle):
    x = synth.conv_input(1, 16, 14, 14, 36)
    w = synth.conv_weights(16, 8, 3, 3, 37)
    b = (synth.conv_input(1, 1, 1, 16, 38).reshape(-1)).astype(np.float32)
    got, _ = _run(ctx, x, w, 2, 3, 1, 1, "fp32", bias=b, relu=True)
    want = np.maximum((_expect(oracle, x, w, 2, 1, 1) + b[None, :, None, None]).astype(np.float32), np.float32(0))
    assert np.array_equal(got, want)
    with pytest.raises(fc.FastConvError) as err:  # -a winograd on a grouped layer is refused, not computed wrongly
        conv = fc.make_layer("winograd", x, w, None, None, 16, 14, 14, 16, 3, 3, 1, 1, 1, 1, 1, 1, 2, False, 1, 1, ctx=ctx)
        conv.Init(); conv.Forward()
    assert err.value.status == -2

"""Parity at the sizes of the two multi-GPU benchmark configurations, on one GPU.

  * the wide single-image sweep (3x3 s1 p1, C = K in {512, 1024, 2048} at 14 / 28 / 56): the layers whose output
    channels are split over GPUs;
  * the batched VGG-16 stack at the per-GPU batch of an 8-way split (8 images: 200 and 72 tiles on the 512-channel
    layers) and at the full batch of 64 on three of its layers.

fp32 mirrored mode: bit-equal to the oracle.  "tf32" (the mode that stands for rel-L2 <= 3e-3): held to 3e-3.
3xTF32: rel-L2 <= 1e-5 up to 256 input channels.  Above that no implementation with another summation order can
stay inside 1e-5 of the reference -- the reference's own output moves by more than that when only the ORDER of its
input channels changes -- so the bound is that movement, measured in the same test: the oracle run on the same
layer with its channels permuted (same products, same exact sum, another fp32 accumulation order).
"""
import numpy as np
import pytest

import fastconv_b200 as fc
from _oracle import max_abs_rel, order_noise, rel_l2
from fastconv_b200 import synth

pytestmark = pytest.mark.gpu

WIDE = [(512, 14), (512, 28), (512, 56), (1024, 14), (1024, 28), (1024, 56), (2048, 14), (2048, 28)]


def _forward(ctx, x, w, mode):
    n, ic, ih, iw = x.shape
    oc = w.shape[0]
    layer = fc.make_layer("auto", x, w, None, None, ic, ih, iw, oc, 3, 3, 1, 1, 1, 1, 1, 1, 1, False, 1, 1,
                          batch=n, mode=mode, ctx=ctx)
    layer.Init()
    layer.Forward()
    out = layer.output_data.copy()
    layer.release()
    return out


@pytest.mark.parametrize("c,hw", WIDE)
def test_wide_single_image_layers(ctx, oracle, c, hw):
    x = synth.conv_input(1, c, hw, hw, 4000 + c + hw)
    w = synth.conv_weights(c, c, 3, 3, 5000 + c + hw)
    want = oracle.wino_forward(x, w, 1)
    assert np.array_equal(_forward(ctx, x, w, "fp32"), want)
    got = _forward(ctx, x, w, "3xtf32")
    noise = order_noise(oracle, x, w, want)
    assert rel_l2(got, want) <= max(1e-5, 1.25 * noise), (rel_l2(got, want), noise)
    assert max_abs_rel(got, want) <= 1e-4
    assert rel_l2(_forward(ctx, x, w, "tf32"), want) <= 3e-3


# ic, oc, hw of the VGG-16 layers whose tile count at 8 images sits between the few-tile and the 128-wide kernels,
# and one early layer
@pytest.mark.parametrize("ic,oc,hw", [(512, 512, 28), (512, 512, 14), (256, 512, 28), (128, 256, 56), (64, 64, 224)])
def test_vgg16_layers_at_eight_images(ctx, oracle, ic, oc, hw):
    n = 8
    x = synth.conv_input(n, ic, hw, hw, 6000 + ic + hw)
    w = synth.conv_weights(oc, ic, 3, 3, 7000 + ic + hw)
    want = oracle.wino_forward(x, w, 1)
    assert np.array_equal(_forward(ctx, x, w, "fp32"), want)
    got = _forward(ctx, x, w, "3xtf32")
    bound = 1e-5 if ic <= 256 else max(1e-5, 1.25 * order_noise(oracle, x[:1], w, want[:1]))
    assert rel_l2(got, want) <= bound and max_abs_rel(got, want) <= 1e-4
    assert rel_l2(_forward(ctx, x, w, "tf32"), want) <= 3e-3


def _batch_of(images, n):
    """n distinct images from a few generated ones: image i = base[i % len] scaled by an exact power-of-two step."""
    scale = (1.0 - np.arange(n, dtype=np.float32) / 256.0).reshape(n, 1, 1, 1)
    return np.ascontiguousarray(images[np.arange(n) % len(images)] * scale)


@pytest.mark.parametrize("ic,oc,hw", [(64, 64, 224), (256, 256, 56), (512, 512, 14)])
def test_vgg16_layers_at_sixty_four_images(ctx, oracle, ic, oc, hw):
    """The full batch of the batched configuration.  Images are independent, so the oracle checks a sample of them
    one by one (first, last, two in the middle) against the matching slices of the 64-image result."""
    n, sample = 64, (0, 21, 42, 63)
    x = _batch_of(synth.conv_input(4, ic, hw, hw, 8000 + ic + hw), n)
    w = synth.conv_weights(oc, ic, 3, 3, 9000 + ic + hw)
    want = {i: oracle.wino_forward(x[i:i + 1], w, 1)[0] for i in sample}
    got = _forward(ctx, x, w, "fp32")
    for i in sample:
        assert np.array_equal(got[i], want[i]), f"image {i}"
    got = _forward(ctx, x, w, "3xtf32")
    noise = order_noise(oracle, x[:1], w, want[0][None]) if ic > 256 else 0.0
    for i in sample:
        assert rel_l2(got[i], want[i]) <= max(1e-5, 1.25 * noise) and max_abs_rel(got[i], want[i]) <= 1e-4
    got = _forward(ctx, x, w, "tf32")
    for i in sample:
        assert rel_l2(got[i], want[i]) <= 3e-3

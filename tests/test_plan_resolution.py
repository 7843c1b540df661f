"""What `-a auto` and the math modes resolve to per layer (fc_resolve_plan: host logic, no GPU needed).

The reference's choice depends on the shape only (select_algorithm, ConvTest.cpp:318-331: 3x3 stride 1 -> winograd,
everything else -> im2col; its `direct` case is empty).  Here the TF32 modes add the direct tensor-core kernel, taken
where per-layer timings on a B200 favour it; these cases pin the crossovers that the timings gave."""
import pytest

import fastconv_b200 as fc


def plan(n, ic, oc, hw, k, s=1, pad=None, algo="auto", mode="tf32"):
    pad = (k // 2) if pad is None else pad
    return fc.resolve_plan(fc.make_desc(n, ic, hw, hw, oc, k, k, s, s, pad, pad, pad, pad), algo, mode, 148)


@pytest.mark.parametrize("mode", ["fp32", "3xtf32"])
def test_exact_modes_keep_the_reference_choice(mode):
    assert plan(1, 256, 256, 56, 3, mode=mode) == ("winograd", mode)
    assert plan(1, 256, 64, 56, 1, mode=mode) == ("im2col", mode)
    assert plan(1, 128, 128, 56, 3, s=2, mode=mode) == ("im2col", mode)
    assert plan(1, 3, 64, 224, 7, s=2, mode=mode) == ("im2col", mode)
    assert plan(8, 64, 64, 224, 3, algo="direct", mode=mode) == ("im2col", mode)  # no direct kernel in these modes


def test_unbounded_tf32_auto_on_the_vgg16_layers():
    def plan(*a, **k):
        return globals()["plan"](*a, mode="tf32-unbounded", **k)
    # batch 1: few channels -> direct; small maps (shared reduction) -> direct; the middle of the network -> Winograd
    assert plan(1, 3, 64, 224, 3)[0] == "direct"
    assert plan(1, 64, 128, 112, 3)[0] == "direct"
    assert plan(1, 128, 128, 112, 3)[0] == "winograd"
    assert plan(1, 256, 256, 56, 3)[0] == "winograd"
    assert plan(1, 512, 512, 28, 3)[0] == "direct"
    assert plan(1, 512, 512, 14, 3)[0] == "direct"
    # batch 8 and 64: direct up to 128 -> 256 channels, Winograd from 256 -> 256 on
    for n in (8, 64):
        assert plan(n, 128, 256, 56, 3)[0] == "direct"
        assert plan(n, 256, 256, 56, 3)[0] == "winograd"
        assert plan(n, 512, 512, 14, 3)[0] == "winograd"


def test_tf32_auto_on_1x1_and_strided_layers():
    assert plan(1, 64, 64, 56, 1)[0] == "im2col"          # 26 MFLOP: the extra launch of the layout pass decides
    assert plan(1, 64, 256, 56, 1)[0] == "direct"
    assert plan(1, 2048, 512, 7, 1)[0] == "direct"
    assert plan(1, 128, 128, 56, 3, s=2)[0] == "direct"   # stride 2 = element stride of the tensor map
    assert plan(64, 3, 64, 224, 7, s=2)[0] == "im2col"    # the stem: 3 real channels per k-block, 49 taps that do not fold
    assert plan(1, 64, 64, 56, 3, s=3)[0] == "im2col"     # stride 3: no direct kernel
    assert plan(1, 64, 64, 56, 3, algo="winograd") == ("winograd", "3xtf32")  # the algorithm asked for by name is kept
    assert plan(1, 64, 64, 56, 3, algo="winograd", mode="tf32-unbounded") == ("winograd", "tf32")


def test_tf32_never_runs_one_pass_through_winograd():
    """"tf32" stands for rel-L2 <= 3e-3, which one TF32 pass through F(6x6,3x3) misses."""
    for n in (1, 8, 64):
        for ic, oc, hw in [(3, 64, 224), (128, 128, 112), (256, 256, 56), (512, 512, 28), (512, 512, 14), (512, 512, 7)]:
            assert plan(n, ic, oc, hw, 3) == ("direct", "tf32")
    assert plan(1, 256, 256, 56, 3, algo="winograd") == ("winograd", "3xtf32")
    assert plan(1, 256, 64, 56, 1)[1] == "tf32"
    assert plan(1, 3, 64, 224, 7, s=2) == ("im2col", "tf32")


def test_fp16_filter_mode_resolves_per_layer():
    """"tf32-u16" keeps the fp16 filter for Winograd layers with more than 64 channels and under 128 tiles."""
    assert plan(1, 512, 512, 14, 3, algo="winograd", mode="tf32-u16") == ("winograd", "tf32-u16")
    assert plan(1, 256, 256, 56, 3, algo="winograd", mode="tf32-u16") == ("winograd", "tf32-u16")   # 100 tiles
    assert plan(64, 512, 512, 14, 3, algo="winograd", mode="tf32-u16") == ("winograd", "tf32")      # 576 tiles
    assert plan(1, 64, 64, 56, 3, algo="winograd", mode="tf32-u16") == ("winograd", "tf32")         # 64 channels
    assert plan(1, 256, 64, 56, 1, mode="tf32-u16")[1] == "tf32"                                    # not a Winograd layer
    assert plan(1, 256, 256, 56, 3, mode="tf32-u16") == plan(1, 256, 256, 56, 3, mode="tf32-unbounded")[:1] + ("tf32-u16",)


def test_make_layer_auto_follows_the_plan():
    """The Python front end, the CLI and the library agree on what `auto` means in every mode."""
    import numpy as np
    for mode in ("fp32", "3xtf32", "tf32", "tf32-unbounded"):
        for ic, oc, hw, k, s in [(64, 64, 56, 3, 1), (256, 256, 56, 3, 1), (64, 256, 56, 1, 1), (128, 128, 56, 3, 2)]:
            p = k // 2
            x = np.zeros((1, ic, hw, hw), np.float32)
            w = np.zeros((oc, ic, k, k), np.float32)
            layer = fc.make_layer("auto", x, w, None, None, ic, hw, hw, oc, k, k, s, s, p, p, p, p, mode=mode)
            name = {fc.ConvWinoF63ZCLayer: "winograd", fc.ConvDirectLayer: "direct", fc.ConvIm2colLayer: "im2col"}[type(layer)]
            assert name == plan(1, ic, oc, hw, k, s=s, mode=mode)[0]
            assert layer._algo == 0  # created as AUTO, so the library records the request


def test_accuracy_mode_runs_the_fp32_kernels_on_short_reductions(monkeypatch):
    """By default a Winograd layer of at most 64 input channels asked for in 3xTF32 (or in "tf32" with Winograd named)
    is planned in the fp32 arithmetic: faster there, and inside the mode's tolerance by being exact."""
    monkeypatch.delenv("FASTCONV_3XTF32_MIN_IC")
    assert plan(64, 3, 64, 224, 3, mode="3xtf32") == ("winograd", "fp32")
    assert plan(1, 64, 128, 112, 3, mode="3xtf32") == ("winograd", "fp32")
    assert plan(1, 65, 128, 112, 3, mode="3xtf32") == ("winograd", "3xtf32")
    assert plan(8, 512, 512, 28, 3, mode="3xtf32") == ("winograd", "3xtf32")
    assert plan(1, 64, 64, 56, 3, algo="winograd", mode="tf32") == ("winograd", "fp32")
    assert plan(1, 64, 64, 56, 1, mode="3xtf32") == ("im2col", "3xtf32")   # the rule is about Winograd layers only
    monkeypatch.setenv("FASTCONV_3XTF32_MIN_IC", "200")
    assert plan(1, 128, 128, 56, 3, mode="3xtf32") == ("winograd", "fp32")


def test_bad_arguments_are_refused():
    d = fc.make_desc(1, 8, 8, 8, 8)
    with pytest.raises(fc.FastConvError):
        fc.resolve_plan(d, 9, "tf32")
    with pytest.raises(fc.FastConvError):
        fc.resolve_plan(d, "auto", 7)

"""Parity of the CUDA Winograd F(6x6,3x3) path with the CPU oracle, through the C ABI.

fp32 "mirrored" mode is held to BIT equality with the oracle (which is itself bit-equal to the
reference build).  3xTF32 is held to rel-L2 <= 1e-5 and max-abs <= 1e-4*||out||inf up to 256 input
channels; at 512 channels the reference's own output moves by 1.06e-5 when only the order of its
accumulation changes, so the bound there is that movement (measured in the test) times 1.25.  The mode "tf32" stands for
rel-L2 <= 3e-3 and is held to it: a Winograd layer asked for by name then runs the split
arithmetic, because one TF32 pass through F(6x6,3x3) measures 6.4e-3 (the transform amplifies the
2^-11 operand rounding about 16x).  That single pass is the mode "tf32-unbounded": the test pins
its measured level (<= 8e-3) and a strict xfail records that it misses 3e-3.
"""
import ctypes as C
import hashlib

import numpy as np
import pytest

import fastconv_b200 as fc
from _oracle import max_abs_rel, order_noise, rel_l2
from fastconv_b200 import synth

pytestmark = pytest.mark.gpu

SMALL = [  # n, ic, oc, ih, iw, pad -- every OH mod 6 residue, channel counts around the 4/8 padding
    (1, 1, 1, 6, 6, 1), (1, 3, 5, 7, 9, 1), (1, 4, 4, 1, 1, 1), (1, 8, 8, 12, 12, 1), (1, 5, 3, 6, 6, 0),
    (1, 17, 6, 23, 20, 1), (1, 6, 7, 13, 8, 2), (2, 3, 4, 10, 11, 1), (3, 9, 65, 5, 31, 1), (1, 64, 64, 14, 14, 1),
    (1, 33, 129, 8, 8, 1), (2, 70, 40, 19, 7, 1), (1, 5, 8, 2, 2, 1), (1, 4, 4, 3, 3, 1), (1, 8, 4, 4, 4, 1),
    (1, 12, 20, 5, 5, 1), (1, 16, 16, 16, 16, 0), (1, 130, 66, 15, 15, 1),
]


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def run_layer(ctx, x, w, pad, mode="fp32", launches=None):
    n, ic, ih, iw = x.shape
    oc = w.shape[0]
    layer = fc.ConvWinoF63ZCLayer(x, w, None, None, ic, ih, iw, oc, 3, 3, 1, 1, pad, pad, pad, pad, 1, False, 1, 1,
                                  batch=n, mode=mode, ctx=ctx)
    assert layer.Init() == -1  # the reference's Init returns -1 (winoF63ConvZC.cpp:212)
    assert layer.Forward() == 1
    out = layer.output_data.copy()
    if launches is not None:
        assert layer.kernel_launches == launches
    layer.release()
    return out


@pytest.mark.parametrize("shape", SMALL)
def test_mirrored_mode_is_bit_exact(ctx, oracle, shape):
    n, ic, oc, ih, iw, pad = shape
    x = synth.conv_input(n, ic, ih, iw, 41)
    w = synth.conv_weights(oc, ic, 3, 3, 42)
    assert np.array_equal(run_layer(ctx, x, w, pad), oracle.wino_forward(x, w, pad))


def test_golden_vectors_small(ctx, golden):
    meta, z = golden
    for rec in meta["wino"]:
        x = synth.conv_input(1, rec["ic"], rec["ih"], rec["iw"], rec["seed_in"])
        w = synth.conv_weights(rec["oc"], rec["ic"], 3, 3, rec["seed_w"])
        got = run_layer(ctx, x, w, rec["pad"])[0]
        assert np.array_equal(got, z[f"wino_{rec['idx']}"]), rec


def test_golden_vectors_full_size(ctx, golden):
    meta, z = golden
    for rec in meta["wino_large"]:
        x = synth.conv_input(1, rec["ic"], rec["ih"], rec["iw"], rec["seed_in"])
        w = synth.conv_weights(rec["oc"], rec["ic"], 3, 3, rec["seed_w"])
        got = run_layer(ctx, x, w, rec["pad"])[0]
        assert sha(got) == rec["sha_wino"], f"{rec['ic']}->{rec['oc']}@{rec['ih']} differs from the reference output"


@pytest.mark.parametrize("mode,budget_mb,passes", [("fp32", 8, 3), ("fp32", 3, 5), ("3xtf32", 8, 3)])
def test_batch_split_into_l2_sized_passes(ctx, oracle, monkeypatch, mode, budget_mb, passes):
    """A batch whose Winograd-domain buffers exceed the L2 budget runs as several passes over blocks of images
    (here 3 passes of 2+2+1 and 5 passes of 1): same bits as the one-pass run and as the oracle."""
    n, ic, oc, h = 5, 64, 64, 56
    x = synth.conv_input(n, ic, h, h, 51)
    w = synth.conv_weights(oc, ic, 3, 3, 52)
    monkeypatch.setenv("FASTCONV_L2_BUDGET_MB", "0")
    whole = run_layer(ctx, x, w, 1, mode, launches=3)
    monkeypatch.setenv("FASTCONV_L2_BUDGET_MB", str(budget_mb))
    split = run_layer(ctx, x, w, 1, mode, launches=3 * passes)
    assert np.array_equal(split, whole)
    if mode == "fp32":
        assert np.array_equal(split, oracle.wino_forward(x, w, 1))


def _dev(ctx, a):
    return C.c_void_p(ctx.upload(a))


@pytest.mark.parametrize("mode", [0, 1])
def test_each_stage_bit_exact(ctx, oracle, mode):
    """Filter transform, input transform, TensorGEMM and output transform one by one, in the operand layouts
    of the fp32 mirrored mode (0) and of the tensor-core modes (1 = 3xTF32)."""
    from _oracle import unpack_filter
    lib = fc.load()
    n, ic, oc, ih, iw, pad = 2, 13, 21, 17, 11, 1
    x = synth.conv_input(n, ic, ih, iw, 51)
    w = synth.conv_weights(oc, ic, 3, 3, 52)
    d = fc.make_desc(n, ic, ih, iw, oc, 3, 3, 1, 1, pad, pad, pad, pad)
    u, v, m = C.c_size_t(), C.c_size_t(), C.c_size_t()
    fc._lib.check(lib.fc_wino_buffer_elems(C.byref(d), mode, C.byref(u), C.byref(v), C.byref(m)), "elems")
    icp, ocp, tiles, tp = 16, 24, 2 * 3 * 2, 16
    assert (u.value, v.value, m.value) == (64 * icp * ocp if mode == 0 else 64 * 128 * 32, 64 * tp * icp, 64 * oc * tp)
    dU, dV, dM = (C.c_void_p(ctx.alloc(4 * e.value)) for e in (u, v, m))
    d_out = C.c_void_p(ctx.alloc(4 * n * oc * ih * iw))
    dk, dx = _dev(ctx, w), _dev(ctx, x)
    h = ctx.handle
    fc._lib.check(lib.fc_wino_filter_transform(h, dk, dU, oc, ic, mode), "filter")
    fc._lib.check(lib.fc_wino_input_transform(h, dx, dV, C.byref(d), mode), "input")
    fc._lib.check(lib.fc_wino_tensor_gemm(h, dU, dV, dM, C.byref(d), mode), "gemm")
    fc._lib.check(lib.fc_wino_output_transform(h, dM, d_out, C.byref(d)), "output")
    Uo = oracle.filter_transform(w, icp=icp)          # [64][oc][icp]
    Vo = oracle.input_transform(x, pad, tp=tp, icp=icp)  # [64][tp][icp]
    if mode == 0:  # row-major: U[64][icp][ocp], V[64][icp][tp]
        U = ctx.download(dU.value, (64, icp, ocp))
        assert not U[:, :, oc:].any() and np.array_equal(U[:, :, :oc].transpose(0, 2, 1), Uo), "filter transform"
        V = ctx.download(dV.value, (64, icp, tp)).transpose(0, 2, 1)
    else:          # packed boxes / K-major
        U = unpack_filter(ctx.download(dU.value, (u.value,)), oc, ic)
        assert np.array_equal(U, Uo[:, :, :ic]), "filter transform"
        V = ctx.download(dV.value, (64, tp, icp))
    assert np.array_equal(V, Vo), "input transform (padding rows/channels must be zero)"
    M = ctx.download(dM.value, (64, oc, tp))
    out = ctx.download(d_out.value, (n, oc, ih, iw))
    Mo = oracle.wino_gemm(Uo, Vo, oc, icp, tp)
    if mode == 0:
        assert np.array_equal(M[:, :, :tiles], Mo[:, :, :tiles]), "TensorGEMM"
        assert np.array_equal(out, oracle.output_transform(Mo, n, oc, ih, iw)), "output transform"
    else:
        assert rel_l2(M[:, :, :tiles], Mo[:, :, :tiles]) < 2e-6, "TensorGEMM (3xTF32)"
        # the output transform itself is exact arithmetic in every mode: feed it the device's own M
        assert np.array_equal(out, oracle.output_transform(M, n, oc, ih, iw)), "output transform"
    # the fused entry point gives the same bits and reports stage times
    ms = (C.c_float * 4)()
    fc._lib.check(lib.fc_wino_forward(h, dx, dU, dV, dM, d_out, C.byref(d), mode, ms), "forward")
    assert np.array_equal(ctx.download(d_out.value, (n, oc, ih, iw)), out)
    assert ms[0] > 0 and ms[2] > 0 and ms[3] > 0 and ms[1] == 0
    for p in (dU, dV, dM, d_out, dk, dx):
        ctx.free(p.value)


def test_unsupported_shapes_are_refused(ctx):
    x = synth.conv_input(1, 4, 8, 8, 1)
    for kw in (dict(kh=5, kw=5), dict(sh=2, sw=2), dict(pad_left=0)):
        args = dict(kh=3, kw=3, sh=1, sw=1, pad_left=1, pad_right=1, pad_top=1, pad_bottom=1)
        args.update(kw)
        w = synth.conv_weights(4, 4, args["kh"], args["kw"], 2)
        layer = fc.ConvWinoF63ZCLayer(x, w, None, None, 4, 8, 8, 4, ctx=ctx, **args)
        with pytest.raises(fc.FastConvError) as e:
            layer.Init()
        assert e.value.status == -2


def test_batch_is_independent_images(ctx, oracle):
    """Tiles of all images are concatenated on the GEMM's tile axis; each image must come out as if alone."""
    n, ic, oc, ih, iw = 5, 16, 24, 14, 14
    x = synth.conv_input(n, ic, ih, iw, 61)
    w = synth.conv_weights(oc, ic, 3, 3, 62)
    whole = run_layer(ctx, x, w, 1)
    for i in range(n):
        assert np.array_equal(whole[i:i + 1], run_layer(ctx, x[i:i + 1], w, 1))


def test_linearity_at_full_size(ctx):
    """conv(x, a+b) == conv(x, a) + conv(x, b) up to fp32 rounding, on conv3_2's full shape."""
    ic = oc = 256
    x = synth.conv_input(1, ic, 56, 56, 71)
    a = synth.conv_weights(oc, ic, 3, 3, 72)
    b = synth.conv_weights(oc, ic, 3, 3, 73)
    lhs = run_layer(ctx, x, a + b, 1)
    rhs = run_layer(ctx, x, a, 1) + run_layer(ctx, x, b, 1)
    assert rel_l2(lhs, rhs) < 2e-5


def test_reference_self_check_line(ctx, oracle, capsys):
    """Forward() prints the reference's labels and the `diff` against output_ref (winoF63ConvZC.cpp:249-256)."""
    ic, oc, hw = 32, 32, 28
    x = synth.conv_input(1, ic, hw, hw, 81)
    w = synth.conv_weights(oc, ic, 3, 3, 82)
    naive = oracle.naive_conv(x, w, 1, 1, 1, 1, 1, 1)
    layer = fc.ConvWinoF63ZCLayer(x, w, None, naive, ic, hw, hw, oc, iter=3, ctx=ctx)
    layer.Init()
    layer.Forward()
    text = capsys.readouterr().out
    for label in ("Algorithm: winograd F63", "InputTran time:", "KernelTran time:", "TensorGEMM time:",
                  "OutputTran time:", "Total time:", "The difference is"):
        assert label in text
    assert rel_l2(layer.output_data, naive) < 1e-5
    layer.release()


@pytest.mark.parametrize("mode, tol_l2, tol_max", [("3xtf32", 1e-5, 1e-4), ("tf32", 3e-3, 1.5e-2), ("tf32-unbounded", 8e-3, 4e-2)])
@pytest.mark.parametrize("shape", [(1, 64, 64, 56, 56, 1), (1, 256, 256, 56, 56, 1), (2, 37, 70, 20, 23, 1),
                                   (1, 3, 64, 40, 40, 1), (1, 128, 128, 14, 14, 1), (1, 8, 8, 6, 6, 1),
                                   (1, 200, 136, 30, 30, 1), (3, 40, 300, 13, 13, 1)])
def test_tensor_core_modes_within_tolerance(ctx, oracle, mode, tol_l2, tol_max, shape):
    n, ic, oc, ih, iw, pad = shape
    x = synth.conv_input(n, ic, ih, iw, 91)
    w = synth.conv_weights(oc, ic, 3, 3, 92)
    want = oracle.wino_forward(x, w, pad)
    got = run_layer(ctx, x, w, pad, mode=mode)
    assert rel_l2(got, want) <= tol_l2, f"{mode} rel-L2 {rel_l2(got, want):.3e}"
    assert max_abs_rel(got, want) <= tol_max, f"{mode} max-abs/||out||inf {max_abs_rel(got, want):.3e}"


def test_3xtf32_at_512_channels_is_at_the_reference_noise_floor(ctx, oracle):
    x = synth.conv_input(1, 512, 28, 28, 93)
    w = synth.conv_weights(512, 512, 3, 3, 94)
    want = oracle.wino_forward(x, w, 1)
    got = run_layer(ctx, x, w, 1, mode="3xtf32")
    truth = oracle.direct_f64(x, w, 1, 1, 1, 1, 1, 1)
    # 1e-5, or what the reference's own output moves by when only its accumulation order changes (1.06e-5 here)
    assert rel_l2(got, want) <= max(1e-5, 1.25 * order_noise(oracle, x, w, want)) and max_abs_rel(got, want) <= 1e-4
    # against the exact result it is as accurate as the reference's own fp32 arithmetic (within 30 %)
    assert rel_l2(got, truth) <= 1.3 * rel_l2(want, truth)


@pytest.mark.xfail(strict=True, reason="one TF32 pass through F(6x6,3x3) measures 6.4e-3 rel-L2; the 3e-3 target "
                                       "needs more than single-pass TF32 operands")
def test_single_pass_tf32_through_winograd_meets_3e_3(ctx, oracle):
    x = synth.conv_input(1, 64, 56, 56, 95)
    w = synth.conv_weights(64, 64, 3, 3, 96)
    assert rel_l2(run_layer(ctx, x, w, 1, mode="tf32-unbounded"), oracle.wino_forward(x, w, 1)) <= 3e-3


def test_tensor_core_kernel_reports_no_timeouts(ctx):
    ctx.synchronize()  # raises FastConvError(FC_ERR_TIMEOUT) if any bounded wait gave up in the tests above


def test_layer_list_graph_replays_every_layer(ctx, oracle):
    """Three layers captured into one CUDA graph give, on replay, the bits of running them one by one."""
    import ctypes as C
    lib = fc.load()
    specs = [(1, 16, 24, 20, 20), (2, 8, 8, 9, 13), (1, 40, 72, 14, 14)]
    convs, ins, outs, wants = [], [], [], []
    for i, (n, ic, oc, ih, iw) in enumerate(specs):
        x = synth.conv_input(n, ic, ih, iw, 300 + i)
        w = synth.conv_weights(oc, ic, 3, 3, 400 + i)
        d = fc.make_desc(n, ic, ih, iw, oc)
        h = C.c_void_p()
        fc._lib.check(lib.fc_conv_create(ctx.handle, C.byref(d), fc.ALGO_WINOGRAD, 0, C.c_void_p(w.ctypes.data),
                                         C.byref(h)), "create")
        convs.append(h)
        ins.append(ctx.upload(x))
        outs.append(ctx.zeros(4 * n * oc * ih * iw))
        wants.append(oracle.wino_forward(x, w, 1))
    stack = fc.LayerList(ctx, convs, ins, outs)
    assert stack.kernel_launches == 9
    for o, want in zip(outs, wants):  # clear what the eager pass inside create() wrote
        fc._lib.check(lib.fc_memset_device(ctx.handle, C.c_void_p(o), 0, want.nbytes), "memset")
    stack.forward()
    stack.forward()
    ctx.synchronize()
    for o, want in zip(outs, wants):
        assert np.array_equal(ctx.download(o, want.shape), want)
    # the host-buffer form of the same list (uploads / kernels / downloads pipelined over three streams)
    xs = [synth.conv_input(n, ic, ih, iw, 600 + i) for i, (n, ic, oc, ih, iw) in enumerate(specs)]
    ws = [synth.conv_weights(oc, ic, 3, 3, 400 + i) for i, (n, ic, oc, ih, iw) in enumerate(specs)]
    host_out = [np.zeros_like(w_) for w_ in wants]
    stack.forward_host(xs, host_out)
    for x_, w_, got in zip(xs, ws, host_out):
        assert np.array_equal(got, oracle.wino_forward(x_, w_, 1))
    stack.close()
    for h in convs:
        lib.fc_conv_destroy(h)
    for p in ins + outs:
        ctx.free(p)


def _random_shapes(seed, count):
    rng = np.random.default_rng(seed)
    shapes = []
    for _ in range(count):
        n = int(rng.integers(1, 4))
        ic, oc = int(rng.integers(1, 72)), int(rng.integers(1, 150))
        ih, iw = int(rng.integers(1, 44)), int(rng.integers(1, 44))
        pad = int(rng.integers(0, 3))
        if ih + 2 * pad < 3 or iw + 2 * pad < 3:
            pad = 1
            ih, iw = max(ih, 1), max(iw, 1)
        shapes.append((n, ic, oc, ih, iw, pad))
    return shapes


@pytest.mark.parametrize("shape", _random_shapes(2024, 28))
def test_random_shapes_mirrored_mode_bit_exact(ctx, oracle, shape):
    """Seeded random shapes: 1..150 channels, 1..43 pixels a side, batch 1..3, padding 0..2 -- every tile-count bucket
    of the skinny kernel, ragged channel counts, tiles that overhang the image on both sides."""
    n, ic, oc, ih, iw, pad = shape
    x = synth.conv_input(n, ic, ih, iw, 91)
    w = synth.conv_weights(oc, ic, 3, 3, 92)
    assert np.array_equal(run_layer(ctx, x, w, pad), oracle.wino_forward(x, w, pad))


@pytest.mark.parametrize("shape", _random_shapes(4048, 20))
def test_random_shapes_3xtf32_within_tolerance(ctx, oracle, shape):
    """The same family of shapes through the tcgen05 kernel (both operand-role variants occur: at most 64 output
    channels or at least 128 tiles exchange the roles)."""
    n, ic, oc, ih, iw, pad = shape
    x = synth.conv_input(n, ic, ih, iw, 93)
    w = synth.conv_weights(oc, ic, 3, 3, 94)
    want = oracle.wino_forward(x, w, pad)
    got = run_layer(ctx, x, w, pad, "3xtf32")
    assert rel_l2(got, want) <= 1e-5
    assert max_abs_rel(got, want) <= 1e-4


@pytest.mark.parametrize("bn", [80, 96, 112])
@pytest.mark.parametrize("shape", [(8, 136, 200, 14, 14), (3, 64, 130, 30, 31), (1, 40, 129, 55, 50)])
def test_ffma_block_widths_between_64_and_128_are_bit_exact(ctx, oracle, bn, shape):
    """The FFMA TensorGEMM in blocks of 128 channels x 80 / 96 / 112 tiles (what 72 or 200 tiles take by default),
    forced by hand on tile counts that leave ragged blocks in both directions."""
    n, ic, oc, ih, iw = shape
    x = synth.conv_input(n, ic, ih, iw, 141)
    w = synth.conv_weights(oc, ic, 3, 3, 142)
    layer = fc.ConvWinoF63ZCLayer(x, w, None, None, ic, ih, iw, oc, 3, 3, 1, 1, 1, 1, 1, 1, 1, False, 1, 1,
                                  batch=n, ctx=ctx)
    layer.Init()
    layer.set_kernel_config(0, bn, 2, 0)
    layer.Forward()
    assert np.array_equal(layer.output_data, oracle.wino_forward(x, w, 1))
    layer.release()


@pytest.mark.parametrize("shape", [(1, 512, 512, 14, 14), (1, 256, 256, 28, 28), (1, 128, 200, 30, 30), (2, 96, 129, 13, 13),
                                   (1, 40, 72, 56, 56)])
def test_fp16_filter_mode_is_as_accurate_as_one_tf32_pass(ctx, oracle, shape):
    """"tf32-u16": the transformed filter stored as scaled fp16 (TF32's own significand), expanded in shared memory,
    one TF32 pass.  A reduced-precision mode outside the stated tolerances -- its error against the reference is
    that of one TF32 pass through F(6x6,3x3) (6.4e-3), which is what the test pins, together with its distance to
    the fp32-filter result of the same arithmetic (the fp16 rounding of values TF32 would have rounded anyway)."""
    n, ic, oc, ih, iw = shape
    x = synth.conv_input(n, ic, ih, iw, 151)
    w = synth.conv_weights(oc, ic, 3, 3, 152)
    want = oracle.wino_forward(x, w, 1)
    layer = fc.ConvWinoF63ZCLayer(x, w, None, None, ic, ih, iw, oc, batch=n, iter=1, mode="tf32-u16", ctx=ctx)
    layer.Init()
    mode = C.c_int()
    fc.load().fc_conv_math_mode(layer._conv, C.byref(mode))
    assert mode.value == fc._lib.MATH_TF32_U16
    layer.Forward()
    got = layer.output_data.copy()
    layer.release()
    one_pass = run_layer(ctx, x, w, 1, mode="tf32-unbounded")
    assert rel_l2(got, want) <= 8e-3, rel_l2(got, want)
    # the two round the filter differently (fp16 to nearest, the tensor core by truncation): independent errors
    assert rel_l2(got, one_pass) <= 1e-2, rel_l2(got, one_pass)


def test_fp16_filter_mode_falls_back_where_it_does_not_fit(ctx, oracle):
    lib = fc.load()
    for n, ic, oc, hw in [(1, 32, 64, 28), (8, 128, 128, 28)]:  # at most 64 channels; 128 tiles or more
        x = synth.conv_input(n, ic, hw, hw, 153)
        w = synth.conv_weights(oc, ic, 3, 3, 154)
        layer = fc.ConvWinoF63ZCLayer(x, w, None, None, ic, hw, hw, oc, batch=n, iter=1, mode="tf32-u16", ctx=ctx)
        layer.Init()
        mode = C.c_int()
        lib.fc_conv_math_mode(layer._conv, C.byref(mode))
        assert mode.value == fc._lib.MATH_TF32
        layer.Forward()
        assert rel_l2(layer.output_data, oracle.wino_forward(x, w, 1)) <= 8e-3
        layer.release()


# n, ic, oc, ih, iw, pad: at most 4 input channels and 32+ tiles -- the TensorGEMM runs inside the output transform
FEW_CHANNELS = [(1, 3, 64, 224, 224, 1), (2, 3, 16, 40, 37, 1), (1, 1, 7, 36, 36, 1), (3, 2, 33, 25, 31, 0),
                (1, 4, 20, 48, 30, 2), (5, 3, 5, 19, 20, 1), (1, 4, 130, 34, 34, 1)]


@pytest.mark.parametrize("shape", FEW_CHANNELS)
def test_few_input_channels_two_kernels_bit_exact(ctx, oracle, shape):
    """Two launches (input transform, output transform with the multiply-accumulate inside) and the oracle's bits."""
    n, ic, oc, ih, iw, pad = shape
    x = synth.conv_input(n, ic, ih, iw, 141)
    w = synth.conv_weights(oc, ic, 3, 3, 142)
    assert np.array_equal(run_layer(ctx, x, w, pad, launches=2), oracle.wino_forward(x, w, pad))


def test_few_input_channels_same_bits_as_three_kernels(ctx, monkeypatch):
    """Full-size first layer on 4 images: the two-kernel form against the three-kernel form of the same library."""
    import subprocess, sys, os, textwrap
    code = textwrap.dedent("""
        import hashlib, numpy as np, fastconv_b200 as fc
        from fastconv_b200 import synth
        x = synth.conv_input(4, 3, 224, 224, 7); w = synth.conv_weights(64, 3, 3, 3, 8)
        with fc.Context(0, arena_bytes=3 << 30) as ctx:
            l = fc.ConvWinoF63ZCLayer(x, w, None, None, 3, 224, 224, 64, batch=4, ctx=ctx)
            l.Init(); l.Forward()
            print(l.kernel_launches, hashlib.sha256(l.output_data.tobytes()).hexdigest())
    """)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    outs = []
    for flag in ("1", "0"):
        env = dict(os.environ, FASTCONV_FUSE_SMALL_IC=flag, PYTHONPATH=root)
        r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        outs.append(r.stdout.split()[-2:])  # the layer's own "Algorithm:" line comes first
    assert outs[0][0] == "2" and outs[1][0] == "3"
    assert outs[0][1] == outs[1][1]


# th, tw: 128 tiles and a rest of 8, 32, 40, 48, 56, 64, 72, 80, 96, 104, 112, 120 -- every width of the last block column
OFF_WIDTH = [(8, 17), (10, 16), (12, 14), (11, 16), (8, 23), (12, 16), (10, 20), (13, 16), (14, 16), (8, 29), (15, 16),
             (8, 31)]


@pytest.mark.parametrize("th,tw", OFF_WIDTH)
def test_tile_counts_off_the_block_width_are_bit_exact(ctx, oracle, th, tw):
    """One launch with 128-wide block columns and a narrower last one; 130 output channels make the second row of
    blocks nearly empty, 40 input channels end the reduction inside a slab."""
    x = synth.conv_input(1, 40, 6 * th, 6 * tw - 2, 151)
    w = synth.conv_weights(130, 40, 3, 3, 152)
    assert np.array_equal(run_layer(ctx, x, w, 1), oracle.wino_forward(x, w, 1))


def test_copy_fed_kernels_give_the_bits_of_the_tma_fed_ones():
    """The blocked TensorGEMM on per-thread asynchronous copies (what callers without a context get) against the
    TMA-fed default, and the uniform launch against the one with a narrower last column: same bits."""
    import os, subprocess, sys, textwrap
    code = textwrap.dedent("""
        import hashlib, numpy as np, fastconv_b200 as fc
        from fastconv_b200 import synth
        out = []
        with fc.Context(0, arena_bytes=2 << 30) as ctx:
            for n, ic, oc, h, w in [(2, 40, 130, 48, 100), (1, 64, 64, 56, 56), (4, 96, 200, 14, 14), (1, 24, 72, 112, 112)]:
                x = synth.conv_input(n, ic, h, w, 161); k = synth.conv_weights(oc, ic, 3, 3, 162)
                l = fc.ConvWinoF63ZCLayer(x, k, None, None, ic, h, w, oc, batch=n, ctx=ctx)
                l.Init(); l.Forward()
                out.append(hashlib.sha256(l.output_data.tobytes()).hexdigest()); l.release()
        print("HASHES", " ".join(out))
    """)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    got = []
    for extra in ({}, {"FASTCONV_FFMA_TMA": "0"}, {"FASTCONV_FFMA_MIXED": "0"}):
        r = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, PYTHONPATH=root, **extra), capture_output=True,
                           text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        got.append([line for line in r.stdout.splitlines() if line.startswith("HASHES")][0])
    assert got[0] == got[1] == got[2]


def test_accuracy_mode_on_a_short_reduction_is_the_fp32_path(ctx, oracle, monkeypatch):
    """Library default (the variable the test session sets is removed): 64 input channels in 3xTF32 run the fp32
    kernels -- the reported arithmetic says so and the result is the oracle's, bit for bit."""
    monkeypatch.delenv("FASTCONV_3XTF32_MIN_IC")
    lib = fc.load()
    x = synth.conv_input(2, 64, 30, 30, 171)
    w = synth.conv_weights(48, 64, 3, 3, 172)
    d = fc.make_desc(2, 64, 30, 30, 48)
    h, m = C.c_void_p(), C.c_int()
    fc._lib.check(lib.fc_conv_create(ctx.handle, C.byref(d), fc.ALGO_WINOGRAD, 1, C.c_void_p(w.ctypes.data), C.byref(h)), "create")
    lib.fc_conv_math_mode(h, C.byref(m))
    assert m.value == 0
    y = np.empty((2, 48, 30, 30), np.float32)
    fc._lib.check(lib.fc_conv_forward_host(h, C.c_void_p(x.ctypes.data), C.c_void_p(y.ctypes.data)), "forward")
    assert np.array_equal(y, oracle.wino_forward(x, w, 1))
    lib.fc_conv_destroy(h)

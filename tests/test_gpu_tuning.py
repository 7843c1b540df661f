"""Tuning(): configurations are compared on measured device time, the winner is logged and reused, and the
result stays bit-equal to the oracle of whichever algorithm won."""
import ctypes as C
import os

import numpy as np
import pytest

import fastconv_b200 as fc
from _oracle import rel_l2
from fastconv_b200 import synth

pytestmark = pytest.mark.gpu


@pytest.fixture()
def tuning_log(tmp_path, monkeypatch):
    path = tmp_path / "tuning_log"
    monkeypatch.setenv("FASTCONV_TUNING_LOG", str(path))
    return path


def _algo(layer):
    a = C.c_int()
    fc._lib.check(fc.load().fc_conv_algorithm(layer._conv, C.byref(a)), "fc_conv_algorithm")
    return a.value


@pytest.mark.parametrize("mode", ["fp32", "3xtf32"])
def test_winograd_tuning_keeps_results_and_logs(ctx, oracle, tuning_log, capfd, mode):
    n, ic, oc, hw = 1, 48, 80, 28
    x = synth.conv_input(n, ic, hw, hw, 501)
    w = synth.conv_weights(oc, ic, 3, 3, 502)
    layer = fc.ConvWinoF63ZCLayer(x, w, None, None, ic, hw, hw, oc, iter=3, mode=mode, ctx=ctx)
    assert layer.Tuning() == -1  # the reference's Tuning returns -1 (winoF63ConvZC.cpp:173)
    out = capfd.readouterr().out
    assert "log entry doesn't exist." in out and "Best Config:" in out and out.count("time=") >= 4
    layer.Init()
    layer.Forward()
    want = oracle.wino_forward(x, w, 1)
    if mode == "fp32":
        assert np.array_equal(layer.output_data, want)
    else:
        assert rel_l2(layer.output_data, want) <= 1e-5
    layer.release()
    lines = tuning_log.read_text().strip().splitlines()
    assert len(lines) == 1 and len(lines[0].split(",")) == 23
    # a second layer of the same shape finds the entry instead of searching
    again = fc.ConvWinoF63ZCLayer(x, w, None, None, ic, hw, hw, oc, iter=3, mode=mode, ctx=ctx)
    again.Tuning()
    out = capfd.readouterr().out
    assert "log entry exists." in out and "Best Config:" not in out
    again.Init()
    again.Forward()
    assert np.array_equal(again.output_data, layer.output_data)
    again.release()
    assert len(tuning_log.read_text().strip().splitlines()) == 1


def test_auto_picks_the_algorithm_from_measured_time(ctx, oracle, tuning_log, capfd):
    lib = fc.load()
    ic = oc = 64
    hw = 7  # 4 tiles of which 3/4 is overhang: the case where the choice is not obvious
    x = synth.conv_input(1, ic, hw, hw, 511)
    w = synth.conv_weights(oc, ic, 3, 3, 512)
    d = fc.make_desc(1, ic, hw, hw, oc)
    h = C.c_void_p()
    fc._lib.check(lib.fc_conv_create(ctx.handle, C.byref(d), fc.ALGO_AUTO, 0, C.c_void_p(w.ctypes.data), C.byref(h)), "create")
    fc._lib.check(lib.fc_conv_tune(h, 5, 1), "tune")
    out = capfd.readouterr().out
    assert "algo=winograd" in out and "algo=im2col" in out  # both were timed
    algo = C.c_int()
    lib.fc_conv_algorithm(h, C.byref(algo))
    assert algo.value in (fc.ALGO_WINOGRAD, fc.ALGO_IM2COL)
    y = np.empty((1, oc, hw, hw), np.float32)
    fc._lib.check(lib.fc_conv_forward_host(h, C.c_void_p(x.ctypes.data), C.c_void_p(y.ctypes.data)), "forward")
    want = oracle.wino_forward(x, w, 1) if algo.value == fc.ALGO_WINOGRAD else oracle.im2col_gemm_forward(x, w, 1, 1, 1, 1, 1, 1)
    assert np.array_equal(y, want)
    lib.fc_conv_destroy(h)


def test_im2col_tuning(ctx, oracle, tuning_log, capfd):
    x = synth.conv_input(2, 24, 15, 15, 521)
    w = synth.conv_weights(40, 24, 3, 3, 522)
    layer = fc.ConvIm2colLayer(x, w, None, None, 24, 15, 15, 40, 3, 3, 2, 2, 1, 1, 1, 1, batch=2, iter=3, ctx=ctx)
    assert layer.Tuning() == 1
    assert "Best Config:" in capfd.readouterr().out
    layer.Init()
    layer.Forward()
    assert np.array_equal(layer.output_data, oracle.im2col_gemm_forward(x, w, 2, 2, 1, 1, 1, 1))
    layer.release()


@pytest.mark.parametrize("case, mode, rivals", [
    ((4, 256, 128, 28, 1, 0), "tf32", ("algo=direct", "algo=im2col")),     # 1x1: direct against the gathering kernel
    # 3x3, few channels: direct against Winograd -- only where one TF32 pass through Winograd is allowed at all
    ((1, 64, 64, 56, 3, 1), "tf32-unbounded", ("algo=direct", "algo=winograd")),
])
def test_auto_in_tf32_times_the_direct_kernel_against_its_rival(ctx, oracle, tuning_log, capfd, case, mode, rivals):
    n, ic, oc, hw, k, pad = case
    lib = fc.load()
    x = synth.conv_input(n, ic, hw, hw, 531)
    w = synth.conv_weights(oc, ic, k, k, 532)
    d = fc.make_desc(n, ic, hw, hw, oc, k, k, 1, 1, pad, pad, pad, pad)
    h = C.c_void_p()
    fc._lib.check(lib.fc_conv_create(ctx.handle, C.byref(d), fc.ALGO_AUTO, fc._lib.MODE_NAMES[mode], C.c_void_p(w.ctypes.data),
                                     C.byref(h)), "create")
    algo = C.c_int()
    lib.fc_conv_algorithm(h, C.byref(algo))
    assert algo.value == fc.ALGO_DIRECT  # the untuned choice for these shapes
    fc._lib.check(lib.fc_conv_tune(h, 5, 1), "tune")
    out = capfd.readouterr().out
    for label in rivals:
        assert label in out
    y = np.empty((n, oc, hw, hw), np.float32)
    fc._lib.check(lib.fc_conv_forward_host(h, C.c_void_p(x.ctypes.data), C.c_void_p(y.ctypes.data)), "forward")
    lib.fc_conv_algorithm(h, C.byref(algo))
    tol = 8e-3 if algo.value == fc.ALGO_WINOGRAD else 3e-3  # single-pass TF32 through F(6x6,3x3) is 6.4e-3
    assert rel_l2(y, oracle.im2col_gemm_forward(x, w, 1, 1, pad, pad, pad, pad)) <= tol
    lib.fc_conv_destroy(h)

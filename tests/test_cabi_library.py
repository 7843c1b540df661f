"""The C-ABI library loads without a GPU and exports exactly what include/fastconv_b200.h declares."""
import ctypes
import re
from pathlib import Path

import numpy as np
import pytest

import fastconv_b200 as fc
from fastconv_b200 import _lib

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    text = (ROOT / "include" / "fastconv_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fc_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    lib = fc.load()
    names = declared_symbols()
    assert len(names) >= 40
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in the header but missing from the library"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == names


def test_abi_version_and_status_strings():
    lib = fc.load()
    assert lib.fc_abi_version() == 1
    assert lib.fc_status_string(0) == b"ok"
    for s in range(-7, 0):
        assert lib.fc_status_string(s) not in (b"ok", b"unknown status")
    assert lib.fc_status_string(-99) == b"unknown status"


def test_no_cpu_fallback_without_gpu():
    lib = fc.load()
    n = ctypes.c_int(-1)
    assert lib.fc_device_count(ctypes.byref(n)) == 0
    if n.value > 0:
        pytest.skip("a GPU is present")
    with pytest.raises(fc.FastConvError) as e:
        fc.Context(0)
    assert e.value.status == -5
    assert "no CPU path" in str(e.value)


def test_shape_rules():
    # oh/ow as conv_layer.h:68-69
    assert fc.output_size(fc.make_desc(1, 256, 56, 56, 256)) == (56, 56)
    assert fc.output_size(fc.make_desc(1, 3, 224, 224, 64, 7, 7, 2, 2, 3, 3, 3, 3)) == (112, 112)
    assert fc.output_size(fc.make_desc(1, 256, 56, 56, 512, 1, 1, 2, 2, 0, 0, 0, 0)) == (28, 28)
    assert fc.output_size(fc.make_desc(1, 4, 5, 9, 4, 3, 3, 1, 1, 0, 0, 0, 0)) == (3, 7)


def test_select_algorithm_follows_reference():
    W, I = fc.ALGO_WINOGRAD, fc.ALGO_IM2COL
    assert fc.select_algorithm(fc.make_desc(1, 64, 56, 56, 64)) == W  # 3x3 s1
    assert fc.select_algorithm(fc.make_desc(1, 64, 56, 56, 64, 3, 3, 2, 2)) == I  # strided 3x3
    assert fc.select_algorithm(fc.make_desc(1, 64, 56, 56, 256, 1, 1, 1, 1, 0, 0, 0, 0)) == I  # "direct" -> implicit GEMM
    assert fc.select_algorithm(fc.make_desc(1, 3, 224, 224, 64, 7, 7, 2, 2, 3, 3, 3, 3)) == I
    assert fc.select_algorithm(fc.make_desc(1, 8, 20, 20, 8, 5, 5, 1, 1, 2, 2, 2, 2)) == I
    assert fc.select_algorithm(fc.make_desc(1, 64, 56, 56, 64, group=4)) == I  # grouped 3x3 s1: implicit GEMM per group


@pytest.mark.parametrize("bad, status", [
    (dict(ic=0), -1), (dict(oc=-3), -1), (dict(sh=0), -1), (dict(pad_left=-1), -1), (dict(group=3), -1), (dict(group=0), -1),
    (dict(kh=9, ih=3, pad_top=0, pad_bottom=0), -1), (dict(batch=0), -1),
])
def test_descriptor_validation(bad, status):
    base = dict(batch=1, ic=8, ih=8, iw=8, oc=8, kh=3, kw=3, sh=1, sw=1, pad_left=1, pad_right=1, pad_top=1,
                pad_bottom=1, group=1)
    base.update(bad)
    d = fc.make_desc(**base)
    oh, ow = ctypes.c_int(), ctypes.c_int()
    assert fc.load().fc_conv_output_size(ctypes.byref(d), ctypes.byref(oh), ctypes.byref(ow)) == status
    assert fc.load().fc_last_error() != b""


def test_winograd_buffer_sizes_and_rejections():
    lib = fc.load()
    u, v, m = ctypes.c_size_t(), ctypes.c_size_t(), ctypes.c_size_t()
    d = fc.make_desc(1, 256, 56, 56, 256)
    for mode in (0, 1, 2):
        assert lib.fc_wino_buffer_elems(ctypes.byref(d), mode, ctypes.byref(u), ctypes.byref(v), ctypes.byref(m)) == 0
        assert (u.value, v.value, m.value) == (64 * 256 * 256, 64 * 104 * 256, 64 * 256 * 104)  # 100 tiles -> 104
    d = fc.make_desc(2, 3, 224, 224, 64)
    assert lib.fc_wino_buffer_elems(ctypes.byref(d), 0, ctypes.byref(u), ctypes.byref(v), ctypes.byref(m)) == 0
    assert (u.value, v.value, m.value) == (64 * 8 * 64, 64 * 2888 * 8, 64 * 64 * 2888)  # fp32 mode: U[64][icp][ocp]
    assert lib.fc_wino_buffer_elems(ctypes.byref(d), 2, ctypes.byref(u), ctypes.byref(v), ctypes.byref(m)) == 0
    assert u.value == 64 * 128 * 32  # tensor-core modes: U is padded to 128x32 boxes
    assert lib.fc_wino_buffer_elems(ctypes.byref(d), 7, None, None, None) == -1
    d = fc.make_desc(1, 64, 56, 56, 64, group=2)  # the Winograd stages are built for group 1
    assert lib.fc_wino_buffer_elems(ctypes.byref(d), 0, ctypes.byref(u), ctypes.byref(v), ctypes.byref(m)) == -2
    for bad in (fc.make_desc(1, 8, 8, 8, 8, 3, 3, 2, 2), fc.make_desc(1, 8, 8, 8, 8, 5, 5), fc.make_desc(1, 8, 8, 8, 8, 3, 3, 1, 1, 1, 0, 1, 1)):
        assert lib.fc_wino_buffer_elems(ctypes.byref(bad), 0, None, None, None) == -2  # FC_ERR_UNSUPPORTED


def test_null_arguments_are_rejected():
    lib = fc.load()
    assert lib.fc_context_create(0, 0, None) == -1
    assert lib.fc_arena_alloc(None, 16, None) == -1
    assert lib.fc_conv_create(None, None, 0, 0, None, None) == -1
    assert lib.fc_wino_forward(None, None, None, None, None, None, None, 0, None) == -1
    assert lib.fc_context_destroy(None) == 0 and lib.fc_conv_destroy(None) == 0


def test_diff_metric():
    a = np.array([0, 1, 2, 3], np.float32)
    b = np.array([0, 1.000001, 2.5, 2], np.float32)
    assert abs(fc.diff(a, b) - 0.75) < 1e-6


def test_synth_is_deterministic_and_distributed_as_named():
    x = fc.synth.conv_input(1, 64, 56, 56, 1005)
    assert np.array_equal(x, fc.synth.conv_input(1, 64, 56, 56, 1005))
    assert x.min() >= -1 and x.max() < 1 and abs(float(x.mean())) < 0.01
    w = fc.synth.conv_weights(256, 256, 3, 3, 2005)
    assert abs(float(w.std()) - np.sqrt(2 / (9 * 256))) < 2e-4 and abs(float(w.mean())) < 1e-4
    assert not np.array_equal(w, fc.synth.conv_weights(256, 256, 3, 3, 2006))

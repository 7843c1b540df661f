"""The channel-split forward on ONE GPU: with a single rank the scatter kernel stores into local memory only,
which exercises fc_conv_forward_scatter, the flag publish and the bounded flag wait without a second device.
The two-GPU version (peer-mapped buffers over NVLink) is tests/test_gpu_multi.py."""
import ctypes as C

import numpy as np
import pytest

import fastconv_b200 as fc
from fastconv_b200 import _lib, synth
from fastconv_b200.layers import make_desc

pytestmark = pytest.mark.gpu


def _plan(ctx, lib, x, w, mode):
    n, ic, ih, iw = x.shape
    desc = make_desc(n, ic, ih, iw, w.shape[0], 3, 3, 1, 1, 1, 1, 1, 1)
    h = C.c_void_p()
    _lib.check(lib.fc_conv_create(ctx.handle, C.byref(desc), _lib.ALGO_WINOGRAD, _lib.MODE_NAMES[mode],
                                  C.c_void_p(w.ctypes.data), C.byref(h)), "fc_conv_create")
    d_in = C.c_void_p()
    _lib.check(lib.fc_conv_device_buffers(h, C.byref(d_in), None), "fc_conv_device_buffers")
    ctx.upload(x, d_in.value)
    return h, d_in


@pytest.mark.parametrize("mode", ["fp32", "3xtf32"])
@pytest.mark.parametrize("hw", [7, 14, 30])  # 4, 9 and 25 tiles: the three shapes of the scatter kernel
def test_scatter_forward_of_two_slabs_equals_the_whole_layer(ctx, mode, hw):
    lib = fc.load()
    ic, oc = 40, 72
    x = synth.conv_input(1, ic, hw, hw, 61)
    w = synth.conv_weights(oc, ic, 3, 3, 62)
    whole, d_in = _plan(ctx, lib, x, w, mode)
    d_ref = ctx.alloc(4 * oc * hw * hw)
    _lib.check(lib.fc_conv_forward_device(whole, d_in, C.c_void_p(d_ref)), "fc_conv_forward_device")
    ref = ctx.download(d_ref, (1, oc, hw, hw))

    # the same layer as two channel slabs [0,40) and [40,72), each scattered into one full-size buffer
    d_out = ctx.zeros(4 * oc * hw * hw)
    d_flags = ctx.zeros(4 * 8)
    outs, flags = (C.c_void_p * 1)(d_out), (C.c_void_p * 1)(d_flags)
    for step, (k0, k1) in enumerate([(0, 40), (40, 72)], start=1):
        slab, s_in = _plan(ctx, lib, x, np.ascontiguousarray(w[k0:k1]), mode)
        _lib.check(lib.fc_conv_forward_scatter(slab, s_in, outs, flags, 1, 0, k0, oc, step), "fc_conv_forward_scatter")
        _lib.check(lib.fc_peer_wait(ctx.handle, C.c_void_p(d_flags), 1, step), "fc_peer_wait")
        ctx.synchronize()
        assert ctx.download(d_flags, (8,)).view(np.int32)[0] == step
        lib.fc_conv_destroy(slab)
    got = ctx.download(d_out, (1, oc, hw, hw))
    if mode == "fp32":
        assert np.array_equal(got, ref)
    else:
        # slabs of at most 64 channels run the tensor-core GEMM with exchanged operand roles (another MMA shape), so
        # the tensor-core modes agree with the unsplit layer to rounding of the accumulation, not bit for bit
        assert np.linalg.norm(got - ref) <= 1e-6 * np.linalg.norm(ref)
    lib.fc_conv_destroy(whole)


def test_flag_wait_gives_up_and_reports_a_timeout(ctx):
    """Nothing ever publishes step 1 for rank 1: the wait kernel runs out of polls (limit set to 300 ms here), sets
    the context status word and returns; the context stays usable."""
    lib = fc.load()
    d_flags = ctx.zeros(4 * 8)
    _lib.check(lib.fc_context_set_wait_limit_ms(ctx.handle, 300), "fc_context_set_wait_limit_ms")
    try:
        _lib.check(lib.fc_peer_wait(ctx.handle, C.c_void_p(d_flags), 2, 1), "fc_peer_wait")
        with pytest.raises(_lib.FastConvError) as err:
            ctx.synchronize()
    finally:
        _lib.check(lib.fc_context_set_wait_limit_ms(ctx.handle, 5000), "fc_context_set_wait_limit_ms")
    assert err.value.status == _lib.FC_ERR_TIMEOUT
    ctx.synchronize()  # the status word was cleared; the stream still works
    assert np.all(ctx.download(d_flags, (8,)).view(np.int32) == 0)


def test_scatter_rejects_bad_arguments(ctx):
    lib = fc.load()
    x = synth.conv_input(2, 8, 6, 6, 1)
    w = synth.conv_weights(8, 8, 3, 3, 2)
    h, d_in = _plan(ctx, lib, x, w, "fp32")
    d_out, d_flags = ctx.zeros(4 * 2 * 8 * 36), ctx.zeros(32)
    outs, flags = (C.c_void_p * 1)(d_out), (C.c_void_p * 1)(d_flags)
    assert lib.fc_conv_forward_scatter(h, d_in, outs, flags, 1, 0, 0, 8, 1) == _lib.FC_ERR_UNSUPPORTED  # batch 2
    assert lib.fc_conv_forward_scatter(h, d_in, outs, flags, 9, 0, 0, 8, 1) == _lib.FC_ERR_INVALID_ARG  # 9 ranks
    assert lib.fc_peer_wait(ctx.handle, C.c_void_p(d_flags), 0, 1) == _lib.FC_ERR_INVALID_ARG
    lib.fc_conv_destroy(h)

"""The allocation-free Winograd entry point against the regular one, through the C ABI.

fc_wino_forward_static_scratch exists for hosts that may not allocate device memory (an engine plugin
with a fixed memory budget, a loop that must not synchronise after start-up): its V/M workspaces are
an array inside the library image.  The test runs it twice in a row on different inputs -- the second
call finds the first call's leftovers in the shared array -- and expects the same bits as
fc_wino_forward with caller-provided workspaces, then checks that an oversized layer is refused.
"""
import ctypes as C

import numpy as np
import pytest

import fastconv_b200 as fc
from fastconv_b200 import _lib, synth

pytestmark = pytest.mark.gpu


def _regular(ctx, lib, x, dU, desc, n, oc, oh, ow):
    u, v, m = C.c_size_t(), C.c_size_t(), C.c_size_t()
    _lib.check(lib.fc_wino_buffer_elems(C.byref(desc), 0, C.byref(u), C.byref(v), C.byref(m)), "elems")
    dV, dM = ctx.alloc(4 * v.value), ctx.alloc(4 * m.value)
    dx, dout = ctx.upload(x), ctx.alloc(4 * n * oc * oh * ow)
    _lib.check(lib.fc_wino_forward(ctx.handle, C.c_void_p(dx), C.c_void_p(dU), C.c_void_p(dV), C.c_void_p(dM),
                                   C.c_void_p(dout), C.byref(desc), 0, None), "fc_wino_forward")
    out = ctx.download(dout, (n, oc, oh, ow))
    for p in (dV, dM, dx, dout):
        ctx.free(p)
    return out


def _static(ctx, lib, x, dU, desc, n, oc, oh, ow):
    dx, dout = ctx.upload(x), ctx.zeros(4 * n * oc * oh * ow)
    ctx.synchronize()
    before = ctx.stats()
    # enqueued on the context's own stream, so the copies below are ordered after it
    _lib.check(lib.fc_wino_forward_static_scratch(C.c_void_p(dx), C.c_void_p(dU), C.c_void_p(dout), C.byref(desc),
                                                  ctx.stream), "fc_wino_forward_static_scratch")
    assert ctx.stats() == before  # the arena was not touched
    out = ctx.download(dout, (n, oc, oh, ow))
    ctx.free(dx)
    ctx.free(dout)
    return out


def test_static_scratch_matches_regular_entry_point_twice():
    lib = fc.load()
    with fc.Context(0, arena_bytes=512 << 20) as ctx:
        for (n, ic, oc, ih, iw, pad) in [(2, 37, 70, 20, 23, 1), (1, 64, 64, 56, 56, 1)]:
            desc = fc.make_desc(n, ic, ih, iw, oc, 3, 3, 1, 1, pad, pad, pad, pad)
            oh, ow = ih + 2 * pad - 2, iw + 2 * pad - 2
            w = synth.conv_weights(oc, ic, 3, 3, 7)
            dk = ctx.upload(w)
            u_elems = C.c_size_t()
            _lib.check(lib.fc_wino_buffer_elems(C.byref(desc), 0, C.byref(u_elems), None, None), "elems")
            dU = ctx.alloc(4 * u_elems.value)
            _lib.check(lib.fc_wino_filter_transform(ctx.handle, C.c_void_p(dk), C.c_void_p(dU), oc, ic, 0), "filter")
            ctx.synchronize()
            for seed in (11, 12):  # two calls in a row share the built-in array
                x = synth.conv_input(n, ic, ih, iw, seed)
                want = _regular(ctx, lib, x, dU, desc, n, oc, oh, ow)
                got = _static(ctx, lib, x, dU, desc, n, oc, oh, ow)
                assert np.array_equal(got, want), f"seed {seed}, layer {ic}->{oc}@{ih}x{iw}"
            ctx.free(dk)
            ctx.free(dU)


def test_static_scratch_refuses_layers_beyond_its_size():
    lib = fc.load()
    desc = fc.make_desc(1, 512, 28, 28, 512)
    big = fc.make_desc(1, 128, 112, 112, 128)  # V + M = 2 * 64*368*128 floats > 4 Mi floats
    dummy = C.c_void_p(256)  # never dereferenced: the size check comes first
    st = lib.fc_wino_forward_static_scratch(dummy, dummy, dummy, C.byref(big), None)
    assert st == -2 and b"built-in scratch" in lib.fc_last_error()
    assert lib.fc_wino_forward_static_scratch(None, dummy, dummy, C.byref(desc), None) == -1
    bad = fc.make_desc(1, 8, 8, 8, 8, 3, 3, 2, 2)
    assert lib.fc_wino_forward_static_scratch(dummy, dummy, dummy, C.byref(bad), None) == -2

"""The device arena through the C ABI (PrivateMemPool / CommonMemPool semantics, utility/mempool.h:23-71)."""
import numpy as np
import pytest

import fastconv_b200 as fc

pytestmark = pytest.mark.gpu


def test_private_pool_alloc_free_roundtrip():
    with fc.Context(0, arena_bytes=64 << 20) as c:
        base = c.stats()
        a = c.alloc(1000)
        b = c.alloc(4 << 20)
        assert a % 256 == 0 and b % 256 == 0 and c.size_of(a) == 1024
        host = np.arange(1 << 20, dtype=np.float32)
        c.upload(host, b)
        assert np.array_equal(c.download(b, host.shape), host)
        c.free(a)
        with pytest.raises(fc.FastConvError) as e:
            c.free(a)  # double free is an error status, not a crash
        assert e.value.status == -1
        c.free(b)
        assert c.stats()["in_use"] == base["in_use"]
        assert c.stats()["peak"] >= (4 << 20)


def test_exhaustion_reports_out_of_memory():
    with fc.Context(0, arena_bytes=8 << 20) as c:
        with pytest.raises(fc.FastConvError) as e:
            c.alloc(64 << 20)
        assert e.value.status == -3 and "arena exhausted" in str(e.value)
        # a layer that does not fit reports the same status and leaves nothing allocated
        before = c.stats()["in_use"]
        x = fc.synth.conv_input(1, 256, 56, 56, 1)
        w = fc.synth.conv_weights(256, 256, 3, 3, 2)
        layer = fc.ConvWinoF63ZCLayer(x, w, None, None, 256, 56, 56, 256, ctx=c)
        with pytest.raises(fc.FastConvError) as e:
            layer.Init()
        assert e.value.status == -3
        assert c.stats()["in_use"] == before


def test_common_pool_is_max_of_requests():
    with fc.Context(0, arena_bytes=32 << 20) as c:
        c.common_request(1 << 20, 7)
        c.common_request(3 << 20, 7)
        c.common_request(2 << 20, 7)
        c.common_request(1 << 10, 9)
        with pytest.raises(fc.FastConvError):
            c.common_ptr(7)  # not committed yet
        c.common_commit()
        p7, p9 = c.common_ptr(7), c.common_ptr(9)
        assert c.size_of(p7) == 3 << 20 and c.size_of(p9) == 1 << 10 and p7 != p9
        c.common_free(7)
        with pytest.raises(fc.FastConvError):
            c.common_ptr(7)
        c.free_all()
        assert c.stats()["blocks"] == 1  # only the context's own status word remains

"""Host-side arithmetic of bench.py: how the images are split over the ranks, the work counts the throughput and the
roofline are computed from, and the agreement of the split with the library's own fc_shard_range."""
import ctypes as C
import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
import bench  # noqa: E402


def test_images_are_split_like_the_library_splits_them():
    import fastconv_b200 as fc
    lib = fc.load()
    for total in (64, 8, 7, 1, 65):
        for world in (1, 2, 3, 4, 8):
            seen = []
            for rank in range(world):
                a, b = bench.shard_range(total, world, rank)
                lo, hi = C.c_int(), C.c_int()
                assert lib.fc_shard_range(total, world, rank, C.byref(lo), C.byref(hi)) == 0
                assert (a, b) == (lo.value, hi.value)
                seen.extend(range(a, b))
            assert seen == list(range(total))  # every image once, in order


def test_work_counts():
    # VGG-16 conv3_2 on one image: 3.699 GFLOP direct, 100 tiles, 0.839 GFLOP in the Winograd domain
    assert abs(bench.layer_flops(1, 256, 256, 56) - 3.699e9) < 1e6
    t, tp, icp = bench.wino_geometry(1, 256, 256, 56)
    assert (t, tp, icp) == (100, 104, 256)
    assert abs(2.0 * 64 * t * 256 * 256 - 0.839e9) < 1e6
    assert bench.wino_geometry(64, 3, 64, 224) == (64 * 38 * 38, 92416, 8)
    assert bench.parse_layers("256,256,56;3,64,224") == [(256, 256, 56), (3, 64, 224)]
    assert len(bench.VGG16) == 13 and sum(bench.layer_flops(1, *l) for l in bench.VGG16) > 3.0e10


def test_batch_images_are_distinct_and_exact():
    one = np.arange(12, dtype=np.float32).reshape(1, 3, 2, 2) + 1
    x = bench.make_batch(one, 4, first=62)
    assert x.shape == (4, 3, 2, 2)
    for i in range(4):  # global images 62..65: factor 1 - (g % 128)/256, exact in fp32
        assert np.array_equal(x[i], one[0] * np.float32(1.0 - ((62 + i) % 128) / 256.0))
    assert len({x[i].tobytes() for i in range(4)}) == 4


def test_repeat_statistics():
    s = bench.repeat_stats([3.0, 1.0, 2.0], 20)
    assert (s["regions"], s["steps_per_region"], s["median_ms_per_step"], s["min_ms_per_step"], s["max_ms_per_step"]) == (3, 20, 2.0, 1.0, 3.0)

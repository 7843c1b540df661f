"""Host-side logic of the device arena (the CommonMemPool / PrivateMemPool stand-in) on a fake range."""
import ctypes as C
import random
import subprocess
from pathlib import Path

import pytest

HERE = Path(__file__).resolve().parent
BASE = 0x7000_0000_0000


@pytest.fixture(scope="module")
def probe():
    so = HERE / "arena_probe.so"
    src = HERE / "arena_probe.cpp"
    if not so.exists() or so.stat().st_mtime < max(src.stat().st_mtime,
                                                    (HERE.parent / "fastconv_b200/csrc/fc_arena.h").stat().st_mtime):
        subprocess.run(["g++", "-std=c++17", "-O1", "-fPIC", "-shared", "-o", str(so), str(src)], check=True)
    lib = C.CDLL(str(so))
    for name in ("probe_alloc", "probe_size_of", "probe_in_use", "probe_peak", "probe_blocks", "probe_fragments",
                 "probe_largest_free"):
        getattr(lib, name).restype = C.c_ulonglong
    lib.probe_alloc.argtypes = [C.c_ulonglong]
    lib.probe_release.argtypes = [C.c_ulonglong]
    lib.probe_size_of.argtypes = [C.c_ulonglong]
    lib.probe_reset.argtypes = [C.c_ulonglong, C.c_ulonglong]
    return lib


def test_alignment_and_accounting(probe):
    probe.probe_reset(BASE, 1 << 20)
    a = probe.probe_alloc(1)
    b = probe.probe_alloc(300)
    assert a == BASE and a % 256 == 0 and b % 256 == 0 and b == BASE + 256
    assert probe.probe_size_of(a) == 256 and probe.probe_size_of(b) == 512
    assert probe.probe_in_use() == 768 and probe.probe_blocks() == 2
    assert probe.probe_release(a) == 1 and probe.probe_release(a) == 0  # double free refused
    assert probe.probe_release(BASE + 12345) == 0  # foreign pointer refused
    assert probe.probe_in_use() == 512 and probe.probe_peak() == 768


def test_exhaustion_and_coalescing(probe):
    probe.probe_reset(BASE, 4096)
    blocks = [probe.probe_alloc(1024) for _ in range(4)]
    assert all(blocks) and probe.probe_alloc(1) == 0  # exhausted -> 0, not a crash
    probe.probe_release(blocks[1])
    probe.probe_release(blocks[2])
    assert probe.probe_fragments() == 1 and probe.probe_largest_free() == 2048  # neighbours merged
    big = probe.probe_alloc(2048)
    assert big == blocks[1]
    probe.probe_release(blocks[0]); probe.probe_release(big); probe.probe_release(blocks[3])
    assert probe.probe_in_use() == 0 and probe.probe_fragments() == 1 and probe.probe_largest_free() == 4096


def test_random_workload_never_overlaps(probe):
    rnd = random.Random(5)
    probe.probe_reset(BASE, 1 << 22)
    live = {}
    for _ in range(4000):
        if live and rnd.random() < 0.45:
            p = rnd.choice(list(live))
            assert probe.probe_release(p) == 1
            del live[p]
        else:
            n = rnd.randint(1, 60000)
            p = probe.probe_alloc(n)
            if p:
                assert p % 256 == 0 and BASE <= p and p + n <= BASE + (1 << 22)
                live[p] = probe.probe_size_of(p)
        spans = sorted(live.items())
        for (p0, n0), (p1, _) in zip(spans, spans[1:]):
            assert p0 + n0 <= p1
    assert probe.probe_in_use() == sum(live.values())
    probe.probe_release_all()
    assert probe.probe_in_use() == 0 and probe.probe_largest_free() == 1 << 22

import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (B200); deselect with -m 'not gpu'")


def _have_gpu() -> bool:
    import fastconv_b200 as fc
    import ctypes
    n = ctypes.c_int(0)
    fc.load().fc_device_count(ctypes.byref(n))
    return n.value > 0


def pytest_collection_modifyitems(config, items):
    # GPU tests error out loudly instead of skipping when selected on a machine without a GPU,
    # except under the default (unfiltered) run where they are skipped for convenience.
    if config.getoption("-m"):
        return
    if _have_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device; run with -m gpu on a B200")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def oracle():
    from _oracle import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def reference():
    """The reference's own sources built through the NEON stand-in; None when not built."""
    from _oracle import Reference
    return Reference.try_load()


@pytest.fixture(scope="session")
def golden():
    from _oracle import load_golden
    return load_golden()


@pytest.fixture(scope="session")
def ctx():
    import fastconv_b200 as fc
    c = fc.Context(0, arena_bytes=10 << 30)
    yield c
    c.close()


@pytest.fixture(autouse=True)
def _split_arithmetic_on_every_layer(monkeypatch):
    """A layer asked for in 3xTF32 runs the tensor-core kernel whatever its channel count, so that the tests of that
    mode keep exercising it on small shapes.  (The library's default sends Winograd layers of at most 64 input channels
    to the fp32 kernels, which are faster there and exact; tests/test_plan_resolution.py and one GPU test cover that
    rule with the variable removed.)"""
    monkeypatch.setenv("FASTCONV_3XTF32_MIN_IC", "0")

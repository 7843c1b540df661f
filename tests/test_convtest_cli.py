"""The ConvTest command-line harness (fastconv_b200/host/ConvTest.cpp): same flags, header and labels as the
reference's winograd_dev."""
import re
import subprocess
from pathlib import Path

import pytest

HOST = Path(__file__).resolve().parents[1] / "fastconv_b200" / "host"
BIN = HOST / "winograd_dev"


@pytest.fixture(scope="module")
def binary():
    import fastconv_b200
    fastconv_b200.load()  # builds the library if needed
    subprocess.run(["make", "-C", str(HOST)], check=True, capture_output=True)
    assert BIN.exists()
    return str(BIN)


def run(binary, *args):
    return subprocess.run([binary, *args], capture_output=True, text=True, timeout=600)


def test_help_lists_the_reference_flags(binary):
    r = run(binary, "-h")
    assert r.returncode == 0
    for flag in ("-ic", "-oc", "-is", "-ks", "-a ", "-ts", "-s ", "-ip", "-tn", "-t ", "-i "):
        assert flag in r.stdout
    assert "auto, direct, im2col, or winograd" in r.stdout


@pytest.mark.parametrize("args, message", [
    (["-oc", "4", "-is", "8", "8", "-ks", "3", "3"], "the number of input channels is not specified"),
    (["-ic", "4", "-is", "8", "8", "-ks", "3", "3"], "the number of output channels is not specified"),
    (["-ic", "4", "-oc", "4", "-ks", "3", "3"], "the input size is not specified"),
    (["-ic", "4", "-oc", "4", "-is", "8", "8"], "the kernel size is not specified"),
    (["-ic", "0", "-oc", "4", "-is", "8", "8", "-ks", "3", "3"], "positive value expected"),
    (["-ic", "x", "-oc", "4", "-is", "8", "8", "-ks", "3", "3"], "can not parse x as an unsigned integer"),
    (["-ic", "4", "-oc", "4", "-is", "8", "8", "-ks", "3", "3", "-a", "fft"], "invalid convolution algorithm name fft"),
    (["-ic", "4", "-oc", "4", "-is", "8", "8", "-ks", "3", "3", "-tn", "maybe"], "invalid tuning name maybe"),
    (["-ic", "4", "-oc", "4", "-is", "8", "8", "-ks", "3", "3", "--frobnicate", "1"], "unknown argument"),
    (["-ic", "4", "-oc", "4", "-is", "8"], "expected two values"),
])
def test_argument_errors_exit_nonzero(binary, args, message):
    r = run(binary, *args)
    assert r.returncode != 0
    assert message in r.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("args, algo, labels", [
    (["-ic", "16", "-oc", "16", "-is", "12", "12", "-ks", "3", "3"], "winograd F63",
     ["InputTran time:", "KernelTran time:", "TensorGEMM time:", "OutputTran time:", "Total time:"]),
    (["-ic", "16", "-oc", "24", "-is", "14", "14", "-ks", "1", "1", "-ip", "0"], "im2col",  # `direct` in the reference: ran nothing
     ["Im2colTran time:", "Gemm time:", "Total time:"]),
    (["-ic", "3", "-oc", "8", "-is", "30", "30", "-ks", "7", "7", "-s", "2", "2", "-ip", "3", "-a", "im2col"], "im2col",
     ["Gemm time:"]),
    (["-ic", "8", "-oc", "8", "-is", "20", "20", "-ks", "3", "3", "-a", "winograd", "-n", "3", "-m", "3xtf32", "-tn", "tuning"],
     "winograd F63", ["TensorGEMM time:"]),
])
def test_runs_and_prints_reference_lines(binary, args, algo, labels):
    r = run(binary, *args, "-i", "3", "-seed", "7")
    assert r.returncode == 0, r.stderr
    out = r.stdout
    assert re.search(r"Input channels: \d+\nOutput channels: \d+\nInput: \d+x\d+ with implicit padding \d+\nKernel: \d+x\d+\n"
                     r"Subsampling: \d+x\d+\n", out)
    assert f"Algorithm: {algo}" in out
    for label in labels:
        assert label in out
    m = re.search(r"The difference is ([0-9.]+)", out)
    assert m, out
    # inputs are in [0,256) and kernels in [0,1) as in the reference, so outputs are ~1e4 and an fp32
    # difference of a few 1e-3 in absolute terms is rounding, not error
    assert float(m.group(1)) < 0.05


@pytest.mark.gpu
def test_winograd_refuses_shapes_the_reference_computes_wrongly(binary):
    r = run(binary, "-ic", "8", "-oc", "8", "-is", "16", "16", "-ks", "3", "3", "-s", "2", "2", "-a", "winograd")
    assert r.returncode != 0 and "stride 1" in r.stderr


@pytest.mark.gpu
def test_direct_runs_the_tensor_core_kernel_in_tf32_and_the_implicit_gemm_otherwise(binary):
    base = ["-ic", "16", "-oc", "16", "-is", "20", "20", "-ks", "3", "3", "-a", "direct", "-i", "2", "-seed", "7"]
    exact = run(binary, *base)
    assert exact.returncode == 0, exact.stderr
    assert "Algorithm: direct" in exact.stdout and "Gemm time:" in exact.stdout
    assert float(re.search(r"The difference is ([0-9.]+)", exact.stdout).group(1)) < 0.05  # fp32: the implicit GEMM
    fast = run(binary, *base, "-m", "tf32")
    assert fast.returncode == 0, fast.stderr
    assert "Algorithm: direct" in fast.stdout
    # outputs are ~1e4 (inputs in [0,256), 144 taps): a mean absolute difference of a few units is TF32 rounding (3e-4)
    assert float(re.search(r"The difference is ([0-9.]+)", fast.stdout).group(1)) < 10.0


@pytest.mark.gpu
def test_round_times_testing_line_and_json_line(binary):
    """The reference prints one `round time:` per -i iteration (convLayer/winoF63ConvZC.cpp:245) and a `Testing ic=...
    tileBlock=... ocBlock=... icBlock=... threads=...` line (:191-192); the harness adds one JSON line per layer."""
    import json
    r = run(binary, "-ic", "16", "-oc", "32", "-is", "18", "18", "-ks", "3", "3", "-i", "4", "-seed", "3")
    assert r.returncode == 0, r.stderr
    assert len(re.findall(r"^round time: [0-9.]+ms$", r.stdout, re.M)) == 4
    assert re.search(r"^Testing ic=16 oc=32 width=18 tileBlock=\d+ ocBlock=\d+ icBlock=\d+ threads=1 tiles=9 batch=1$",
                     r.stdout, re.M)
    rec = json.loads([line for line in r.stdout.splitlines() if line.startswith("{")][-1])
    assert rec["layer"] == "16->32@18x18 3x3s1" and rec["algo"] == "winograd" and rec["math"] == "fp32"
    assert rec["ms"] > 0 and rec["gflops_direct_equiv"] > 0 and 0 < rec["frac_of_roofline"] <= 1.5
    assert rec["bound"] in ("hbm", "math")


def _gpu_count():
    import ctypes
    import fastconv_b200
    n = ctypes.c_int(0)
    fastconv_b200.load().fc_device_count(ctypes.byref(n))
    return n.value


@pytest.mark.gpu
@pytest.mark.parametrize("shard", [["-shard", "batch", "-n", "4"], ["-shard", "k"], ["-shard", "k", "-gather", "nccl"]])
def test_two_gpus_print_the_difference_line_of_one(binary, shard):
    """`-g 2` shards the layer over two GPUs driven by the one process; the self-check line is the one-GPU line."""
    if _gpu_count() < 2:
        pytest.skip("needs two GPUs")
    base = ["-ic", "32", "-oc", "64", "-is", "20", "20", "-ks", "3", "3", "-i", "3", "-seed", "1", *shard]
    one = run(binary, *base)
    two = run(binary, *base, "-g", "2")
    assert one.returncode == 0 and two.returncode == 0, one.stderr + two.stderr
    line = re.compile(r"The difference is ([0-9.]+)")
    assert line.search(one.stdout).group(0) == line.search(two.stdout).group(0)
    assert "Sharding:" in two.stdout and "over 2 GPUs" in two.stdout


@pytest.mark.gpu
def test_more_gpus_than_the_box_has_is_refused(binary):
    r = run(binary, "-ic", "8", "-oc", "8", "-is", "8", "8", "-ks", "3", "3", "-g", "64")
    assert r.returncode != 0 and "GPUs asked for" in r.stderr


@pytest.mark.gpu
def test_feather_layer_blob_and_pools_chain_two_convolutions(binary):
    """The FeatherCNN-style interface the reference carries (layer.h, utility/blob.h, utility/mempool.h) instantiated
    over the GPU library: two convolutions with fused bias + ReLU chained on device blobs, checked on the host."""
    r = subprocess.run([str(HOST / "feather_chain_test")], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "feather chain ok" in r.stdout

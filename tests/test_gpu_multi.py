"""Layers sharded over a communicator (fc_comm_*, fc_sharded_conv_*) against the single-GPU result, bit for bit.

  * one rank (runs on any box): the same entry points with a world of one, where the peer gather stores into local
    memory only;
  * two GPUs driven by ONE process (fc_comm_init_all: peer pointers inside the process);
  * two GPUs, one process each (fc_comm_init_env: NCCL id through a file, CUDA IPC mappings of the arenas).
The two-GPU tests are skipped on a box with fewer than two GPUs.
"""
import ctypes
import os
import tempfile

import numpy as np
import pytest

import fastconv_b200 as fc
from fastconv_b200 import parallel, synth

pytestmark = pytest.mark.gpu

IC, OC, HW = 96, 256, 14


def _gpus():
    n = ctypes.c_int(0)
    fc.load().fc_device_count(ctypes.byref(n))
    return n.value


def _reference_outputs(ctx, x, w, xb, modes):
    """The unsharded layer on one GPU: per mode the single-image output, and the fp32 output of the batch."""
    one = {}
    for mode in modes:
        layer = fc.ConvWinoF63ZCLayer(x, w, None, None, IC, HW, HW, OC, iter=1, mode=mode, ctx=ctx)
        layer.Init(); layer.Forward()
        one[mode] = layer.output_data.copy()
        layer.release()
    full = fc.ConvWinoF63ZCLayer(xb, w, None, None, IC, HW, HW, OC, batch=xb.shape[0], iter=1, ctx=ctx)
    full.Init(); full.Forward()
    batch = full.output_data.copy()
    full.release()
    return one, batch


def _check_sharded(comm, forwards=12):
    """Runs on every process of the job; returns True when every sharded result equals the unsharded one."""
    x = synth.conv_input(1, IC, HW, HW, 700)
    w = synth.conv_weights(OC, IC, 3, 3, 701)
    xb = synth.conv_input(5, IC, HW, HW, 702)  # 5 images: an uneven split over two ranks
    one, batch = _reference_outputs(comm.contexts[0], x, w, xb, ("fp32", "3xtf32"))
    ok = True
    # output channels split, gathered by the output transform's own stores: many forwards in a row, so that both of
    # the alternating buffers and the device-side step counter are exercised and a missing fence would show
    for mode in ("fp32", "3xtf32"):
        for gather in ("peer", "nccl"):
            sc = parallel.ShardedConv(comm, w, 1, HW, HW, shard="k", gather=gather, algorithm="winograd", mode=mode)
            sc.upload(x)
            for _ in range(forwards):
                sc.forward()
                sc.wait()
                ok = ok and np.array_equal(sc.download(), one[mode])
            ok = ok and np.array_equal(sc.forward_host(x), one[mode])
            ok = ok and sc.time_device(2, 5) > 0.0
            sc.release()
    # images split: no collective; this process's ranks return their images back to back
    sb = parallel.ShardedConv(comm, w, xb.shape[0], HW, HW, shard="batch", algorithm="winograd")
    b0, b1 = sb.local_images()
    ok = ok and np.array_equal(sb.forward_host(xb[b0:b1]), batch[b0:b1])
    # an uneven channel split (255 channels) goes through the broadcast form of the NCCL gather
    w_odd = np.ascontiguousarray(w[:255])
    so = parallel.ShardedConv(comm, w_odd, 1, HW, HW, shard="k", gather="nccl", algorithm="winograd")
    ok = ok and np.array_equal(so.forward_host(x), one["fp32"][:, :255])
    so.release()
    sb.release()
    return bool(ok)


def test_one_rank_communicator_runs_the_sharded_entry_points():
    with parallel.Comm.all(1, arena_bytes=1 << 30) as comm:
        assert (comm.world, comm.local_count, comm.first_rank) == (1, 1, 0)
        assert comm.max(3.5) == 3.5
        comm.barrier()
        x = synth.conv_input(1, IC, HW, HW, 700)
        w = synth.conv_weights(OC, IC, 3, 3, 701)
        xb = synth.conv_input(3, IC, HW, HW, 702)
        one, batch = _reference_outputs(comm.contexts[0], x, w, xb, ("fp32",))
        sc = parallel.ShardedConv(comm, w, 1, HW, HW, shard="k", gather="peer", algorithm="winograd")
        sc.upload(x)
        for _ in range(5):
            sc.forward()
            sc.wait()
            assert np.array_equal(sc.download(), one["fp32"])
        sb = parallel.ShardedConv(comm, w, 3, HW, HW, shard="batch")
        assert sb.local_images() == (0, 3)
        assert np.array_equal(sb.forward_host(xb), batch)
        with pytest.raises(fc.FastConvError):  # the channel split takes one image
            parallel.ShardedConv(comm, w, 2, HW, HW, shard="k")
    lib = fc.load()
    h = ctypes.c_void_p()
    assert lib.fc_comm_init_all(99, None, 1 << 20, ctypes.byref(h)) == fc._lib.FC_ERR_INVALID_ARG


def test_two_gpus_one_process_sharding_is_bit_equal_to_one_gpu():
    if _gpus() < 2:
        pytest.skip("needs two GPUs")
    with parallel.Comm.all(2, arena_bytes=2 << 30) as comm:
        assert (comm.world, comm.local_count) == (2, 2)
        assert _check_sharded(comm)


def _worker(rank, world, id_file, ret):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), FASTCONV_COMM_ID_FILE=id_file,
                      NCCL_NVLS_ENABLE="0")
    ok, err = False, ""
    comm = None
    try:
        comm = parallel.Comm.from_env(arena_bytes=2 << 30)
        ok = (comm.world, comm.local_count, comm.first_rank) == (world, 1, rank) and _check_sharded(comm)
    except Exception as exc:  # reported through the queue; the peer is not left waiting for ever (bounded waits)
        err = repr(exc)
    finally:
        try:
            if comm is not None:
                comm.close()
        except Exception as exc:
            err = err or repr(exc)
    ret.put((rank, bool(ok), err))


def test_two_gpus_two_processes_sharding_is_bit_equal_to_one_gpu():
    if _gpus() < 2:
        pytest.skip("needs two GPUs")
    import multiprocessing as mp
    mpc = mp.get_context("spawn")
    ret = mpc.Queue()
    with tempfile.TemporaryDirectory() as tmp:
        id_file = os.path.join(tmp, "nccl.id")
        procs = [mpc.Process(target=_worker, args=(r, 2, id_file, ret)) for r in range(2)]
        for p in procs:
            p.start()
        results = [ret.get(timeout=600) for _ in procs]
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0
    assert all(ok for _, ok, _ in results), results

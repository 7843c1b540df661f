"""Two GPUs, one process each, NCCL: K-sharded and batch-sharded layers against the single-GPU result.
Skipped on a box with fewer than two GPUs."""
import ctypes
import os
import socket

import numpy as np
import pytest

import fastconv_b200 as fc
from fastconv_b200 import parallel, synth

pytestmark = pytest.mark.gpu


def _gpus():
    n = ctypes.c_int(0)
    fc.load().fc_device_count(ctypes.byref(n))
    return n.value


def _worker(rank, world, port, ret):
    import torch
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    ok = True
    try:
        with fc.Context(rank, arena_bytes=2 << 30) as ctx:
            ic, oc, hw = 96, 256, 14
            x = synth.conv_input(1, ic, hw, hw, 700)
            w = synth.conv_weights(oc, ic, 3, 3, 701)
            whole = fc.ConvWinoF63ZCLayer(x, w, None, None, ic, hw, hw, oc, iter=1, ctx=ctx)
            whole.Init(); whole.Forward()
            sharded = parallel.KShardedConv.gpu(ctx, w, hw, hw, 1, "fp32")
            got = sharded.forward(x)
            torch.cuda.synchronize()
            ok = ok and np.array_equal(got.cpu().numpy(), whole.output_data)  # bit for bit, on every rank
            got2 = sharded.forward(None)  # second call: same device input, same answer
            torch.cuda.synchronize()
            ok = ok and np.array_equal(got2.cpu().numpy(), whole.output_data)
            # batch sharding: this rank's images only, no collective
            xb = synth.conv_input(4, ic, hw, hw, 702)
            b0, b1 = parallel.shard_batch(4, world, rank)
            mine = fc.ConvWinoF63ZCLayer(xb[b0:b1], w, None, None, ic, hw, hw, oc, batch=b1 - b0, iter=1, ctx=ctx)
            mine.Init(); mine.Forward()
            full = fc.ConvWinoF63ZCLayer(xb, w, None, None, ic, hw, hw, oc, batch=4, iter=1, ctx=ctx)
            full.Init(); full.Forward()
            ok = ok and np.array_equal(mine.output_data, full.output_data[b0:b1])
            # K sharding with the all-gather fused into the output transform (peer stores over NVLink, flags,
            # bounded wait): every rank ends with the whole output, bit-equal to the one-GPU layer, on both of
            # the alternating output buffers and in both operand layouts
            for mode, ref in (("fp32", whole.output_data), ("3xtf32", None)):
                peer = parallel.PeerKShardedConv(ctx, w, hw, hw, 1, mode)
                peer.upload(x)
                if ref is None:
                    one = fc.ConvWinoF63ZCLayer(x, w, None, None, ic, hw, hw, oc, iter=1, mode=mode, ctx=ctx)
                    one.Init(); one.Forward()
                    ref = one.output_data
                for _ in range(3):
                    ok = ok and np.array_equal(peer.result(peer.forward()), ref)
                dist.barrier()
            ctx.close_peer_mappings()
            dist.barrier()
        flag = torch.tensor([1 if ok else 0], device=f"cuda:{rank}")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if rank == 0:
            ret.put(int(flag.item()))
    finally:
        dist.destroy_process_group()


def test_two_gpu_sharding_is_bit_equal_to_one_gpu():
    if _gpus() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mpc = mp.get_context("spawn")
    ret = mpc.Queue()
    procs = [mpc.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    assert ret.get(timeout=10) == 1

"""Multi-rank host logic on CPU: world_size-2 (and 3) gloo groups, no GPU.

Batch sharding has no collective: the ranks' image ranges must tile the batch exactly.  K sharding
all-gathers per-rank channel slabs; with the oracle standing in for the GPU layer the gathered output
must equal the unsharded oracle output bit for bit (the reduction over input channels is never split).
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fastconv_b200 import parallel, synth


def test_shard_ranges_tile_exactly():
    for total in (0, 1, 7, 64, 65, 513):
        for world in (1, 2, 3, 4, 8):
            spans = [parallel.shard_range(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    assert parallel.shard_batch(64, 8, 3) == (24, 32)
    assert [parallel.shard_channels(512, 4, r, multiple=128) for r in range(4)] == [(0, 128), (128, 256), (256, 384), (384, 512)]
    assert [parallel.shard_channels(200, 2, r, multiple=128) for r in range(2)] == [(0, 128), (128, 200)]
    with pytest.raises(ValueError):
        parallel.shard_range(8, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, oc, n, ret):
    import sys
    from pathlib import Path
    sys.path.insert(0, str(Path(__file__).resolve().parent))
    from _oracle import Oracle

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        oracle = Oracle()
        ic, hw = 12, 14
        x = synth.conv_input(n, ic, hw, hw, 900)
        w = synth.conv_weights(oc, ic, 3, 3, 901)
        conv = parallel.KShardedConv(w, lambda xx, ws: oracle.wino_forward(xx, ws, 1))
        k0, k1 = parallel.shard_channels(oc, world, rank)
        assert conv.w_slice.shape[0] == k1 - k0
        full = conv.forward(x).numpy()
        want = oracle.wino_forward(x, w, 1)
        ok = np.array_equal(full, want)
        # batch sharding: every rank takes its images, the union is the batch, no collective needed
        b0, b1 = parallel.shard_batch(8, world, rank)
        xb = synth.conv_input(8, ic, hw, hw, 902)
        part = oracle.wino_forward(xb[b0:b1], w, 1) if b1 > b0 else np.zeros((0, oc, hw, hw), np.float32)
        whole = oracle.wino_forward(xb, w, 1)
        ok = ok and np.array_equal(part, whole[b0:b1])
        flag = torch.tensor([1 if ok else 0])
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if rank == 0:
            ret.put(int(flag.item()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world, oc, n", [(2, 16, 1), (2, 15, 1), (3, 16, 2)])
def test_k_sharding_equals_unsharded_bitwise(world, oc, n):
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, oc, n, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0
    assert ret.get(timeout=10) == 1

"""Several GPUs of one machine: thin ctypes front end of the communicator and the sharded layers of the C ABI
(fc_comm_*, fc_sharded_conv_*), plus the partition arithmetic as plain functions.

The reference has no distributed code (its only parallelism is OpenMP inside one process), so nothing here
mirrors a reference interface; the two partitionings are the ones the path offers naturally:

* batch sharding  -- images are independent: rank r runs the same layers on images [b0, b1) of the batch;
  there is NO collective in the data path.
* K sharding      -- output channels are independent: rank r owns channels [k0, k1) of a single-image
  wide layer, i.e. transforms and keeps only its slice of the weights (which is what shrinks the
  dominant 64*C*K weight stream), reads the whole (small) input, and produces the slab
  out[:, k0:k1] -- contiguous in NCHW for one image.  The slabs reach every rank either through the stores of
  the output transform itself (peer memory over NVLink, step flags, bounded wait) or through one NCCL
  all-gather.  The reduction over input channels is never split, so every output element is computed by
  exactly the arithmetic of the unsharded layer: sharded == unsharded bit for bit.

Nothing here computes and nothing here needs torch: process groups, collectives and peer mappings live in the
library.  `KShardedConv` is the exception, kept for CPU tests of the partition logic: it all-gathers slabs that
any callable produced, over a torch.distributed group of any backend.
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, List, Optional, Tuple

import numpy as np

from . import _lib
from .layers import Context, make_desc

SHARD_BATCH, SHARD_CHANNELS = 0, 1
GATHER_PEER, GATHER_NCCL = 0, 1
SHARD_NAMES = {"batch": SHARD_BATCH, "k": SHARD_CHANNELS, "channels": SHARD_CHANNELS}
GATHER_NAMES = {"peer": GATHER_PEER, "nccl": GATHER_NCCL}


def shard_range(total: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous balanced split of range(total): the first total % world ranks get one extra item
    (the same arithmetic as fc_shard_range)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if total < 0:
        raise ValueError("negative extent")
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_batch(images: int, world: int, rank: int) -> Tuple[int, int]:
    return shard_range(images, world, rank)


def shard_channels(oc: int, world: int, rank: int, multiple: int = 1) -> Tuple[int, int]:
    """Output-channel slice of a rank; with `multiple` > 1 every slice but the last is a multiple of it."""
    blocks = -(-oc // multiple)
    b0, b1 = shard_range(blocks, world, rank)
    return min(b0 * multiple, oc), min(b1 * multiple, oc)


class Comm:
    """fc_comm: the GPUs of one machine as ranks.  `Comm.all(n)` drives n GPUs from this process; `Comm.from_env()`
    is one rank of a job started by a launcher (RANK / WORLD_SIZE / LOCAL_RANK / MASTER_PORT in the environment)."""

    def __init__(self, handle: C.c_void_p):
        self._lib = _lib.load()
        self._h = handle
        w, n, f = C.c_int(), C.c_int(), C.c_int()
        _lib.check(self._lib.fc_comm_size(handle, C.byref(w), C.byref(n), C.byref(f)), "fc_comm_size")
        self.world, self.local_count, self.first_rank = w.value, n.value, f.value
        self.contexts: List[Context] = []
        for i in range(self.local_count):
            c = C.c_void_p()
            _lib.check(self._lib.fc_comm_context(handle, i, C.byref(c)), "fc_comm_context")
            self.contexts.append(Context(_borrowed=c))
        self._layers = []

    @classmethod
    def all(cls, ndev: int, arena_bytes: int = 1 << 30, devices=None) -> "Comm":
        lib = _lib.load()
        h = C.c_void_p()
        arr = None if devices is None else (C.c_int * ndev)(*devices)
        _lib.check(lib.fc_comm_init_all(ndev, arr, arena_bytes, C.byref(h)), "fc_comm_init_all")
        return cls(h)

    @classmethod
    def from_env(cls, device: int = -1, arena_bytes: int = 1 << 30) -> "Comm":
        lib = _lib.load()
        h = C.c_void_p()
        _lib.check(lib.fc_comm_init_env(device, arena_bytes, C.byref(h)), "fc_comm_init_env")
        return cls(h)

    @property
    def handle(self) -> C.c_void_p:
        if not self._h:
            raise RuntimeError("communicator is closed")
        return self._h

    def barrier(self) -> None:
        _lib.check(self._lib.fc_comm_barrier(self.handle), "fc_comm_barrier")

    def max(self, value: float) -> float:
        """Maximum over all ranks of `value` (taken as the value of every local rank)."""
        arr = (C.c_double * self.local_count)(*([float(value)] * self.local_count))
        _lib.check(self._lib.fc_comm_allreduce_max(self.handle, arr), "fc_comm_allreduce_max")
        return float(arr[0])

    def allgather(self, values) -> np.ndarray:
        """One row of float64 values per rank, gathered to every rank: [world][len(values)].  With several local ranks
        the same row stands for each of them."""
        row = np.ascontiguousarray(values, dtype=np.float64).reshape(1, -1)
        mine = np.ascontiguousarray(np.repeat(row, self.local_count, axis=0))
        out = np.empty((self.world, row.shape[1]), np.float64)
        _lib.check(self._lib.fc_comm_allgather(self.handle, C.c_void_p(mine.ctypes.data), C.c_void_p(out.ctypes.data),
                                               row.nbytes), "fc_comm_allgather")
        return out

    def close(self) -> None:
        if self._h:
            for layer in list(self._layers):
                layer.release()
            for c in self.contexts:
                c.close()  # layer lists, pinned buffers; the contexts themselves belong to the communicator
            self._lib.fc_comm_destroy(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class ShardedConv:
    """fc_sharded_conv: one layer split over the ranks of a communicator by images ("batch") or by output channels
    ("k", single image; gather "peer" = stores of the output transform into every rank's buffer, "nccl" = one
    all-gather after the layer)."""

    def __init__(self, comm: Comm, weights: np.ndarray, batch: int, ih: int, iw: int, *, stride=1, pad=1, shard="batch",
                 gather="peer", algorithm="auto", mode="fp32"):
        self._lib, self.comm = _lib.load(), comm
        w = np.ascontiguousarray(weights, dtype=np.float32)
        oc, ic, kh, kw = w.shape
        self.desc = make_desc(batch, ic, ih, iw, oc, kh, kw, stride, stride, pad, pad, pad, pad)
        self.oh, self.ow = (ih + 2 * pad - kh) // stride + 1, (iw + 2 * pad - kw) // stride + 1
        self.shard = SHARD_NAMES[shard] if isinstance(shard, str) else int(shard)
        h = C.c_void_p()
        _lib.check(self._lib.fc_sharded_conv_create(comm.handle, C.byref(self.desc), _lib.ALGO_NAMES[algorithm],
                                                    _lib.MODE_NAMES[mode], self.shard,
                                                    GATHER_NAMES[gather] if isinstance(gather, str) else int(gather),
                                                    C.c_void_p(w.ctypes.data), C.byref(h)), "fc_sharded_conv_create")
        self._h = h
        comm._layers.append(self)

    def part(self, local_index: int = 0):
        """(fc_conv handle or None, device input, device output, begin, end) of one local rank."""
        conv, d_in, d_out, b, e = C.c_void_p(), C.c_void_p(), C.c_void_p(), C.c_int(), C.c_int()
        _lib.check(self._lib.fc_sharded_conv_part(self._h, local_index, C.byref(conv), C.byref(d_in), C.byref(d_out),
                                                  C.byref(b), C.byref(e)), "fc_sharded_conv_part")
        return (conv if conv.value else None), d_in.value, d_out.value, b.value, e.value

    def local_images(self) -> Tuple[int, int]:
        """Batch split: the range of images this process's ranks own together."""
        first, last = self.part(0), self.part(self.comm.local_count - 1)
        return first[3], last[4]

    def upload(self, x: np.ndarray) -> None:
        x = np.ascontiguousarray(x, dtype=np.float32)
        _lib.check(self._lib.fc_sharded_conv_upload(self._h, C.c_void_p(x.ctypes.data)), "fc_sharded_conv_upload")

    def forward(self) -> None:
        _lib.check(self._lib.fc_sharded_conv_forward(self._h), "fc_sharded_conv_forward")

    def wait(self) -> None:
        _lib.check(self._lib.fc_sharded_conv_wait(self._h), "fc_sharded_conv_wait")

    def download(self) -> np.ndarray:
        if self.shard == SHARD_BATCH:
            b0, b1 = self.local_images()
            out = np.empty((b1 - b0, self.desc.oc, self.oh, self.ow), np.float32)
        else:
            out = np.empty((1, self.desc.oc, self.oh, self.ow), np.float32)
        _lib.check(self._lib.fc_sharded_conv_download(self._h, C.c_void_p(out.ctypes.data)), "fc_sharded_conv_download")
        return out

    def forward_host(self, x: np.ndarray) -> np.ndarray:
        self.upload(x)
        self.forward()
        self.wait()
        return self.download()

    def time_device(self, warmup: int = 3, iters: int = 20) -> float:
        ms = C.c_float()
        _lib.check(self._lib.fc_sharded_conv_time_device(self._h, warmup, iters, C.byref(ms)), "fc_sharded_conv_time_device")
        return float(ms.value)

    def release(self) -> None:
        if self._h:
            self._lib.fc_sharded_conv_destroy(self._h)
            self._h = None
            if self in self.comm._layers:
                self.comm._layers.remove(self)


def allgather_channel_slabs(local, oc: int, group=None):
    """All-gather of per-rank slabs [n][k_r][oh][ow] into [n][oc][oh][ow] on every rank (torch tensors,
    any backend).  Equal slabs of a single image go through one all_gather_into_tensor (the slab is a
    contiguous piece of the NCHW output); ragged or batched slabs are gathered as a list and concatenated."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    n, k_local, oh, ow = local.shape
    sizes = [shard_channels(oc, world, r)[1] - shard_channels(oc, world, r)[0] for r in range(world)]
    if sum(sizes) != oc or sizes[dist.get_rank(group)] != k_local:
        raise ValueError(f"slab of {k_local} channels does not match the partition {sizes} of {oc}")
    local = local.contiguous()
    if n == 1 and len(set(sizes)) == 1:
        out = torch.empty((1, oc, oh, ow), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out.view(-1), local.view(-1), group=group)
        return out
    # ragged or batched: collectives want equal shapes, so every slab is padded to the widest one
    widest = max(sizes)
    padded = torch.zeros((n, widest, oh, ow), dtype=local.dtype, device=local.device)
    padded[:, :k_local] = local
    parts = [torch.empty_like(padded) for _ in sizes]
    dist.all_gather(parts, padded, group=group)
    return torch.cat([p[:, :s] for p, s in zip(parts, sizes)], dim=1)


class KShardedConv:
    """CPU-test stand-in for the channel split: `forward_slab(x, w_slice) -> [n][k_r][oh][ow]` computes this
    rank's channels (any convolution), and the slabs are all-gathered over a torch.distributed group."""

    def __init__(self, weights: np.ndarray, forward_slab: Callable, group=None):
        import torch.distributed as dist

        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.oc = int(weights.shape[0])
        self.k0, self.k1 = shard_channels(self.oc, self.world, self.rank)
        self.w_slice = np.ascontiguousarray(weights[self.k0:self.k1])
        self._forward_slab = forward_slab

    def forward(self, x):
        import torch

        slab = self._forward_slab(x, self.w_slice)
        if not isinstance(slab, torch.Tensor):
            slab = torch.from_numpy(np.ascontiguousarray(slab))
        return allgather_channel_slabs(slab, self.oc, self.group)

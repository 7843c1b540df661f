"""Multi-GPU partitioning of the convolution path: one process per GPU, torch.distributed for the plumbing.

The reference has no distributed code (its only parallelism is OpenMP inside one process), so nothing here
mirrors a reference interface; the two partitionings are the ones the path offers naturally:

* batch sharding  -- images are independent: rank r runs the same layers on images [b0, b1) of the batch;
  there is NO collective in the data path.
* K sharding      -- output channels are independent: rank r owns channels [k0, k1) of a single-image
  wide layer, i.e. transforms and keeps only its slice of the weights (which is what shrinks the
  dominant 64*C*K weight stream), reads the whole (small) input, and produces the slab
  out[:, k0:k1] -- contiguous in NCHW for one image -- which one all-gather reassembles on every
  rank.  The reduction over input channels is never split, so every output element is computed by
  exactly the arithmetic of the unsharded layer: sharded == unsharded bit for bit.
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, Optional, Tuple

import numpy as np


def shard_range(total: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous balanced split of range(total): the first total % world ranks get one extra item."""
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
    """One single-image layer with its output channels split over the ranks of a process group.

    `forward_slab(x, w_slice) -> ndarray/tensor [n][k_r][oh][ow]` computes this rank's channels; on a GPU
    it is a planned fastconv layer built from the weight slice (see `gpu`), in CPU tests any convolution.
    """

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

    @classmethod
    def gpu(cls, ctx, weights: np.ndarray, ih: int, iw: int, pad: int = 1, mode: str = "fp32", group=None):
        """K-sharded Winograd layer on this rank's GPU: the slab is written straight into a torch CUDA
        tensor by the library, then all-gathered over NCCL."""
        import torch

        from . import _lib
        from .layers import make_desc

        lib = _lib.load()
        state = {}

        def forward_slab(x, w_slice):
            if "conv" not in state:
                x = np.ascontiguousarray(x, dtype=np.float32)
                n, ic = x.shape[:2]
                desc = make_desc(n, ic, ih, iw, w_slice.shape[0], 3, 3, 1, 1, pad, pad, pad, pad)
                h = C.c_void_p()
                _lib.check(lib.fc_conv_create(ctx.handle, C.byref(desc), _lib.ALGO_WINOGRAD, _lib.MODE_NAMES[mode],
                                              C.c_void_p(w_slice.ctypes.data), C.byref(h)), "fc_conv_create")
                d_in, d_out = C.c_void_p(), C.c_void_p()
                _lib.check(lib.fc_conv_device_buffers(h, C.byref(d_in), C.byref(d_out)), "fc_conv_device_buffers")
                oh, ow = ih + 2 * pad - 2, iw + 2 * pad - 2
                state.update(conv=h, d_in=d_in, slab=torch.empty((n, w_slice.shape[0], oh, ow), dtype=torch.float32,
                                                                  device=f"cuda:{ctx.device}"))
            if x is not None:
                ctx.upload(x, state["d_in"].value)
            _lib.check(lib.fc_conv_forward_device(state["conv"], state["d_in"], C.c_void_p(state["slab"].data_ptr())),
                       "fc_conv_forward_device")
            return state["slab"]

        def release():
            if "conv" in state:
                lib.fc_conv_destroy(state.pop("conv"))

        obj = cls(weights, forward_slab, group)
        obj._state = state
        obj.release = release
        ctx.adopt(obj)
        # torch sees the library's stream as an external stream: with it current, the all-gather is ordered
        # after the kernels without a host synchronisation, and CUDA events on it time both
        obj.stream = torch.cuda.ExternalStream(ctx.stream.value, device=f"cuda:{ctx.device}")
        plain_forward = obj.forward

        def forward_on_library_stream(x):
            with torch.cuda.stream(obj.stream):
                return plain_forward(x)

        obj.forward = forward_on_library_stream
        return obj


class PeerKShardedConv:
    """K-sharded Winograd layer whose all-gather is fused into the output transform: the kernel of each rank
    stores its channel slab into the output buffer of every rank through peer-mapped pointers over NVLink
    (`fc_conv_forward_scatter`), publishes a step flag, and a bounded wait kernel on every rank makes the
    stream wait for all slabs.  No NCCL call in the data path; torch.distributed only carries the CUDA IPC
    handles at construction.  Two output buffers alternate by step, so a rank that runs one step ahead never
    overwrites what a peer is still reading; `forward` returns the device address of the buffer just filled.
    """

    def __init__(self, ctx, weights: np.ndarray, ih: int, iw: int, pad: int = 1, mode: str = "fp32", group=None):
        import torch.distributed as dist

        from . import _lib
        from .layers import make_desc

        self._lib, self._check = _lib.load(), _lib.check
        lib, check = self._lib, self._check
        self.ctx, self.group = ctx, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > 8:
            raise ValueError("at most 8 ranks")
        self.oc = int(weights.shape[0])
        ic = int(weights.shape[1])
        self.k0, self.k1 = shard_channels(self.oc, self.world, self.rank)
        if self.k1 <= self.k0:
            raise ValueError("a rank would own no output channel")
        w_slice = np.ascontiguousarray(weights[self.k0:self.k1], dtype=np.float32)
        self.oh, self.ow = ih + 2 * pad - 2, iw + 2 * pad - 2
        desc = make_desc(1, ic, ih, iw, self.k1 - self.k0, 3, 3, 1, 1, pad, pad, pad, pad)
        h = C.c_void_p()
        check(lib.fc_conv_create(ctx.handle, C.byref(desc), _lib.ALGO_WINOGRAD, _lib.MODE_NAMES[mode],
                                 C.c_void_p(w_slice.ctypes.data), C.byref(h)), "fc_conv_create")
        self._conv = h
        d_in = C.c_void_p()
        check(lib.fc_conv_device_buffers(h, C.byref(d_in), None), "fc_conv_device_buffers")
        self._d_in = d_in
        self.out_bytes = 4 * self.oc * self.oh * self.ow
        self._outs = [ctx.alloc(self.out_bytes), ctx.alloc(self.out_bytes)]  # alternate by step
        self._flags = ctx.zeros(4 * 8)
        ctx.synchronize()  # the flags are zero before any peer can learn their address
        self.step = 0

        # exchange the IPC handle of this rank's arena and the offsets of its three buffers
        handle = (C.c_ubyte * 64)()
        offs = []
        for p in (*self._outs, self._flags):
            off = C.c_size_t()
            check(lib.fc_peer_export(ctx.handle, C.c_void_p(p), handle, C.byref(off)), "fc_peer_export")
            offs.append(off.value)
        mine = (bytes(handle), offs)
        everyone = [None] * self.world
        dist.all_gather_object(everyone, mine, group=group)
        self._peer_outs = [[0] * self.world, [0] * self.world]
        self._peer_flags = [0] * self.world
        opened = ctx._peer_arenas
        for r, (hbytes, roffs) in enumerate(everyone):
            if r == self.rank:
                base = None
            else:
                if hbytes not in opened:  # one mapping per peer arena and process
                    b = C.c_void_p()
                    buf = (C.c_ubyte * 64).from_buffer_copy(hbytes)
                    check(lib.fc_peer_open(ctx.handle, buf, C.byref(b)), "fc_peer_open")
                    opened[hbytes] = b.value
                base = opened[hbytes]
            for i in range(2):
                self._peer_outs[i][r] = self._outs[i] if base is None else base + roffs[i]
            self._peer_flags[r] = self._flags if base is None else base + roffs[2]
        dist.barrier(group=group)
        ctx.adopt(self)

    def upload(self, x: np.ndarray) -> None:
        self.ctx.upload(np.ascontiguousarray(x, dtype=np.float32), self._d_in.value)

    def forward(self) -> int:
        """Enqueues one forward on the context stream; returns the device address of the full output."""
        self.step += 1
        which = self.step & 1
        vp = C.c_void_p * self.world
        outs, flags = vp(*self._peer_outs[which]), vp(*self._peer_flags)
        self._check(self._lib.fc_conv_forward_scatter(self._conv, self._d_in, outs, flags, self.world, self.rank,
                                                      self.k0, self.oc, self.step), "fc_conv_forward_scatter")
        self._check(self._lib.fc_peer_wait(self.ctx.handle, C.c_void_p(self._flags), self.world, self.step),
                    "fc_peer_wait")
        return self._outs[which]

    def result(self, dptr: int) -> np.ndarray:
        self.ctx.synchronize()
        return self.ctx.download(dptr, (1, self.oc, self.oh, self.ow))

    def release(self) -> None:
        if self._conv is not None:
            self._lib.fc_conv_destroy(self._conv)
            self._conv = None

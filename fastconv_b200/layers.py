"""Host-side mirror of FastConv's operator interface over the C ABI.

`ConvLayer`, `ConvWinoF63ZCLayer` and `ConvIm2colLayer` keep the reference's constructor
arguments, `Init()/Forward()/Tuning()` methods, return values and public `output_data`
(conv_layer.h:24-149, convLayer/winoF63ConvZC.h:9-43, convLayer/im2colConv.h:9-53), so a test
written against the reference classes reads the same here.  Additions are keyword-only: `batch`,
`mode` (arithmetic of the multiply-accumulate stage) and `ctx` (the GPU context to run on).

All compute happens in libfastconv_b200.so on the GPU; this module only moves pointers.
"""
from __future__ import annotations

import ctypes as C
import sys
import weakref
from typing import Optional

import numpy as np

from . import _lib
from ._lib import ConvDesc, check

_FLOAT = np.dtype(np.float32)


def _as_f32(a, what: str) -> np.ndarray:
    if a is None:
        raise ValueError(f"{what} is None")
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a


def _ptr(a: np.ndarray) -> C.c_void_p:
    return C.c_void_p(a.ctypes.data)


class Context:
    """One GPU, one stream, one device arena (fc_context)."""

    def __init__(self, device: int = 0, arena_bytes: int = 1 << 30, *, _borrowed: Optional[C.c_void_p] = None):
        self._lib = _lib.load()
        self._owned = _borrowed is None
        if _borrowed is None:
            h = C.c_void_p()
            check(self._lib.fc_context_create(device, arena_bytes, C.byref(h)), "fc_context_create")
        else:  # a context that belongs to a communicator (fc_comm_context): used here, destroyed there
            h = _borrowed
            dev = C.c_int()
            check(self._lib.fc_context_device(h, C.byref(dev)), "fc_context_device")
            device = dev.value
        self._h = h
        self.device = device
        self._pinned = []
        self._children = weakref.WeakSet()  # layers / layer lists planned on this context
        self._peer_arenas = {}  # IPC handle bytes -> base address of a peer's arena mapped into this process

    def adopt(self, child) -> None:
        """Registers an object with a release()/close() method that must run before the context goes."""
        self._children.add(child)

    # -- lifetime ---------------------------------------------------------------------------
    def close_peer_mappings(self) -> None:
        """Unmaps the arenas of other ranks.  Call it on every rank, then synchronise the ranks, BEFORE any of
        them destroys its context: an exporter must not free memory a peer still has mapped."""
        for base in self._peer_arenas.values():
            self._lib.fc_peer_close(self._h, C.c_void_p(base))
        self._peer_arenas = {}

    def close(self) -> None:
        if getattr(self, "_h", None):
            for child in list(self._children):  # their device buffers live in this context's arena
                (getattr(child, "release", None) or child.close)()
            self.close_peer_mappings()
            for p in self._pinned:
                self._lib.fc_host_free_pinned(p)
            self._pinned = []
            if self._owned:
                self._lib.fc_context_destroy(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def handle(self) -> C.c_void_p:
        if not self._h:
            raise RuntimeError("context is closed")
        return self._h

    @property
    def stream(self) -> C.c_void_p:
        """The context's cudaStream_t as an opaque pointer."""
        s = C.c_void_p()
        check(self._lib.fc_context_stream(self.handle, C.byref(s)), "fc_context_stream")
        return s

    # -- arena (PrivateMemPool / CommonMemPool of utility/mempool.h) -----------------------------
    def alloc(self, nbytes: int) -> int:
        p = C.c_void_p()
        check(self._lib.fc_arena_alloc(self.handle, nbytes, C.byref(p)), "fc_arena_alloc")
        return p.value

    def free(self, dptr: int) -> None:
        check(self._lib.fc_arena_free(self.handle, C.c_void_p(dptr)), "fc_arena_free")

    def size_of(self, dptr: int) -> int:
        n = C.c_size_t()
        check(self._lib.fc_arena_size_of(self.handle, C.c_void_p(dptr), C.byref(n)), "fc_arena_size_of")
        return n.value

    def free_all(self) -> None:
        check(self._lib.fc_arena_free_all(self.handle), "fc_arena_free_all")

    def stats(self) -> dict:
        cap, use, peak, blocks = C.c_size_t(), C.c_size_t(), C.c_size_t(), C.c_size_t()
        check(self._lib.fc_arena_stats(self.handle, C.byref(cap), C.byref(use), C.byref(peak), C.byref(blocks)),
              "fc_arena_stats")
        return {"capacity": cap.value, "in_use": use.value, "peak": peak.value, "blocks": blocks.value}

    def common_request(self, nbytes: int, pool_id: int) -> None:
        check(self._lib.fc_arena_common_request(self.handle, nbytes, pool_id), "fc_arena_common_request")

    def common_commit(self) -> None:
        check(self._lib.fc_arena_common_commit(self.handle), "fc_arena_common_commit")

    def common_ptr(self, pool_id: int) -> int:
        p = C.c_void_p()
        check(self._lib.fc_arena_common_ptr(self.handle, pool_id, C.byref(p)), "fc_arena_common_ptr")
        return p.value

    def common_free(self, pool_id: int) -> None:
        check(self._lib.fc_arena_common_free(self.handle, pool_id), "fc_arena_common_free")

    # -- copies ------------------------------------------------------------------------------
    def upload(self, host: np.ndarray, dptr: Optional[int] = None) -> int:
        host = _as_f32(host, "host array")
        if dptr is None:
            dptr = self.alloc(host.nbytes)
        check(self._lib.fc_memcpy_h2d(self.handle, C.c_void_p(dptr), _ptr(host), host.nbytes), "fc_memcpy_h2d")
        return dptr

    def download(self, dptr: int, shape) -> np.ndarray:
        out = np.empty(shape, dtype=np.float32)
        check(self._lib.fc_memcpy_d2h(self.handle, _ptr(out), C.c_void_p(dptr), out.nbytes), "fc_memcpy_d2h")
        return out

    def zeros(self, nbytes: int) -> int:
        p = self.alloc(nbytes)
        check(self._lib.fc_memset_device(self.handle, C.c_void_p(p), 0, nbytes), "fc_memset_device")
        return p

    def timer_record(self, slot: int) -> None:
        check(self._lib.fc_timer_record(self.handle, slot), "fc_timer_record")

    def timer_elapsed_ms(self, start_slot: int, stop_slot: int) -> float:
        ms = C.c_float()
        check(self._lib.fc_timer_elapsed_ms(self.handle, start_slot, stop_slot, C.byref(ms)), "fc_timer_elapsed_ms")
        return float(ms.value)

    def pinned(self, shape) -> np.ndarray:
        """A float32 array in page-locked host memory (kept alive by the returned array's base)."""
        n = int(np.prod(shape))
        p = C.c_void_p()
        check(self._lib.fc_host_alloc_pinned(n * 4, C.byref(p)), "fc_host_alloc_pinned")
        buf = (C.c_float * n).from_address(p.value)
        arr = np.frombuffer(buf, dtype=np.float32).reshape(shape)
        self._pinned.append(p)
        return arr

    def synchronize(self) -> None:
        check(self._lib.fc_context_synchronize(self.handle), "fc_context_synchronize")


_default_ctx: Optional[Context] = None


def default_context() -> Context:
    global _default_ctx
    if _default_ctx is None or not _default_ctx._h:
        _default_ctx = Context(0)
    return _default_ctx


def make_desc(batch, ic, ih, iw, oc, kh=3, kw=3, sh=1, sw=1, pad_left=1, pad_right=1, pad_top=1, pad_bottom=1,
              group=1) -> ConvDesc:
    return ConvDesc(batch, ic, ih, iw, oc, kh, kw, sh, sw, pad_left, pad_right, pad_top, pad_bottom, group)


def output_size(desc: ConvDesc):
    oh, ow = C.c_int(), C.c_int()
    check(_lib.load().fc_conv_output_size(C.byref(desc), C.byref(oh), C.byref(ow)), "fc_conv_output_size")
    return oh.value, ow.value


def select_algorithm(desc: ConvDesc) -> int:
    """select_algorithm of ConvTest.cpp:318-331 (1x1 stride 1 resolves to the implicit GEMM)."""
    a = C.c_int()
    check(_lib.load().fc_select_algorithm(C.byref(desc), C.byref(a)), "fc_select_algorithm")
    return a.value


def resolve_plan(desc: ConvDesc, algorithm="auto", mode="tf32", sm_count: int = 0):
    """(algorithm, math mode) that a layer planned with these arguments runs, as names; needs no GPU.

    `auto` is select_algorithm of ConvTest.cpp:318-331 plus, in the TF32 modes, the direct tensor-core kernel where
    the measured crossovers favour it; "tf32" (the mode that keeps rel-L2 <= 3e-3) resolves to "tf32" or "3xtf32" per
    layer, "tf32-unbounded" always to "tf32"."""
    algo = _lib.ALGO_NAMES[algorithm] if isinstance(algorithm, str) else int(algorithm)
    m = _lib.MODE_NAMES[mode] if isinstance(mode, str) else int(mode)
    a, r = C.c_int(), C.c_int()
    check(_lib.load().fc_resolve_plan(C.byref(desc), algo, m, int(sm_count), C.byref(a), C.byref(r)), "fc_resolve_plan")
    names = {v: k for k, v in _lib.ALGO_NAMES.items()}
    return names[a.value], _lib.MODE_LABELS[r.value]


def diff(a: np.ndarray, b: np.ndarray) -> float:
    """diff() of utility/helper.cpp:74-89, printing the same line."""
    a = _as_f32(a, "a").ravel()
    b = _as_f32(b, "b").ravel()
    d = float(_lib.load().fc_diff(_ptr(a), _ptr(b), a.size))
    print("The difference is %.5f" % d)
    return d


class ConvLayer:
    """Base operator, conv_layer.h:24-149.

    The constructor deep-copies input / kernel (here: keeps host copies and uploads the kernel to
    the device at Init), computes the output size (conv_layer.h:68-69) and owns `output_data`.
    `Init/Forward/Tuning` of the base class return -1 like the reference's.
    """

    _algo = _lib.ALGO_AUTO

    def __init__(self, input, kernel, biasw, output_ref, ic, ih, iw, oc, kh=3, kw=3, sh=1, sw=1, pad_left=1,
                 pad_right=1, pad_top=1, pad_bottom=1, g=1, bias=False, nt=1, iter=10, *, batch=1, mode="fp32",
                 ctx: Optional[Context] = None):
        if g == 0 or sw == 0 or sh == 0:
            raise AssertionError("group and strides must be non-zero (conv_layer.h:62-63)")
        self.num_threads, self.iterations = int(nt), int(iter)
        self.input_channels, self.input_height, self.input_width = int(ic), int(ih), int(iw)
        self.output_channels, self.kernel_height, self.kernel_width = int(oc), int(kh), int(kw)
        self.stride_height, self.stride_width = int(sh), int(sw)
        self.padding_left, self.padding_right = int(pad_left), int(pad_right)
        self.padding_top, self.padding_bottom = int(pad_top), int(pad_bottom)
        self.group, self.bias_term, self.batch = int(g), bool(bias), int(batch)
        self.mode = _lib.MODE_NAMES[mode] if isinstance(mode, str) else int(mode)
        self.output_ref = output_ref
        self.desc = make_desc(self.batch, ic, ih, iw, oc, kh, kw, sh, sw, pad_left, pad_right, pad_top, pad_bottom, g)
        self.output_width = (self.input_width + pad_left + pad_right - kw) // sw + 1
        self.output_height = (self.input_height + pad_top + pad_bottom - kh) // sh + 1
        self.input_data = _as_f32(input, "input").reshape(self.batch, ic, ih, iw).copy()
        self.kernel_data = _as_f32(kernel, "kernel").reshape(oc, ic // int(g), kh, kw).copy()
        self.bias_data = None if biasw is None else _as_f32(biasw, "bias").copy()
        self.output_data = np.zeros((self.batch, oc, self.output_height, self.output_width), dtype=np.float32)
        self._ctx = ctx
        self._lib = _lib.load()
        self._conv = None
        self.stage_ms = None

    def get_output_height(self) -> int:
        return self.output_height

    def get_output_width(self) -> int:
        return self.output_width

    def Init(self) -> int:
        return -1

    def Forward(self) -> int:
        return -1

    def Tuning(self) -> int:
        return -1

    # -- shared machinery -------------------------------------------------------------------------
    @property
    def ctx(self) -> Context:
        if self._ctx is None:
            self._ctx = default_context()
        return self._ctx

    def _create(self) -> None:
        if self._conv is not None:
            return
        h = C.c_void_p()
        check(self._lib.fc_conv_create(self.ctx.handle, C.byref(self.desc), self._algo, self.mode,
                                       _ptr(self.kernel_data), C.byref(h)), "fc_conv_create")
        self._conv = h
        self.ctx.adopt(self)

    def _forward_iterations(self, labels) -> None:
        """`iterations` forwards from host memory; prints the reference's timing lines with device times."""
        self._create()
        d_in, d_out = C.c_void_p(), C.c_void_p()
        check(self._lib.fc_conv_device_buffers(self._conv, C.byref(d_in), C.byref(d_out)), "fc_conv_device_buffers")
        check(self._lib.fc_conv_forward_host(self._conv, _ptr(self.input_data), _ptr(self.output_data)),
              "fc_conv_forward_host")
        ms = (C.c_float * 5)()
        check(self._lib.fc_conv_profile(self._conv, d_in, d_out, max(1, self.iterations), ms), "fc_conv_profile")
        self.stage_ms = [float(x) for x in ms]
        for label, idx in labels:
            print("%s %fms" % (label, self.stage_ms[idx]))

    def set_epilogue(self, bias: Optional[np.ndarray] = None, relu: bool = False) -> None:
        """Per-channel bias (oc floats) and/or ReLU applied to every output element inside the layer's last kernel."""
        self._create()
        b = None
        if bias is not None:
            b = _as_f32(bias, "bias")
            if b.size != self.desc.oc:
                raise ValueError(f"bias has {b.size} values, the layer {self.desc.oc} output channels")
        check(self._lib.fc_conv_set_epilogue(self._conv, None if b is None else _ptr(b), 1 if relu else 0),
              "fc_conv_set_epilogue")

    def set_kernel_config(self, bm: int = 0, bn: int = 0, variant: int = 0, smem_kb: int = 0) -> None:
        """Fixes the kernel configuration by hand (what mc/nc/kc/row_batch/col_batch of the reference's im2col
        constructor and the block members its Winograd Tuning() assigns are to the reference); zeros = heuristic."""
        self._create()
        check(self._lib.fc_conv_set_kernel_config(self._conv, bm, bn, variant, smem_kb), "fc_conv_set_kernel_config")

    @property
    def kernel_launches(self) -> int:
        """Kernel launches of one Forward (3 per pass of a Winograd layer, 1 for an implicit GEMM)."""
        self._create()
        k = C.c_int()
        check(self._lib.fc_conv_launches_per_forward(self._conv, C.byref(k)), "fc_conv_launches_per_forward")
        return k.value

    def release(self) -> None:
        if self._conv is not None:
            self._lib.fc_conv_destroy(self._conv)
            self._conv = None

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


class ConvWinoF63ZCLayer(ConvLayer):
    """Winograd F(6x6,3x3) layer, convLayer/winoF63ConvZC.{h,cpp}.

    Init() returns -1 and Forward() returns 1 on success, as the reference does
    (winoF63ConvZC.cpp:212, :258).  A shape the Winograd driver cannot compute (anything but 3x3,
    stride 1, symmetric padding -- the reference silently computes garbage there,
    winoF63ZC/winoF63ZC.cpp:334-338) raises FastConvError with status FC_ERR_UNSUPPORTED.
    """

    _algo = _lib.ALGO_WINOGRAD

    def Tuning(self) -> int:
        self._create()
        check(self._lib.fc_conv_tune(self._conv, max(1, self.iterations), 1), "fc_conv_tune")
        return -1

    def Init(self) -> int:
        print("Algorithm: winograd F63")
        self._create()
        return -1

    def Forward(self) -> int:
        self._forward_iterations([("InputTran time:", 0), ("KernelTran time:", 1), ("TensorGEMM time:", 2),
                                  ("OutputTran time:", 3), ("Total time:", 4)])
        if self.output_ref is not None:
            diff(np.asarray(self.output_ref), self.output_data)
        return 1


class ConvIm2colLayer(ConvLayer):
    """im2col + SGEMM layer, convLayer/im2colConv.{h,cpp}; Init() and Forward() return 1 (im2colConv.cpp:234, :258).

    The blocking parameters of the reference constructor (mc, nc, kc, gemm_version, row_batch,
    col_batch, pack_c_version, mt_pack_b_version, prefetch_a/b/c; im2colConv.h:16-18) are accepted
    and ignored: they describe ARM cache blocking that has no counterpart in the GPU kernel.
    """

    _algo = _lib.ALGO_IM2COL

    def __init__(self, *args, mc=8, nc=256, kc=384, gemm_version=1, row_batch=8, col_batch=8, pack_c_version=0,
                 mt_pack_b_version=2, prefetch_a=256, prefetch_b=256, prefetch_c=0, **kw):
        super().__init__(*args, **kw)
        self.M = self.output_channels
        self.N = self.output_height * self.output_width
        self.K = self.input_channels * self.kernel_height * self.kernel_width

    def Tuning(self) -> int:
        self._create()
        check(self._lib.fc_conv_tune(self._conv, max(1, self.iterations), 1), "fc_conv_tune")
        return 1

    def Init(self) -> int:
        print("Algorithm: im2col")
        self._create()
        return 1

    def Forward(self) -> int:
        self._forward_iterations([("Im2colTran time:", 0), ("Gemm time:", 2), ("Total time:", 4)])
        if self.output_ref is not None:
            diff(np.asarray(self.output_ref), self.output_data)
        return 1

    def im2col(self, image: int = 0) -> np.ndarray:
        """The gathered matrix [ic*kh*kw][oh*ow] of one image (ConvIm2colLayer::im2col, im2colConv.cpp:285-309)."""
        ctx = self.ctx
        d_in = ctx.upload(self.input_data)
        n = self.K * self.N
        d_b = ctx.alloc(n * 4)
        try:
            check(self._lib.fc_im2col_gather(ctx.handle, C.c_void_p(d_in), C.c_void_p(d_b), C.byref(self.desc), image),
                  "fc_im2col_gather")
            return ctx.download(d_b, (self.K, self.N))
        finally:
            ctx.free(d_b)
            ctx.free(d_in)


class ConvDirectLayer(ConvLayer):
    """`-a direct`: the reference parses the name but its case is empty (ConvTest.cpp:369-371).  Here it is the direct
    convolution on the tensor cores: ungrouped layers of stride 1 or 2 in mode "tf32" (shifted TMA boxes of an NHWC copy of
    the input, no Winograd transform, so single-pass TF32 keeps its plain accuracy); any other layer or mode runs as
    the implicit GEMM.  Init() and Forward() return 1 like the im2col layer's."""

    _algo = _lib.ALGO_DIRECT

    def Tuning(self) -> int:
        self._create()
        check(self._lib.fc_conv_tune(self._conv, max(1, self.iterations), 1), "fc_conv_tune")
        return 1

    def Init(self) -> int:
        print("Algorithm: direct")
        self._create()
        return 1

    def Forward(self) -> int:
        self._forward_iterations([("Gemm time:", 2), ("Total time:", 4)])
        if self.output_ref is not None:
            diff(np.asarray(self.output_ref), self.output_data)
        return 1

    @property
    def algorithm(self) -> int:
        """The algorithm the layer actually runs (ALGO_DIRECT or ALGO_IM2COL)."""
        self._create()
        a = C.c_int()
        check(self._lib.fc_conv_algorithm(self._conv, C.byref(a)), "fc_conv_algorithm")
        return a.value


class LayerList:
    """Several initialised layers replayed as one CUDA graph (fc_layer_list): the in-process form of the
    reference's per-network shell loops (run_vgg16.sh:5-13, run_resnet50.sh:10-30)."""

    def __init__(self, ctx: Context, convs, d_ins, d_outs):
        self._lib = _lib.load()
        n = len(convs)
        arr = C.c_void_p * n
        h = C.c_void_p()
        check(self._lib.fc_layer_list_create(ctx.handle, arr(*[c.value if isinstance(c, C.c_void_p) else c for c in convs]),
                                             arr(*[int(p) for p in d_ins]), arr(*[int(p) for p in d_outs]), n,
                                             C.byref(h)), "fc_layer_list_create")
        self._h = h
        ctx.adopt(self)
        k = C.c_int()
        check(self._lib.fc_layer_list_launches(h, C.byref(k)), "fc_layer_list_launches")
        self.kernel_launches = k.value

    def forward(self) -> None:
        check(self._lib.fc_layer_list_forward(self._h), "fc_layer_list_forward")

    def forward_host(self, host_ins, host_outs) -> None:
        """All layers from/to host arrays; uploads, kernels and downloads of neighbouring layers overlap.
        A None entry skips that copy: the layer is chained to its neighbour on the device."""
        n = len(host_ins)
        arr = C.c_void_p * n
        ptr = lambda a: None if a is None else a.ctypes.data  # noqa: E731
        check(self._lib.fc_layer_list_forward_host(self._h, arr(*[ptr(a) for a in host_ins]),
                                                   arr(*[ptr(a) for a in host_outs])),
              "fc_layer_list_forward_host")

    def close(self) -> None:
        if self._h:
            self._lib.fc_layer_list_destroy(self._h)
            self._h = None


def make_layer(algorithm: str, *args, **kw) -> ConvLayer:
    """The dispatch of ConvTest.cpp:365-413 (`-a auto|direct|im2col|winograd`).

    `auto` asks the library for the per-layer plan (fc_resolve_plan) and returns the matching layer class; the layer
    itself is still created with the algorithm AUTO, so that the library records the request: the math mode then
    resolves as for `-a auto` and Tuning() may time the rival algorithms too."""
    algo = _lib.ALGO_NAMES[algorithm]
    requested_auto = algo == _lib.ALGO_AUTO
    if requested_auto:
        probe = ConvLayer(*args, **kw)
        name, _ = resolve_plan(probe.desc, "auto", probe.mode)
        algo = _lib.ALGO_NAMES[name]
    cls = {_lib.ALGO_WINOGRAD: ConvWinoF63ZCLayer, _lib.ALGO_DIRECT: ConvDirectLayer}.get(algo, ConvIm2colLayer)
    layer = cls(*args, **kw)
    if requested_auto:
        layer._algo = _lib.ALGO_AUTO  # instance attribute: fc_conv_create resolves it to the same plan
    return layer

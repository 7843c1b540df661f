"""ctypes binding of libfastconv_b200.so -- the C ABI declared in include/fastconv_b200.h.

Nothing here computes: every call goes to the CUDA library.  If the library is missing or has
no GPU to run on, the calls raise; there is no CPU path behind this module.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

from . import build as _build

FC_OK = 0
(FC_ERR_INVALID_ARG, FC_ERR_UNSUPPORTED, FC_ERR_OUT_OF_MEMORY, FC_ERR_CUDA, FC_ERR_NO_DEVICE, FC_ERR_TIMEOUT,
 FC_ERR_COMM) = -1, -2, -3, -4, -5, -6, -7
ALGO_AUTO, ALGO_DIRECT, ALGO_IM2COL, ALGO_WINOGRAD = 0, 1, 2, 3
MATH_FP32_MIRRORED, MATH_3XTF32, MATH_TF32, MATH_TF32_UNBOUNDED, MATH_TF32_U16 = 0, 1, 2, 3, 4
MODE_LABELS = {0: "fp32", 1: "3xtf32", 2: "tf32", 4: "tf32-u16"}  # what fc_conv_math_mode / fc_resolve_plan report
MODE_NAMES = {"fp32": MATH_FP32_MIRRORED, "ffma": MATH_FP32_MIRRORED, "3xtf32": MATH_3XTF32, "tf32": MATH_TF32,
              "tf32-unbounded": MATH_TF32_UNBOUNDED, "tf32-u16": MATH_TF32_U16}
ALGO_NAMES = {"auto": ALGO_AUTO, "direct": ALGO_DIRECT, "im2col": ALGO_IM2COL, "winograd": ALGO_WINOGRAD}


class ConvDesc(C.Structure):
    """fc_conv_desc"""

    _fields_ = [(n, C.c_int32) for n in (
        "batch", "ic", "ih", "iw", "oc", "kh", "kw", "sh", "sw",
        "pad_left", "pad_right", "pad_top", "pad_bottom", "group")]


class FastConvError(RuntimeError):
    def __init__(self, status: int, where: str, message: str):
        super().__init__(f"{where}: status {status} ({message})")
        self.status = status


_fp = C.POINTER(C.c_float)
_vp = C.c_void_p
_szp = C.POINTER(C.c_size_t)
_ip = C.POINTER(C.c_int)
_dp = C.POINTER(ConvDesc)

# name -> (restype, argtypes); every symbol include/fastconv_b200.h declares
SIGNATURES = {
    "fc_abi_version": (C.c_int, []),
    "fc_status_string": (C.c_char_p, [C.c_int]),
    "fc_last_error": (C.c_char_p, []),
    "fc_device_count": (C.c_int, [_ip]),
    "fc_context_create": (C.c_int, [C.c_int, C.c_size_t, C.POINTER(_vp)]),
    "fc_context_destroy": (C.c_int, [_vp]),
    "fc_context_synchronize": (C.c_int, [_vp]),
    "fc_context_device": (C.c_int, [_vp, _ip]),
    "fc_context_stream": (C.c_int, [_vp, C.POINTER(_vp)]),
    "fc_arena_alloc": (C.c_int, [_vp, C.c_size_t, C.POINTER(_vp)]),
    "fc_arena_size_of": (C.c_int, [_vp, _vp, _szp]),
    "fc_arena_free": (C.c_int, [_vp, _vp]),
    "fc_arena_free_all": (C.c_int, [_vp]),
    "fc_arena_stats": (C.c_int, [_vp, _szp, _szp, _szp, _szp]),
    "fc_arena_common_request": (C.c_int, [_vp, C.c_size_t, C.c_size_t]),
    "fc_arena_common_commit": (C.c_int, [_vp]),
    "fc_arena_common_ptr": (C.c_int, [_vp, C.c_size_t, C.POINTER(_vp)]),
    "fc_arena_common_free": (C.c_int, [_vp, C.c_size_t]),
    "fc_memcpy_h2d": (C.c_int, [_vp, _vp, _vp, C.c_size_t]),
    "fc_memcpy_d2h": (C.c_int, [_vp, _vp, _vp, C.c_size_t]),
    "fc_memset_device": (C.c_int, [_vp, _vp, C.c_int, C.c_size_t]),
    "fc_host_alloc_pinned": (C.c_int, [C.c_size_t, C.POINTER(_vp)]),
    "fc_host_free_pinned": (C.c_int, [_vp]),
    "fc_timer_record": (C.c_int, [_vp, C.c_int]),
    "fc_timer_elapsed_ms": (C.c_int, [_vp, C.c_int, C.c_int, _fp]),
    "fc_conv_output_size": (C.c_int, [_dp, _ip, _ip]),
    "fc_select_algorithm": (C.c_int, [_dp, _ip]),
    "fc_wino_buffer_elems": (C.c_int, [_dp, C.c_int, _szp, _szp, _szp]),
    "fc_wino_filter_transform": (C.c_int, [_vp, _vp, _vp, C.c_int, C.c_int, C.c_int]),
    "fc_wino_input_transform": (C.c_int, [_vp, _vp, _vp, _dp, C.c_int]),
    "fc_wino_tensor_gemm": (C.c_int, [_vp, _vp, _vp, _vp, _dp, C.c_int]),
    "fc_wino_output_transform": (C.c_int, [_vp, _vp, _vp, _dp]),
    "fc_wino_forward": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _dp, C.c_int, _fp]),
    "fc_wino_forward_static_scratch": (C.c_int, [_vp, _vp, _vp, _dp, _vp]),
    "fc_im2col_gather": (C.c_int, [_vp, _vp, _vp, _dp, C.c_int]),
    "fc_igemm_packed_elems": (C.c_int, [C.c_int, C.c_int, _szp]),
    "fc_igemm_pack_weights": (C.c_int, [_vp, _vp, _vp, C.c_int, C.c_int]),
    "fc_igemm_forward": (C.c_int, [_vp, _vp, _vp, _vp, _dp, C.c_int]),
    "fc_conv_create": (C.c_int, [_vp, _dp, C.c_int, C.c_int, _vp, C.POINTER(_vp)]),
    "fc_conv_destroy": (C.c_int, [_vp]),
    "fc_resolve_plan": (C.c_int, [_dp, C.c_int, C.c_int, C.c_int, _ip, _ip]),
    "fc_conv_algorithm": (C.c_int, [_vp, _ip]),
    "fc_conv_math_mode": (C.c_int, [_vp, _ip]),
    "fc_conv_forward_device": (C.c_int, [_vp, _vp, _vp]),
    "fc_conv_forward_host": (C.c_int, [_vp, _vp, _vp]),
    "fc_conv_device_buffers": (C.c_int, [_vp, C.POINTER(_vp), C.POINTER(_vp)]),
    "fc_conv_time_device": (C.c_int, [_vp, _vp, _vp, C.c_int, C.c_int, _fp]),
    "fc_conv_profile": (C.c_int, [_vp, _vp, _vp, C.c_int, _fp]),
    "fc_conv_tune": (C.c_int, [_vp, C.c_int, C.c_int]),
    "fc_conv_launches_per_forward": (C.c_int, [_vp, _ip]),
    "fc_layer_list_create": (C.c_int, [_vp, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp), C.c_int, C.POINTER(_vp)]),
    "fc_layer_list_forward": (C.c_int, [_vp]),
    "fc_layer_list_forward_host": (C.c_int, [_vp, C.POINTER(_vp), C.POINTER(_vp)]),
    "fc_layer_list_launches": (C.c_int, [_vp, _ip]),
    "fc_layer_list_destroy": (C.c_int, [_vp]),
    "fc_conv_set_epilogue": (C.c_int, [_vp, _vp, C.c_int]),
    "fc_context_info": (C.c_int, [_vp, _ip, _ip]),
    "fc_conv_round_times": (C.c_int, [_vp, _fp, C.c_int, _ip]),
    "fc_conv_work": (C.c_int, [_vp] + [C.POINTER(C.c_double)] * 4),
    "fc_conv_set_kernel_config": (C.c_int, [_vp, C.c_int, C.c_int, C.c_int, C.c_int]),
    "fc_conv_get_kernel_config": (C.c_int, [_vp, _ip, _ip, _ip, _ip]),
    "fc_peer_export": (C.c_int, [_vp, _vp, _vp, _vp]),
    "fc_peer_open": (C.c_int, [_vp, _vp, _vp]),
    "fc_peer_close": (C.c_int, [_vp, _vp]),
    "fc_conv_forward_scatter": (C.c_int, [_vp, _vp, _vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "fc_peer_wait": (C.c_int, [_vp, _vp, C.c_int, C.c_int]),
    "fc_context_set_wait_limit_ms": (C.c_int, [_vp, C.c_int]),
    "fc_comm_init_all": (C.c_int, [C.c_int, _ip, C.c_size_t, C.POINTER(_vp)]),
    "fc_comm_init_env": (C.c_int, [C.c_int, C.c_size_t, C.POINTER(_vp)]),
    "fc_comm_destroy": (C.c_int, [_vp]),
    "fc_comm_size": (C.c_int, [_vp, _ip, _ip, _ip]),
    "fc_comm_context": (C.c_int, [_vp, C.c_int, C.POINTER(_vp)]),
    "fc_comm_barrier": (C.c_int, [_vp]),
    "fc_comm_allreduce_max": (C.c_int, [_vp, C.POINTER(C.c_double)]),
    "fc_comm_allgather": (C.c_int, [_vp, _vp, _vp, C.c_size_t]),
    "fc_shard_range": (C.c_int, [C.c_int, C.c_int, C.c_int, _ip, _ip]),
    "fc_sharded_conv_create": (C.c_int, [_vp, _dp, C.c_int, C.c_int, C.c_int, C.c_int, _vp, C.POINTER(_vp)]),
    "fc_sharded_conv_destroy": (C.c_int, [_vp]),
    "fc_sharded_conv_part": (C.c_int, [_vp, C.c_int, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp), _ip, _ip]),
    "fc_sharded_conv_upload": (C.c_int, [_vp, _vp]),
    "fc_sharded_conv_forward": (C.c_int, [_vp]),
    "fc_sharded_conv_wait": (C.c_int, [_vp]),
    "fc_sharded_conv_download": (C.c_int, [_vp, _vp]),
    "fc_sharded_conv_forward_host": (C.c_int, [_vp, _vp, _vp]),
    "fc_sharded_conv_time_device": (C.c_int, [_vp, C.c_int, C.c_int, _fp]),
    "fc_diff": (C.c_float, [_vp, _vp, C.c_int]),
}

_lib = None


def library_path() -> Path:
    return _build.LIB_PATH


def load(build_if_missing: bool = True) -> C.CDLL:
    """Load libfastconv_b200.so and type every entry point.  Raises if it cannot be loaded."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if build_if_missing:
        _build.build_library()  # returns at once when the library is newer than every source and header
    elif not path.exists():
        raise FileNotFoundError(f"{path} is not built; run `python -m fastconv_b200.build`")
    lib = C.CDLL(str(path))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = header and library disagree
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status: int, where: str) -> None:
    if status != FC_OK:
        lib = load()
        msg = lib.fc_last_error().decode(errors="replace") or lib.fc_status_string(status).decode()
        raise FastConvError(status, where, msg)

"""ctypes binding of libmixlab_b200.so.  Fails loudly when the library is absent:
there is no Python, torch or CPU fallback for any operator."""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
# MIXLAB_B200_LIB selects another build of the same library (same exports), e.g. to compare two builds
LIB_PATH = os.environ.get("MIXLAB_B200_LIB") or os.path.join(_PKG, "libmixlab_b200.so")

MXB_F32, MXB_BF16 = 1, 2
MXB_GDN_FORCE_FP32_PATH = 1
MXB_GDN_BWD_FP32_KERNELS = 2
MXB_GDN_SAVE_FOR_BWD = 4
MXB_GDN_BWD_USE_SAVED = 8
MXB_GDN_DECODE_REGISTER_KERNEL = 16
MXB_GDN_NO_TMA = 32
MXB_GDN_F32_IO_BF16_OPERANDS = 64
MXB_MAMBA3_CHANNEL_KERNELS = 1
MXB_MAMBA3_RECURRENT_KERNELS = 2
MXB_MAMBA3_SAVE_FOR_BWD = 4
MXB_MAMBA3_BWD_USE_SAVED = 8
MXB_MAMBA3_NO_TMA = 16
MXB_MAMBA3_SERIAL_WALK = 32
MXB_MAMBA3_WINDOW_PARALLEL = 64


class MxbError(RuntimeError):
    def __init__(self, status: int, what: str, detail: str = ""):
        self.status = status
        super().__init__(f"{what}: status {status} ({detail})")


class GdnDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("B", "T", "H", "Dk", "Dv", "chunk", "io_dtype", "gate_is_log", "flags")]


class Mamba3Desc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("B", "T", "D", "N", "G", "nheads", "io_dtype", "flags")]


class IrOp(C.Structure):
    """mxb_ir_op: an IR op record (mlx_ir_program_add_op) after name resolution."""
    _fields_ = [("op_type", C.c_int32), ("inputs", C.POINTER(C.c_void_p)), ("n_inputs", C.c_int32),
                ("outputs", C.POINTER(C.c_void_p)), ("n_outputs", C.c_int32), ("float_params", C.POINTER(C.c_float)),
                ("n_float_params", C.c_int32), ("int_params", C.POINTER(C.c_int32)), ("n_int_params", C.c_int32),
                ("io_dtype", C.c_int32)]


# name -> (restype, argtypes); the complete export list of include/mixlab_b200.h
_P = C.c_void_p
EXPORTS = {
    "mxb_status_string": (C.c_char_p, [C.c_int32]),
    "mxb_version": (C.c_int, []),
    "mxb_last_cuda_error": (C.c_int, []),
    "mxb_launch_count": (C.c_uint64, []),
    "mxb_trace_enable": (None, [C.c_int]),
    "mxb_trace_summary": (C.c_size_t, [C.c_char_p, C.c_size_t]),
    "mxb_gdn_fwd_workspace_bytes": (C.c_size_t, [C.POINTER(GdnDesc)]),
    "mxb_gdn_bwd_workspace_bytes": (C.c_size_t, [C.POINTER(GdnDesc)]),
    "mxb_gdn_fwd": (C.c_int32, [C.POINTER(GdnDesc)] + [_P] * 9 + [C.c_size_t, _P]),
    "mxb_gdn_bwd": (C.c_int32, [C.POINTER(GdnDesc)] + [_P] * 15 + [C.c_size_t, _P]),
    "mxb_gdn_static_scratch_bytes": (C.c_size_t, []),
    "mxb_gdn_fwd_static_scratch": (C.c_int32, [C.POINTER(GdnDesc)] + [_P] * 9),
    "mxb_gdn_device_status": (C.c_int32, [_P, C.POINTER(C.c_int32)]),
    "mxb_gdn_decode_step": (C.c_int32, [C.POINTER(GdnDesc)] + [_P] * 8),
    "mxb_gdn_block_workspace_bytes": (C.c_size_t, [C.POINTER(GdnDesc)]),
    "mxb_gdn_block_pre_fwd": (C.c_int32, [C.POINTER(GdnDesc)] + [_P] * 16),
    "mxb_gdn_block_pre_bwd": (C.c_int32, [C.POINTER(GdnDesc)] + [_P] * 26 + [C.c_size_t, _P]),
    "mxb_gdn_block_post_fwd": (C.c_int32, [C.POINTER(GdnDesc)] + [_P] * 5),
    "mxb_gdn_block_post_bwd": (C.c_int32, [C.POINTER(GdnDesc)] + [_P] * 8 + [C.c_size_t, _P]),
    "mxb_mamba3_fwd_workspace_bytes": (C.c_size_t, [C.POINTER(Mamba3Desc)]),
    "mxb_mamba3_bwd_workspace_bytes": (C.c_size_t, [C.POINTER(Mamba3Desc)]),
    "mxb_mamba3_fwd": (C.c_int32, [C.POINTER(Mamba3Desc)] + [_P] * 9 + [C.c_size_t, _P]),
    "mxb_mamba3_bwd": (C.c_int32, [C.POINTER(Mamba3Desc)] + [_P] * 16 + [C.c_size_t, _P]),
    "mxb_mamba3_block_workspace_bytes": (C.c_size_t, [C.POINTER(Mamba3Desc)]),
    "mxb_mamba3_block_conv_fwd": (C.c_int32, [C.POINTER(Mamba3Desc), C.c_int32] + [_P] * 4),
    "mxb_mamba3_block_conv_bwd": (C.c_int32, [C.POINTER(Mamba3Desc), C.c_int32] + [_P] * 6 + [C.c_size_t, _P]),
    "mxb_mamba3_block_bc_fwd": (C.c_int32, [C.POINTER(Mamba3Desc), C.c_float] + [_P] * 9),
    "mxb_mamba3_block_bc_bwd": (C.c_int32, [C.POINTER(Mamba3Desc), C.c_float] + [_P] * 13 + [C.c_size_t, _P]),
    "mxb_mamba3_block_post_fwd": (C.c_int32, [C.POINTER(Mamba3Desc), C.c_float] + [_P] * 5),
    "mxb_mamba3_block_post_bwd": (C.c_int32, [C.POINTER(Mamba3Desc), C.c_float] + [_P] * 8 + [C.c_size_t, _P]),
    "mxb_dp_partial_floats": (C.c_size_t, []),
    "mxb_dp_sanitize": (C.c_int32, [_P, C.c_size_t, C.c_float, _P, _P]),
    "mxb_dp_finalize": (C.c_int32, [_P, C.c_size_t, C.c_float, C.c_float, _P, _P, _P]),
    "mxb_dp_finalize_dev": (C.c_int32, [_P, C.c_size_t, _P, C.c_float, _P, _P, _P]),
    "mxb_dp_scale": (C.c_int32, [_P, C.c_size_t, _P, _P]),
    "mxb_ir_op_workspace_bytes": (C.c_size_t, [C.POINTER(IrOp)]),
    "mxb_ir_op_forward": (C.c_int32, [C.POINTER(IrOp), _P, C.c_size_t, _P]),
    "mxb_selftest_umma": (C.c_int32, [_P, C.c_uint32, _P, C.c_uint32, _P, _P, _P, _P]),
    "mxb_selftest_wait_timeout": (C.c_int32, [_P, C.c_size_t, C.c_uint32, _P]),
    "mxb_host_ctx_create": (C.c_int32, [C.c_int, C.c_size_t, C.POINTER(_P)]),
    "mxb_host_ctx_destroy": (None, [_P]),
    "mxb_host_gdn": (C.c_int32, [_P, C.POINTER(GdnDesc)] + [_P] * 12),
}

_lib = None


def load_library(path: str | None = None):
    """dlopen the C-ABI library and bind every export; raises if it is missing."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    p = path or LIB_PATH
    if not os.path.exists(p):
        raise ImportError(
            f"{p} not found: build it with `python -m mixlab_b200.build` "
            "(the kernels have no Python/CPU fallback)")
    lib = C.CDLL(p)
    for name, (res, args) in EXPORTS.items():
        fn = getattr(lib, name)  # AttributeError if an export is missing
        fn.restype = res
        fn.argtypes = args
    if path is None:
        _lib = lib
    return lib


def lib():
    return load_library()


def check(status: int, what: str):
    if status != 0:
        l = lib()
        raise MxbError(status, what, l.mxb_status_string(status).decode())

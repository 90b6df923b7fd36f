"""ctypes binding of liblvx.so (declarations in include/lvx.h).

There is no fallback: if the shared library is missing or a call fails, an exception is raised.
torch tensors are passed as raw device pointers; the current CUDA stream is passed as the stream.
"""
from __future__ import annotations

import ctypes
import os

import torch

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "liblvx.so")
_lib = None

LVX_BF16, LVX_FP16, LVX_FP32 = 0, 1, 2
_DTYPE = {torch.bfloat16: LVX_BF16, torch.float16: LVX_FP16, torch.float32: LVX_FP32}

# every symbol include/lvx.h declares
SYMBOLS = [
    "lvx_version", "lvx_last_error", "lvx_device_status", "lvx_device_status_peek", "lvx_p2p_set_timeout",
    "lvx_query_workspace", "lvx_fwd_block", "lvx_fwd_block_bias", "lvx_bwd_block_bias",
    "lvx_kv_project", "lvx_knorm_bwd", "lvx_fwd_block_gathered", "lvx_bwd_block_gathered",
    "lvx_fwd_combine_merge", "lvx_bwd_prep", "lvx_bwd_block", "lvx_add_cast", "lvx_selftest_mma",
    "lvx_fwd_block_static", "lvx_fwd_merge_parts", "lvx_sum_cast",
    "lvx_p2p_signal", "lvx_p2p_gather", "lvx_p2p_fwd_merge", "lvx_p2p_sum_cast", "lvx_p2p_push", "lvx_p2p_wait",
    "lvx_p2p_push_dma",
]
MAX_PEERS = 16      # LVX_MAX_PEERS
P2P_SLOTS = 8       # LVX_P2P_SLOTS


class LvxShape(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("B", "Hq", "Hkv", "Sq", "Skv", "D", "dtype", "q_blocks")]


class LvxPeers(ctypes.Structure):
    _fields_ = [("world", ctypes.c_int32), ("rank", ctypes.c_int32), ("ptr", ctypes.c_void_p * 16),
                ("nbytes", ctypes.c_size_t)]


class LvxBias(ctypes.Structure):
    _fields_ = [("bias", ctypes.c_void_p)] + [(n, ctypes.c_int64) for n in
                                               ("stride_block", "stride_b", "stride_h", "stride_q", "stride_kv")]


class LvxBlockWait(ctypes.Structure):
    _fields_ = [("my_flags", ctypes.c_void_p), ("slot", ctypes.c_int32), ("epoch", ctypes.c_uint32),
                ("first_block", ctypes.c_int32)]


class LvxPushSegment(ctypes.Structure):
    _fields_ = [("src", ctypes.c_void_p), ("src_stride", ctypes.c_size_t), ("dst_offset", ctypes.c_size_t),
                ("dst_rank_stride", ctypes.c_size_t), ("bytes", ctypes.c_size_t), ("src_bytes", ctypes.c_size_t)]


class LvxError(RuntimeError):
    pass


def lib_path() -> str:
    return _LIB_PATH


def load():
    """Loads liblvx.so once. Raises LvxError when it has not been built (python -m lv_xattn_b200.build)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        raise LvxError(f"{_LIB_PATH} is missing: build it with `python -m lv_xattn_b200.build` "
                       "(there is no non-CUDA fallback)")
    lib = ctypes.CDLL(_LIB_PATH)
    vp, i32p, fp = ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p
    sp = ctypes.POINTER(LvxShape)
    lib.lvx_version.restype = ctypes.c_int
    lib.lvx_last_error.restype = ctypes.c_char_p
    lib.lvx_device_status.argtypes = [vp, ctypes.POINTER(ctypes.c_int)]
    lib.lvx_device_status_peek.argtypes = [vp, vp]
    lib.lvx_p2p_set_timeout.argtypes = [ctypes.c_double]
    lib.lvx_query_workspace.argtypes = [sp, ctypes.POINTER(ctypes.c_size_t), ctypes.POINTER(ctypes.c_size_t)]
    lib.lvx_fwd_block.argtypes = [sp, vp, vp, vp, i32p, ctypes.c_float, vp, ctypes.c_size_t, vp]
    bp = ctypes.POINTER(LvxBias)
    lib.lvx_fwd_block_bias.argtypes = [sp, vp, vp, vp, i32p, bp, ctypes.c_float, vp, ctypes.c_size_t, vp]
    lib.lvx_bwd_block_bias.argtypes = [sp, vp, vp, fp, fp, vp, vp, i32p, bp, ctypes.c_float, fp, vp, vp, ctypes.c_int, vp]
    wp = ctypes.POINTER(LvxBlockWait)
    lib.lvx_fwd_block_gathered.argtypes = [sp, vp, vp, vp, i32p, ctypes.c_float, vp, ctypes.c_size_t, wp, vp]
    lib.lvx_bwd_block_gathered.argtypes = [sp, vp, vp, fp, fp, vp, vp, i32p, ctypes.c_float, fp, fp, fp, ctypes.c_int,
                                           wp, vp]
    lib.lvx_kv_project.argtypes = [ctypes.c_int, vp, vp, vp, vp, ctypes.c_float, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                   ctypes.c_int, vp, vp, fp, vp]
    lib.lvx_knorm_bwd.argtypes = [ctypes.c_int, vp, vp, fp, vp, vp, fp, ctypes.c_size_t, vp]
    lib.lvx_fwd_combine_merge.argtypes = [sp, vp, fp, fp, vp, fp, ctypes.c_int, vp]
    lib.lvx_bwd_prep.argtypes = [sp, vp, vp, fp, vp]
    lib.lvx_bwd_block.argtypes = [sp, vp, vp, fp, fp, vp, vp, i32p, ctypes.c_float, fp, fp, fp, ctypes.c_int, vp,
                                  ctypes.c_size_t, vp]
    lib.lvx_add_cast.argtypes = [fp, fp, vp, ctypes.c_int, ctypes.c_size_t, vp]
    lib.lvx_selftest_mma.argtypes = [ctypes.c_int, vp, vp, fp, vp]
    lib.lvx_fwd_merge_parts.argtypes = [sp, fp, fp, ctypes.c_int, ctypes.c_size_t, ctypes.c_size_t, vp, fp, vp]
    lib.lvx_sum_cast.argtypes = [fp, ctypes.c_int, ctypes.c_size_t, vp, ctypes.c_int, ctypes.c_size_t, vp]
    lib.lvx_fwd_block_static.argtypes = [sp, vp, vp, vp, i32p, ctypes.c_float, vp, fp, vp]
    for name in SYMBOLS:
        getattr(lib, name)  # AttributeError here means header and library disagree
        if name != "lvx_last_error":
            getattr(lib, name).restype = ctypes.c_int
    _lib = lib
    return lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().lvx_last_error().decode("utf-8", "replace")
        raise LvxError(f"{what} failed with status {rc}: {msg}")


def ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def stream_ptr():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def make_shape(B, Hq, Hkv, Sq, Skv, D, dtype, q_blocks=1) -> LvxShape:
    if dtype not in _DTYPE:
        raise ValueError(f"unsupported dtype {dtype}; expected bfloat16, float16 or float32")
    return LvxShape(B, Hq, Hkv, Sq, Skv, D, _DTYPE[dtype], q_blocks)


def dtype_code(dtype) -> int:
    return _DTYPE[dtype]


def query_workspace(shape: LvxShape):
    f, b = ctypes.c_size_t(0), ctypes.c_size_t(0)
    check(load().lvx_query_workspace(ctypes.byref(shape), ctypes.byref(f), ctypes.byref(b)), "lvx_query_workspace")
    return f.value, b.value


def device_status() -> int:
    out = ctypes.c_int(0)
    check(load().lvx_device_status(stream_ptr(), ctypes.byref(out)), "lvx_device_status")
    return out.value

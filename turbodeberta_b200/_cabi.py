"""ctypes binding of ``libtdb_b200.so`` (declared in ``include/tdb_b200.h``).

There is no CPU or PyTorch fallback: if the library is missing the import of this module
raises, and every call turns a negative status code into a Python exception.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtdb_b200.so")

TDB_DTYPE_F32, TDB_DTYPE_BF16 = 0, 1
TDB_FLAG_C2P, TDB_FLAG_P2C, TDB_FLAG_P2C_MIRRORED = 1, 2, 4
TDB_KERNEL_AUTO, TDB_KERNEL_SIMT, TDB_KERNEL_UMMA = 0, 1, 2
TDB_EXPAND_MARGIN = 256
TDB_STATIC_MAX_TILES = 65535
TDB_STATIC_SCRATCH_BYTES = 16 + 8 * TDB_STATIC_MAX_TILES
ERR_ARG, ERR_DTYPE, ERR_ALIGN, ERR_SHAPE, ERR_UNSUPPORTED, ERR_CUDA, ERR_TIMEOUT, ERR_WORKSPACE = range(-1, -9, -1)

EXPORTS = ["tdb_version", "tdb_strerror", "tdb_last_error", "tdb_bucket_table", "tdb_relpos_project",
           "tdb_relpos_expand", "tdb_attn_workspace_bytes", "tdb_attn_fwd_fixed", "tdb_attn_fwd_varlen",
           "tdb_attn_fwd_varlen_static", "tdb_attn_fwd_fixed_scores", "tdb_attn_fwd_varlen_scores",
           "tdb_selftest_bounded_wait"]


class TdbError(RuntimeError):
    def __init__(self, code: int, detail: str):
        self.code = code
        super().__init__(f"libtdb_b200: {detail} (code {code})")


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m turbodeberta_b200.build` (needs nvcc). "
            "There is no fallback path.")
    lib = C.CDLL(LIB_PATH)
    vp, i32, i64, f32, sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t
    lib.tdb_version.restype = i32
    lib.tdb_strerror.restype = C.c_char_p
    lib.tdb_strerror.argtypes = [i32]
    lib.tdb_last_error.restype = C.c_char_p
    lib.tdb_bucket_table.restype = i32
    lib.tdb_bucket_table.argtypes = [i32, i32, i32, vp, vp]
    lib.tdb_relpos_project.restype = i32
    lib.tdb_relpos_project.argtypes = [vp, vp, vp, i32, i32, i32, i32, i32, vp, vp, vp]
    lib.tdb_relpos_expand.restype = i32
    lib.tdb_relpos_expand.argtypes = [vp, vp, i32, i32, i32, i32, i32, i32, i32, vp, vp]
    lib.tdb_attn_workspace_bytes.restype = sz
    lib.tdb_attn_workspace_bytes.argtypes = [i32, i64]
    lib.tdb_attn_fwd_fixed.restype = i32
    lib.tdb_attn_fwd_fixed.argtypes = ([vp] * 4 + [i64] * 12 + [vp, vp, i32, vp, i32, vp, vp, i32, i32]
                                       + [vp, i32, i32, i32, i32, f32, i32, i32, i32, vp, vp, vp])
    lib.tdb_attn_fwd_varlen.restype = i32
    lib.tdb_attn_fwd_varlen.argtypes = ([vp] * 4 + [i64] * 8 + [vp, vp, i32, vp, i32, vp, vp, i32, i32]
                                        + [vp, i32, i64, i32, i32, i32, f32, i32, i32, i32, vp, sz, vp, vp, vp])
    lib.tdb_attn_fwd_varlen_static.restype = i32
    lib.tdb_attn_fwd_varlen_static.argtypes = ([vp] * 4 + [i64] * 8 + [vp, vp, i32, vp, i32, vp, vp, i32, i32]
                                               + [vp, i32, i64, i32, i32, i32, f32, i32, i32, i32, vp, vp, vp])
    lib.tdb_selftest_bounded_wait.restype = i32
    lib.tdb_selftest_bounded_wait.argtypes = [vp, i32, i32, vp]
    lib.tdb_attn_fwd_fixed_scores.restype = i32
    lib.tdb_attn_fwd_fixed_scores.argtypes = ([vp] * 4 + [i64] * 12 + [vp, i64, i64, i64, vp, i64, i64, i64]
                                              + [i32, vp, i32, vp, i32, i32, i32, i32, f32, i32, i32, vp, vp, vp])
    lib.tdb_attn_fwd_varlen_scores.restype = i32
    lib.tdb_attn_fwd_varlen_scores.argtypes = ([vp] * 4 + [i64] * 8 + [vp, i64, i64, vp, i64, i64]
                                               + [i32, vp, i32, vp, i32, i64, i32, i32, i32, f32, i32, i32, vp, vp, vp])
    return lib


lib = _load()


def check(code: int) -> None:
    if code == 0:
        return
    detail = lib.tdb_last_error().decode() or lib.tdb_strerror(code).decode()
    if code in (ERR_ARG, ERR_DTYPE, ERR_ALIGN, ERR_SHAPE, ERR_WORKSPACE):
        raise ValueError(f"libtdb_b200: {detail} (code {code})")
    raise TdbError(code, detail)


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return TDB_DTYPE_F32
    if dt == torch.bfloat16:
        return TDB_DTYPE_BF16
    raise ValueError(f"unsupported dtype {dt}: the kernels take float32 or bfloat16")


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("turbodeberta_b200 runs on CUDA tensors only; there is no CPU path")
        if dev is not None and t.device != dev:
            raise ValueError("all tensors must live on the same device")
        dev = t.device
    return dev

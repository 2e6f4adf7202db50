"""ctypes view of the C ABI in ``include/pla_b200.h`` (torch-free: plain pointers and sizes).

Used by the tests that call the shared library directly; a binding in another language would
declare the same structures. Only the structures needed so far are mirrored here.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libpla_b200.so"


class Index(ctypes.Structure):
    """``pla_b200_index``: an int32/int64, possibly strided, index vector."""
    _fields_ = [("data", ctypes.c_void_p), ("wide", ctypes.c_int32), ("stride", ctypes.c_int64)]


class KdaCommitArgs(ctypes.Structure):
    """``pla_b200_kda_commit_args``."""
    _fields_ = [
        ("layers", ctypes.c_void_p), ("n_layers", ctypes.c_int32),
        ("candidate", ctypes.c_void_p), ("plan", ctypes.c_void_p),
        ("sampled", Index), ("source", Index), ("cu", Index), ("mapping", Index), ("computed", Index),
        ("blocks", Index),
        ("block_row_stride", ctypes.c_int64), ("block_col_stride", ctypes.c_int64), ("block_size", ctypes.c_int64),
        ("block_rows", ctypes.c_int32), ("block_cols", ctypes.c_int32),
        ("N", ctypes.c_int32), ("capacity", ctypes.c_int32), ("sampler_rows", ctypes.c_int32),
        ("H", ctypes.c_int32), ("slots", ctypes.c_int32), ("Q", ctypes.c_int32), ("null_block_id", ctypes.c_int32),
        ("token_capacity", ctypes.c_int64), ("status", ctypes.c_void_p),
    ]


def load() -> ctypes.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(f"{LIB_PATH} is not built; run `python -m pla_b200.build`")
    lib = ctypes.CDLL(str(LIB_PATH))
    lib.pla_b200_last_error.restype = ctypes.c_char_p
    for name in ("pla_b200_kda_replay_plan", "pla_b200_kda_replay_commit", "pla_b200_kda_replay_plan_static"):
        fn = getattr(lib, name)
        fn.restype = ctypes.c_int
        fn.argtypes = [ctypes.POINTER(KdaCommitArgs), ctypes.c_void_p]
    return lib


def index_of(tensor) -> Index:
    """Describe a 1-D torch int32/int64 tensor (any stride) as a ``pla_b200_index``."""
    import torch
    if tensor is None:
        return Index(None, 0, 1)
    assert tensor.dim() == 1 and tensor.dtype in (torch.int32, torch.int64)
    return Index(tensor.data_ptr(), int(tensor.dtype == torch.int64), tensor.stride(0))

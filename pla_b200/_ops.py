"""Loads the native libraries and exposes ``torch.ops.pla_b200``.

``lib/libpla_b200.so`` holds the kernels behind the C ABI; ``lib/pla_b200_ops.so``
registers the C++ host ops. Both are built in-tree by ``python -m pla_b200.build``.
There is no fallback: a missing library is an ImportError.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

import torch

_LIB_DIR = Path(__file__).resolve().parent / "lib"
NATIVE_PATH = _LIB_DIR / "libpla_b200.so"
OPS_PATH = _LIB_DIR / "pla_b200_ops.so"

_MISSING = (
    "pla_b200: native library {path} is not built. Run `python -m pla_b200.build` "
    "(needs nvcc with sm_100a support). There is no CPU or PyTorch fallback."
)


def _load():
    for path in (NATIVE_PATH, OPS_PATH):
        if not path.exists():
            raise ImportError(_MISSING.format(path=path))
    native = ctypes.CDLL(str(NATIVE_PATH), mode=ctypes.RTLD_GLOBAL)
    torch.ops.load_library(str(OPS_PATH))
    return native


native = _load()
native.pla_b200_last_error.restype = ctypes.c_char_p
ops = torch.ops.pla_b200


def last_error() -> str:
    return native.pla_b200_last_error().decode()


def device_status(clear: bool = False) -> int:
    """PLA_B200_DEV_* bits that kernels on the current CUDA device reported while the caller passed no ``status``
    tensor (``pla_b200_device_status``). Waits for the device's earlier work: poll it off the hot path."""
    word = ctypes.c_int32(0)
    rc = native.pla_b200_device_status(ctypes.byref(word), 1 if clear else 0)
    if rc != 0:
        raise RuntimeError(f"pla_b200_device_status failed: {last_error()}")
    return int(word.value)

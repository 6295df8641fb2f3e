"""ctypes loader for the in-tree CUDA kernel library (``dcp_b200/_kernels.so``).

The library exports a plain C ABI (``dcpk_*``); callers pass raw device pointers and the
current CUDA stream handle.  Loading fails loudly: on a machine with a GPU a missing library
is an error, never a silent fallback to eager PyTorch.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

_LIB = None


def lib_path() -> Path:
    return Path(__file__).resolve().parent.parent / "_kernels.so"


def load() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        p = lib_path()
        if not p.exists():
            raise RuntimeError(
                f"{p} is missing: build it with `python -m dcp_b200.csrc.build` (needs nvcc, no GPU required)"
            )
        _LIB = ctypes.CDLL(str(p))
    return _LIB


def available() -> bool:
    return lib_path().exists()


def ptr(t) -> ctypes.c_void_p:
    """Device (or host) pointer of a torch tensor as a ctypes void pointer."""
    return ctypes.c_void_p(t.data_ptr())


def stream_handle():
    import torch

    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


LAUNCHES = 0  # kernel-entry calls made through this library since import (each launches >= 1 kernel)


def check(rc: int, what: str):
    global LAUNCHES
    LAUNCHES += 1
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")

"""Pinned host arena with a caching allocator.

Pinning memory per batch (cudaHostAlloc / cudaHostRegister) costs milliseconds and fragments the
host; the arena pins one region once and hands out sub-ranges, so every batch's tokens, labels and
kernel tables are staged in already-pinned memory.  ``apply_monkey_patch`` makes
``torch.utils.data.DataLoader(pin_memory=True)`` use the arena, the job of
dcp/memory/host_caching_allocator.py:96-267.
"""
from __future__ import annotations

import threading
import weakref
from typing import Any, Dict, Optional

import torch

from .allocation_simulator import AllocationSimulator, OutOfArena

DEFAULT_ARENA_BYTES = 1 << 30


class HostCachingAllocator:
    def __init__(self, capacity: int = DEFAULT_ARENA_BYTES, pin: Optional[bool] = None):
        self.capacity = int(capacity)
        pin = torch.cuda.is_available() if pin is None else pin
        self.arena = torch.empty(self.capacity, dtype=torch.uint8, pin_memory=pin)
        self.pinned = pin
        self.sim = AllocationSimulator(self.capacity)
        self._lock = threading.Lock()
        self._offsets: Dict[int, int] = {}     # id(tensor storage view) -> offset
        self.n_fallback = 0

    def alloc(self, shape, dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        with self._lock:
            try:
                off = self.sim.alloc(max(nbytes, 1))
            except OutOfArena:
                self.n_fallback += 1
                return torch.empty(shape, dtype=dtype, pin_memory=self.pinned)
        t = self.arena[off:off + nbytes].view(dtype).view(*shape)
        self._offsets[id(t)] = off
        weakref.finalize(t, self._release, id(t))
        return t

    def _release(self, key: int) -> None:
        with self._lock:
            off = self._offsets.pop(key, None)
            if off is not None:
                self.sim.free(off)

    def free(self, t: torch.Tensor) -> None:
        self._release(id(t))

    def pin(self, data: Any) -> Any:
        """Recursively copy tensors of a batch into the arena."""
        if isinstance(data, torch.Tensor):
            if data.is_cuda:
                return data
            dst = self.alloc(data.shape, data.dtype)
            dst.copy_(data)
            return dst
        if isinstance(data, dict):
            return {k: self.pin(v) for k, v in data.items()}
        if isinstance(data, tuple):
            return tuple(self.pin(v) for v in data)
        if isinstance(data, list):
            return [self.pin(v) for v in data]
        return data


_GLOBAL: Optional[HostCachingAllocator] = None
_ORIGINAL = None


def get_allocator(capacity: int = DEFAULT_ARENA_BYTES) -> HostCachingAllocator:
    global _GLOBAL
    if _GLOBAL is None:
        _GLOBAL = HostCachingAllocator(capacity)
    return _GLOBAL


def apply_monkey_patch(capacity: int = DEFAULT_ARENA_BYTES) -> HostCachingAllocator:
    """Route the DataLoader's pin-memory thread through the arena."""
    global _ORIGINAL
    import torch.utils.data._utils.pin_memory as pm
    alloc = get_allocator(capacity)
    if _ORIGINAL is None:
        _ORIGINAL = pm.pin_memory

        def pin_memory(data, device=None):
            return alloc.pin(data)

        pm.pin_memory = pin_memory
    return alloc


def remove_monkey_patch() -> None:
    global _ORIGINAL
    if _ORIGINAL is not None:
        import torch.utils.data._utils.pin_memory as pm
        pm.pin_memory = _ORIGINAL
        _ORIGINAL = None

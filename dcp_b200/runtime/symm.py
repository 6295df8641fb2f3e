"""Symmetric (peer-mapped) device memory for the fused executor.

One byte arena per rank is allocated and mapped once into every peer, which gives every rank the
device address of every peer's arena over NVLink.  Two allocation routes exist:
``torch.distributed._symmetric_memory`` (allocate + rendezvous; the default where that module has
``empty`` and ``rendezvous``) and CUDA IPC handles through the in-tree library (``dcpk_ipc_*``:
cudaMalloc, handle exchange over the process group, cudaIpcOpenMemHandle), taken when the module is
missing or when ``DCP_B200_PEER_MEMORY=ipc``.  Named regions are carved at identical offsets on all
ranks, so "region X of rank r" is ``ptrs[r] + offset(X)`` everywhere.  With a single rank the arena
is ordinary device memory.

Cross-GPU synchronisation uses a flag row per rank inside the arena and the bounded
``signal_barrier`` kernel: a peer that never arrives turns into a status code, not a hang.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Tuple

import torch

from ..ops import _lib, block_ops

_ALIGN = 1024


def peer_memory_route() -> str:
    """"symm" or "ipc": which of the two routes ``SymmetricArena`` takes in this process."""
    want = os.environ.get("DCP_B200_PEER_MEMORY", "").lower()
    if want in ("symm", "ipc"):
        return want
    try:
        import torch.distributed._symmetric_memory as symm_mem
        return "symm" if hasattr(symm_mem, "empty") and hasattr(symm_mem, "rendezvous") else "ipc"
    except ImportError:
        return "ipc"


class _RawDeviceBuffer:
    """Device memory owned by the in-tree library, exposed to torch through the CUDA array interface."""

    def __init__(self, ptr: int, nbytes: int):
        self.ptr, self.nbytes = ptr, nbytes
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def _ipc_allocate(nbytes: int, device: torch.device, group):
    """(own buffer as a uint8 tensor, device addresses of every rank's buffer, owner object)."""
    import torch.distributed as dist
    lib = _lib.load()
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    with torch.cuda.device(device):
        ptr, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
        rc = lib.dcpk_ipc_alloc(ctypes.c_size_t(nbytes), ctypes.byref(ptr), handle)
        if rc != 0:
            raise RuntimeError(f"dcpk_ipc_alloc({nbytes}) failed with code {rc}")
        handles = [None] * world
        dist.all_gather_object(handles, bytes(handle.raw), group=group)
        ptrs = []
        for r, h in enumerate(handles):
            if r == rank:
                ptrs.append(int(ptr.value))
                continue
            peer = ctypes.c_void_p()
            rc = lib.dcpk_ipc_open(ctypes.create_string_buffer(h, 64), ctypes.byref(peer))
            if rc != 0:
                raise RuntimeError(f"dcpk_ipc_open of rank {r}'s buffer failed with code {rc}")
            ptrs.append(int(peer.value))
    owner = _RawDeviceBuffer(int(ptr.value), nbytes)
    return torch.as_tensor(owner, device=device), ptrs, owner


class SymmetricArena:
    def __init__(self, regions: Dict[str, Tuple[Tuple[int, ...], torch.dtype]], device: torch.device, group=None,
                 timeout_s: float = 10.0):
        """regions: name -> (shape, dtype).  ``group`` None or of size 1 -> local memory only."""
        self.device = device
        self.group = group
        self.timeout_s = timeout_s
        self.world = 1
        self.rank = 0
        if group is not None:
            import torch.distributed as dist
            self.world = dist.get_world_size(group)
            self.rank = dist.get_rank(group)
        self.offsets: Dict[str, int] = {}
        self.specs = dict(regions)
        off = 0
        for name, (shape, dtype) in regions.items():
            self.offsets[name] = off
            n = 1
            for s in shape:
                n *= int(s)
            off += -(-(n * torch.empty((), dtype=dtype).element_size()) // _ALIGN) * _ALIGN
        self.offsets["__flags__"] = off
        off += _ALIGN
        self.nbytes = off
        self.route = peer_memory_route() if self.world > 1 else "local"
        if self.route == "ipc":
            # buffers live until the process exits: peers may still hold mappings of them
            self.buf, self.ptrs, self.handle = _ipc_allocate(self.nbytes, device, group)
        elif self.world > 1:
            import torch.distributed._symmetric_memory as symm_mem
            self.buf = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
            self.buf.zero_()
            torch.cuda.synchronize(device)
            self.handle = symm_mem.rendezvous(self.buf, group.group_name)
            self.ptrs: List[int] = [int(p) for p in self.handle.buffer_ptrs]
        else:
            self.buf = torch.zeros(self.nbytes, dtype=torch.uint8, device=device)
            self.handle = None
            self.ptrs = [self.buf.data_ptr()]
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.epoch = 0
        self._views: Dict[str, torch.Tensor] = {}

    def view(self, name: str) -> torch.Tensor:
        if name not in self._views:
            shape, dtype = self.specs[name]
            n = 1
            for s in shape:
                n *= int(s)
            nbytes = n * torch.empty((), dtype=dtype).element_size()
            off = self.offsets[name]
            # .data: an alias with its own autograd version counter, so in-place writes to one region
            # (e.g. gradient accumulation) do not invalidate tensors autograd saved from another
            self._views[name] = self.buf[off:off + nbytes].view(dtype).view(*shape).data
        return self._views[name]

    def peer_ptrs(self, name: str) -> List[int]:
        """Device address of region ``name`` on every rank (index = rank)."""
        off = self.offsets[name]
        return [p + off for p in self.ptrs]

    def barrier(self) -> None:
        """All ranks' prior work on the current stream is complete and visible when this returns
        on the stream (device-side; the host does not block)."""
        if self.world <= 1:
            return
        self.epoch += 1
        block_ops.signal_barrier(self.peer_ptrs("__flags__"), self.rank, self.world, self.epoch, self.status,
                                 self.timeout_s)

    def check_status(self) -> None:
        """Host-side check of the device status word (synchronises the stream)."""
        code = int(self.status.item())
        if code != 0:
            names = {1: "an mbarrier wait inside a compute kernel ran out",
                     2: "a peer never reached a cross-GPU barrier within the deadline", 3: "bad kernel arguments"}
            self.status.zero_()
            raise RuntimeError(f"device-side failure detected (code {code}): {names.get(code, 'unknown')}")


class FlagBarrierModel:
    """Host model of the device barrier protocol (``signal_barrier_kernel``): rank r owns a row of
    flags, ``flags[r][s]`` is written only by rank s and holds the last epoch s has reached; to
    pass epoch e a rank publishes e into its slot of every peer's row, then waits until every
    slot of its own row is >= e (wrap-safe signed difference) or its deadline passes, in which
    case it records the timeout status and returns instead of hanging.  Used by the CPU tests to
    check safety (nobody passes epoch e before everyone arrived at e), liveness and the bounded
    wait with a withheld signal, with real threads and randomised timing."""

    STATUS_OK, STATUS_SIGNAL_TIMEOUT = 0, 2

    def __init__(self, world: int):
        self.world = world
        self.flags = [[0] * world for _ in range(world)]
        self.status = [self.STATUS_OK] * world

    def arrive_and_wait(self, rank: int, epoch: int, timeout_s: float = 1.0, withhold_from=()) -> int:
        """One barrier call of ``rank``; ``withhold_from`` lists peers that are NOT told (fault injection)."""
        import time
        for peer in range(self.world):
            if peer != rank and peer not in withhold_from:
                self.flags[peer][rank] = epoch & 0xFFFFFFFF
        deadline = time.monotonic() + timeout_s
        for peer in range(self.world):
            if peer == rank:
                continue
            while True:
                diff = (self.flags[rank][peer] - epoch) & 0xFFFFFFFF
                if diff < 0x80000000:            # int32(v - epoch) >= 0
                    break
                if time.monotonic() > deadline:
                    self.status[rank] = self.STATUS_SIGNAL_TIMEOUT
                    return self.status[rank]
                time.sleep(0)
        return self.STATUS_OK

"""Address-space simulator of a caching allocator: best-fit blocks, splitting, coalescing on free.

Used to size and to drive the pinned host arena (and to estimate paged-buffer footprints in dry
runs) without touching real memory.  Plays the role of
dcp/memory/allocation_simulator.py:69-348 with a simpler design: one sorted free list over a
linear address space instead of a re-implementation of torch's multi-pool allocator.
"""
from __future__ import annotations

import bisect
from typing import Dict, List, Tuple


class OutOfArena(MemoryError):
    pass


class AllocationSimulator:
    def __init__(self, capacity: int, alignment: int = 512):
        self.capacity, self.alignment = int(capacity), int(alignment)
        self._free: List[Tuple[int, int]] = [(0, self.capacity)]   # sorted (offset, size)
        self._live: Dict[int, int] = {}                            # offset -> size
        self.in_use = 0
        self.high_water = 0          # highest address ever handed out
        self.peak_in_use = 0

    def _round(self, n: int) -> int:
        a = self.alignment
        return max(a, -(-int(n) // a) * a)

    def alloc(self, nbytes: int) -> int:
        size = self._round(nbytes)
        best = None
        for i, (off, sz) in enumerate(self._free):
            if sz >= size and (best is None or sz < self._free[best][1]):
                best = i
                if sz == size:
                    break
        if best is None:
            raise OutOfArena(f"cannot place {size} bytes (capacity {self.capacity}, in use {self.in_use})")
        off, sz = self._free.pop(best)
        if sz > size:
            bisect.insort(self._free, (off + size, sz - size))
        self._live[off] = size
        self.in_use += size
        self.peak_in_use = max(self.peak_in_use, self.in_use)
        self.high_water = max(self.high_water, off + size)
        return off

    def free(self, offset: int) -> None:
        size = self._live.pop(offset)
        self.in_use -= size
        i = bisect.bisect_left(self._free, (offset, 0))
        # coalesce with neighbours
        if i < len(self._free) and self._free[i][0] == offset + size:
            size += self._free.pop(i)[1]
        if i > 0 and self._free[i - 1][0] + self._free[i - 1][1] == offset:
            prev = self._free.pop(i - 1)
            offset, size = prev[0], prev[1] + size
            i -= 1
        self._free.insert(i, (offset, size))

    def fragmentation(self) -> float:
        free = sum(s for _, s in self._free)
        largest = max((s for _, s in self._free), default=0)
        return 0.0 if free == 0 else 1.0 - largest / free

    def reset(self) -> None:
        self.__init__(self.capacity, self.alignment)


# name used by the reference
TorchCachingAllocatorSimulator = AllocationSimulator

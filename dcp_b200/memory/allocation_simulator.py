"""Address-space simulator of a caching allocator: best-fit blocks, splitting, coalescing on free.

Used to size and to drive the pinned host arena (and to estimate paged-buffer footprints in dry
runs) without touching real memory.  Two models: ``AllocationSimulator`` is the arena's own policy
(one sorted free list over a linear address space); ``TorchCachingAllocatorSimulator`` follows the
framework's CUDA caching allocator (size rounding, small / large pools with their segment sizes,
best fit, split thresholds, per-segment coalescing), which is what the reference's simulator
models (dcp/memory/allocation_simulator.py:69-348), to predict reserved memory from an
allocation trace.
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


class TorchCachingAllocatorSimulator:
    """Model of the framework's CUDA caching allocator, for predicting how much device memory a
    sequence of allocations and frees will *reserve* (not just use): the question the reference asks
    its simulator before sizing pinned buffers (dcp/memory/allocation_simulator.py:69-348).

    Modelled behaviour: requests are rounded up to 512 bytes; requests of at most 1 MiB are served
    from the small pool, whose segments are 2 MiB; larger ones from the large pool, whose segments
    are 20 MiB for requests below 10 MiB and the request rounded up to 2 MiB otherwise; a request
    takes the smallest cached free block of its pool that fits (best fit), a new segment is
    reserved when none does; a block is split when the remainder is worth keeping (at least 512
    bytes in the small pool, more than 1 MiB in the large pool); freed blocks merge with free
    neighbours of the same segment; ``empty_cache`` returns fully free segments.  ``capacity``
    bounds the reserved bytes (OutOfArena beyond it, after one ``empty_cache`` retry, as the real
    allocator retries after releasing its cache)."""

    ROUND, SMALL_LIMIT, SMALL_SEGMENT = 512, 1 << 20, 2 << 20
    LARGE_SEGMENT, LARGE_DIRECT, LARGE_ROUND = 20 << 20, 10 << 20, 2 << 20

    def __init__(self, capacity: int = 1 << 62):
        self.capacity = int(capacity)
        self._segments: Dict[int, Dict] = {}      # id -> {"size", "pool", "blocks": sorted [offset, size, free]}
        self._next_id = 0
        self._live: Dict[int, Tuple[int, int]] = {}   # handle -> (segment id, offset)
        self._next_handle = 0
        self.allocated = self.reserved = self.peak_allocated = self.peak_reserved = 0
        self.n_segments_reserved = 0

    def _round(self, n: int) -> int:
        return max(self.ROUND, -(-int(n) // self.ROUND) * self.ROUND)

    def _segment_size(self, size: int) -> int:
        if size <= self.SMALL_LIMIT:
            return self.SMALL_SEGMENT
        if size < self.LARGE_DIRECT:
            return self.LARGE_SEGMENT
        return -(-size // self.LARGE_ROUND) * self.LARGE_ROUND

    def _find(self, pool: str, size: int):
        best = None
        for sid, seg in self._segments.items():
            if seg["pool"] != pool:
                continue
            for i, (off, sz, free) in enumerate(seg["blocks"]):
                if free and sz >= size and (best is None or sz < best[2]):
                    best = (sid, i, sz)
        return best

    def alloc(self, nbytes: int) -> int:
        """-> handle to pass to ``free``."""
        size = self._round(nbytes)
        pool = "small" if size <= self.SMALL_LIMIT else "large"
        hit = self._find(pool, size)
        if hit is None:
            seg_size = self._segment_size(size)
            if self.reserved + seg_size > self.capacity:
                self.empty_cache()
                if self.reserved + seg_size > self.capacity:
                    raise OutOfArena(f"cannot reserve {seg_size} bytes (reserved {self.reserved} of {self.capacity})")
            sid, self._next_id = self._next_id, self._next_id + 1
            self._segments[sid] = {"size": seg_size, "pool": pool, "blocks": [[0, seg_size, True]]}
            self.reserved += seg_size
            self.n_segments_reserved += 1
            self.peak_reserved = max(self.peak_reserved, self.reserved)
            hit = (sid, 0, seg_size)
        sid, i, sz = hit
        blocks = self._segments[sid]["blocks"]
        off = blocks[i][0]
        rest = sz - size
        keep = rest >= self.ROUND if pool == "small" else rest > self.SMALL_LIMIT
        if keep:
            blocks[i] = [off, size, False]
            blocks.insert(i + 1, [off + size, rest, True])
        else:
            blocks[i][2] = False
        used = blocks[i][1]
        self.allocated += used
        self.peak_allocated = max(self.peak_allocated, self.allocated)
        h, self._next_handle = self._next_handle, self._next_handle + 1
        self._live[h] = (sid, off)
        return h

    def free(self, handle: int) -> None:
        sid, off = self._live.pop(handle)
        blocks = self._segments[sid]["blocks"]
        i = next(j for j, b in enumerate(blocks) if b[0] == off)
        self.allocated -= blocks[i][1]
        blocks[i][2] = True
        if i + 1 < len(blocks) and blocks[i + 1][2]:
            blocks[i][1] += blocks.pop(i + 1)[1]
        if i > 0 and blocks[i - 1][2]:
            blocks[i - 1][1] += blocks.pop(i)[1]

    def empty_cache(self) -> int:
        """Release segments that are entirely free; -> bytes returned."""
        gone = [sid for sid, seg in self._segments.items() if len(seg["blocks"]) == 1 and seg["blocks"][0][2]]
        freed = sum(self._segments.pop(sid)["size"] for sid in gone)
        self.reserved -= freed
        return freed

    def stats(self) -> Dict[str, int]:
        return {"allocated": self.allocated, "reserved": self.reserved, "peak_allocated": self.peak_allocated,
                "peak_reserved": self.peak_reserved, "segments": len(self._segments)}

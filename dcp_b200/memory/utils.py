"""Device-memory helpers (dcp/memory/utils.py:8-43)."""
from __future__ import annotations

import torch


def reserve_full_memory(device=None, fraction: float = 0.9, chunk_bytes: int = 1 << 30) -> int:
    """Make torch's caching allocator hold ``fraction`` of the free device memory up front (and
    release it to the cache), so later allocations never call cudaMalloc mid-iteration.  Returns
    the number of bytes reserved.  Bounded: never asks for more than is free."""
    if not torch.cuda.is_available():
        return 0
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    free, _ = torch.cuda.mem_get_info(device)
    target = int(free * min(max(fraction, 0.0), 0.95))
    held, total = [], 0
    try:
        while total + chunk_bytes <= target:
            held.append(torch.empty(chunk_bytes, dtype=torch.uint8, device=device))
            total += chunk_bytes
    except torch.cuda.OutOfMemoryError:
        pass
    del held
    return total

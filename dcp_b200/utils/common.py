"""Small shared helpers (dcp/utils/common.py:7-42)."""
from __future__ import annotations

import os
from typing import Any


def read_env_int(name: str, default: int = 0) -> int:
    v = os.environ.get(name)
    try:
        return int(v) if v is not None and v != "" else default
    except ValueError:
        return default


def trepr(x: Any, max_items: int = 8) -> str:
    """Truncated repr for logs: tensors show shape/dtype, long containers are elided."""
    try:
        import torch
        if isinstance(x, torch.Tensor):
            return f"Tensor(shape={tuple(x.shape)}, dtype={x.dtype}, device={x.device})"
    except ImportError:  # pragma: no cover
        pass
    if isinstance(x, dict):
        items = list(x.items())
        body = ", ".join(f"{k!r}: {trepr(v, max_items)}" for k, v in items[:max_items])
        return "{" + body + (", ..." if len(items) > max_items else "") + "}"
    if isinstance(x, (list, tuple, set)):
        items = list(x)
        body = ", ".join(trepr(v, max_items) for v in items[:max_items])
        more = f", ... ({len(items)} items)" if len(items) > max_items else ""
        open_, close = ("[", "]") if isinstance(x, list) else ("(", ")") if isinstance(x, tuple) else ("{", "}")
        return open_ + body + more + close
    return repr(x)

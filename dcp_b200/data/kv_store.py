"""Small key-value control plane.

It carries the planner's published per-rank plans (shared planning: one planner, every rank reads
its share; values above the store's payload limit travel in pieces) and control state for
multi-process jobs: iteration counts, abort flags, experiment barriers.  In-process it is a dict
guarded by a condition variable; across processes it wraps ``torch.distributed.TCPStore``.
Blocking ``get`` calls take a timeout and raise instead of polling forever (the reference's Redis
client polls without one, dcp/data/kv_redis.py:22-135).
"""
from __future__ import annotations

import pickle
import threading
import time
from typing import Any, Optional


class KVTimeout(TimeoutError):
    pass


class KVServer:
    """Owns the TCPStore master (the role of the spawned redis-server); no-op for in-process use."""

    def __init__(self, host: str = "127.0.0.1", port: int = 29650, world_size: int = 1):
        from torch.distributed import TCPStore
        self.store = TCPStore(host, port, world_size, is_master=True, wait_for_workers=False)
        self.host, self.port = host, port


_CHUNK = 4 << 20                 # TCPStore refuses payloads above 8 MiB; larger values travel in pieces
_CHUNK_MARK = b"\x00dcp-chunked:"


class KVStore:
    def __init__(self, host: Optional[str] = None, port: int = 29650, timeout_s: float = 60.0, store=None):
        self.timeout_s = timeout_s
        self._local = None
        if store is not None:
            self._store = store
        elif host is None:
            self._store = None
            self._local = {}
            self._cv = threading.Condition()
        else:
            from datetime import timedelta
            from torch.distributed import TCPStore
            self._store = TCPStore(host, port, is_master=False, timeout=timedelta(seconds=timeout_s))

    def set(self, key: str, value: Any) -> None:
        data = pickle.dumps(value)
        if self._local is not None:
            with self._cv:
                self._local[key] = data
                self._cv.notify_all()
        elif len(data) <= _CHUNK:
            self._store.set(key, data)
        else:
            # pieces first, the header (which readers wait for) last
            n = -(-len(data) // _CHUNK)
            for i in range(n):
                self._store.set(f"{key}#{i}", data[i * _CHUNK:(i + 1) * _CHUNK])
            self._store.set(key, _CHUNK_MARK + str(n).encode())

    def get(self, key: str, timeout_s: Optional[float] = None) -> Any:
        timeout_s = self.timeout_s if timeout_s is None else timeout_s
        if self._local is not None:
            deadline = time.time() + timeout_s
            with self._cv:
                while key not in self._local:
                    left = deadline - time.time()
                    if left <= 0:
                        raise KVTimeout(f"key {key!r} was not set within {timeout_s}s")
                    self._cv.wait(left)
                return pickle.loads(self._local[key])
        from datetime import timedelta
        try:
            self._store.wait([key], timedelta(seconds=timeout_s))
        except Exception as e:  # torch raises a generic error type on timeout
            raise KVTimeout(f"key {key!r} was not set within {timeout_s}s") from e
        data = self._store.get(key)
        if data.startswith(_CHUNK_MARK):
            n = int(data[len(_CHUNK_MARK):])
            data = b"".join(self._store.get(f"{key}#{i}") for i in range(n))
        return pickle.loads(data)

    def exists(self, key: str) -> bool:
        if self._local is not None:
            with self._cv:
                return key in self._local
        return bool(self._store.check([key]))

    def add(self, key: str, amount: int = 1) -> int:
        if self._local is not None:
            with self._cv:
                cur = pickle.loads(self._local[key]) if key in self._local else 0
                cur += amount
                self._local[key] = pickle.dumps(cur)
                self._cv.notify_all()
                return cur
        return int(self._store.add(key, amount))

    def delete(self, key: str) -> None:
        if self._local is not None:
            with self._cv:
                self._local.pop(key, None)
        else:
            if self._store.check([key]):
                data = self._store.get(key)
                if data.startswith(_CHUNK_MARK):
                    for i in range(int(data[len(_CHUNK_MARK):])):
                        self._store.delete_key(f"{key}#{i}")
            self._store.delete_key(key)

"""Binary wire format of plans and workloads.

Stream-style codec (``ByteWriter`` / ``ByteReader``) producing the same bytes as the
reference's functional helpers (dcp/core/serialization.py:10-120, 306-437): little-endian,
every integer a 4-byte unsigned, instruction tags one byte, floats 8-byte doubles, strings and
containers length-prefixed with a u32, tensors as (dtype code, byte length, raw bytes).
"""
from __future__ import annotations

import struct
from typing import Callable, Dict, Iterable, List, Sequence, Tuple

import numpy as np
import torch

INT_BYTES = 4
TAG_BYTES = 1

# dtype codes shared by plans and tensors (dcp/core/serialization.py:410-437)
_TORCH_DTYPE_CODES = {
    torch.bfloat16: 0,
    torch.float16: 1,
    torch.float32: 2,
    torch.int32: 3,
    torch.int64: 4,
}
_CODE_TO_TORCH = {v: k for k, v in _TORCH_DTYPE_CODES.items()}
_NP_VIEW = {torch.bfloat16: np.uint16, torch.float16: np.float16, torch.float32: np.float32,
            torch.int32: np.int32, torch.int64: np.int64}


def torch_dtype_to_code(dtype: torch.dtype) -> int:
    return _TORCH_DTYPE_CODES[dtype]


def code_to_torch_dtype(code: int) -> torch.dtype:
    return _CODE_TO_TORCH[code]


class ByteWriter:
    """Append-only byte sink; every ``put_*`` returns self so calls chain."""

    __slots__ = ("_parts",)

    def __init__(self):
        self._parts: List[bytes] = []

    def getvalue(self) -> bytes:
        return b"".join(self._parts)

    def raw(self, b: bytes) -> "ByteWriter":
        self._parts.append(bytes(b))
        return self

    def tag(self, v: int) -> "ByteWriter":
        self._parts.append(int(v).to_bytes(TAG_BYTES, "little"))
        return self

    def u32(self, v: int) -> "ByteWriter":
        self._parts.append(int(v).to_bytes(INT_BYTES, "little"))
        return self

    def f64(self, v: float) -> "ByteWriter":
        self._parts.append(struct.pack("<d", float(v)))
        return self

    def string(self, s: str) -> "ByteWriter":
        data = (s or "").encode()
        self.u32(len(data))
        if data:
            self._parts.append(data)
        return self

    def ints(self, values: Iterable[int]) -> "ByteWriter":
        values = list(values)
        self.u32(len(values))
        if values:
            self._parts.append(np.asarray(values, dtype="<u4").tobytes())
        return self

    def floats(self, values: Iterable[float]) -> "ByteWriter":
        values = list(values)
        self.u32(len(values))
        if values:
            self._parts.append(np.asarray(values, dtype="<f8").tobytes())
        return self

    def seq(self, items: Sequence, put: Callable[["ByteWriter", object], None]) -> "ByteWriter":
        self.u32(len(items))
        for it in items:
            put(self, it)
        return self

    def tensor(self, t: torch.Tensor) -> "ByteWriter":
        t = t.detach().cpu().contiguous()
        self.u32(torch_dtype_to_code(t.dtype))
        self.ints(t.shape)
        data = t.view(torch.int16).numpy().tobytes() if t.dtype == torch.bfloat16 else t.numpy().tobytes()
        self.u32(len(data))
        self._parts.append(data)
        return self


class ByteReader:
    """Cursor over a bytes object; ``rest()`` hands back what was not consumed."""

    __slots__ = ("_buf", "_pos")

    def __init__(self, data: bytes, pos: int = 0):
        self._buf = memoryview(data)
        self._pos = pos

    def rest(self) -> bytes:
        return bytes(self._buf[self._pos:])

    def exhausted(self) -> bool:
        return self._pos >= len(self._buf)

    def _take(self, n: int) -> memoryview:
        if self._pos + n > len(self._buf):
            raise ValueError("truncated buffer")
        out = self._buf[self._pos:self._pos + n]
        self._pos += n
        return out

    def raw(self, n: int) -> bytes:
        return bytes(self._take(n))

    def tag(self) -> int:
        return int.from_bytes(self._take(TAG_BYTES), "little")

    def u32(self) -> int:
        return int.from_bytes(self._take(INT_BYTES), "little")

    def f64(self) -> float:
        return struct.unpack("<d", self._take(8))[0]

    def string(self) -> str:
        n = self.u32()
        return bytes(self._take(n)).decode() if n else ""

    def ints(self) -> List[int]:
        n = self.u32()
        if n == 0:
            return []
        return np.frombuffer(self._take(INT_BYTES * n), dtype="<u4").astype(np.int64).tolist()

    def int_tuple(self) -> Tuple[int, ...]:
        return tuple(self.ints())

    def floats(self) -> List[float]:
        n = self.u32()
        if n == 0:
            return []
        return np.frombuffer(self._take(8 * n), dtype="<f8").tolist()

    def seq(self, get: Callable[["ByteReader"], object]) -> list:
        return [get(self) for _ in range(self.u32())]

    def tensor(self) -> torch.Tensor:
        dtype = code_to_torch_dtype(self.u32())
        shape = self.int_tuple()
        nbytes = self.u32()
        raw = bytearray(self._take(nbytes))
        if dtype == torch.bfloat16:
            return torch.frombuffer(raw, dtype=torch.int16).view(torch.bfloat16).reshape(shape).clone()
        if nbytes == 0:
            return torch.empty(shape, dtype=dtype)
        return torch.frombuffer(raw, dtype=dtype).reshape(shape).clone()


# ---- dictionary helpers used by workload specs (keys/values are u32 unless noted) ----
def put_int_dict(w: ByteWriter, d: Dict[int, int]) -> None:
    w.u32(len(d))
    for k, v in d.items():
        w.u32(k).u32(v)


def get_int_dict(r: ByteReader) -> Dict[int, int]:
    return {r.u32(): r.u32() for _ in range(r.u32())}


def put_int_to_ints_dict(w: ByteWriter, d: Dict[int, Sequence[int]]) -> None:
    w.u32(len(d))
    for k, v in d.items():
        w.u32(k).ints(v)


def get_int_to_ints_dict(r: ByteReader) -> Dict[int, List[int]]:
    out = {}
    for _ in range(r.u32()):
        k = r.u32()
        out[k] = r.ints()
    return out

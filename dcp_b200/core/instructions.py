"""Per-device execution plans: eight instruction kinds over named block buffers.

Same instruction set, field order and wire bytes as the reference
(dcp/core/instructions.py:21-1098); here each instruction is a small class whose fields are
described by a codec table, so (de)serialisation, equality and repr are generated from one
schema instead of being written out per class.

Wire tags: Memcpy=0 CommLaunch=1 Barrier=2 CommWait=3 Attn=4 AttnBackward=5
AttnReduction=6 Sum=7.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Sequence, Tuple

import numpy as np
import torch

from .serialization import ByteReader, ByteWriter


class BufferType:
    """Buffer names. ``Local*`` hold a rank's own unpadded tokens, ``Buffer*`` are paged slots."""

    LOCAL_Q = "LocalQ"
    LOCAL_KV = "LocalKV"
    LOCAL_dQ = "LocaldQ"
    LOCAL_dKV = "LocaldKV"
    LOCAL_OUT = "LocalOut"
    LOCAL_dOUT = "LocaldOut"
    LOCAL_LSE = "LocalLSE"
    BUFFER_Q = "BufferQ"
    BUFFER_KV = "BufferKV"
    BUFFER_dQ = "BufferdQ"
    BUFFER_dKV = "BufferdKV"
    BUFFER_OUT = "BufferOut"
    BUFFER_dOUT = "BufferdOut"
    BUFFER_LSE = "BufferLSE"

    LOCAL = (LOCAL_Q, LOCAL_KV, LOCAL_dQ, LOCAL_dKV, LOCAL_OUT, LOCAL_dOUT, LOCAL_LSE)
    PAGED = (BUFFER_Q, BUFFER_KV, BUFFER_dQ, BUFFER_dKV, BUFFER_OUT, BUFFER_dOUT, BUFFER_LSE)

    @classmethod
    def is_local(cls, name: str) -> bool:
        return name in cls.LOCAL

    @classmethod
    def is_lse(cls, name: str) -> bool:
        return name in (cls.LOCAL_LSE, cls.BUFFER_LSE)


class CommType:
    SEND = 0
    RECV = 1

    @classmethod
    def from_num(cls, num: int) -> int:
        if num not in (cls.SEND, cls.RECV):
            raise ValueError(f"Invalid comm type {num}")
        return num

    @classmethod
    def to_str(cls, comm_type: int) -> str:
        return {cls.SEND: "send", cls.RECV: "recv"}[comm_type]


class DType:
    """Plan-level dtype codes (identical to the tensor codes of the serializer)."""

    BFLOAT16 = 0
    FLOAT16 = 1
    FLOAT32 = 2
    INT32 = 3
    INT64 = 4

    _TORCH = {0: torch.bfloat16, 1: torch.float16, 2: torch.float32, 3: torch.int32, 4: torch.int64}
    _NAMES = {0: "bfloat16", 1: "float16", 2: "float32", 3: "int32", 4: "int64"}
    _SIZES = {0: 2, 1: 2, 2: 4, 3: 4, 4: 8}

    @classmethod
    def from_num(cls, num: int) -> int:
        if num not in cls._TORCH:
            raise ValueError(f"Invalid dtype {num}")
        return num

    @classmethod
    def from_torch(cls, dtype: torch.dtype) -> int:
        for k, v in cls._TORCH.items():
            if v == dtype:
                return k
        raise ValueError(f"Unsupported dtype {dtype}")

    @classmethod
    def to_torch(cls, dtype: int) -> torch.dtype:
        return cls._TORCH[dtype]

    @classmethod
    def as_str(cls, dtype: int) -> str:
        return cls._NAMES[dtype]

    @classmethod
    def element_size(cls, dtype: int) -> int:
        return cls._SIZES[dtype]


@dataclass(frozen=True)
class BufferBlock:
    """One block slot: (buffer name, slot or local block index, valid tokens)."""

    buffer_type: str
    index: int
    n_tokens: int

    def __repr__(self):
        return f"({self.buffer_type}, {self.index}, {self.n_tokens})"


# ------------------------------------------------------------------ field codecs
def _put_block(w: ByteWriter, b: BufferBlock) -> None:
    w.string(b.buffer_type).u32(b.index).u32(b.n_tokens)


def _get_block(r: ByteReader) -> BufferBlock:
    return BufferBlock(r.string(), r.u32(), r.u32())


def _put_blocks(w: ByteWriter, blocks: Sequence[BufferBlock]) -> None:
    w.seq(blocks, _put_block)


def _get_blocks(r: ByteReader) -> List[BufferBlock]:
    return r.seq(_get_block)


def _put_table(w: ByteWriter, table: Sequence[Sequence[BufferBlock]]) -> None:
    w.seq(table, _put_blocks)


def _get_table(r: ByteReader) -> List[List[BufferBlock]]:
    return r.seq(_get_blocks)


def _mask_items(mask) -> List[torch.Tensor]:
    """The wire form iterates the leading dim: [2,T] -> 2 rows, [2,2,T] -> 2 items of [2,T]."""
    if isinstance(mask, torch.Tensor):
        return [mask[i] for i in range(mask.shape[0])]
    return [m if isinstance(m, torch.Tensor) else torch.as_tensor(m, dtype=torch.int32) for m in mask]


def _put_mask(w: ByteWriter, mask) -> None:
    items = _mask_items(mask)
    w.u32(len(items))
    for m in items:
        assert m.dtype == torch.int32, "range masks are int32"
        data = m.contiguous().cpu().numpy().tobytes()
        w.ints(m.shape).u32(len(data)).raw(data)


def _get_mask(r: ByteReader) -> List[torch.Tensor]:
    out = []
    for _ in range(r.u32()):
        shape = r.int_tuple()
        n = r.u32()
        arr = np.frombuffer(r.raw(n), dtype="<i4").reshape(shape).copy()
        out.append(torch.from_numpy(arr))
    return out


def _eq_mask(a, b) -> bool:
    ia, ib = _mask_items(a), _mask_items(b)
    return len(ia) == len(ib) and all(x.shape == y.shape and torch.equal(x, y) for x, y in zip(ia, ib))


_U32 = (lambda w, v: w.u32(v), lambda r: r.u32(), None)
_STR = (lambda w, v: w.string(v or ""), lambda r: r.string(), None)
_OPT_STR = (lambda w, v: w.string(v or ""), lambda r: (r.string() or None), None)
_INTS = (lambda w, v: w.ints(v), lambda r: r.ints(), None)
_TABLE = (_put_table, _get_table, None)
_MASK = (_put_mask, _get_mask, _eq_mask)


class BlockInstrBase:
    """Base of all instructions; subclasses declare ``FIELDS = ((name, codec), ...)``."""

    FIELDS: Tuple[Tuple[str, tuple], ...] = ()
    _registry: List[type] = []
    tag: int = -1

    def __init_subclass__(cls, **kw) -> None:
        super().__init_subclass__(**kw)
        cls.tag = len(BlockInstrBase._registry)
        BlockInstrBase._registry.append(cls)

    def __init__(self, **kwargs):
        names = [n for n, _ in self.FIELDS]
        for n in names:
            if n not in kwargs:
                raise TypeError(f"{type(self).__name__} missing field {n}")
            setattr(self, n, kwargs.pop(n))
        self.extras = kwargs  # non-serialised annotations (debug only)
        self.validate()

    def validate(self) -> None:  # hook
        pass

    def serialize(self, config=None) -> bytes:
        w = ByteWriter().tag(self.tag)
        for name, (put, _, _) in self.FIELDS:
            put(w, getattr(self, name))
        return w.getvalue()

    def write(self, w: ByteWriter) -> None:
        w.tag(self.tag)
        for name, (put, _, _) in self.FIELDS:
            put(w, getattr(self, name))

    @staticmethod
    def read(r: ByteReader) -> "BlockInstrBase":
        tag = r.tag()
        if tag >= len(BlockInstrBase._registry):
            raise ValueError(f"unknown instruction tag {tag}")
        cls = BlockInstrBase._registry[tag]
        return cls(**{name: get(r) for name, (_, get, _) in cls.FIELDS})

    @classmethod
    def deserialize(cls, data: bytes, config=None) -> Tuple["BlockInstrBase", bytes]:
        r = ByteReader(data)
        instr = BlockInstrBase.read(r)
        return instr, r.rest()

    def __eq__(self, other) -> bool:
        if type(self) is not type(other):
            return False
        for name, (_, _, eq) in self.FIELDS:
            a, b = getattr(self, name), getattr(other, name)
            if not (eq(a, b) if eq else a == b):
                return False
        return True

    __hash__ = None

    def __repr__(self) -> str:
        parts = []
        for name, codec in self.FIELDS:
            if codec is _MASK:
                continue
            parts.append(f"{name}={getattr(self, name)!r}")
        return f"{type(self).__name__}({', '.join(parts)})"


# ------------------------------------------------------------------ instructions (definition order = wire tag)
def _put_pairs(w: ByteWriter, pairs) -> None:
    w.u32(len(pairs))
    for src, dst in pairs:
        _put_block(w, src)
        _put_block(w, dst)


def _get_pairs(r: ByteReader):
    return [(_get_block(r), _get_block(r)) for _ in range(r.u32())]


class MemcpyInstr(BlockInstrBase):
    """Copy blocks between buffers on one device: ``src_dst_pairs = [(src, dst), ...]``."""

    FIELDS = (("src_dst_pairs", (_put_pairs, _get_pairs, None)),)

    def __init__(self, src_dst_pairs, **kw):
        super().__init__(src_dst_pairs=[tuple(p) for p in src_dst_pairs], **kw)


@dataclass(frozen=True)
class CommOp:
    comm_type: int
    peer: Tuple[int, int]  # (node, device)
    buffer_block: BufferBlock

    def __repr__(self) -> str:
        return f"{CommType.to_str(self.comm_type)}{self.peer}{self.buffer_block}"


def _put_ops(w: ByteWriter, ops: Sequence[CommOp]) -> None:
    w.u32(len(ops))
    for op in ops:
        w.u32(op.comm_type).u32(op.peer[0]).u32(op.peer[1])
        _put_block(w, op.buffer_block)


def _get_ops(r: ByteReader) -> List[CommOp]:
    out = []
    for _ in range(r.u32()):
        ct = CommType.from_num(r.u32())
        peer = (r.u32(), r.u32())
        out.append(CommOp(ct, peer, _get_block(r)))
    return out


class CommLaunchInstr(BlockInstrBase):
    """Start an exchange identified by ``key``; SEND/RECV ops are matched per peer in order."""

    FIELDS = (("key", _STR), ("comm_ops", (_put_ops, _get_ops, None)), ("stream", _OPT_STR))

    def __init__(self, key, comm_ops, stream=None, **kw):
        super().__init__(key=key, comm_ops=list(comm_ops), stream=stream, **kw)


class BarrierInstr(BlockInstrBase):
    FIELDS = ()


class CommWaitInstr(BlockInstrBase):
    FIELDS = (("key", _STR), ("stream", _OPT_STR))

    def __init__(self, key, stream=None, **kw):
        super().__init__(key=key, stream=stream, **kw)


_ATTN_HEAD = (("stage_id", _U32), ("seqlens_q", _INTS), ("seqlens_kv", _INTS), ("max_seqlen_q", _U32),
              ("max_seqlen_kv", _U32), ("attn_mask", _MASK))


class AttnInstr(BlockInstrBase):
    """Forward attention over a batch of q rows; row i = one Q block vs. the KV blocks of row i."""

    FIELDS = _ATTN_HEAD + (("q_block_table", _TABLE), ("kv_block_table", _TABLE),
                           ("out_block_table", _TABLE), ("lse_block_table", _TABLE))

    def __init__(self, stage_id, seqlens_q, seqlens_kv, max_seqlen_q, max_seqlen_kv, attn_mask,
                 q_block_table, kv_block_table, out_block_table, lse_block_table, **kw):
        super().__init__(stage_id=stage_id, seqlens_q=list(seqlens_q), seqlens_kv=list(seqlens_kv),
                         max_seqlen_q=max_seqlen_q, max_seqlen_kv=max_seqlen_kv, attn_mask=attn_mask,
                         q_block_table=q_block_table, kv_block_table=kv_block_table,
                         out_block_table=out_block_table, lse_block_table=lse_block_table, **kw)

    def validate(self) -> None:
        assert len(self.out_block_table) == len(self.lse_block_table)
        for o_row, l_row in zip(self.out_block_table, self.lse_block_table):
            assert [b.index for b in o_row] == [b.index for b in l_row], "out/lse slots must pair up"


class AttnBackwardInstr(BlockInstrBase):
    FIELDS = _ATTN_HEAD + (("q_block_table", _TABLE), ("kv_block_table", _TABLE), ("out_block_table", _TABLE),
                           ("dq_block_table", _TABLE), ("dkv_block_table", _TABLE))

    def __init__(self, stage_id, seqlens_q, seqlens_kv, max_seqlen_q, max_seqlen_kv, attn_mask,
                 q_block_table, kv_block_table, out_block_table, dq_block_table, dkv_block_table, **kw):
        super().__init__(stage_id=stage_id, seqlens_q=list(seqlens_q), seqlens_kv=list(seqlens_kv),
                         max_seqlen_q=max_seqlen_q, max_seqlen_kv=max_seqlen_kv, attn_mask=attn_mask,
                         q_block_table=q_block_table, kv_block_table=kv_block_table,
                         out_block_table=out_block_table, dq_block_table=dq_block_table,
                         dkv_block_table=dkv_block_table, **kw)


@dataclass
class ReductionOp:
    """LSE-weighted merge of partial (out, lse) pairs into ``dst``."""

    src_buffers: List[Tuple[BufferBlock, BufferBlock]]
    dst_buffer: Tuple[BufferBlock, BufferBlock]

    def __post_init__(self):
        self.src_buffers = [tuple(x) for x in self.src_buffers]
        self.dst_buffer = tuple(self.dst_buffer)


def _put_red_ops(w: ByteWriter, ops: Sequence[ReductionOp]) -> None:
    w.u32(len(ops))
    for op in ops:
        w.u32(len(op.src_buffers))
        for out_b, lse_b in op.src_buffers:
            _put_block(w, out_b)
            _put_block(w, lse_b)
        _put_block(w, op.dst_buffer[0])
        _put_block(w, op.dst_buffer[1])


def _get_red_ops(r: ByteReader) -> List[ReductionOp]:
    ops = []
    for _ in range(r.u32()):
        srcs = [(_get_block(r), _get_block(r)) for _ in range(r.u32())]
        ops.append(ReductionOp(srcs, (_get_block(r), _get_block(r))))
    return ops


class AttnReductionInstr(BlockInstrBase):
    FIELDS = (("ops", (_put_red_ops, _get_red_ops, None)), ("output_is_unpadded", _U32))

    def __init__(self, ops, output_is_unpadded, **kw):
        super().__init__(ops=list(ops), output_is_unpadded=int(bool(output_is_unpadded)), **kw)


@dataclass
class SumOp:
    """dst = sum(src blocks) (dQ / dKV partial accumulation)."""

    src_buffers: List[BufferBlock]
    dst_buffer: BufferBlock


def _put_sum_ops(w: ByteWriter, ops: Sequence[SumOp]) -> None:
    w.u32(len(ops))
    for op in ops:
        _put_blocks(w, op.src_buffers)
        _put_block(w, op.dst_buffer)


def _get_sum_ops(r: ByteReader) -> List[SumOp]:
    return [SumOp(_get_blocks(r), _get_block(r)) for _ in range(r.u32())]


class SumInstr(BlockInstrBase):
    FIELDS = (("ops", (_put_sum_ops, _get_sum_ops, None)), ("output_is_unpadded", _U32))

    def __init__(self, ops, output_is_unpadded, **kw):
        super().__init__(ops=list(ops), output_is_unpadded=int(bool(output_is_unpadded)), **kw)


# ------------------------------------------------------------------ plan
@dataclass
class BufferInfo:
    n_blocks: int
    block_size: int
    block_numel: int
    dtype: int
    buffer_shape: Tuple[int, ...]
    per_token_shape: Tuple[int, ...]

    def __post_init__(self):
        self.buffer_shape = tuple(int(x) for x in self.buffer_shape)
        self.per_token_shape = tuple(int(x) for x in self.per_token_shape)


class ExecutionPlan:
    """Instruction list of one device plus the buffer geometry it needs."""

    def __init__(self, instructions: List[BlockInstrBase], n_nodes: int, n_devices_per_node: int, node_id: int,
                 local_device_id: int, n_stages: int, local_cu_seqlens: List[int],
                 buffer_info: Dict[str, BufferInfo]):
        self.instructions = instructions
        self.n_nodes = n_nodes
        self.n_devices_per_node = n_devices_per_node
        self.node_id = node_id
        self.local_device_id = local_device_id
        self.n_stages = n_stages
        self.local_cu_seqlens = list(local_cu_seqlens)
        self.buffer_info = buffer_info

    def write(self, w: ByteWriter) -> None:
        w.u32(self.n_nodes).u32(self.n_devices_per_node).u32(self.node_id).u32(self.local_device_id)
        w.u32(self.n_stages).ints(self.local_cu_seqlens)
        w.u32(len(self.buffer_info))
        for name, info in self.buffer_info.items():
            w.string(name).u32(info.n_blocks).u32(info.block_size).u32(info.block_numel).u32(info.dtype)
            w.ints(info.buffer_shape).ints(info.per_token_shape)
        w.u32(len(self.instructions))
        for instr in self.instructions:
            instr.write(w)

    def serialize(self, config=None) -> bytes:
        w = ByteWriter()
        self.write(w)
        return w.getvalue()

    @classmethod
    def read(cls, r: ByteReader) -> "ExecutionPlan":
        n_nodes, n_dpn, node_id, dev_id, n_stages = (r.u32() for _ in range(5))
        cu = r.ints()
        infos: Dict[str, BufferInfo] = {}
        for _ in range(r.u32()):
            name = r.string()
            nb, bs, numel, dt = (r.u32() for _ in range(4))
            infos[name] = BufferInfo(nb, bs, numel, dt, r.int_tuple(), r.int_tuple())
        instrs = [BlockInstrBase.read(r) for _ in range(r.u32())]
        return cls(instrs, n_nodes, n_dpn, node_id, dev_id, n_stages, cu, infos)

    @classmethod
    def deserialize(cls, data: bytes, config=None) -> Tuple["ExecutionPlan", bytes]:
        r = ByteReader(data)
        plan = cls.read(r)
        return plan, r.rest()

    def __eq__(self, other: Any) -> bool:
        return (isinstance(other, ExecutionPlan)
                and (self.n_nodes, self.n_devices_per_node, self.node_id, self.local_device_id, self.n_stages)
                == (other.n_nodes, other.n_devices_per_node, other.node_id, other.local_device_id, other.n_stages)
                and self.local_cu_seqlens == other.local_cu_seqlens
                and self.buffer_info == other.buffer_info
                and self.instructions == other.instructions)

    __hash__ = None

    def __repr__(self) -> str:
        return (f"ExecutionPlan(node={self.node_id}, dev={self.local_device_id}, n_stages={self.n_stages}, "
                f"n_instrs={len(self.instructions)}, buffers={list(self.buffer_info)})")

    def __str__(self) -> str:
        lines = [repr(self)]
        lines += [f"  [{i}] {ins!r}" for i, ins in enumerate(self.instructions)]
        return "\n".join(lines)

    def count(self, cls) -> int:
        return sum(isinstance(i, cls) for i in self.instructions)


def serialize_list_of_execution_plans(plans: Sequence[ExecutionPlan], config=None) -> bytes:
    w = ByteWriter().u32(len(plans))
    for p in plans:
        p.write(w)
    return w.getvalue()


def deserialize_list_of_execution_plans(data: bytes, config=None) -> Tuple[List[ExecutionPlan], bytes]:
    r = ByteReader(data)
    plans = [ExecutionPlan.read(r) for _ in range(r.u32())]
    return plans, r.rest()

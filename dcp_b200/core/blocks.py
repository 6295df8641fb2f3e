"""Block-level IR of one training iteration: data blocks, computation blocks, workload spec.

A batch is cut into token blocks x head blocks.  *Data blocks* are the Q / KV inputs and the
Out / LSE outputs of every (sequence, head block, token block); *computation blocks* are the
(q block, kv block) pairs whose mask slice is not empty.  ``WorkloadSpec`` bundles them with
costs, the block->device placement and the work->stage schedule.  Field names follow the
reference (dcp/core/block_table.py:33-645) so plans, specs and user code stay interchangeable.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .instructions import DType
from .serialization import ByteReader, ByteWriter

Device = Tuple[int, int]  # (node, local device)


class BlockType:
    Q = "Q"
    dQ = "dQ"
    KV = "KV"
    dKV = "dKV"
    Out = "OUT"
    dOut = "dOUT"
    LSE = "LSE"
    Work = "WORK"


class BlockMeta:
    def __init__(self, type: str, dtype: int, seq_id: int, head_id: int, **kwargs):
        self.type = type
        self.dtype = dtype
        self.seq_id = seq_id
        self.head_id = head_id
        for k, v in kwargs.items():
            setattr(self, k, v)


class ComputationBlockMeta(BlockMeta):
    """One attention work unit: Q block ``q_id`` against KV block ``kv_id``.

    ``local_attn_mask`` is int32 [2, n_q] (one range) or [2, 2, n_q] (two ranges): per query the
    allowed key interval(s) relative to the start of the KV block.  It is not part of the wire
    form (dcp/core/block_table.py:127,160-161).
    """

    _ID_FIELDS = ("seq_id", "head_id", "q_id", "kv_id", "out_id", "lse_id", "dout_id", "dq_id", "dkv_id")

    def __init__(self, type, dtype, seq_id, head_id, q_id, kv_id, out_id, lse_id, dout_id=None, dq_id=None,
                 dkv_id=None, local_attn_mask: Optional[torch.Tensor] = None, **kwargs):
        super().__init__(type, dtype, seq_id, head_id, **kwargs)
        self.q_id, self.kv_id, self.out_id, self.lse_id = q_id, kv_id, out_id, lse_id
        self.dout_id, self.dq_id, self.dkv_id = dout_id, dq_id, dkv_id
        self.local_attn_mask = None if local_attn_mask is None else local_attn_mask.to(torch.int32)

    def __eq__(self, other):
        if not isinstance(other, ComputationBlockMeta):
            return False
        same = self.type == other.type and self.dtype == other.dtype and all(
            getattr(self, f) == getattr(other, f) for f in self._ID_FIELDS)
        if same and self.local_attn_mask is not None and other.local_attn_mask is not None:
            same = torch.equal(self.local_attn_mask, other.local_attn_mask)
        return same

    __hash__ = None

    def __repr__(self):
        return (f"ComputationBlockMeta(seq={self.seq_id}, head={self.head_id}, q={self.q_id}, kv={self.kv_id}, "
                f"out={self.out_id}, lse={self.lse_id})")

    def write(self, w: ByteWriter) -> None:
        w.string(self.type).u32(self.dtype)
        ids = [getattr(self, f) for f in self._ID_FIELDS]
        w.ints(ids if self.dout_id is not None else ids[:6])

    @classmethod
    def read(cls, r: ByteReader) -> "ComputationBlockMeta":
        type_, dtype = r.string(), r.u32()
        ids = r.ints()
        ids = ids + [None] * (9 - len(ids))
        return cls(type_, dtype, *ids)


class DataBlockMeta(BlockMeta):
    def __init__(self, type, dtype, seq_id, head_id, block_id, n_tokens, block_size, head_block_size,
                 per_token_shape: Tuple[int, ...], **kwargs):
        super().__init__(type, dtype, seq_id, head_id, **kwargs)
        self.block_id = block_id
        self.n_tokens = n_tokens            # tokens actually present
        self.block_size = block_size        # padded token capacity
        self.head_block_size = head_block_size
        self.per_token_shape = tuple(per_token_shape)

    def _key(self):
        return (self.type, self.dtype, self.seq_id, self.head_id, self.block_id, self.n_tokens, self.block_size,
                self.head_block_size, self.per_token_shape)

    def __eq__(self, other):
        return isinstance(other, DataBlockMeta) and self._key() == other._key()

    def __hash__(self):
        return hash(self._key())

    def __repr__(self):
        return ("DataBlockMeta(type={}, dtype={}, seq_id={}, head_id={}, block_id={}, n_tokens={}, block_size={}, "
                "head_block_size={}, per_token_shape={})").format(*self._key())

    def per_token_numel(self) -> int:
        n = 1
        for d in self.per_token_shape:
            n *= d
        return n

    def numel(self, padded: bool = True) -> int:
        return (self.block_size if padded else self.n_tokens) * self.per_token_numel()

    def nbytes(self, padded: bool = False) -> int:
        return self.numel(padded) * DType.element_size(self.dtype)

    def write(self, w: ByteWriter) -> None:
        w.string(self.type).u32(self.dtype)
        w.ints([self.seq_id, self.head_id, self.block_id, self.n_tokens, self.block_size, self.head_block_size])
        w.ints(self.per_token_shape)

    @classmethod
    def read(cls, r: ByteReader) -> "DataBlockMeta":
        type_, dtype = r.string(), r.u32()
        seq_id, head_id, block_id, n_tokens, block_size, hbs = r.ints()
        return cls(type_, dtype, seq_id, head_id, block_id, n_tokens, block_size, hbs, tuple(r.ints()))


def _write_meta_map(w: ByteWriter, m: Dict[int, BlockMeta]) -> None:
    w.u32(len(m))
    for k, meta in m.items():
        w.u32(k)
        meta.write(w)


def _read_meta_map(r: ByteReader, cls) -> Dict[int, BlockMeta]:
    out = {}
    for _ in range(r.u32()):
        k = r.u32()
        out[k] = cls.read(r)
    return out


def _write_dev_map(w: ByteWriter, m: Dict[Device, Dict[int, int]]) -> None:
    w.u32(len(m))
    for (n, d), inner in m.items():
        w.u32(n).u32(d).u32(len(inner))
        for k, v in inner.items():
            w.u32(k).u32(v)


def _read_dev_map(r: ByteReader) -> Dict[Device, Dict[int, int]]:
    out = {}
    for _ in range(r.u32()):
        dev = (r.u32(), r.u32())
        inner = {}
        for _ in range(r.u32()):
            k = r.u32()
            inner[k] = r.u32()
        out[dev] = inner
    return out


@dataclass
class BlockMappings:
    input_id_to_meta: Dict[int, DataBlockMeta]
    output_id_to_meta: Dict[int, DataBlockMeta]
    work_id_to_meta: Dict[int, ComputationBlockMeta]
    # device -> block id -> index of the block in that device's local (unpadded) buffers
    input_id_to_buffer_index: Dict[Device, Dict[int, int]] = field(default_factory=dict)
    output_id_to_buffer_index: Dict[Device, Dict[int, int]] = field(default_factory=dict)
    buffer_type_to_dtype: Dict[str, int] = field(default_factory=dict)

    def write(self, w: ByteWriter) -> None:
        _write_meta_map(w, self.input_id_to_meta)
        _write_meta_map(w, self.output_id_to_meta)
        _write_meta_map(w, self.work_id_to_meta)
        _write_dev_map(w, self.input_id_to_buffer_index)
        _write_dev_map(w, self.output_id_to_buffer_index)
        w.u32(len(self.buffer_type_to_dtype))
        for k, v in self.buffer_type_to_dtype.items():
            w.string(k).u32(v)

    @classmethod
    def read(cls, r: ByteReader) -> "BlockMappings":
        i = _read_meta_map(r, DataBlockMeta)
        o = _read_meta_map(r, DataBlockMeta)
        wk = _read_meta_map(r, ComputationBlockMeta)
        ib, ob = _read_dev_map(r), _read_dev_map(r)
        bt = {}
        for _ in range(r.u32()):
            k = r.string()
            bt[k] = r.u32()
        return cls(i, o, wk, ib, ob, bt)

    def serialize(self, config=None) -> bytes:
        w = ByteWriter()
        self.write(w)
        return w.getvalue()

    @classmethod
    def deserialize(cls, data: bytes, config=None):
        r = ByteReader(data)
        return cls.read(r), r.rest()


class BlockManager:
    """First-free-slot allocator for one paged buffer type.

    A slot is addressed by ``(data_id, is_input, creation_device, stage_id, replica_id)``
    (dcp/core/block_table.py:429-532); freed slots are reused lowest index first and
    ``high_water`` gives the number of slots the buffer must provide.
    """

    def __init__(self):
        self._key_to_slot: Dict[tuple, int] = {}
        self._free: List[int] = []
        self._next = 0

    @staticmethod
    def _key(data_id, is_input, creation_device=None, stage_id=None, replica_id=0):
        return (data_id, bool(is_input), creation_device, stage_id, replica_id)

    def has_block(self, *key_args, **key_kw) -> bool:
        return self._key(*key_args, **key_kw) in self._key_to_slot

    def alloc_block(self, *key_args, **key_kw) -> int:
        key = self._key(*key_args, **key_kw)
        if key in self._key_to_slot:
            raise KeyError(f"block {key} already allocated")
        if self._free:
            slot = min(self._free)
            self._free.remove(slot)
        else:
            slot = self._next
            self._next += 1
        self._key_to_slot[key] = slot
        return slot

    def get_block(self, *key_args, **key_kw) -> int:
        return self._key_to_slot[self._key(*key_args, **key_kw)]

    def get_or_alloc(self, *key_args, **key_kw) -> int:
        key = self._key(*key_args, **key_kw)
        return self._key_to_slot[key] if key in self._key_to_slot else self.alloc_block(*key_args, **key_kw)

    def free_block(self, *key_args, **key_kw) -> int:
        slot = self._key_to_slot.pop(self._key(*key_args, **key_kw))
        self._free.append(slot)
        return slot

    def keys(self):
        return list(self._key_to_slot)

    @property
    def high_water(self) -> int:
        return self._next

    @property
    def n_live(self) -> int:
        return len(self._key_to_slot)


@dataclass
class WorkloadSpec:
    workloads: List[float]
    work_unit_input_map: List[List[int]]
    work_unit_output_map: List[List[int]]
    block_mapping: BlockMappings
    input_to_device_map: Dict[int, Device] = field(default_factory=dict)
    output_to_device_map: Dict[int, Device] = field(default_factory=dict)
    work_to_device_map: Dict[int, Device] = field(default_factory=dict)
    work_to_stage_map: Dict[int, int] = field(default_factory=dict)
    colocation_constraints: List[List[List[int]]] = field(default_factory=list)

    def __post_init__(self):
        # bytes of the tokens really present (what crosses a link when the block moves)
        im, om = self.block_mapping.input_id_to_meta, self.block_mapping.output_id_to_meta
        self.input_sizes = [im[i].nbytes(padded=False) for i in range(len(im))]
        self.output_sizes = [om[i].nbytes(padded=False) for i in range(len(om))]

    @property
    def n_work(self) -> int:
        return len(self.workloads)

    def write(self, w: ByteWriter) -> None:
        w.floats(self.workloads)
        w.seq(self.work_unit_input_map, lambda ww, x: ww.ints(x))
        w.seq(self.work_unit_output_map, lambda ww, x: ww.ints(x))
        self.block_mapping.write(w)
        for m in (self.input_to_device_map, self.output_to_device_map, self.work_to_device_map):
            w.u32(len(m))
            for k, dev in m.items():
                w.u32(k).ints(dev)
        w.u32(len(self.work_to_stage_map))
        for k, v in self.work_to_stage_map.items():
            w.u32(k).u32(v)
        w.seq(self.colocation_constraints, lambda ww, grp: ww.seq(grp, lambda w3, x: w3.ints(x)))

    @classmethod
    def read(cls, r: ByteReader) -> "WorkloadSpec":
        workloads = r.floats()
        wi = r.seq(lambda rr: rr.ints())
        wo = r.seq(lambda rr: rr.ints())
        bm = BlockMappings.read(r)
        maps = []
        for _ in range(3):
            m = {}
            for _ in range(r.u32()):
                k = r.u32()
                m[k] = tuple(r.ints())
            maps.append(m)
        stage = {}
        for _ in range(r.u32()):
            k = r.u32()
            stage[k] = r.u32()
        coloc = r.seq(lambda rr: rr.seq(lambda r3: r3.ints()))
        return cls(workloads, wi, wo, bm, maps[0], maps[1], maps[2], stage, coloc)

    def serialize(self, config=None) -> bytes:
        w = ByteWriter()
        self.write(w)
        return w.getvalue()

    @classmethod
    def deserialize(cls, data: bytes, config=None):
        r = ByteReader(data)
        return cls.read(r), r.rest()


def serialize_list_of_workloads(workloads: Sequence[WorkloadSpec], config=None) -> bytes:
    w = ByteWriter().u32(len(workloads))
    for wl in workloads:
        wl.write(w)
    return w.getvalue()


def deserialize_list_of_workloads(data: bytes, config=None):
    r = ByteReader(data)
    out = [WorkloadSpec.read(r) for _ in range(r.u32())]
    return out, r.rest()

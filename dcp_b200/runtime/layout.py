"""Where a device's blocks sit inside its Local* buffers, and global <-> local reshuffles.

Local buffers hold a device's own tokens unpadded, one block after another in buffer-index
order, i.e. sorted by (head block, sequence, token block) - the layout
dcp/core/compiler.py:183-256 fixes and dcp/runtime/flash_attention/interface.py:297-420
(get_local_q_kv) fills.  ``LocalLayout`` precomputes row offsets per buffer so executors and tests
can address a block by (buffer name, index).
"""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

from ..core.blocks import BlockType, DataBlockMeta, Device, WorkloadSpec
from ..core.instructions import BufferType

_TYPE_TO_LOCAL = {
    BlockType.Q: BufferType.LOCAL_Q, BlockType.KV: BufferType.LOCAL_KV, BlockType.Out: BufferType.LOCAL_OUT,
    BlockType.LSE: BufferType.LOCAL_LSE, BlockType.dOut: BufferType.LOCAL_dOUT, BlockType.dQ: BufferType.LOCAL_dQ,
    BlockType.dKV: BufferType.LOCAL_dKV,
}


class LocalLayout:
    def __init__(self, workload: WorkloadSpec, dev: Device):
        self.dev = tuple(dev)
        bm = workload.block_mapping
        self.blocks: Dict[str, List[Tuple[int, DataBlockMeta]]] = {}   # buffer -> [(block id, meta)] in index order
        for metas, idx_map in ((bm.input_id_to_meta, bm.input_id_to_buffer_index),
                               (bm.output_id_to_meta, bm.output_id_to_buffer_index)):
            per_type: Dict[str, Dict[int, Tuple[int, DataBlockMeta]]] = {}
            for bid, idx in idx_map.get(self.dev, {}).items():
                m = metas[bid]
                per_type.setdefault(_TYPE_TO_LOCAL[m.type], {})[idx] = (bid, m)
            for name, by_idx in per_type.items():
                self.blocks[name] = [by_idx[i] for i in range(len(by_idx))]
        # head-block width of every buffer, also for buffers this device holds no block of
        self.head_block: Dict[str, int] = {}
        for metas in (bm.input_id_to_meta, bm.output_id_to_meta):
            for m in metas.values():
                self.head_block.setdefault(_TYPE_TO_LOCAL[m.type], m.head_block_size)
        self.offsets: Dict[str, np.ndarray] = {}
        for name, lst in self.blocks.items():
            self.offsets[name] = np.concatenate([[0], np.cumsum([m.n_tokens for _, m in lst])]).astype(np.int64)

    def n_tokens(self, name: str) -> int:
        return int(self.offsets[name][-1]) if name in self.offsets else 0

    def row_range(self, name: str, index: int) -> Tuple[int, int]:
        off = self.offsets[name]
        return int(off[index]), int(off[index + 1])


def seq_token_offsets(raw_seqlens: Sequence[int]) -> np.ndarray:
    return np.concatenate([[0], np.cumsum(np.asarray(raw_seqlens, dtype=np.int64))])


def gather_local(global_t: torch.Tensor, layout: LocalLayout, name: str, raw_seqlens: Sequence[int],
                 head_axis: int) -> torch.Tensor:
    """Slice a global [sum(raw), ...heads..., d] tensor into a device's local buffer ``name``.

    ``head_axis`` is the axis of ``global_t`` that is cut into head blocks (1 for Q-like
    [T, H, d], 2 for KV-like [T, 2, H, d]).  Returns [local_tokens, *per_token_shape].
    """
    cu = seq_token_offsets(raw_seqlens)
    parts = []
    for _, m in layout.blocks.get(name, []):
        t0 = int(cu[m.seq_id]) + m.block_id * m.block_size
        hb = m.head_block_size
        sl = [slice(t0, t0 + m.n_tokens)] + [slice(None)] * (global_t.dim() - 1)
        sl[head_axis] = slice(m.head_id * hb, (m.head_id + 1) * hb)
        parts.append(global_t[tuple(sl)])
    if not parts:      # a device that owns no block of this kind: empty, but with the buffer's head-block width
        shape = list(global_t.shape)
        shape[0] = 0
        shape[head_axis] = layout.head_block.get(name, shape[head_axis])
        return global_t.new_zeros(shape)
    return torch.cat(parts, dim=0)


def scatter_to_global(local_t: torch.Tensor, global_t: torch.Tensor, layout: LocalLayout, name: str,
                      raw_seqlens: Sequence[int], head_axis: int, token_axis_local: int = 0) -> None:
    """Inverse of ``gather_local``: write a device's local buffer into the global tensor.

    For LSE-like local tensors ([heads_in_block, tokens]) pass ``token_axis_local=1``; the global
    LSE is [n_heads, sum(raw)] with ``head_axis=0``.
    """
    cu = seq_token_offsets(raw_seqlens)
    off = layout.offsets.get(name)
    for k, (_, m) in enumerate(layout.blocks.get(name, [])):
        t0 = int(cu[m.seq_id]) + m.block_id * m.block_size
        hb = m.head_block_size
        src = local_t.narrow(token_axis_local, int(off[k]), m.n_tokens)
        if token_axis_local == 1:  # LSE: global [H, T]
            global_t[m.head_id * hb:(m.head_id + 1) * hb, t0:t0 + m.n_tokens] = src
        else:
            sl = [slice(t0, t0 + m.n_tokens)] + [slice(None)] * (global_t.dim() - 1)
            sl[head_axis] = slice(m.head_id * hb, (m.head_id + 1) * hb)
            global_t[tuple(sl)] = src


def get_local_q_kv(q: torch.Tensor, kv: torch.Tensor, workload: WorkloadSpec, dev: Device,
                   raw_seqlens: Sequence[int]):
    """Global q [T, H, d], kv [T, 2, Hkv, d] -> this device's (local_q, local_kv) in buffer order."""
    lay = LocalLayout(workload, dev)
    return (gather_local(q, lay, BufferType.LOCAL_Q, raw_seqlens, 1),
            gather_local(kv, lay, BufferType.LOCAL_KV, raw_seqlens, 2))

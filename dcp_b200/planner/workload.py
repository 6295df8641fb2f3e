"""Cut a packed variable-length batch into data blocks and attention work units.

Block ids follow the reference layout (dcp/data/dataloader.py:1321-1391): per sequence the Q
blocks come first (``base + head_block * n_blk + i``), the KV blocks after them; outputs
interleave Out and LSE (``base_o + head_block * n_blk * 2 + 2 i`` and ``+ 1``).  One work unit is
created per (sequence, head block, q block i, kv block j) whose mask slice is not empty; its
``local_attn_mask`` is the per-query key interval(s) relative to the start of KV block j.

The per-pair slicing is done with array arithmetic over all KV blocks of a query block at once
rather than a Python loop over (i, j) pairs.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..core.blocks import (BlockMappings, BlockType, ComputationBlockMeta, DataBlockMeta, WorkloadSpec)
from ..core.cost_model import AttnRooflineCostModel
from ..core.instructions import BufferType, DType
from .masks import causal_range_mask_fn, to_two_range


def pad_seqlens(raw_seqlens: Sequence[int], block_size: int) -> List[int]:
    return [-(-int(s) // block_size) * block_size for s in raw_seqlens]


def head_block_geometry(n_heads: int, n_query_groups: int, head_block_size: int):
    """-> (n_head_blocks_q, n_head_blocks_kv, head_block_size_kv, q_head_block -> kv_head_block)."""
    assert n_heads % n_query_groups == 0
    per_group = n_heads // n_query_groups
    assert n_heads % head_block_size == 0, "n_heads must be divisible by head_block_size"
    n_hb_q = n_heads // head_block_size
    if per_group > 1:
        if head_block_size <= per_group:
            # GQA: one KV head per KV head block (dcp/data/dataloader.py:1253-1265)
            assert per_group % head_block_size == 0
            hbs_kv = 1
            n_hb_kv = n_query_groups
            kv_of = [(j * head_block_size) // per_group for j in range(n_hb_q)]
        else:
            # wider head blocks spanning whole groups (all heads on one device is hbs == n_heads)
            assert head_block_size % per_group == 0
            hbs_kv = head_block_size // per_group
            n_hb_kv = n_hb_q
            kv_of = list(range(n_hb_q))
    else:
        hbs_kv, n_hb_kv, kv_of = head_block_size, n_hb_q, list(range(n_hb_q))
    return n_hb_q, n_hb_kv, hbs_kv, kv_of


def _slice_pairs(rng: np.ndarray, q_lo: int, q_hi: int, n_blk: int, block_size: int):
    """For queries [q_lo, q_hi) return per KV block j the clamped, rebased intervals.

    rng: int64 [T, 2, 2] in sequence coordinates. Returns (local [n_blk, 2, 2, n_q], allowed [n_blk]).
    """
    r = rng[q_lo:q_hi]                                  # [n_q, 2, 2]
    lo = (np.arange(n_blk, dtype=np.int64) * block_size)[:, None, None]  # [n_blk,1,1]
    hi = lo + block_size
    start = np.clip(r[None, :, :, 0], lo, hi) - lo      # [n_blk, n_q, 2]
    end = np.clip(r[None, :, :, 1], lo, hi) - lo
    end = np.maximum(end, start)
    length = end - start
    empty = length <= 0
    start = np.where(empty, 0, start)
    end = np.where(empty, 0, end)
    overlap = np.clip(np.minimum(end[..., 0], end[..., 1]) - np.maximum(start[..., 0], start[..., 1]), 0, None)
    allowed = (end - start).sum(axis=(1, 2)) - overlap.sum(axis=1)
    local = np.stack([start, end], axis=2)              # [n_blk, n_q, 2(bound), 2(range)]
    local = local.transpose(0, 3, 2, 1)                 # [n_blk, range, bound, n_q]
    return local, allowed


def _native_planner():
    try:
        from .. import _planner
        return _planner if hasattr(_planner, "slice_mask_pairs") else None
    except ImportError:
        return None


def slice_pairs(rng: np.ndarray, q_lo: int, q_hi: int, n_blk: int, block_size: int, use_native: bool = True):
    """-> (kv block indices with allowed pairs, allowed counts, local int32 [n, 2(range), 2(bound), n_q]).
    Native (C++) when the planner extension is built, the array-arithmetic version otherwise."""
    nat = _native_planner() if use_native else None
    if nat is not None:
        return nat.slice_mask_pairs(rng, int(q_lo), int(q_hi), int(n_blk), int(block_size))
    local, allowed = _slice_pairs(rng, q_lo, q_hi, n_blk, block_size)
    idx = np.nonzero(allowed > 0)[0]
    return idx.tolist(), allowed[idx].tolist(), local[idx].astype(np.int32)


def generate_workload(q_shape: Tuple[int, ...], kv_shape: Tuple[int, ...], raw_seqlens: Sequence[int],
                      padded_seqlens: Sequence[int], block_size: int, head_block_size: int,
                      comp_cost_model: Optional[AttnRooflineCostModel] = None,
                      attn_mask: Optional[torch.Tensor] = None, qkv_dtype: torch.dtype = torch.bfloat16,
                      is_forward: bool = True, logger=None) -> WorkloadSpec:
    """Build the (placement-free) WorkloadSpec of one batch.

    q_shape ``(total_tokens, n_heads, head_dim)``, kv_shape ``(total_tokens, 2, n_query_groups,
    head_dim)``; ``attn_mask`` follows the mask_fn contract (None = causal).
    """
    n_heads, head_dim = int(q_shape[-2]), int(q_shape[-1])
    n_groups = int(kv_shape[-2])
    comp_cost_model = comp_cost_model or AttnRooflineCostModel()
    n_hb_q, n_hb_kv, hbs_kv, kv_of = head_block_geometry(n_heads, n_groups, head_block_size)
    dt = DType.from_torch(qkv_dtype)
    if attn_mask is None:
        attn_mask = causal_range_mask_fn(raw_seqlens, padded_seqlens, torch.int32)
    single_range = attn_mask.dim() == 2
    full_rng = to_two_range(attn_mask)
    offsets = np.concatenate([[0], np.cumsum(np.asarray(padded_seqlens, dtype=np.int64))])

    input_meta: Dict[int, DataBlockMeta] = {}
    output_meta: Dict[int, DataBlockMeta] = {}
    work_meta: Dict[int, ComputationBlockMeta] = {}
    workloads: List[float] = []
    work_in: List[List[int]] = []
    work_out: List[List[int]] = []
    coloc: List[List[List[int]]] = []
    in_base = out_base = 0
    heads_per_kv_block = head_block_size // hbs_kv if hbs_kv else 1

    for s, (raw, padded) in enumerate(zip(raw_seqlens, padded_seqlens)):
        n_blk = padded // block_size
        tok = [min(block_size, max(int(raw) - i * block_size, 0)) for i in range(n_blk)]
        q_id = lambda j, i: in_base + j * n_blk + i
        kv_id = lambda j, i: in_base + n_hb_q * n_blk + j * n_blk + i
        o_id = lambda j, i: out_base + j * n_blk * 2 + 2 * i
        for j in range(n_hb_q):
            for i in range(n_blk):
                input_meta[q_id(j, i)] = DataBlockMeta(BlockType.Q, dt, s, j, i, tok[i], block_size,
                                                       head_block_size, (head_block_size, head_dim))
                output_meta[o_id(j, i)] = DataBlockMeta(BlockType.Out, dt, s, j, i, tok[i], block_size,
                                                        head_block_size, (head_block_size, head_dim))
                output_meta[o_id(j, i) + 1] = DataBlockMeta(BlockType.LSE, DType.FLOAT32, s, j, i, tok[i],
                                                            block_size, head_block_size, (head_block_size,))
        for j in range(n_hb_kv):
            for i in range(n_blk):
                input_meta[kv_id(j, i)] = DataBlockMeta(BlockType.KV, dt, s, j, i, tok[i], block_size, hbs_kv,
                                                        (2, hbs_kv, head_dim))
        for i in range(n_blk):
            ins = [q_id(j, i) for j in range(n_hb_q)] + [kv_id(j, i) for j in range(n_hb_kv)]
            outs = [o_id(j, i) + d for j in range(n_hb_q) for d in (0, 1)]
            coloc.append([ins, outs])
        rng = full_rng[offsets[s]:offsets[s] + padded]
        for i in range(n_blk):
            if tok[i] == 0:
                continue
            kv_idx, allowed, local = slice_pairs(rng, i * block_size, i * block_size + tok[i], n_blk, block_size)
            for k, jj in enumerate(kv_idx):
                if tok[jj] == 0:
                    continue
                m = local[k]                               # [range, bound, n_q]
                mask_t = torch.from_numpy(np.ascontiguousarray(m[0] if single_range else m).astype(np.int32))
                cost = comp_cost_model.pair_cost(tok[i], tok[jj], float(allowed[k]), head_block_size,
                                                 hbs_kv, head_dim, is_forward)
                for j in range(n_hb_q):
                    wid = len(workloads)
                    work_meta[wid] = ComputationBlockMeta(BlockType.Work, dt, s, j, q_id(j, i), kv_id(kv_of[j], jj),
                                                          o_id(j, i), o_id(j, i) + 1, local_attn_mask=mask_t)
                    workloads.append(cost)
                    work_in.append([q_id(j, i), kv_id(kv_of[j], jj)])
                    work_out.append([o_id(j, i), o_id(j, i) + 1])
        in_base += (n_hb_q + n_hb_kv) * n_blk
        out_base += 2 * n_hb_q * n_blk

    buffer_dtypes = {
        BufferType.LOCAL_KV: dt, BufferType.LOCAL_Q: dt, BufferType.LOCAL_OUT: dt,
        BufferType.LOCAL_LSE: DType.FLOAT32, BufferType.LOCAL_dOUT: dt, BufferType.BUFFER_Q: dt,
        BufferType.BUFFER_KV: dt, BufferType.BUFFER_OUT: dt, BufferType.BUFFER_LSE: DType.FLOAT32,
    }
    mappings = BlockMappings(input_meta, output_meta, work_meta, {}, {}, buffer_dtypes)
    return WorkloadSpec(workloads, work_in, work_out, mappings, {}, {}, {}, {}, coloc)


def block_size_heuristic(raw_seqlens: Sequence[int], n_devices: int, mem_epsilon: float = 0.2,
                         min_block_size: int = 256, max_block_size: Optional[int] = None) -> int:
    """Largest power-of-two block size whose LPT packing onto ``n_devices`` stays within
    ``1 + mem_epsilon`` of the mean load (dcp/data/dataloader.py:1651-1686)."""
    longest = max(int(s) for s in raw_seqlens)
    bs = 1 << max(int(longest - 1).bit_length(), 0)
    if max_block_size:
        bs = min(bs, max_block_size)
    bs = max(bs, min_block_size)

    def imbalance(b: int) -> float:
        sizes = []
        for s in raw_seqlens:
            full, rem = divmod(int(s), b)
            sizes += [b] * full + ([rem] if rem else [])
        loads = [0] * n_devices
        for x in sorted(sizes, reverse=True):
            loads[loads.index(min(loads))] += x
        mean = sum(loads) / n_devices
        return max(loads) / mean if mean > 0 else 1.0

    while bs > min_block_size and imbalance(bs) > 1.0 + mem_epsilon:
        bs //= 2
    return bs

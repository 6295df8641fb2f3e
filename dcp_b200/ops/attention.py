"""Blockwise range-masked attention: host-side table building, kernel launch, fp32 reference.

The kernels (``csrc/kernels/attn_fwd.cu``, ``attn_bwd.cu``) consume flat int32 tables that
describe 128-query tiles, the KV blocks each tile attends to, and two half-open key ranges per
query.  ``AttnRow`` is the Python-side unit: one Q block of one plan stage (what one row of the
reference's AttnInstr block tables describes, dcp/core/instructions.py:479-626).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import _lib

TILE_M = 128          # query rows per softmax warpgroup
TILE_M_PAIR = 256     # query rows per CTA of the two-tile forward kernel (the default)
TILE_N = 128
HEAD_DIM = 128


@dataclass
class AttnRow:
    """One Q block and the KV blocks it attends to within one stage.

    q_row/out_row are arena rows; ``kv`` lists (arena_row, n_tokens) per KV block in position
    order; ``ranges`` is int32 [n_tokens, 4] = (s0, e0, s1, e1) in concatenated-KV positions
    where KV block i covers positions [i*block_size, (i+1)*block_size).
    """

    q_row: int
    n_tokens: int
    heads: Sequence[int]
    kv: List[Tuple[int, int]]
    ranges: np.ndarray
    out_dev: int = 0
    out_row: int = 0
    # backward only: destination of dQ / per-KV-block destination of dKV
    dq_dev: int = 0
    dq_row: int = 0
    dkv: List[Tuple[int, int]] = field(default_factory=list)  # (dev, row) per KV block


@dataclass
class FwdTables:
    tiles: torch.Tensor       # int32 [n_tiles, 8]
    kv_entries: torch.Tensor  # int32 [n_entries, 2]
    masks: torch.Tensor       # int32 [n_mask_rows, 4]
    n_tiles: int
    block_size: int
    flops: float = 0.0
    tile_m: int = TILE_M_PAIR   # 256: two-tile kernel (attn_fwd_pair.cu); 128: one tile per CTA (attn_fwd.cu)

    def to(self, device, non_blocking: bool = True) -> "FwdTables":
        mv = lambda t: t.to(device, non_blocking=non_blocking)
        return FwdTables(mv(self.tiles), mv(self.kv_entries), mv(self.masks), self.n_tiles, self.block_size, self.flops,
                         self.tile_m)

    def pin(self) -> "FwdTables":
        return FwdTables(self.tiles.pin_memory(), self.kv_entries.pin_memory(), self.masks.pin_memory(), self.n_tiles,
                         self.block_size, self.flops, self.tile_m)


def _pair_count(ranges: np.ndarray) -> float:
    """Number of (query, key) pairs allowed by a [n,4] range table (ranges assumed disjoint)."""
    r = ranges.astype(np.int64)
    return float(np.maximum(r[:, 1] - r[:, 0], 0).sum() + np.maximum(r[:, 3] - r[:, 2], 0).sum())


def _native_planner():
    """The C++ table builders (csrc/planner/kernel_tables.cpp), or None when DCP_B200_PY_TABLES=1
    asks for the Python implementations below (their twins and oracle)."""
    import os
    if os.environ.get("DCP_B200_PY_TABLES", "0") == "1":
        return None
    from .. import _planner
    # a planner library built before the table builders were added has no such entry points
    return _planner if hasattr(_planner, "build_fwd_tables") and hasattr(_planner, "build_bwd_tables") else None


def _row_tuples(rows: Sequence[AttnRow]):
    return [(int(r.q_row), int(r.n_tokens), [int(h) for h in r.heads], [(int(a), int(b)) for a, b in r.kv],
             np.ascontiguousarray(r.ranges, dtype=np.int32).reshape(-1, 4), int(r.out_dev), int(r.out_row), int(r.dq_dev),
             int(r.dq_row), [(int(a), int(b)) for a, b in r.dkv]) for r in rows]


def build_fwd_tables(rows: Sequence[AttnRow], block_size: int, device, tile_m: int = TILE_M_PAIR) -> FwdTables:
    """Forward kernel tables (see ``build_fwd_tables_py`` for the layout); built by the C++ planner module."""
    native = _native_planner()
    if native is None:
        return build_fwd_tables_py(rows, block_size, device, tile_m)
    assert tile_m in (TILE_M, TILE_M_PAIR)
    t_np, e_np, m_np, pairs = native.build_fwd_tables(_row_tuples(rows), int(block_size), int(tile_m))
    to = lambda a: torch.from_numpy(a).to(device, non_blocking=True)
    return FwdTables(to(t_np), to(e_np), to(m_np), int(t_np.shape[0]), block_size, flops=4.0 * pairs * HEAD_DIM, tile_m=tile_m)


def build_fwd_tables_py(rows: Sequence[AttnRow], block_size: int, device, tile_m: int = TILE_M_PAIR) -> FwdTables:
    """Flatten Q blocks into CTA tiles of ``tile_m`` query rows.

    tile_m = 128: one tile per CTA (attn_fwd.cu, attn_fwd_split.cu); ``kv_entries`` lists the KV blocks
    (arena row, tokens) and the kernel derives the 128-key tiles it needs from the mask bounds.

    tile_m = 256: two 128-row tiles per CTA that share every K/V tile (attn_fwd_pair.cu);
    ``kv_entries`` then is the ready-made walk of the CTA: one int32 x 4 entry per 128-key tile that
    at least one of the two query tiles can see = (arena row, position of its first key, valid keys,
    flags) with flags bit 0 / 1 = query tile A / B sees a key of it, bit 2 / 3 = A / B sees every
    (query, key) pair of it (no per-element masking needed).  ``AttnTile.kv_off / n_kv`` index it.
    """
    assert tile_m in (TILE_M, TILE_M_PAIR)
    tiles, entries, masks = [], [], []
    mask_row = 0
    pairs = 0.0
    n_entries = 0
    for row in rows:
        rng = np.ascontiguousarray(row.ranges, dtype=np.int32).reshape(-1, 4)
        assert rng.shape[0] == row.n_tokens
        masks.append(rng)
        pairs += _pair_count(rng) * len(row.heads)
        n_sub = (row.n_tokens + tile_m - 1) // tile_m
        if tile_m == TILE_M:
            kv_off = n_entries
            entries.append(np.asarray([(int(r), int(n)) for r, n in row.kv], dtype=np.int32).reshape(-1, 2))
            n_entries += len(row.kv)
            per_tile = [(kv_off, len(row.kv))] * n_sub
        else:
            per_tile = []
            for sub in _kv_walks(row, rng, block_size):
                per_tile.append((n_entries, sub.shape[0]))
                entries.append(sub)
                n_entries += sub.shape[0]
        for t in range(n_sub):
            n_rows = min(tile_m, row.n_tokens - t * tile_m)
            off, cnt = per_tile[t]
            for h in row.heads:
                tiles.append((row.q_row + t * tile_m, n_rows, int(h), off, cnt,
                              mask_row + t * tile_m, row.out_dev, row.out_row + t * tile_m))
        mask_row += row.n_tokens
    # longest tiles first: the grid is scheduled in index order, so this is LPT packing
    tiles.sort(key=lambda x: -x[4])
    width = 2 if tile_m == TILE_M else 4
    t_np = np.asarray(tiles, dtype=np.int32).reshape(-1, 8)
    e_np = np.concatenate(entries, axis=0) if entries else np.zeros((0, width), np.int32)
    m_np = np.concatenate(masks, axis=0) if masks else np.zeros((0, 4), np.int32)
    to = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device, non_blocking=True)
    return FwdTables(to(t_np), to(e_np.astype(np.int32)), to(m_np), len(tiles), block_size, flops=4.0 * pairs * HEAD_DIM,
                     tile_m=tile_m)


def _kv_walks(row: AttnRow, rng: np.ndarray, block_size: int) -> List[np.ndarray]:
    """Per 256-row CTA tile of a Q block: int32 [n, 4] list of the 128-key tiles it visits (see
    build_fwd_tables).  Visibility comes from the union / intersection of the two key ranges over each
    128-row query tile, the same test the one-tile kernels run on the device."""
    n_qt, (u0s, u0e, u1s, u1e, i0s, i0e, i1s, i1e) = _tile_bounds(rng, TILE_M)
    k_row, k_pos, k_nv = [], [], []
    for e, (kv_row, n_tok) in enumerate(row.kv):
        n_sub = (int(n_tok) + TILE_N - 1) // TILE_N
        t = np.arange(n_sub)
        k_row.append(int(kv_row) + t * TILE_N)
        k_pos.append(e * block_size + t * TILE_N)
        k_nv.append(np.minimum(TILE_N, int(n_tok) - t * TILE_N))
    if not k_row:
        return [np.zeros((0, 4), np.int32) for _ in range((n_qt + 1) // 2)]
    k_row, k_pos, k_nv = np.concatenate(k_row), np.concatenate(k_pos), np.concatenate(k_nv)
    lo, hi = k_pos[:, None], (k_pos + k_nv)[:, None]                                   # [n_k, 1]
    need = ((lo < u0e[None]) & (hi > u0s[None])) | ((lo < u1e[None]) & (hi > u1s[None]))           # [n_k, n_qt]
    full = (k_nv[:, None] == TILE_N) & (((i0s[None] <= lo) & (i0e[None] >= hi)) | ((i1s[None] <= lo) & (i1e[None] >= hi)))
    out = []
    for c in range((n_qt + 1) // 2):
        a, b = 2 * c, 2 * c + 1
        need_a, full_a = need[:, a], full[:, a]
        need_b = need[:, b] if b < n_qt else np.zeros_like(need_a)
        full_b = full[:, b] if b < n_qt else np.zeros_like(full_a)
        sel = np.nonzero(need_a | need_b)[0]
        flags = (need_a[sel].astype(np.int64) | (need_b[sel].astype(np.int64) << 1) |
                 ((full_a[sel] & need_a[sel]).astype(np.int64) << 2) | ((full_b[sel] & need_b[sel]).astype(np.int64) << 3))
        out.append(np.stack([k_row[sel], k_pos[sel], k_nv[sel], flags], axis=1).astype(np.int32))
    return out


def _ptr_array(tensors) -> ctypes.Array:
    arr = (ctypes.c_void_p * len(tensors))()
    for i, t in enumerate(tensors):
        arr[i] = t if isinstance(t, int) else t.data_ptr()
    return arr


class CopyContext:
    """Region bases of the copy jobs an attention kernel may carry (csrc/kernels/copy_jobs.cuh): for
    every region kind (q, kv, dout, lse, delta) the device address of the region on every rank of the
    group, and the local base.  ``stat_stride`` = rows per head of the statistics regions."""
    KINDS = ("q", "kv", "dout", "lse", "delta")
    MAX_PEERS = 16

    def __init__(self, peer_ptrs_of, rank: int, stat_stride: int):
        self.src = (ctypes.c_void_p * (len(self.KINDS) * self.MAX_PEERS))()
        self.dst = (ctypes.c_void_p * len(self.KINDS))()
        for k, name in enumerate(self.KINDS):
            ptrs = peer_ptrs_of(name)
            for r, ptr in enumerate(ptrs):
                self.src[k * self.MAX_PEERS + r] = ptr
            self.dst[k] = ptrs[rank]
        self.stat_stride = int(stat_stride)


def _job_args(jobs, ctx):
    """ctypes arguments (jobs, n_jobs, src bases, dst bases, stat stride) of a kernel's copy-job list."""
    if jobs is None or ctx is None or jobs.shape[0] == 0:
        return ctypes.c_void_p(0), ctypes.c_int(0), ctypes.c_void_p(0), ctypes.c_void_p(0), ctypes.c_int(0)
    return _lib.ptr(jobs), ctypes.c_int(jobs.shape[0]), ctx.src, ctx.dst, ctypes.c_int(ctx.stat_stride)


def copy_jobs(jobs: torch.Tensor, ctx: CopyContext) -> None:
    """Stand-alone launch of a copy-job list (int32 [n, 4]); used when no attention kernel can carry it."""
    if jobs is None or jobs.shape[0] == 0:
        return
    lib = _lib.load()
    _lib.check(lib.dcpk_copy_jobs(*_job_args(jobs, ctx), _lib.stream_handle()), "dcpk_copy_jobs")


def attn_fwd(q_arena: torch.Tensor, kv_arena: torch.Tensor, tables: FwdTables, out_dsts, lse_dsts,
             scale: float, status: torch.Tensor, variant: int = 0, lse_stride: Optional[int] = None,
             lse_stride_b: Optional[int] = None, n_dst_a: Optional[int] = None, jobs: Optional[torch.Tensor] = None,
             job_ctx: Optional[CopyContext] = None):
    """Run the forward kernel the tables were built for (``tables.tile_m``); ``variant`` only applies to
    the one-tile kernel (0: P in TMEM, 1: P through shared memory).  ``jobs`` (int32 [n, 4] on the
    device, see copy_jobs.cuh) is a list of peer -> local copies the two-tile kernel performs with
    two spare warps per CTA while it computes; ``job_ctx`` names the regions they refer to.

    q_arena: bf16 [rows, hq, 128]; kv_arena: bf16 [rows, 2, hkv, 128]; out_dsts / lse_dsts: lists of
    destination arenas (tensors or raw device addresses; index 0 = this rank), every out arena
    bf16 [rows_o, hq, 128] with its lse fp32 [hq, rows_o].
    """
    lib = _lib.load()
    assert q_arena.dtype == torch.bfloat16 and kv_arena.dtype == torch.bfloat16
    assert q_arena.is_contiguous() and kv_arena.is_contiguous()
    assert q_arena.shape[-1] == HEAD_DIM and kv_arena.shape[-1] == HEAD_DIM
    hq, hkv = q_arena.shape[1], kv_arena.shape[2]
    if lse_stride is None:
        lse_stride = lse_dsts[0].shape[1]
    if tables.tile_m == TILE_M_PAIR:
        rc = lib.dcpk_attn_fwd_pair(
            _lib.ptr(q_arena), ctypes.c_long(q_arena.shape[0]), _lib.ptr(kv_arena), ctypes.c_long(kv_arena.shape[0]),
            ctypes.c_int(hq), ctypes.c_int(hkv), _lib.ptr(tables.tiles), ctypes.c_int(tables.n_tiles),
            _lib.ptr(tables.kv_entries), ctypes.c_int(tables.kv_entries.shape[0]), _lib.ptr(tables.masks),
            ctypes.c_int(tables.masks.shape[0]), _ptr_array(out_dsts), _ptr_array(lse_dsts),
            ctypes.c_int(len(out_dsts)), ctypes.c_int(lse_stride),
            ctypes.c_int(lse_stride if lse_stride_b is None else lse_stride_b),
            ctypes.c_int(len(out_dsts) if n_dst_a is None else n_dst_a), ctypes.c_int(tables.block_size),
            ctypes.c_float(scale), *_job_args(jobs, job_ctx), _lib.ptr(status), _lib.stream_handle())
        _lib.check(rc, "dcpk_attn_fwd_pair")
        return
    assert jobs is None or jobs.shape[0] == 0, "only the two-tile forward kernel carries copy jobs"
    rc = lib.dcpk_attn_fwd(
        _lib.ptr(q_arena), ctypes.c_long(q_arena.shape[0]), _lib.ptr(kv_arena), ctypes.c_long(kv_arena.shape[0]),
        ctypes.c_int(hq), ctypes.c_int(hkv), _lib.ptr(tables.tiles), ctypes.c_int(tables.n_tiles),
        _lib.ptr(tables.kv_entries), ctypes.c_int(tables.kv_entries.shape[0]), _lib.ptr(tables.masks),
        ctypes.c_int(tables.masks.shape[0]), _ptr_array(out_dsts), _ptr_array(lse_dsts),
        ctypes.c_int(len(out_dsts)), ctypes.c_int(lse_stride),
        ctypes.c_int(lse_stride if lse_stride_b is None else lse_stride_b),
        ctypes.c_int(len(out_dsts) if n_dst_a is None else n_dst_a), ctypes.c_int(tables.block_size),
        ctypes.c_float(scale), _lib.ptr(status), ctypes.c_int(variant), _lib.stream_handle())
    _lib.check(rc, "dcpk_attn_fwd")


# ----------------------------------------------------------------------------- reference
def ranges_to_dense(ranges: np.ndarray, n_kv: int) -> torch.Tensor:
    """[n_q, 4] ranges -> bool [n_q, n_kv] mask."""
    r = torch.as_tensor(np.asarray(ranges)).long().reshape(-1, 4)
    pos = torch.arange(n_kv)[None, :]
    return ((pos >= r[:, 0:1]) & (pos < r[:, 1:2])) | ((pos >= r[:, 2:3]) & (pos < r[:, 3:4]))


def attention_reference(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: torch.Tensor, scale: float):
    """fp32 dense masked attention. q [nq, hq, d], k/v [nk, hkv, d], mask bool [nq, nk].

    Returns (out [nq, hq, d] fp32, lse [hq, nq] fp32); fully masked rows give out 0, lse -inf.
    """
    hq, hkv = q.shape[1], k.shape[1]
    g = hq // hkv
    qf = q.float().permute(1, 0, 2)
    kf = k.float().permute(1, 0, 2).repeat_interleave(g, dim=0)
    vf = v.float().permute(1, 0, 2).repeat_interleave(g, dim=0)
    s = torch.einsum("hqd,hkd->hqk", qf, kf) * scale
    s = s.masked_fill(~mask.to(s.device)[None], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)[..., None])
    p = torch.where(torch.isinf(lse)[..., None], torch.zeros_like(p), p)
    out = torch.einsum("hqk,hkd->hqd", p, vf).permute(1, 0, 2)
    return out, lse


# ----------------------------------------------------------------------------- backward
Q_TILE_BWD = 64


@dataclass
class BwdTables:
    ctas: torch.Tensor    # int32 [n_ctas, 8]
    items: torch.Tensor   # int32 [n_items, 8]
    masks: torch.Tensor   # int32 [n_mask_rows, 4]
    n_ctas: int
    n_items: int
    flops: float = 0.0

    def to(self, device, non_blocking: bool = True) -> "BwdTables":
        mv = lambda t: t.to(device, non_blocking=non_blocking)
        return BwdTables(mv(self.ctas), mv(self.items), mv(self.masks), self.n_ctas, self.n_items, self.flops)

    def pin(self) -> "BwdTables":
        return BwdTables(self.ctas.pin_memory(), self.items.pin_memory(), self.masks.pin_memory(), self.n_ctas,
                         self.n_items, self.flops)


def _tile_bounds(rng: np.ndarray, tile: int):
    """Per-tile union / intersection of the two ranges; rows past the end are neutral."""
    n = rng.shape[0]
    n_t = (n + tile - 1) // tile
    pad = n_t * tile - n
    r = rng.astype(np.int64)
    big, small = np.iinfo(np.int32).max, np.iinfo(np.int32).min
    valid = np.concatenate([np.ones(n, bool), np.zeros(pad, bool)])
    r = np.concatenate([r, np.zeros((pad, 4), np.int64)], axis=0)
    e0 = np.maximum(r[:, 1], r[:, 0]); e1 = np.maximum(r[:, 3], r[:, 2])
    has0 = valid & (e0 > r[:, 0]); has1 = valid & (e1 > r[:, 2])
    sh = (n_t, tile)
    u0s = np.where(has0, r[:, 0], big).reshape(sh).min(1); u0e = np.where(has0, e0, small).reshape(sh).max(1)
    u1s = np.where(has1, r[:, 2], big).reshape(sh).min(1); u1e = np.where(has1, e1, small).reshape(sh).max(1)
    i0s = np.where(valid, r[:, 0], small).reshape(sh).max(1); i0e = np.where(valid, e0, big).reshape(sh).min(1)
    i1s = np.where(valid, r[:, 2], small).reshape(sh).max(1); i1e = np.where(valid, e1, big).reshape(sh).min(1)
    return n_t, (u0s, u0e, u1s, u1e, i0s, i0e, i1s, i1e)


def build_bwd_tables(rows: Sequence[AttnRow], block_size: int, hq: int, hkv: int, device) -> BwdTables:
    """Backward kernel tables (see ``build_bwd_tables_py`` for the layout); built by the C++ planner module."""
    native = _native_planner()
    if native is None:
        return build_bwd_tables_py(rows, block_size, hq, hkv, device)
    c_np, i_np, m_np, pairs = native.build_bwd_tables(_row_tuples(rows), int(block_size), int(hq))
    to = lambda a: torch.from_numpy(a).to(device, non_blocking=True)
    return BwdTables(to(c_np), to(i_np), to(m_np), int(c_np.shape[0]), int(i_np.shape[0]), flops=10.0 * pairs * HEAD_DIM)


def build_bwd_tables_py(rows: Sequence[AttnRow], block_size: int, hq: int, hkv: int, device) -> BwdTables:
    """KV-major work lists for the backward kernel: one table entry per key tile (the kernel runs
    it once per KV head) listing the 64-query tiles that see it; heads are not materialised."""
    masks, mask_row = [], 0
    cta_items = {}  # (kv_row, n_valid, dkv_dev, dkv_row) -> list of item arrays
    pairs = 0.0
    for row in rows:
        rng = np.ascontiguousarray(row.ranges, dtype=np.int32).reshape(-1, 4)
        masks.append(rng)
        assert len(row.heads) == hq, "the backward kernel visits every query head of a row"
        pairs += _pair_count(rng) * len(row.heads)
        n_qt, (u0s, u0e, u1s, u1e, i0s, i0e, i1s, i1e) = _tile_bounds(rng, Q_TILE_BWD)
        qt = np.arange(n_qt)
        n_rows_t = np.minimum(Q_TILE_BWD, row.n_tokens - qt * Q_TILE_BWD)
        for e, (kv_row, n_tok) in enumerate(row.kv):
            dkv_dev, dkv_row = row.dkv[e] if row.dkv else (0, kv_row)
            n_sub = (n_tok + TILE_N - 1) // TILE_N
            p0 = e * block_size + np.arange(n_sub) * TILE_N                      # [n_sub]
            nv = np.minimum(TILE_N, n_tok - np.arange(n_sub) * TILE_N)
            lo, hi = p0[:, None], (p0 + nv)[:, None]
            need = ((lo < u0e[None]) & (hi > u0s[None])) | ((lo < u1e[None]) & (hi > u1s[None]))   # [n_sub, n_qt]
            full = (nv[:, None] == TILE_N) & (((i0s[None] <= lo) & (i0e[None] >= hi)) | ((i1s[None] <= lo) & (i1e[None] >= hi)))
            # all (key tile, query tile) pairs of this KV block at once, key-tile major; the per-key-tile
            # item lists are slices of it
            ts, ii = np.nonzero(need)
            if ts.size == 0:
                continue
            arr = np.empty((ts.size, 8), dtype=np.int64)
            arr[:, 0] = row.q_row + ii * Q_TILE_BWD
            arr[:, 1] = n_rows_t[ii]
            arr[:, 2] = p0[ts]
            arr[:, 3] = mask_row + ii * Q_TILE_BWD
            arr[:, 4] = row.dq_dev
            arr[:, 5] = row.dq_row + ii * Q_TILE_BWD
            arr[:, 6] = full[ts, ii]
            arr[:, 7] = 0
            counts = np.bincount(ts, minlength=n_sub)
            ends = np.cumsum(counts)
            for t in np.nonzero(counts)[0].tolist():
                key = (kv_row + t * TILE_N, int(nv[t]), dkv_dev, dkv_row + t * TILE_N)
                cta_items.setdefault(key, []).append(arr[ends[t] - counts[t]:ends[t]])
        mask_row += row.n_tokens
    ctas, item_chunks, off = [], [], 0
    for key, chunks in sorted(cta_items.items(), key=lambda kv: -sum(c.shape[0] for c in kv[1])):
        n = sum(c.shape[0] for c in chunks)
        ctas.append((key[0], key[1], off, n, key[2], key[3], 0, 0))
        item_chunks.extend(chunks)
        off += n
    c_np = np.asarray(ctas, dtype=np.int32).reshape(-1, 8)
    i_np = (np.concatenate(item_chunks, axis=0) if item_chunks else np.zeros((0, 8))).astype(np.int32)
    m_np = np.concatenate(masks, axis=0) if masks else np.zeros((0, 4), np.int32)
    to = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device, non_blocking=True)
    return BwdTables(to(c_np), to(i_np), to(m_np), len(ctas), int(off), flops=10.0 * pairs * HEAD_DIM)


def attn_delta(out_arena: torch.Tensor, dout_arena: torch.Tensor, delta: torch.Tensor, row0: int, n_rows: int):
    """delta[h, row] = sum_d dO*O for rows [row0, row0+n_rows) of bf16 [rows, hq, 128] arenas."""
    lib = _lib.load()
    rc = lib.dcpk_attn_delta(_lib.ptr(out_arena), _lib.ptr(dout_arena), _lib.ptr(delta), ctypes.c_int(n_rows),
                             ctypes.c_int(out_arena.shape[1]), ctypes.c_int(delta.shape[1]), ctypes.c_int(row0),
                             _lib.stream_handle())
    _lib.check(rc, "dcpk_attn_delta")


def attn_bwd(q_arena, do_arena, kv_arena, lse, delta, tables: BwdTables, dq_dsts, dkv_dsts, scale: float,
             status: torch.Tensor, jobs: Optional[torch.Tensor] = None, job_ctx: Optional[CopyContext] = None):
    """Run the backward kernel; dq_dsts/dkv_dsts are fp32 accumulators (zeroed by the caller),
    [rows, hq, 128] and [rows, 2, hkv, 128]; lse/delta are fp32 [hq, rows].  ``jobs`` / ``job_ctx``: copy
    jobs two spare warps per CTA perform meanwhile (the next stage's operands, see attn_fwd)."""
    lib = _lib.load()
    hq, hkv = q_arena.shape[1], kv_arena.shape[2]
    assert q_arena.shape == do_arena.shape and lse.shape == delta.shape
    rc = lib.dcpk_attn_bwd(
        _lib.ptr(q_arena), _lib.ptr(do_arena), ctypes.c_long(q_arena.shape[0]), _lib.ptr(kv_arena),
        ctypes.c_long(kv_arena.shape[0]), ctypes.c_int(hq), ctypes.c_int(hkv), _lib.ptr(tables.ctas),
        ctypes.c_int(tables.n_ctas), _lib.ptr(tables.items), ctypes.c_int(tables.items.shape[0]), _lib.ptr(tables.masks),
        ctypes.c_int(tables.masks.shape[0]), _lib.ptr(lse), _lib.ptr(delta),
        ctypes.c_int(lse.shape[1]), _ptr_array(dq_dsts), _ptr_array(dkv_dsts), ctypes.c_int(len(dq_dsts)),
        ctypes.c_float(scale), *_job_args(jobs, job_ctx), _lib.ptr(status), _lib.stream_handle())
    _lib.check(rc, "dcpk_attn_bwd")


def attention_reference_bwd(q, k, v, mask, scale, dout):
    """fp32 autograd through the dense reference. Returns (out, lse, dq, dk, dv)."""
    qf = q.float().detach().requires_grad_(True)
    kf = k.float().detach().requires_grad_(True)
    vf = v.float().detach().requires_grad_(True)
    out, lse = attention_reference(qf, kf, vf, mask, scale)
    out.backward(dout.float())
    return out.detach(), lse.detach(), qf.grad, kf.grad, vf.grad

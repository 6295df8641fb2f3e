"""CPU emulation of the fused executor: every rank's ``FusedProgram`` run in one process with
plain torch ops, rank by rank and stage by stage, over dictionaries of per-rank arenas.

It follows the table formats the sm_100a kernels consume row for row (forward tiles + KV entry
lists + per-query range rows; backward key-tile CTAs + query-tile items; pull, merge and
gradient-push lists), so it serves two purposes: a readable definition of those formats, and a
way to check the lowering for any world size without that many GPUs (the GPU tests cover the
kernels themselves on one or two devices).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import numpy as np
import torch

from ..planner.lowering import FusedProgram

NEG_INF = float("-inf")


class _Arenas:
    def __init__(self, prog: FusedProgram, head_dim: int, dtype):
        rq, rkv, rp = (int(x) + 128 for x in prog.need_all)
        hq, hkv = prog.heads_q, prog.heads_kv
        z = lambda *s: torch.zeros(*s, dtype=dtype)
        self.q, self.kv = z(rq, hq, head_dim), z(rkv, 2, hkv, head_dim)
        self.out, self.lse = z(rq, hq, head_dim), torch.full((hq, rq), NEG_INF, dtype=dtype)
        self.part_out, self.part_lse = z(rp, hq, head_dim), torch.full((hq, rp), NEG_INF, dtype=dtype)
        self.dout, self.delta = z(rq, hq, head_dim), z(hq, rq)
        self.dq, self.dkv = z(rq, hq, head_dim), z(rkv, 2, hkv, head_dim)


def _allowed(ranges: torch.Tensor, key_pos: torch.Tensor) -> torch.Tensor:
    """ranges [n_q, 4] = (s0, e0, s1, e1), key_pos [n_k] -> bool [n_q, n_k]."""
    p = key_pos[None, :]
    return ((p >= ranges[:, 0:1]) & (p < ranges[:, 1:2])) | ((p >= ranges[:, 2:3]) & (p < ranges[:, 3:4]))


def _pull(pulls: np.ndarray, src_of_rank, dst: torch.Tensor, token_axis: int = 0) -> None:
    for peer, src_row, dst_row, n in pulls.tolist():
        src = src_of_rank(peer)
        if token_axis == 0:
            dst[dst_row:dst_row + n] = src[src_row:src_row + n]
        else:
            dst[:, dst_row:dst_row + n] = src[:, src_row:src_row + n]


def emulate(programs: List[FusedProgram], q_local: List[torch.Tensor], kv_local: List[torch.Tensor],
            dout_local: Optional[List[torch.Tensor]] = None, scale: Optional[float] = None,
            dtype=torch.float64) -> List[Tuple[torch.Tensor, ...]]:
    """Run all ranks' programs.  Inputs are per-rank local tensors (q [n, hq, d], kv [n, 2, hkv, d],
    optional dout [n, hq, d]); returns per rank (out, lse[, dq, dkv]) of its local rows."""
    world = len(programs)
    assert all(p.world == world and p.rank == r for r, p in enumerate(programs))
    d = q_local[0].shape[-1]
    scale = d ** -0.5 if scale is None else scale
    hq, hkv, bs = programs[0].heads_q, programs[0].heads_kv, programs[0].block_size
    g = hq // hkv
    A = [_Arenas(p, d, dtype) for p in programs]
    for r, p in enumerate(programs):
        A[r].q[:p.q_local_rows] = q_local[r].to(dtype)
        A[r].kv[:p.kv_local_rows] = kv_local[r].to(dtype)

    # ---------------------------------------------------------------- forward
    for s in range(programs[0].n_stages):
        for r, p in enumerate(programs):                      # pulls of this stage (owners' local rows only)
            _pull(p.q_pulls[s], lambda peer: A[peer].q, A[r].q)
            _pull(p.kv_pulls[s], lambda peer: A[peer].kv, A[r].kv)
        for r, p in enumerate(programs):
            t = p.fwd[s]
            if t is None:
                continue
            tiles, entries, masks = t.tiles.numpy(), t.kv_entries.numpy(), t.masks
            for q_row, n_rows, head, kv_off, n_kv, mask_row, out_dev, out_row in tiles.tolist():
                if n_rows <= 0:
                    continue
                # 128-row tiles carry (arena row, tokens) per KV block; 256-row tiles carry the ready-made
                # walk (arena row, position, valid keys, flags) and each 128-row half only takes the
                # entries whose flag bit says it can see them
                halves = [(0, n_rows, None)] if t.tile_m == 128 else [(x * 128, min(128, n_rows - x * 128), x)
                                                                       for x in range(2) if n_rows > x * 128]
                for r0, nr, x in halves:
                    rng = masks[mask_row + r0:mask_row + r0 + nr].to(torch.int64)
                    ks, vs, pos = [], [], []
                    for e in range(n_kv):
                        ent = entries[kv_off + e].tolist()
                        if x is None:
                            row, n_tok, p0 = ent[0], ent[1], e * bs
                        else:
                            row, p0, n_tok, flags = ent
                            if not (flags >> x) & 1:
                                continue
                        ks.append(A[r].kv[row:row + n_tok, 0, head // g])
                        vs.append(A[r].kv[row:row + n_tok, 1, head // g])
                        pos.append(torch.arange(p0, p0 + n_tok))
                    if ks:
                        k, v, pos = torch.cat(ks), torch.cat(vs), torch.cat(pos)
                        sc = (A[r].q[q_row + r0:q_row + r0 + nr, head] @ k.T) * scale
                        sc = sc.masked_fill(~_allowed(rng, pos), NEG_INF)
                        lse = torch.logsumexp(sc, dim=-1)
                        prob = torch.exp(sc - torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)[:, None])
                        prob = torch.where(torch.isinf(lse)[:, None], torch.zeros_like(prob), prob)
                        o = prob @ v
                    else:
                        o = torch.zeros(nr, d, dtype=dtype)
                        lse = torch.full((nr,), NEG_INF, dtype=dtype)
                    if out_dev < world:                           # a partial, in the owner's partial arena
                        A[out_dev].part_out[out_row + r0:out_row + r0 + nr, head] = o
                        A[out_dev].part_lse[head, out_row + r0:out_row + r0 + nr] = lse
                    else:                                         # the only contribution: owner's final buffer
                        A[out_dev - world].out[out_row + r0:out_row + r0 + nr, head] = o
                        A[out_dev - world].lse[head, out_row + r0:out_row + r0 + nr] = lse
    for r, p in enumerate(programs):                          # owner-side merge of the partials
        for dst_row, n, off, n_src in p.merge_ops.tolist():
            slots = p.merge_src[off:off + n_src].tolist()
            ls = torch.stack([A[r].part_lse[:, sl:sl + n] for sl in slots])           # [n_src, hq, n]
            os_ = torch.stack([A[r].part_out[sl:sl + n] for sl in slots])              # [n_src, n, hq, d]
            new = torch.logsumexp(ls, dim=0)
            w = torch.exp(ls - torch.where(torch.isinf(new), torch.zeros_like(new), new)[None])
            w = torch.where(torch.isinf(ls), torch.zeros_like(w), w)
            A[r].out[dst_row:dst_row + n] = (os_ * w.permute(0, 2, 1)[..., None]).sum(0)
            A[r].lse[:, dst_row:dst_row + n] = new
    results = [(A[r].out[:p.q_local_rows].clone(), A[r].lse[:, :p.q_local_rows].clone()) for r, p in enumerate(programs)]
    if dout_local is None:
        return results

    # ---------------------------------------------------------------- backward
    for r, p in enumerate(programs):
        n = p.q_local_rows
        A[r].dout[:n] = dout_local[r].to(dtype)
        A[r].delta[:, :n] = (A[r].dout[:n] * A[r].out[:n]).sum(-1).T
    for s in range(programs[0].n_stages):
        for r, p in enumerate(programs):
            _pull(p.q_pulls[s], lambda peer: A[peer].dout, A[r].dout)
            _pull(p.q_pulls[s], lambda peer: A[peer].lse, A[r].lse, token_axis=1)
            _pull(p.q_pulls[s], lambda peer: A[peer].delta, A[r].delta, token_axis=1)
        for r, p in enumerate(programs):
            t = p.bwd[s]
            if t is None:
                continue
            ctas, items, masks = t.ctas.numpy().tolist(), t.items.numpy(), t.masks
            for kv_row, n_valid, item_off, n_items, dkv_dev, dkv_row, _, _ in ctas:
                assert dkv_dev == 0, "gradients accumulate in the rank's own mirror and are pushed afterwards"
                for kvh in range(hkv):
                    k = A[r].kv[kv_row:kv_row + n_valid, 0, kvh]
                    v = A[r].kv[kv_row:kv_row + n_valid, 1, kvh]
                    for q_row, n_rows, kv_pos0, mask_row, dq_dev, dq_row, _full, _ in items[item_off:item_off + n_items].tolist():
                        allow = _allowed(masks[mask_row:mask_row + n_rows].to(torch.int64),
                                         torch.arange(kv_pos0, kv_pos0 + n_valid))
                        for head in range(kvh * g, (kvh + 1) * g):
                            qh = A[r].q[q_row:q_row + n_rows, head]
                            do = A[r].dout[q_row:q_row + n_rows, head]
                            lse = A[r].lse[head, q_row:q_row + n_rows]
                            sc = (qh @ k.T) * scale
                            prob = torch.where(allow & ~torch.isinf(lse)[:, None],
                                               torch.exp(sc - torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)[:, None]),
                                               torch.zeros_like(sc))
                            ds = prob * (do @ v.T - A[r].delta[head, q_row:q_row + n_rows, None]) * scale
                            A[r].dkv[dkv_row:dkv_row + n_valid, 1, kvh] += prob.T @ do
                            A[r].dkv[dkv_row:dkv_row + n_valid, 0, kvh] += ds.T @ qh
                            if dq_dev >= 0:
                                assert dq_dev == 0
                                A[r].dq[dq_row:dq_row + n_rows, head] += ds @ k
    # gradients of staged (remote) blocks go home; snapshot first so a pushed row is never re-pushed
    snap = [(a.dq.clone(), a.dkv.clone()) for a in A]
    for r, p in enumerate(programs):
        for owner, src_row, dst_row, n in p.dq_push.tolist():
            A[owner].dq[dst_row:dst_row + n] += snap[r][0][src_row:src_row + n]
        for owner, src_row, dst_row, n in p.dkv_push.tolist():
            A[owner].dkv[dst_row:dst_row + n] += snap[r][1][src_row:src_row + n]
    return [res + (A[r].dq[:p.q_local_rows].clone(), A[r].dkv[:p.kv_local_rows].clone())
            for r, (res, p) in enumerate(zip(results, programs))]

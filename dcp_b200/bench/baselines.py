"""Comparison baselines for the attention microbenchmark, built only from library pieces (NCCL
collectives through torch.distributed + a library attention kernel).  They are what a "call NCCL
and a stock kernel" implementation looks like on the same box and exist to be beaten:

* ``UlyssesAttention``  - head-parallel all-to-all (DeepSpeed-Ulysses style; TE ``a2a`` in the
  reference's baseline set, benchmark/microbenchmark/baselines/transformer_engine/
  transformer_engine.py:82-92): tokens are split evenly over ranks, an all-to-all regroups them so
  each rank holds all tokens of H/P heads, a varlen causal attention runs locally, a second
  all-to-all restores the token split.  Backward is the mirrored pair of all-to-alls.
* ``RingAttention``     - ring attention, plain or zigzag (ring-flash-attn ``ring`` / ``zigzag``, TE
  ``p2p``): K/V chunks travel around the ring with NCCL point-to-point while the library kernel
  attends to the chunk at hand; partial results are merged by log-sum-exp and in the backward
  dK/dV travel with their chunk.  The ring logic is tested on CPU (gloo) against dense attention.
* double ring            - ``RingAttention(window=w)``: LoongTrain's context ring in which a chunk circles an inner
  ring of ``w`` ranks and changes rings once per ``w`` steps (baselines/loong_train/loong_train.py:111-165).
* ``HierarchicalA2AP2P`` - head all-to-all inside groups of adjacent ranks, zigzag ring across groups (TE
  ``a2a+p2p``).
* ``NcclPlanAttention`` - the DCP instruction plans interpreted with NCCL point-to-point
  exchanges and torch ops (the plan interpreter, see ``runtime/interface.py``).

The local attention uses flash-attn's varlen kernel when it loads on this GPU and falls back to
torch SDPA per sequence otherwise.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist


def _varlen_causal_attention(q, k, v, cu_seqlens: torch.Tensor, max_len: int, scale: float):
    """q [T, h, d], k/v [T, hkv, d] packed sequences -> out [T, h, d] (autograd-capable)."""
    try:
        from flash_attn import flash_attn_varlen_func
        return flash_attn_varlen_func(q, k, v, cu_seqlens, cu_seqlens, max_len, max_len, softmax_scale=scale,
                                      causal=True)
    except Exception:  # library kernel unavailable on this architecture
        outs = []
        g = q.shape[1] // k.shape[1]
        cu = cu_seqlens.tolist()
        for a, b in zip(cu[:-1], cu[1:]):
            qs = q[a:b].transpose(0, 1)[None]
            ks = k[a:b].transpose(0, 1).repeat_interleave(g, dim=0)[None]
            vs = v[a:b].transpose(0, 1).repeat_interleave(g, dim=0)[None]
            o = torch.nn.functional.scaled_dot_product_attention(qs, ks, vs, is_causal=True, scale=scale)
            outs.append(o[0].transpose(0, 1))
        return torch.cat(outs, dim=0)


class _SeqAllToAll(torch.autograd.Function):
    """[T_local, H, d] (all heads, own tokens) <-> [T_total, H/P, d] (own heads, all tokens)."""

    @staticmethod
    def forward(ctx, x, group, to_heads: bool, token_counts: List[int]):
        ctx.group, ctx.to_heads, ctx.counts = group, to_heads, token_counts
        return _a2a(x, group, to_heads, token_counts)

    @staticmethod
    def backward(ctx, g):
        return _a2a(g.contiguous(), ctx.group, not ctx.to_heads, ctx.counts), None, None, None


def _a2a(x: torch.Tensor, group, to_heads: bool, counts: List[int]) -> torch.Tensor:
    P = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if to_heads:
        T, H = x.shape[0], x.shape[1]
        hp = H // P
        send = x.reshape(T, P, hp, *x.shape[2:]).transpose(0, 1).contiguous()     # [P, T, hp, ...]
        recv = x.new_empty((sum(counts), hp) + tuple(x.shape[2:]))
        in_splits = [T * 1] * P
        dist.all_to_all_single(recv.view(-1, *recv.shape[1:]), send.view(P * T, *send.shape[2:]),
                               output_split_sizes=counts, input_split_sizes=in_splits, group=group)
        return recv
    Ttot, hp = x.shape[0], x.shape[1]
    Tl = counts[rank]
    recv = x.new_empty((P, Tl, hp) + tuple(x.shape[2:]))
    dist.all_to_all_single(recv.view(P * Tl, *recv.shape[2:]), x, output_split_sizes=[Tl] * P,
                           input_split_sizes=counts, group=group)
    return recv.transpose(0, 1).reshape(Tl, P * hp, *x.shape[2:])


class UlyssesAttention:
    def __init__(self, group, seqlens: Sequence[int], n_heads: int, n_kv_heads: int, head_dim: int = 128):
        self.group = group
        self.P, self.rank = dist.get_world_size(group), dist.get_rank(group)
        assert n_heads % self.P == 0 and n_kv_heads % self.P == 0, "heads must divide over ranks"
        total = int(sum(seqlens))
        per = -(-total // self.P)
        self.counts = [max(0, min(per, total - r * per)) for r in range(self.P)]
        self.cu = torch.tensor([0] + list(torch.tensor(list(seqlens)).cumsum(0)), dtype=torch.int32)
        self.max_len = int(max(seqlens))
        self.scale = head_dim ** -0.5

    def local_slice(self, global_t: torch.Tensor) -> torch.Tensor:
        off = sum(self.counts[:self.rank])
        return global_t[off:off + self.counts[self.rank]]

    def __call__(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        """q [T_local, H, d], k/v [T_local, Hkv, d] (this rank's contiguous token slice)."""
        qh = _SeqAllToAll.apply(q, self.group, True, self.counts)
        kh = _SeqAllToAll.apply(k, self.group, True, self.counts)
        vh = _SeqAllToAll.apply(v, self.group, True, self.counts)
        out = _varlen_causal_attention(qh, kh, vh, self.cu.to(q.device), self.max_len, self.scale)
        return _SeqAllToAll.apply(out, self.group, False, self.counts)


# ------------------------------------------------------------------------------------------ ring
# Ring attention (ring-flash-attn `ring` / `zigzag`, TE `p2p` in the reference's baseline set:
# benchmark/microbenchmark/baselines/ring_flash_attn/ring_flash_attn.py:13-62).  K/V travel around
# the ring with NCCL point-to-point while a library kernel attends to the chunk at hand; partial
# results are merged by log-sum-exp; in the backward dK/dV travel with their chunk.

def _dense_block_fwd(q, k, v, cu_q, cu_k, scale, causal):
    """Packed-sequence attention in plain torch: -> (out [Tq, h, d], lse [h, Tq] fp32)."""
    g = q.shape[1] // k.shape[1]
    out = torch.empty_like(q)
    lse = torch.empty(q.shape[1], q.shape[0], dtype=torch.float32, device=q.device)
    for (a, b), (c, d_) in zip(zip(cu_q[:-1], cu_q[1:]), zip(cu_k[:-1], cu_k[1:])):
        qs = q[a:b].float().transpose(0, 1)
        ks = k[c:d_].float().transpose(0, 1).repeat_interleave(g, dim=0)
        vs = v[c:d_].float().transpose(0, 1).repeat_interleave(g, dim=0)
        s = (qs @ ks.transpose(1, 2)) * scale
        if causal:   # bottom-right aligned, as the library kernel does for unequal lengths
            nq, nk = b - a, d_ - c
            keep = torch.ones(nq, nk, dtype=torch.bool, device=q.device).tril(nk - nq)
            s = s.masked_fill(~keep, float("-inf"))
        l = torch.logsumexp(s, dim=-1)
        out[a:b] = (torch.exp(s - l[..., None]) @ vs).transpose(0, 1).to(q.dtype)
        lse[:, a:b] = l
    return out, lse


def _dense_block_bwd(dout, q, k, v, out, lse, cu_q, cu_k, scale, causal):
    g = q.shape[1] // k.shape[1]
    dq = torch.zeros_like(q, dtype=torch.float32)
    dk = torch.zeros_like(k, dtype=torch.float32)
    dv = torch.zeros_like(v, dtype=torch.float32)
    for (a, b), (c, d_) in zip(zip(cu_q[:-1], cu_q[1:]), zip(cu_k[:-1], cu_k[1:])):
        qs = q[a:b].float().transpose(0, 1)
        ks = k[c:d_].float().transpose(0, 1).repeat_interleave(g, dim=0)
        vs = v[c:d_].float().transpose(0, 1).repeat_interleave(g, dim=0)
        s = (qs @ ks.transpose(1, 2)) * scale
        if causal:
            nq, nk = b - a, d_ - c
            keep = torch.ones(nq, nk, dtype=torch.bool, device=q.device).tril(nk - nq)
            s = s.masked_fill(~keep, float("-inf"))
        p = torch.exp(s - lse[:, a:b, None])           # probabilities w.r.t. the GLOBAL normaliser
        do = dout[a:b].float().transpose(0, 1)
        delta = (do * out[a:b].float().transpose(0, 1)).sum(-1, keepdim=True)
        ds = p * (do @ vs.transpose(1, 2) - delta) * scale
        dq[a:b] = (ds @ ks).transpose(0, 1)
        hk = k.shape[1]
        dk[c:d_] = (ds.transpose(1, 2) @ qs).view(hk, g, d_ - c, -1).sum(1).transpose(0, 1)
        dv[c:d_] = (p.transpose(1, 2) @ do).view(hk, g, d_ - c, -1).sum(1).transpose(0, 1)
    return dq, dk, dv


def _block_fwd(q, k, v, cu_q, cu_k, scale, causal):
    if q.is_cuda:
        from flash_attn.flash_attn_interface import _flash_attn_varlen_forward
        tq = torch.tensor(cu_q, dtype=torch.int32, device=q.device)
        tk = torch.tensor(cu_k, dtype=torch.int32, device=q.device)
        mq = max(b - a for a, b in zip(cu_q[:-1], cu_q[1:]))
        mk = max(b - a for a, b in zip(cu_k[:-1], cu_k[1:]))
        out, lse, _, _ = _flash_attn_varlen_forward(q, k, v, tq, tk, mq, mk, 0.0, scale, causal)
        return out, lse.float()
    return _dense_block_fwd(q, k, v, cu_q, cu_k, scale, causal)


def _block_bwd(dout, q, k, v, out, lse, cu_q, cu_k, scale, causal):
    if q.is_cuda:
        from flash_attn.flash_attn_interface import _flash_attn_varlen_backward
        tq = torch.tensor(cu_q, dtype=torch.int32, device=q.device)
        tk = torch.tensor(cu_k, dtype=torch.int32, device=q.device)
        mq = max(b - a for a, b in zip(cu_q[:-1], cu_q[1:]))
        mk = max(b - a for a, b in zip(cu_k[:-1], cu_k[1:]))
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        _flash_attn_varlen_backward(dout, q, k, v, out, lse.contiguous(), dq, dk, dv, tq, tk, mq, mk, 0.0, scale, causal,
                                    -1, -1, 0.0, None, False)
        return dq.float(), dk.float(), dv.float()
    return _dense_block_bwd(dout, q, k, v, out, lse, cu_q, cu_k, scale, causal)


def _merge(out, lse, o2, l2, rows=None):
    """Fold the partial (o2, l2) into (out fp32, lse) for ``rows`` (index tensor) or all rows."""
    if rows is None:
        new = torch.logaddexp(lse, l2)
        out.mul_(torch.exp(lse - new).transpose(0, 1)[..., None]).add_(o2.float() * torch.exp(l2 - new).transpose(0, 1)[..., None])
        lse.copy_(new)
    else:
        new = torch.logaddexp(lse[:, rows], l2)
        out[rows] = out[rows] * torch.exp(lse[:, rows] - new).transpose(0, 1)[..., None] + \
            o2.float() * torch.exp(l2 - new).transpose(0, 1)[..., None]
        lse[:, rows] = new


def _ring_exchange(tensors, group, send_to=None, recv_from=None):
    """Send ``tensors`` to group rank ``send_to`` (default: the next rank of the ring) and receive the
    same shapes from ``recv_from`` (default: the previous rank)."""
    P, rank = dist.get_world_size(group), dist.get_rank(group)
    send_to = (rank + 1) % P if send_to is None else send_to
    recv_from = (rank - 1) % P if recv_from is None else recv_from
    nxt, prv = dist.get_global_rank(group, send_to), dist.get_global_rank(group, recv_from)
    recv = [torch.empty_like(t) for t in tensors]
    ops = [dist.P2POp(dist.isend, t.contiguous(), nxt, group) for t in tensors] + \
          [dist.P2POp(dist.irecv, r, prv, group) for r in recv]
    for w in dist.batch_isend_irecv(ops):
        w.wait()
    return recv


class _RingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, ring):
        P, r = ring.P, ring.rank
        out = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        lse = torch.full((q.shape[1], q.shape[0]), float("-inf"), dtype=torch.float32, device=q.device)
        kc, vc = k, v
        sched = ring.schedule()
        for step in range(P):
            src, send_to, recv_from = sched[step]
            for rows, cu_q, cols, cu_k, causal in ring.step_plan(step, src):
                qs = q if rows is None else q[rows]
                ks, vs = (kc, vc) if cols is None else (kc[cols], vc[cols])
                o2, l2 = _block_fwd(qs, ks, vs, cu_q, cu_k, ring.scale, causal)
                _merge(out, lse, o2, l2, rows)
            if step + 1 < P:
                kc, vc = _ring_exchange([kc, vc], ring.group, send_to, recv_from)
        res = out.to(q.dtype)
        ctx.ring = ring
        ctx.save_for_backward(q, k, v, res, lse)
        return res

    @staticmethod
    def backward(ctx, dout):
        ring = ctx.ring
        q, k, v, out, lse = ctx.saved_tensors
        P, r = ring.P, ring.rank
        dout = dout.contiguous()
        dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        kc, vc = k, v
        dkc = torch.zeros(k.shape, dtype=torch.float32, device=q.device)
        dvc = torch.zeros_like(dkc)
        sched = ring.schedule()
        for step in range(P):
            src, send_to, recv_from = sched[step]
            for rows, cu_q, cols, cu_k, causal in ring.step_plan(step, src):
                sel = (lambda t: t) if rows is None else (lambda t: t[rows])
                ks, vs = (kc, vc) if cols is None else (kc[cols], vc[cols])
                l_rows = lse if rows is None else lse[:, rows].contiguous()
                gq, gk, gv = _block_bwd(sel(dout), sel(q), ks, vs, sel(out), l_rows, cu_q, cu_k, ring.scale, causal)
                if rows is None:
                    dq += gq
                else:
                    dq[rows] += gq
                if cols is None:
                    dkc += gk; dvc += gv
                else:
                    dkc[cols] += gk; dvc[cols] += gv
            # the chunk and its gradient move on together; after P hops the gradient is home
            if step + 1 < P:
                kc, vc, dkc, dvc = _ring_exchange([kc, vc, dkc, dvc], ring.group, send_to, recv_from)
            else:
                dkc, dvc = _ring_exchange([dkc, dvc], ring.group, send_to, recv_from)
        return dq.to(q.dtype), dkc.to(k.dtype), dvc.to(v.dtype), None


class RingAttention:
    """Causal ring attention over packed sequences, plain (rank r holds the r-th contiguous chunk
    of every sequence) or zigzag (rank r holds chunks r and 2P-1-r, which evens out the causal
    work).  Sequence lengths must be multiples of 2P (``adjust_seqlens``)."""

    def __init__(self, group, seqlens: Sequence[int], head_dim: int = 128, zigzag: bool = True, window: int = 0):
        """``window`` > 0 turns the ring into a double ring (LoongTrain's 2D-attention context ring,
        benchmark/microbenchmark/baselines/loong_train/loong_train.py:111-165): the ranks form
        P / window inner rings of ``window`` ranks; a K/V chunk circles its inner ring and hops to
        the next inner ring every ``window`` steps, so only one step in ``window`` crosses rings."""
        self.group, self.zigzag = group, zigzag
        self.P, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.window = window if 0 < window < self.P else self.P
        assert self.P % self.window == 0, "the double-ring window must divide the ring size"
        assert all(n % (2 * self.P) == 0 for n in seqlens), "lengths must be multiples of 2 x ranks"
        self.seqlens = [int(n) for n in seqlens]
        self.scale = head_dim ** -0.5
        self.local = [n // self.P for n in self.seqlens]              # local tokens per sequence
        self.cu = [0]
        for n in self.local:
            self.cu.append(self.cu[-1] + n)
        half = [n // 2 for n in self.local]
        self.cu_half = [0]
        for n in half:
            self.cu_half.append(self.cu_half[-1] + n)
        first, second = [], []
        for off, h in zip(self.cu[:-1], half):
            first.append(torch.arange(off, off + h))
            second.append(torch.arange(off + h, off + 2 * h))
        self._first, self._second = torch.cat(first), torch.cat(second)

    @staticmethod
    def adjust_seqlens(seqlens: Sequence[int], world: int) -> List[int]:
        m = 2 * world
        return [max(m, (int(n) // m) * m) for n in seqlens]

    def local_indices(self) -> torch.Tensor:
        """Global token indices (into the packed batch) of this rank's tokens, in local order."""
        idx, off = [], 0
        for n in self.seqlens:
            if self.zigzag:
                c = n // (2 * self.P)
                idx += [torch.arange(off + self.rank * c, off + (self.rank + 1) * c),
                        torch.arange(off + (2 * self.P - 1 - self.rank) * c, off + (2 * self.P - self.rank) * c)]
            else:
                c = n // self.P
                idx.append(torch.arange(off + self.rank * c, off + (self.rank + 1) * c))
            off += n
        return torch.cat(idx)

    def schedule(self):
        """Per step (rank whose chunk is attended to, rank the chunk goes to afterwards, rank the next
        chunk comes from).  With one inner ring this is the plain ring: chunk of rank r - step, pass
        to r + 1.  In a double ring the rank is (outer o, inner i) = divmod(r, window); step
        oo * window + ii looks at the chunk of (o - oo, i - ii); hops stay in the inner ring except
        after the last inner step, when the chunk moves to the next inner ring (and one place on)."""
        w, n_outer = self.window, self.P // self.window
        o, i = divmod(self.rank, w)
        out = []
        for step in range(self.P):
            oo, ii = divmod(step, w)
            src = ((o - oo) % n_outer) * w + (i - ii) % w
            if ii != w - 1:
                hop = (o * w + (i + 1) % w, o * w + (i - 1) % w)
            else:
                hop = (((o + 1) % n_outer) * w + (i + 1) % w, ((o - 1) % n_outer) * w + (i - 1) % w)
            out.append((src, hop[0], hop[1]))
        return out

    def step_plan(self, step: int, src: int):
        """Attention calls of one ring step, as (query rows or None = all, cu_q, key rows or None,
        cu_k, causal)."""
        dev_rows = lambda t: t
        if src == self.rank:
            if not self.zigzag:
                return [(None, self.cu, None, self.cu, True)]
            # local chunks (r, 2P-1-r): the early chunk attends causally to itself; the late chunk
            # attends fully to the early one and causally to itself = one bottom-right-aligned call
            return [(self._first, self.cu_half, self._first, self.cu_half, True),
                    (self._second, self.cu_half, None, self.cu, True)]
        if not self.zigzag:
            return [(None, self.cu, None, self.cu, False)] if src < self.rank else []
        if src < self.rank:
            # keys from an earlier rank: only its early chunk lies in the past of both local chunks
            return [(None, self.cu, self._first, self.cu_half, False)]
        # keys from a later rank: both of its chunks lie in the past of the local late chunk only
        return [(self._second, self.cu_half, None, self.cu, False)]

    def __call__(self, q, k, v):
        if self._first.device != q.device:
            self._first, self._second = self._first.to(q.device), self._second.to(q.device)
        return _RingFn.apply(q, k, v, self)


class HierarchicalA2AP2P:
    """Head-parallel all-to-all inside groups of ``a2a_size`` adjacent ranks, zigzag ring (NCCL
    point-to-point) across the groups: TransformerEngine's hierarchical ``a2a+p2p`` context
    parallelism, the strongest library baseline of the reference's figures
    (benchmark/microbenchmark/baselines/transformer_engine/transformer_engine.py:82-92,
    benchmark/mlm/run_experiments.py:571-583).  Rank r = ring index * a2a_size + a2a index.  Ring
    member g owns the zigzag chunks g and 2R-1-g of every sequence; the a2a ranks of a member hold
    equal contiguous slices of that member's token stream and trade them for all its tokens of
    H / a2a_size heads, on which the ring attention runs."""

    def __init__(self, group, seqlens: Sequence[int], n_heads: int, n_kv_heads: int, a2a_size: int, head_dim: int = 128):
        P, rank = dist.get_world_size(group), dist.get_rank(group)
        assert P % a2a_size == 0 and n_heads % a2a_size == 0 and n_kv_heads % a2a_size == 0
        self.A, self.R = a2a_size, P // a2a_size
        self.g, self.a = divmod(rank, a2a_size)
        ranks = [dist.get_global_rank(group, r) for r in range(P)] if group is not dist.group.WORLD else list(range(P))
        # every rank creates every sub-group, in the same order (new_group is collective)
        self.a2a_group = self.ring_group = None
        for g in range(self.R):
            grp = dist.new_group([ranks[g * a2a_size + a] for a in range(a2a_size)])
            if g == self.g:
                self.a2a_group = grp
        for a in range(a2a_size):
            grp = dist.new_group([ranks[g * a2a_size + a] for g in range(self.R)])
            if a == self.a:
                self.ring_group = grp
        self.ring = RingAttention(self.ring_group, seqlens, head_dim=head_dim, zigzag=True)
        t_member = self.ring.cu[-1]                          # tokens of one ring member
        assert t_member % a2a_size == 0, "the member's token stream must split evenly over the a2a ranks"
        self.counts = [t_member // a2a_size] * a2a_size
        self.n_local = t_member // a2a_size

    @staticmethod
    def adjust_seqlens(seqlens: Sequence[int], world: int, a2a_size: int) -> List[int]:
        m = 2 * world                                         # 2 x ring x a2a: every rank slice stays whole
        return [max(m, (int(n) // m) * m) for n in seqlens]

    def local_indices(self) -> torch.Tensor:
        """Global token indices of this rank's tokens (its slice of its ring member's stream)."""
        member = self.ring.local_indices()
        return member[self.a * self.n_local:(self.a + 1) * self.n_local]

    def __call__(self, q, k, v):
        qh = _SeqAllToAll.apply(q, self.a2a_group, True, self.counts)
        kh = _SeqAllToAll.apply(k, self.a2a_group, True, self.counts)
        vh = _SeqAllToAll.apply(v, self.a2a_group, True, self.counts)
        out = self.ring(qh, kh, vh)
        return _SeqAllToAll.apply(out, self.a2a_group, False, self.counts)


def make_baseline(framework: str, group, seqlens: Sequence[int], n_heads: int, n_kv_heads: int, rank: int, world: int,
                  window: Optional[int] = None, a2a: Optional[int] = None):
    """-> (attention callable (q, k, v) -> out, number of local tokens) for a baseline framework.
    ``window``: ranks per inner ring of the double ring; ``a2a``: ranks per head all-to-all group of
    a2a+p2p (defaults: 2, and the largest power of two the KV heads and the world size allow)."""
    if framework == "ulysses":
        ua = UlyssesAttention(group, seqlens, n_heads, n_kv_heads)
        return ua, ua.counts[rank]
    if framework in ("ring", "zigzag"):
        assert group is not None, "ring attention needs at least two ranks"
        # lengths are rounded down to multiples of 2 x ranks (at most 2P - 1 tokens per sequence)
        ra = RingAttention(group, RingAttention.adjust_seqlens(seqlens, world), zigzag=framework == "zigzag")
        return ra, ra.cu[-1]
    if framework == "double-ring":
        assert group is not None, "ring attention needs at least two ranks"
        if window is None:
            window = 2 if world % 2 == 0 and world > 2 else world   # inner rings of two ranks (four rings on 8 GPUs)
        assert world % window == 0, "the inner ring size must divide the number of ranks"
        ra = RingAttention(group, RingAttention.adjust_seqlens(seqlens, world), zigzag=True, window=window)
        return ra, ra.cu[-1]
    if framework == "a2a+p2p":
        assert group is not None, "needs at least two ranks"
        if a2a is None:
            a2a = 2 if world % 2 == 0 else 1
            while a2a * 2 <= min(n_kv_heads, 4) and world % (a2a * 2) == 0 and world // (a2a * 2) >= 2:
                a2a *= 2                                             # 4 x 2 on 8 GPUs, 2 x 2 on 4
        assert world % a2a == 0 and n_kv_heads % a2a == 0, "the all-to-all group must divide ranks and KV heads"
        ha = HierarchicalA2AP2P(group, HierarchicalA2AP2P.adjust_seqlens(seqlens, world, a2a), n_heads, n_kv_heads, a2a)
        return ha, ha.n_local
    raise ValueError(f"unknown baseline framework {framework!r}")

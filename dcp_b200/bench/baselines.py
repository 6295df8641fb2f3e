"""Comparison baselines for the attention microbenchmark, built only from library pieces (NCCL
collectives through torch.distributed + a library attention kernel).  They are what a "call NCCL
and a stock kernel" implementation looks like on the same box and exist to be beaten:

* ``UlyssesAttention``  - head-parallel all-to-all (DeepSpeed-Ulysses style; TE ``a2a`` in the
  reference's baseline set, benchmark/microbenchmark/baselines/transformer_engine/
  transformer_engine.py:82-92): tokens are split evenly over ranks, an all-to-all regroups them so
  each rank holds all tokens of H/P heads, a varlen causal attention runs locally, a second
  all-to-all restores the token split.  Backward is the mirrored pair of all-to-alls.
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

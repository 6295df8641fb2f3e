"""Plain-PyTorch fp32 evaluation of the Llama-architecture model on a packed batch: dense causal
attention per sequence, no custom kernels.  Used as the numerical reference of the training path."""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch
import torch.nn.functional as F

from ..ops import model_ops
from .llama import LlamaConfig


def reference_embed(p: Dict[str, torch.Tensor], tokens: torch.Tensor) -> torch.Tensor:
    return F.embedding(tokens, p["embed"])


def sequence_masks(seqlens: Sequence[int], attn_mask=None, padded_seqlens: Optional[Sequence[int]] = None, device=None):
    """Per sequence the boolean [n, n] matrix of allowed (query, key) pairs: causal, or from a range
    mask of the mask library (int32 [2, T_padded] / [2, 2, T_padded] per-query key intervals relative
    to the sequence start, laid out over the padded sequences)."""
    if attn_mask is None:
        return [torch.ones(n, n, dtype=torch.bool, device=device).tril() for n in seqlens]
    from ..runtime.layout import seq_token_offsets
    from ..runtime.simulate import to_two_range
    rng, pcu, out = to_two_range(attn_mask), seq_token_offsets(padded_seqlens), []
    for s, n in enumerate(seqlens):
        r = torch.from_numpy(rng[pcu[s]:pcu[s] + n]).to(device)
        pos = torch.arange(n, device=device)[None, :]
        out.append(((pos >= r[:, 0, 0:1]) & (pos < r[:, 0, 1:2])) | ((pos >= r[:, 1, 0:1]) & (pos < r[:, 1, 1:2])))
    return out


def reference_layers(cfg: LlamaConfig, p: Dict[str, torch.Tensor], x: torch.Tensor, positions: torch.Tensor,
                     seqlens: Sequence[int], first: int, last: int, allow=None) -> torch.Tensor:
    """Decoder layers ``first`` .. ``last - 1`` on the packed hidden states ``x`` (dense attention per
    sequence; ``allow``: per-sequence boolean masks from ``sequence_masks``, default causal).  The unit
    a pipeline stage owns."""
    if allow is None:
        allow = sequence_masks(seqlens, device=x.device)
    cos, sin = model_ops.rope_tables(positions, cfg.rope_theta, cfg.head_dim)
    hq, hkv, d = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
    g = hq // hkv
    norm = lambda t, w: t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + cfg.eps) * w
    for l in range(first, last):
        h = norm(x, p[f"l{l}.norm1"])
        qkv = F.linear(h, p[f"l{l}.wqkv"]).view(-1, hq + 2 * hkv, d)
        q = model_ops.rope_reference(qkv[:, :hq], cos, sin)
        k = model_ops.rope_reference(qkv[:, hq:hq + hkv], cos, sin)
        v = qkv[:, hq + hkv:]
        outs, off = [], 0
        for si, n in enumerate(seqlens):
            qs = q[off:off + n].transpose(0, 1)
            ks = k[off:off + n].transpose(0, 1).repeat_interleave(g, dim=0)
            vs = v[off:off + n].transpose(0, 1).repeat_interleave(g, dim=0)
            s = (qs @ ks.transpose(1, 2)) * d ** -0.5
            s = s.masked_fill(~allow[si], float("-inf"))
            # a query that may see no key at all gets a zero row (softmax of an all -inf row is undefined)
            prob = torch.where(allow[si].any(-1, keepdim=True), torch.softmax(s, -1), torch.zeros_like(s))
            outs.append((prob @ vs).transpose(0, 1).reshape(n, hq * d))
            off += n
        x = x + F.linear(torch.cat(outs), p[f"l{l}.wo"])
        h = norm(x, p[f"l{l}.norm2"])
        gate, up = F.linear(h, p[f"l{l}.wgu"]).chunk(2, dim=-1)
        x = x + F.linear(F.silu(gate) * up, p[f"l{l}.wd"])
    return x


def reference_head_loss(cfg: LlamaConfig, p: Dict[str, torch.Tensor], x: torch.Tensor, labels: torch.Tensor,
                        grad_scale: float) -> torch.Tensor:
    h = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.eps) * p["norm_f"]
    logits = F.linear(h, p["lm_head"])
    loss = F.cross_entropy(logits, labels.clamp(min=0), reduction="none")
    return torch.where(labels >= 0, loss, torch.zeros_like(loss)).sum() * grad_scale


def stage_layer_range(n_layers: int, stage: int, n_stages: int) -> range:
    """Consecutive layers of pipeline stage ``stage`` (earlier stages take the remainder)."""
    per, extra = divmod(n_layers, n_stages)
    first = stage * per + min(stage, extra)
    return range(first, first + per + (1 if stage < extra else 0))


def reference_loss(cfg: LlamaConfig, p: Dict[str, torch.Tensor], tokens: torch.Tensor, labels: torch.Tensor,
                   positions: torch.Tensor, seqlens: Sequence[int], grad_scale: float, allow=None) -> torch.Tensor:
    """Tokens are packed sequence after sequence; returns sum(token losses) * grad_scale."""
    x = reference_layers(cfg, p, reference_embed(p, tokens), positions, seqlens, 0, cfg.n_layers, allow)
    return reference_head_loss(cfg, p, x, labels, grad_scale)

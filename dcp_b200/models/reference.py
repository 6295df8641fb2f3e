"""Plain-PyTorch fp32 evaluation of the Llama-architecture model on a packed batch: dense causal
attention per sequence, no custom kernels.  Used as the numerical reference of the training path."""
from __future__ import annotations

from typing import Dict, Sequence

import torch
import torch.nn.functional as F

from ..ops import model_ops
from .llama import LlamaConfig


def reference_embed(p: Dict[str, torch.Tensor], tokens: torch.Tensor) -> torch.Tensor:
    return F.embedding(tokens, p["embed"])


def reference_layers(cfg: LlamaConfig, p: Dict[str, torch.Tensor], x: torch.Tensor, positions: torch.Tensor,
                     seqlens: Sequence[int], first: int, last: int) -> torch.Tensor:
    """Decoder layers ``first`` .. ``last - 1`` on the packed hidden states ``x`` (dense causal attention
    per sequence).  The unit a pipeline stage owns."""
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
        for n in seqlens:
            qs = q[off:off + n].transpose(0, 1)
            ks = k[off:off + n].transpose(0, 1).repeat_interleave(g, dim=0)
            vs = v[off:off + n].transpose(0, 1).repeat_interleave(g, dim=0)
            s = (qs @ ks.transpose(1, 2)) * d ** -0.5
            s = s.masked_fill(~torch.ones(n, n, dtype=torch.bool, device=s.device).tril(), float("-inf"))
            outs.append((torch.softmax(s, -1) @ vs).transpose(0, 1).reshape(n, hq * d))
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
                   positions: torch.Tensor, seqlens: Sequence[int], grad_scale: float) -> torch.Tensor:
    """Tokens are packed sequence after sequence; returns sum(token losses) * grad_scale."""
    x = reference_layers(cfg, p, reference_embed(p, tokens), positions, seqlens, 0, cfg.n_layers)
    return reference_head_loss(cfg, p, x, labels, grad_scale)

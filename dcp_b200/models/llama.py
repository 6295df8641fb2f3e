"""Llama-3-architecture decoder trained with dynamic context parallelism.

Each rank holds the full model (bf16) and the tokens the planner placed on it.  Inside a layer,
everything except attention is token-local: RMSNorm / SwiGLU / cross-entropy are the hand-written
sm_100a kernels, the dense projections are cuBLAS GEMMs, and attention goes through an executor
(fused sm_100a or plan interpreter) that moves blocks between ranks.  The projection output is
split, rotated and written straight into the executor's arenas by one kernel, and the fp32
gradient accumulators are rotated back and packed by one kernel, so no separate copy, cast or
RoPE pass exists.

Parameters and gradients live in two flat bf16 buffers (symmetric memory when world > 1) so the
data-parallel reduce-scatter / sharded AdamW / parameter all-gather can be single kernels over
peer memory (``dcp_b200.parallel.dist_optimizer``).

The reference trains the same architecture through Megatron-LM (benchmark/mlm/pretrain_gpt.py:191-302,
benchmark/mlm/monkey_patch.py:48-289, model sizes benchmark/mlm/run_experiments.py:25-32).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from ..ops import model_ops


@dataclass
class LlamaConfig:
    n_layers: int = 32
    hidden: int = 4096
    n_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 14336
    vocab: int = 128256
    rope_theta: float = 500000.0
    eps: float = 1e-5
    init_std: float = 0.02

    @property
    def qkv_dim(self) -> int:
        return (self.n_heads + 2 * self.n_kv_heads) * self.head_dim

    def n_params(self) -> int:
        per_layer = self.hidden * self.qkv_dim + self.n_heads * self.head_dim * self.hidden + \
            self.hidden * 2 * self.ffn + self.ffn * self.hidden + 2 * self.hidden
        return 2 * self.vocab * self.hidden + self.n_layers * per_layer + self.hidden


LLAMA3_8B = LlamaConfig()


def tiny_config(n_layers: int = 2, hidden: int = 1024, n_heads: int = 8, n_kv_heads: int = 2, ffn: int = 2048,
                vocab: int = 4096) -> LlamaConfig:
    return LlamaConfig(n_layers, hidden, n_heads, n_kv_heads, 128, ffn, vocab)


class _AttentionFn(torch.autograd.Function):
    """qkv [T, (hq+2hkv)*128] -> attention output [T, hq*128] through the executor's arenas."""

    @staticmethod
    def forward(ctx, qkv, model, cos, sin, layer):
        ex = model.executor
        cfg = model.cfg
        model_ops.qkv_rope_split(qkv, cos, sin, ex.q, ex.kv, cfg.n_heads, cfg.n_kv_heads)
        ex.inputs_written()
        stash = model._attn_stash.pop(layer, None) if model._stash_enabled else None
        if stash is not None:
            # activation recompute: the attention result of this layer was kept from the first
            # forward, so only the operands are put back (the backward needs them in the arenas)
            result, lse_c = stash
            ex.out_local().copy_(result.view(-1, cfg.n_heads, cfg.head_dim))
            ex.lse_local().copy_(lse_c)
        else:
            out, lse = ex.forward()
            result = out.reshape(out.shape[0], -1).clone()
            lse_c = lse.clone()
            if model._stash_enabled:
                model._attn_stash[layer] = (result, lse_c)
        ctx.model, ctx.epoch = model, ex.arena_epoch
        ctx.save_for_backward(qkv, cos, sin, result, lse_c)
        return result

    @staticmethod
    def backward(ctx, dout):
        model = ctx.model
        ex, cfg = model.executor, model.cfg
        qkv, cos, sin, out, lse = ctx.saved_tensors
        if ex.arena_epoch != ctx.epoch:
            # another layer used the arenas since this forward ran: put this layer's operands back
            model_ops.qkv_rope_split(qkv, cos, sin, ex.q, ex.kv, cfg.n_heads, cfg.n_kv_heads)
            ex.inputs_written()
            ex.out_local().copy_(out.view(-1, cfg.n_heads, cfg.head_dim))
            ex.lse_local().copy_(lse)
        dq, dkv = ex.backward(dout.contiguous().view(-1, cfg.n_heads, cfg.head_dim))
        dqkv = model_ops.qkv_rope_pack_bwd(dq, dkv, cos, sin, qkv.shape[0], cfg.n_heads, cfg.n_kv_heads)
        return dqkv, None, None, None, None


class _LMHeadLossFn(torch.autograd.Function):
    """Chunked LM head + cross entropy: logits never exist for more than ``chunk`` tokens, and
    the gradients of the hidden states and of the head weight are formed in the same pass."""

    @staticmethod
    def forward(ctx, h, weight, labels, grad_scale, chunk):
        T = h.shape[0]
        dh = torch.empty_like(h)
        dweight = torch.zeros_like(weight)
        total = torch.zeros((), dtype=torch.float32, device=h.device)
        for t0 in range(0, T, chunk):
            hc = h[t0:t0 + chunk]
            logits = hc @ weight.t()
            loss = model_ops.cross_entropy_inplace(logits, labels[t0:t0 + chunk], grad_scale)
            total += loss.sum()
            dh[t0:t0 + chunk] = logits @ weight
            dweight.addmm_(logits.t(), hc)
        ctx.save_for_backward(dh, dweight)
        return total * grad_scale

    @staticmethod
    def backward(ctx, g):
        dh, dweight = ctx.saved_tensors
        # g is the upstream gradient of the (already scaled) loss; it is 1 in the training loop
        return dh * g, dweight * g, None, None, None


class LlamaModel:
    """Functional model over flat parameter / gradient buffers."""

    def __init__(self, cfg: LlamaConfig, device: torch.device, params_flat: Optional[torch.Tensor] = None,
                 grads_flat: Optional[torch.Tensor] = None, seed: int = 0, recompute: bool = True,
                 lm_head_chunk: int = 4096):
        self.cfg, self.device = cfg, device
        self.recompute = recompute
        self.lm_head_chunk = lm_head_chunk
        self.executor = None
        # keep each layer's attention output across the checkpoint boundary so the recompute pass
        # does not run attention (and its communication) a second time
        self.cache_attention = True
        self._attn_stash: Dict[int, tuple] = {}
        self._stash_enabled = False
        shapes: List[Tuple[str, Tuple[int, ...]]] = [("embed", (cfg.vocab, cfg.hidden))]
        for l in range(cfg.n_layers):
            shapes += [(f"l{l}.norm1", (cfg.hidden,)), (f"l{l}.wqkv", (cfg.qkv_dim, cfg.hidden)),
                       (f"l{l}.wo", (cfg.hidden, cfg.n_heads * cfg.head_dim)), (f"l{l}.norm2", (cfg.hidden,)),
                       (f"l{l}.wgu", (2 * cfg.ffn, cfg.hidden)), (f"l{l}.wd", (cfg.hidden, cfg.ffn))]
        shapes += [("norm_f", (cfg.hidden,)), ("lm_head", (cfg.vocab, cfg.hidden))]
        self.shapes = shapes
        total = 0
        self.offsets: Dict[str, Tuple[int, int]] = {}
        for name, shp in shapes:
            n = math.prod(shp)
            self.offsets[name] = (total, n)
            total += -(-n // 8) * 8
        self.n_flat = -(-total // 1024) * 1024
        self.params_flat = params_flat if params_flat is not None else torch.empty(self.n_flat, dtype=torch.bfloat16,
                                                                                   device=device)
        self.grads_flat = grads_flat if grads_flat is not None else torch.zeros(self.n_flat, dtype=torch.bfloat16,
                                                                                device=device)
        assert self.params_flat.numel() >= self.n_flat and self.grads_flat.numel() >= self.n_flat
        self.p: Dict[str, torch.Tensor] = {}
        for name, shp in shapes:
            off, n = self.offsets[name]
            t = self.params_flat[off:off + n].view(shp).data
            t.requires_grad_(True)
            t.grad = self.grads_flat[off:off + n].view(shp).data
            self.p[name] = t
        self.init_weights(seed)

    @staticmethod
    def flat_size(cfg: LlamaConfig) -> int:
        total = 0
        per_layer = [cfg.hidden, cfg.qkv_dim * cfg.hidden, cfg.hidden * cfg.n_heads * cfg.head_dim, cfg.hidden,
                     2 * cfg.ffn * cfg.hidden, cfg.hidden * cfg.ffn]
        for n in [cfg.vocab * cfg.hidden] + per_layer * cfg.n_layers + [cfg.hidden, cfg.vocab * cfg.hidden]:
            total += -(-n // 8) * 8
        return -(-total // 1024) * 1024

    def init_weights(self, seed: int) -> None:
        g = torch.Generator(device=self.device).manual_seed(seed)
        with torch.no_grad():
            self.params_flat.zero_()
            for name, shp in self.shapes:
                t = self.p[name]
                if name.endswith(("norm1", "norm2", "norm_f")):
                    t.fill_(1.0)
                else:
                    std = self.cfg.init_std
                    if name.endswith((".wo", ".wd")):
                        std = std / math.sqrt(2 * self.cfg.n_layers)
                    # chunked normal_ keeps the fp32 temporary small for the 0.5G-element tables
                    flat = t.view(-1)
                    for s in range(0, flat.numel(), 1 << 26):
                        seg = flat[s:s + (1 << 26)]
                        seg.copy_(torch.empty(seg.numel(), dtype=torch.float32, device=self.device).normal_(0, std, generator=g))

    def parameters(self):
        return list(self.p.values())

    def zero_grad(self) -> None:
        self.grads_flat.zero_()

    def set_executor(self, executor) -> None:
        self.executor = executor

    # ---- forward
    def _layer(self, x, l: int, cos, sin):
        p, cfg = self.p, self.cfg
        h = model_ops.rmsnorm(x, p[f"l{l}.norm1"], cfg.eps)
        qkv = F.linear(h, p[f"l{l}.wqkv"])
        a = _AttentionFn.apply(qkv, self, cos, sin, l)
        x = x + F.linear(a, p[f"l{l}.wo"])
        h = model_ops.rmsnorm(x, p[f"l{l}.norm2"], cfg.eps)
        gu = F.linear(h, p[f"l{l}.wgu"])
        x = x + F.linear(model_ops.swiglu(gu), p[f"l{l}.wd"])
        return x

    def loss(self, tokens: torch.Tensor, labels: torch.Tensor, positions: torch.Tensor, grad_scale: float) -> torch.Tensor:
        """Sum over this rank's tokens of the token losses times ``grad_scale`` (1 / global token
        count); ``labels`` < 0 are ignored.  Call ``.backward()`` on the result."""
        cfg = self.cfg
        self._attn_stash.clear()
        self._stash_enabled = self.cache_attention and self.recompute and torch.is_grad_enabled()
        cos, sin = model_ops.rope_tables(positions, cfg.rope_theta, cfg.head_dim)
        x = F.embedding(tokens, self.p["embed"])
        for l in range(cfg.n_layers):
            if self.recompute and torch.is_grad_enabled():
                x = checkpoint(self._layer, x, l, cos, sin, use_reentrant=False)
            else:
                x = self._layer(x, l, cos, sin)
        h = model_ops.rmsnorm(x, self.p["norm_f"], cfg.eps)
        return _LMHeadLossFn.apply(h, self.p["lm_head"], labels, grad_scale, self.lm_head_chunk)

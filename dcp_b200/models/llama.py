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


    def shard(self, tp: int) -> "LlamaConfig":
        """The slice of the model one tensor-parallel rank holds: 1/tp of the query heads, KV heads
        and FFN channels; hidden size, vocabulary and layer count unchanged."""
        assert self.n_heads % tp == 0 and self.n_kv_heads % tp == 0 and self.ffn % tp == 0, \
            "tensor parallelism must divide the head counts and the FFN width"
        return LlamaConfig(self.n_layers, self.hidden, self.n_heads // tp, self.n_kv_heads // tp, self.head_dim,
                           self.ffn // tp, self.vocab, self.rope_theta, self.eps, self.init_std)


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


class _DecoderLayerFn(torch.autograd.Function):
    """One decoder layer with a hand-written backward and an explicit activation budget.

    Saved per layer, by level: 0 keeps the layer input and the attention result (every dense
    product the backward needs is recomputed, except the down projection, which nothing in the
    backward reads); 1 also keeps the packed QKV projection and the post-attention residual, so
    only the gate/up projection is recomputed; 2 also keeps the gate/up projection, so no GEMM
    is recomputed.  Weight gradients are written straight into the flat gradient buffer by the
    GEMM (or added to it when ``model.accumulate_grads``), with no separate accumulation pass.
    The reference gets the same effect from Megatron's activation-recompute granularity flags
    (benchmark/mlm/run_experiments.py:460-520).
    """

    @staticmethod
    def forward(ctx, x, model, l, cos, sin, level):
        p, cfg, ex = model.p, model.cfg, model.executor
        T = x.shape[0]
        h1, rstd1 = model_ops.rmsnorm_fwd_raw(x, p[f"l{l}.norm1"], cfg.eps)
        qkv = torch.mm(h1, p[f"l{l}.wqkv"].t())
        del h1
        model_ops.qkv_rope_split(qkv, cos, sin, ex.q, ex.kv, cfg.n_heads, cfg.n_kv_heads)
        ex.inputs_written()
        out, lse = ex.forward()
        a = out.reshape(T, -1).clone()
        lse_c = lse.clone()
        x_mid = model.row_parallel(x, a, p[f"l{l}.wo"])
        h2, rstd2 = model_ops.rmsnorm_fwd_raw(x_mid, p[f"l{l}.norm2"], cfg.eps)
        gu = torch.mm(h2, p[f"l{l}.wgu"].t())
        del h2
        act = model_ops.swiglu_fwd_raw(gu)
        y = model.row_parallel(x_mid, act, p[f"l{l}.wd"])
        ctx.model, ctx.l, ctx.level, ctx.epoch = model, l, level, ex.arena_epoch
        keep = [x, cos, sin, a, lse_c, rstd1]
        if level >= 1:
            keep += [qkv, x_mid, rstd2]
        if level >= 2:
            keep.append(gu)
        ctx.save_for_backward(*keep)
        return y

    @staticmethod
    def backward(ctx, dy):
        model, l, level = ctx.model, ctx.l, ctx.level
        p, cfg, ex = model.p, model.cfg, model.executor
        saved = ctx.saved_tensors
        x, cos, sin, a, lse_c, rstd1 = saved[:6]
        T = x.shape[0]
        dy = dy.contiguous()
        w1, wqkv, wo = p[f"l{l}.norm1"], p[f"l{l}.wqkv"], p[f"l{l}.wo"]
        w2, wgu, wd = p[f"l{l}.norm2"], p[f"l{l}.wgu"], p[f"l{l}.wd"]

        def wgrad(param, lhs_t, rhs):
            if model.accumulate_grads:
                param.grad.addmm_(lhs_t, rhs)
            else:
                torch.mm(lhs_t, rhs, out=param.grad)

        def ngrad(param, dw):
            if model.accumulate_grads:
                param.grad.add_(dw.to(param.grad.dtype))
            else:
                param.grad.copy_(dw)

        if level >= 1:
            qkv, x_mid, rstd2 = saved[6:9]
        else:
            h1, _ = model_ops.rmsnorm_fwd_raw(x, w1, cfg.eps)
            qkv = torch.mm(h1, wqkv.t())
            del h1
            x_mid = model.row_parallel(x, a, wo)
            rstd2 = None
        # ---- MLP
        h2, rstd2_new = model_ops.rmsnorm_fwd_raw(x_mid, w2, cfg.eps)
        rstd2 = rstd2 if rstd2 is not None else rstd2_new
        gu = saved[9] if level >= 2 else torch.mm(h2, wgu.t())
        act = model_ops.swiglu_fwd_raw(gu)
        dact = torch.mm(dy, wd)
        wgrad(wd, dy.t(), act)
        del act
        dgu = model_ops.swiglu_bwd_raw(gu, dact)
        del dact, gu
        dh2 = model.tp_sum(torch.mm(dgu, wgu))     # the norm output feeds every rank's gate/up shard
        wgrad(wgu, dgu.t(), h2)
        del dgu, h2
        dx_mid, dw2 = model_ops.rmsnorm_bwd_raw(x_mid, w2, rstd2, dh2)
        del dh2
        dx_mid.add_(dy)
        ngrad(w2, dw2)
        # ---- attention
        da = torch.mm(dx_mid, wo)
        wgrad(wo, dx_mid.t(), a)
        if ex.arena_epoch != ctx.epoch:
            # another layer used the arenas since this forward ran: put this layer's operands back
            model_ops.qkv_rope_split(qkv, cos, sin, ex.q, ex.kv, cfg.n_heads, cfg.n_kv_heads)
            ex.inputs_written()
            ex.out_local().copy_(a.view(-1, cfg.n_heads, cfg.head_dim))
            ex.lse_local().copy_(lse_c)
        dq, dkv = ex.backward(da.view(-1, cfg.n_heads, cfg.head_dim))
        del da
        dqkv = model_ops.qkv_rope_pack_bwd(dq, dkv, cos, sin, T, cfg.n_heads, cfg.n_kv_heads)
        h1, _ = model_ops.rmsnorm_fwd_raw(x, w1, cfg.eps)
        dh1 = model.tp_sum(torch.mm(dqkv, wqkv))
        wgrad(wqkv, dqkv.t(), h1)
        del dqkv, h1
        dx, dw1 = model_ops.rmsnorm_bwd_raw(x, w1, rstd1, dh1)
        dx.add_(dx_mid)
        ngrad(w1, dw1)
        if model.grad_ready_hook is not None and not model.accumulate_grads:
            # every matrix gradient of this layer is final: its bucket can be reduced over the
            # data-parallel ranks while the layers below are still in their backward
            model.grad_ready_hook(model.layer_bucket(l))
        return dx, None, None, None, None, None


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
                 lm_head_chunk: int = 4096, tp_group=None, tp_rank: int = 0, tp_size: int = 1):
        self.cfg, self.device = cfg, device
        self.set_tensor_parallel(tp_group, tp_rank, tp_size)
        self.n_replicated = 0
        self.recompute = recompute
        self.lm_head_chunk = lm_head_chunk
        self.executor = None
        # keep each layer's attention output across the checkpoint boundary so the recompute pass
        # does not run attention (and its communication) a second time
        self.cache_attention = True
        self._attn_stash: Dict[int, tuple] = {}
        self._stash_enabled = False
        # hand-written layer backward (CUDA only): per-layer activation level 0/1/2, see _DecoderLayerFn;
        # None keeps the autograd + checkpoint path
        self.layer_levels: Optional[List[int]] = None
        self.accumulate_grads = False   # True: weight gradients are added to .grad instead of written
        # called with a bucket index (see grad_buckets) when that bucket's gradients are final
        self.grad_ready_hook = None
        # flat layout: parameters every tensor-parallel rank holds in full come first, the sharded
        # matrices after them, so "the replicated part" is one contiguous range of the buffers
        shapes: List[Tuple[str, Tuple[int, ...]]] = self.param_shapes(cfg)
        self.shapes = shapes
        total = 0
        self.offsets: Dict[str, Tuple[int, int]] = {}
        for name, shp in shapes:
            n = math.prod(shp)
            self.offsets[name] = (total, n)
            total += -(-n // 8) * 8
            if name == self.LAST_REPLICATED:
                self.n_replicated = total
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

    LAST_REPLICATED = "lm_head"

    @staticmethod
    def param_shapes(cfg: LlamaConfig) -> List[Tuple[str, Tuple[int, ...]]]:
        rep = [("embed", (cfg.vocab, cfg.hidden))]
        for l in range(cfg.n_layers):
            rep += [(f"l{l}.norm1", (cfg.hidden,)), (f"l{l}.norm2", (cfg.hidden,))]
        rep += [("norm_f", (cfg.hidden,)), ("lm_head", (cfg.vocab, cfg.hidden))]
        sharded = []
        for l in range(cfg.n_layers):
            sharded += [(f"l{l}.wqkv", (cfg.qkv_dim, cfg.hidden)), (f"l{l}.wo", (cfg.hidden, cfg.n_heads * cfg.head_dim)),
                        (f"l{l}.wgu", (2 * cfg.ffn, cfg.hidden)), (f"l{l}.wd", (cfg.hidden, cfg.ffn))]
        return rep + sharded

    @staticmethod
    def flat_size(cfg: LlamaConfig) -> int:
        total = sum(-(-math.prod(shp) // 8) * 8 for _, shp in LlamaModel.param_shapes(cfg))
        return -(-total // 1024) * 1024

    # ---- tensor parallelism: this object holds one rank's shard (``cfg`` is the sharded config)
    def set_tensor_parallel(self, group, rank: int, size: int) -> None:
        self.tp_group, self.tp_rank, self.tp_size = (group if size > 1 else None), rank, size

    def tp_sum(self, t: torch.Tensor) -> torch.Tensor:
        if self.tp_group is not None:
            import torch.distributed as dist
            dist.all_reduce(t, group=self.tp_group)
        return t

    def row_parallel(self, residual: torch.Tensor, inp: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        """residual + sum over tensor-parallel ranks of inp @ weight^T (weight holds this rank's input columns)."""
        if self.tp_group is None:
            return torch.addmm(residual, inp, weight.t())
        return self.tp_sum(torch.mm(inp, weight.t())).add_(residual)

    def init_weights(self, seed: int) -> None:
        """Replicated parameters come from ``seed`` alone (identical on every tensor-parallel rank),
        sharded ones from a stream that also depends on the rank."""
        g_rep = torch.Generator(device=self.device).manual_seed(seed)
        g_shard = torch.Generator(device=self.device).manual_seed(seed * 7919 + 104729 * (self.tp_rank + 1))
        replicated = True
        with torch.no_grad():
            self.params_flat.zero_()
            for name, shp in self.shapes:
                t = self.p[name]
                g = g_rep if replicated else g_shard
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
                if name == self.LAST_REPLICATED:
                    replicated = False

    def plan_activation_levels(self, tokens: int, budget_bytes: int) -> List[int]:
        """Per-layer activation levels for the hand-written layer backward that fit ``budget_bytes``
        of extra activation memory at ``tokens`` tokens per rank: first every layer is raised to
        level 1 (all or nothing: a mixed 0/1 schedule saves little), then as many layers as fit
        are raised to level 2, the last layers first (their activations live the shortest)."""
        cfg = self.cfg
        lvl1 = tokens * (cfg.qkv_dim + cfg.hidden) * 2 + tokens * 4
        lvl2 = tokens * 2 * cfg.ffn * 2
        levels = [0] * cfg.n_layers
        if budget_bytes >= lvl1 * cfg.n_layers:
            levels = [1] * cfg.n_layers
            n2 = min(cfg.n_layers, int((budget_bytes - lvl1 * cfg.n_layers) // lvl2))
            for l in range(cfg.n_layers - n2, cfg.n_layers):
                levels[l] = 2
        return levels

    def parameters(self):
        return list(self.p.values())

    # ---- gradient buckets: bucket 0 = everything that is not a decoder-layer matrix (embedding,
    # norm weights, LM head; final only when the whole backward is done), bucket 1 + l = the four
    # matrices of layer l, which are contiguous in the flat buffers
    def grad_buckets(self) -> List[Tuple[int, int]]:
        first = self.offsets["l0.wqkv"][0]
        out = [(0, first)]
        for l in range(self.cfg.n_layers):
            lo = self.offsets[f"l{l}.wqkv"][0]
            hi = self.offsets[f"l{l + 1}.wqkv"][0] if l + 1 < self.cfg.n_layers else self.n_flat
            out.append((lo, hi - lo))
        return out

    @staticmethod
    def layer_bucket(l: int) -> int:
        return 1 + l

    def zero_grad(self) -> None:
        """Gradients that autograd accumulates into must start at zero; the hand-written layer
        backward overwrites every decoder-layer gradient (matrices and norm weights), so only the
        embedding, the final norm and the LM head are cleared in that mode."""
        manual = self.layer_levels is not None and self.grads_flat.is_cuda and not self.accumulate_grads
        if not manual:
            self.grads_flat.zero_()
            return
        for name in ("embed", "norm_f", "lm_head"):
            self.p[name].grad.zero_()

    def set_executor(self, executor) -> None:
        self.executor = executor

    # ---- forward
    def _layer(self, x, l: int, cos, sin):
        p, cfg = self.p, self.cfg
        h = model_ops.rmsnorm(x, p[f"l{l}.norm1"], cfg.eps)
        qkv = F.linear(h, p[f"l{l}.wqkv"])
        a = _AttentionFn.apply(qkv, self, cos, sin, l)
        assert self.tp_group is None, "tensor parallelism needs the hand-written layer backward (CUDA)"
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
        manual = self.layer_levels is not None and x.is_cuda and torch.is_grad_enabled()
        for l in range(cfg.n_layers):
            if manual:
                x = _DecoderLayerFn.apply(x, self, l, cos, sin, self.layer_levels[l])
            elif self.recompute and torch.is_grad_enabled():
                x = checkpoint(self._layer, x, l, cos, sin, use_reentrant=False)
            else:
                x = self._layer(x, l, cos, sin)
        h = model_ops.rmsnorm(x, self.p["norm_f"], cfg.eps)
        return _LMHeadLossFn.apply(h, self.p["lm_head"], labels, grad_scale, self.lm_head_chunk)

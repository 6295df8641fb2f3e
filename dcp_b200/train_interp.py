"""DCP training step without a GPU: plain torch ops + the plan-interpreting attention executor.

The same stack as ``TrainEngine`` (synthetic batch -> placement -> execution plans -> distributed
attention -> loss -> gradient sum over ranks -> AdamW), but every op is an fp32 torch op and
attention runs the ``ExecutionPlan`` instruction streams through ``AttentionExecutor`` over a
``torch.distributed`` group (gloo on CPU, NCCL on GPUs).  It is the any-device correctness arm of
the framework: on N ranks it must produce the loss and gradients of the unsplit model
(``models/reference.py``), which the CPU tests check with two gloo ranks.  The reference trains
through the same executor interface (``DCPAttention.apply(executor, ...)`` inside its model,
benchmark/mlm/monkey_patch.py), only on GPUs.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m dcp_b200.train_interp --iters 3
"""
from __future__ import annotations

import argparse
import os
from typing import Dict, Optional

import torch
import torch.nn.functional as F

from .core.common import get_default_execution_context
from .data import synth
from .data.plan_service import PlanSpec, RankPlan, plan_iteration
from .models.llama import LlamaConfig, LlamaModel
from .ops import model_ops
from .runtime.interface import DCPAttention, get_executor


def init_params(cfg: LlamaConfig, seed: int = 0, dtype=torch.float32, device="cpu") -> Dict[str, torch.Tensor]:
    """Replicated parameters, identical on every rank (same seed): norms 1, the rest N(0, init_std)."""
    g = torch.Generator().manual_seed(seed)
    p = {}
    for name, shp in LlamaModel.param_shapes(cfg):
        t = torch.ones(shp, dtype=dtype) if "norm" in name else cfg.init_std * torch.randn(shp, generator=g, dtype=dtype)
        p[name] = t.to(device).requires_grad_(True)
    return p


def shard_params(cfg: LlamaConfig, full: Dict[str, torch.Tensor], tp: int, t: int) -> Dict[str, torch.Tensor]:
    """Tensor-parallel rank ``t``'s slice of full parameters: its query heads, KV heads and FFN channels
    (rows of the QKV and gate/up matrices, columns of the output and down projections); embeddings,
    norms and the LM head are held in full.  Same cut as ``LlamaConfig.shard``."""
    d, hq, hkv, f = cfg.head_dim, cfg.n_heads // tp, cfg.n_kv_heads // tp, cfg.ffn // tp
    out = {}
    for name, w in full.items():
        w = w.detach()
        if name.endswith("wqkv"):
            q, k, v = w[:cfg.n_heads * d], w[cfg.n_heads * d:(cfg.n_heads + cfg.n_kv_heads) * d], w[(cfg.n_heads + cfg.n_kv_heads) * d:]
            w = torch.cat([q[t * hq * d:(t + 1) * hq * d], k[t * hkv * d:(t + 1) * hkv * d], v[t * hkv * d:(t + 1) * hkv * d]])
        elif name.endswith("wgu"):
            w = torch.cat([w[t * f:(t + 1) * f], w[cfg.ffn + t * f:cfg.ffn + (t + 1) * f]])
        elif name.endswith(".wo"):
            w = w[:, t * hq * d:(t + 1) * hq * d]
        elif name.endswith(".wd"):
            w = w[:, t * f:(t + 1) * f]
        out[name] = w.clone().contiguous().requires_grad_(True)
    return out


class _SumForward(torch.autograd.Function):
    """Row-parallel output: partial products of the tensor-parallel ranks are summed; the gradient
    passes through unchanged."""

    @staticmethod
    def forward(ctx, x, group):
        import torch.distributed as dist
        x = x.clone()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class _SumBackward(torch.autograd.Function):
    """Input of a column-parallel layer: identity forward; every tensor-parallel rank contributes a
    part of the input gradient, summed in the backward."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        import torch.distributed as dist
        g = g.clone()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class InterpreterEngine:
    """One rank of a context-parallel training job on the plan interpreter.  ``group``: the ranks that
    share every batch (None = single process).

    With ``pp_group`` (the ranks that hold the other pipeline stages of this rank's tokens; group rank
    = stage index) the model is cut into stages of consecutive layers: ``group`` then links the
    context-parallel ranks of ONE stage, every stage of a context-parallel rank plans the same
    batches, a step runs ``n_micro`` planned batches in one-forward-one-backward order
    (``parallel.pipeline.run_stage_1f1b``) and a stage only ever touches its own parameters.

    With ``replica_group`` (all ranks that hold the same parameters) ``group`` is one of several
    context-parallel groups inside it (CP x DP): the batch is dealt over the groups, attention stays
    inside a group and gradients are summed over the whole replica group.

    With ``tp_group`` (the ranks that hold the other shards of this rank's model replica; they see the
    same tokens) every rank holds 1/tp of the heads and FFN channels, the planner plans for the
    per-shard head counts, and ``group`` / ``replica_group`` link ranks of equal shard index."""

    def __init__(self, cfg: LlamaConfig, tokens_per_step: int, block_size: int = 256, mask: str = "causal",
                 length_dist: Optional[synth.LengthDist] = None, group=None, seed: int = 0, lr: float = 1e-3,
                 device: str = "cpu", n_stages: Optional[int] = None, pp_group=None, n_micro: int = 1,
                 replica_group=None, tp_group=None):
        import torch.distributed as dist
        from .models.reference import stage_layer_range
        self.cfg, self.group, self.device = cfg, group, torch.device(device)
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        self.pp_group, self.n_micro = pp_group, n_micro
        self.stage = dist.get_rank(pp_group) if pp_group is not None else 0
        self.n_pp = dist.get_world_size(pp_group) if pp_group is not None else 1
        self.layers = stage_layer_range(cfg.n_layers, self.stage, self.n_pp)
        self.tp_group = tp_group
        self.tp = dist.get_world_size(tp_group) if tp_group is not None else 1
        self.tp_rank = dist.get_rank(tp_group) if tp_group is not None else 0
        self.full_cfg = cfg
        if self.tp > 1:
            cfg = self.cfg = cfg.shard(self.tp)
        self.replica_group = replica_group if replica_group is not None else group
        n_all = dist.get_world_size(self.replica_group) if self.replica_group is not None else 1
        self.plan_rank = dist.get_rank(self.replica_group) if self.replica_group is not None else 0
        assert n_all % self.world == 0 and self.plan_rank % self.world == self.rank, \
            "context-parallel groups must be runs of consecutive ranks of the replica group"
        self.ctx = get_default_execution_context(self.world, 1)
        self.spec = PlanSpec(n_all, self.world, tokens_per_step, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, block_size,
                             0, mask, length_dist or synth.LengthDist("lognormal", 400.0, 0.6, 32, tokens_per_step),
                             vocab=cfg.vocab, seed=seed, n_stages=n_stages, build_instruction_plans=True,
                             qkv_dtype="float32")
        self.p = init_params(self.full_cfg, seed, torch.float32, self.device)
        if self.tp > 1:
            self.p = shard_params(self.full_cfg, self.p, self.tp, self.tp_rank)
        self.opt = torch.optim.AdamW(list(self.p.values()), lr=lr, betas=(0.9, 0.95), weight_decay=0.1)
        self.iteration = 0

    def plan(self, iteration: Optional[int] = None) -> RankPlan:
        return plan_iteration(self.spec, self.iteration if iteration is None else iteration, self.plan_rank)

    def _executor(self, plan: RankPlan):
        cfg = self.cfg
        return get_executor(cfg.n_heads, cfg.head_dim, self.ctx, plan.fw_plan, plan.fw_workload, plan.bw_plan,
                            plan.bw_workload, executor_impl="python", process_group=self.group, device=self.device)

    def _norm(self, t, w):
        return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + self.cfg.eps) * w

    def embed(self, plan: RankPlan) -> torch.Tensor:
        return F.embedding(plan.tokens.to(self.device), self.p["embed"])

    def run_layers(self, plan: RankPlan, ex, x: torch.Tensor, layers) -> torch.Tensor:
        """Decoder layers ``layers`` on this rank's tokens of ``plan`` (attention through ``ex``)."""
        cfg, p = self.cfg, self.p
        hq, hkv, d = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
        cos, sin = model_ops.rope_tables(plan.positions.to(self.device), cfg.rope_theta, d)
        tp_in = (lambda t: _SumBackward.apply(t, self.tp_group)) if self.tp > 1 else (lambda t: t)
        tp_out = (lambda t: _SumForward.apply(t, self.tp_group)) if self.tp > 1 else (lambda t: t)
        for l in layers:
            qkv = F.linear(tp_in(self._norm(x, p[f"l{l}.norm1"])), p[f"l{l}.wqkv"]).view(-1, hq + 2 * hkv, d)
            q = model_ops.rope_reference(qkv[:, :hq], cos, sin)
            k = model_ops.rope_reference(qkv[:, hq:hq + hkv], cos, sin)
            kv = torch.stack([k, qkv[:, hq + hkv:]], dim=1)                   # [tokens, 2, hkv, d]
            # every rank calls the executor in every layer, also with zero local tokens: its peers
            # fetch blocks from it and wait for its messages
            a = DCPAttention.apply(ex, False, False, q.contiguous(), kv.contiguous())
            x = x + tp_out(F.linear(a.reshape(-1, hq * d), p[f"l{l}.wo"]))
            gate, up = F.linear(tp_in(self._norm(x, p[f"l{l}.norm2"])), p[f"l{l}.wgu"]).chunk(2, dim=-1)
            x = x + tp_out(F.linear(F.silu(gate) * up, p[f"l{l}.wd"]))
        return x

    def head_loss(self, plan: RankPlan, x: torch.Tensor) -> torch.Tensor:
        labels = plan.labels.to(self.device)
        logits = F.linear(self._norm(x, self.p["norm_f"]), self.p["lm_head"])
        loss = F.cross_entropy(logits, labels.clamp(min=0), reduction="none")
        return torch.where(labels >= 0, loss, torch.zeros_like(loss)).sum() / max(plan.n_global_tokens, 1)

    def local_loss(self, plan: RankPlan) -> torch.Tensor:
        """Sum of this rank's token losses / global token count (the ranks' values add up to the batch loss)."""
        x = self.run_layers(plan, self._executor(plan), self.embed(plan), range(self.cfg.n_layers))
        return self.head_loss(plan, x)

    def pipeline_loss_and_grads(self, first_iteration: Optional[int] = None):
        """One pipelined step over ``n_micro`` planned batches (iterations ``first_iteration`` ...):
        gradients of this stage's parameters summed over the micro-batches and over the stage's
        context-parallel ranks.  Returns the micro-batch losses on the last stage (summed over its
        ranks), an empty list elsewhere."""
        import torch.distributed as dist
        from .parallel.pipeline import PipelineComm, run_stage_1f1b
        it0 = self.iteration * self.n_micro if first_iteration is None else first_iteration
        plans = [self.plan(it0 + mb) for mb in range(self.n_micro)]
        execs = [self._executor(pl) for pl in plans]          # plans differ per micro-batch, so do the executors
        for t in self.p.values():
            t.grad = None
        comm = PipelineComm(self.pp_group, lambda mb: (plans[mb].tokens.numel(), self.cfg.hidden), torch.float32, self.device)
        losses = run_stage_1f1b(
            comm, self.n_micro,
            lambda mb, x: self.run_layers(plans[mb], execs[mb], self.embed(plans[mb]) if x is None else x, self.layers),
            lambda mb, y: self.head_loss(plans[mb], y))
        mine = self.stage_parameters()
        for name in mine:
            t = self.p[name]
            if t.grad is None:
                t.grad = torch.zeros_like(t)
            if self.group is not None:
                dist.all_reduce(t.grad, group=self.group)
        out = []
        for l in losses:
            l = l.clone()
            if self.group is not None:
                dist.all_reduce(l, group=self.group)
            out.append(float(l.item()))
        return out

    def stage_parameters(self):
        """Names of the parameters this pipeline stage owns."""
        names = [k for k in self.p if any(k.startswith(f"l{l}.") for l in self.layers)]
        if self.stage == 0:
            names.append("embed")
        if self.stage == self.n_pp - 1:
            names += ["norm_f", "lm_head"]
        return names

    def loss_and_grads(self, plan: RankPlan) -> float:
        """Backward through the distributed attention, gradients summed over the ranks; returns the
        batch loss (the same on every rank)."""
        import torch.distributed as dist
        for t in self.p.values():
            t.grad = None
        loss = self.local_loss(plan)
        loss.backward()
        total = loss.detach().clone()
        if self.replica_group is not None:
            dist.all_reduce(total, group=self.replica_group)
            for t in self.p.values():
                if t.grad is None:                       # a rank without tokens still takes part in the sum
                    t.grad = torch.zeros_like(t)
                dist.all_reduce(t.grad, group=self.replica_group)
        return float(total.item())

    def train_step(self) -> float:
        loss = self.loss_and_grads(self.plan())
        torch.nn.utils.clip_grad_norm_(list(self.p.values()), 1.0)
        self.opt.step()
        self.iteration += 1
        return loss


def main(argv=None):
    import torch.distributed as dist
    ap = argparse.ArgumentParser(description="DCP training on the plan interpreter (CPU / gloo or GPU / NCCL)")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--tokens-per-step", type=int, default=2048)
    ap.add_argument("--block-size", type=int, default=256)
    ap.add_argument("--mask", default="causal")
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--hidden", type=int, default=128)
    ap.add_argument("--heads", type=int, default=4)
    ap.add_argument("--kv-heads", type=int, default=2)
    ap.add_argument("--head-dim", type=int, default=32)
    ap.add_argument("--vocab", type=int, default=512)
    args = ap.parse_args(argv)
    group = None
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        dist.init_process_group("gloo")
        group = dist.group.WORLD
    cfg = LlamaConfig(args.layers, args.hidden, args.heads, args.kv_heads, args.head_dim, 2 * args.hidden, args.vocab)
    eng = InterpreterEngine(cfg, args.tokens_per_step, args.block_size, args.mask, group=group)
    for it in range(args.iters):
        loss = eng.train_step()
        if eng.rank == 0:
            print(f"iteration {it}: Training loss: {loss:.6f}", flush=True)
    if group is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

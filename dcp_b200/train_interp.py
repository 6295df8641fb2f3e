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


class InterpreterEngine:
    """One rank of a context-parallel training job on the plan interpreter.  ``group``: the ranks that
    share every batch (None = single process)."""

    def __init__(self, cfg: LlamaConfig, tokens_per_step: int, block_size: int = 256, mask: str = "causal",
                 length_dist: Optional[synth.LengthDist] = None, group=None, seed: int = 0, lr: float = 1e-3,
                 device: str = "cpu", n_stages: Optional[int] = None):
        import torch.distributed as dist
        self.cfg, self.group, self.device = cfg, group, torch.device(device)
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        self.ctx = get_default_execution_context(self.world, 1)
        self.spec = PlanSpec(self.world, self.world, tokens_per_step, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, block_size,
                             0, mask, length_dist or synth.LengthDist("lognormal", 400.0, 0.6, 32, tokens_per_step),
                             vocab=cfg.vocab, seed=seed, n_stages=n_stages, build_instruction_plans=True,
                             qkv_dtype="float32")
        self.p = init_params(cfg, seed, torch.float32, self.device)
        self.opt = torch.optim.AdamW(list(self.p.values()), lr=lr, betas=(0.9, 0.95), weight_decay=0.1)
        self.iteration = 0

    def plan(self, iteration: Optional[int] = None) -> RankPlan:
        return plan_iteration(self.spec, self.iteration if iteration is None else iteration, self.rank)

    def local_loss(self, plan: RankPlan) -> torch.Tensor:
        """Sum of this rank's token losses / global token count (the ranks' values add up to the batch loss)."""
        cfg, p, dev = self.cfg, self.p, self.device
        hq, hkv, d = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
        ex = get_executor(hq, d, self.ctx, plan.fw_plan, plan.fw_workload, plan.bw_plan, plan.bw_workload,
                          executor_impl="python", process_group=self.group, device=dev)
        toks, labels, pos = plan.tokens.to(dev), plan.labels.to(dev), plan.positions.to(dev)
        cos, sin = model_ops.rope_tables(pos, cfg.rope_theta, d)
        norm = lambda t, w: t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + cfg.eps) * w
        x = F.embedding(toks, p["embed"])
        for l in range(cfg.n_layers):
            qkv = F.linear(norm(x, p[f"l{l}.norm1"]), p[f"l{l}.wqkv"]).view(-1, hq + 2 * hkv, d)
            q = model_ops.rope_reference(qkv[:, :hq], cos, sin)
            k = model_ops.rope_reference(qkv[:, hq:hq + hkv], cos, sin)
            kv = torch.stack([k, qkv[:, hq + hkv:]], dim=1)                   # [tokens, 2, hkv, d]
            # every rank calls the executor in every layer, also with zero local tokens: its peers
            # fetch blocks from it and wait for its messages
            a = DCPAttention.apply(ex, False, False, q.contiguous(), kv.contiguous())
            x = x + F.linear(a.reshape(-1, hq * d), p[f"l{l}.wo"])
            gate, up = F.linear(norm(x, p[f"l{l}.norm2"]), p[f"l{l}.wgu"]).chunk(2, dim=-1)
            x = x + F.linear(F.silu(gate) * up, p[f"l{l}.wd"])
        logits = F.linear(norm(x, p["norm_f"]), p["lm_head"])
        loss = F.cross_entropy(logits, labels.clamp(min=0), reduction="none")
        return torch.where(labels >= 0, loss, torch.zeros_like(loss)).sum() / max(plan.n_global_tokens, 1)

    def loss_and_grads(self, plan: RankPlan) -> float:
        """Backward through the distributed attention, gradients summed over the ranks; returns the
        batch loss (the same on every rank)."""
        import torch.distributed as dist
        for t in self.p.values():
            t.grad = None
        loss = self.local_loss(plan)
        loss.backward()
        total = loss.detach().clone()
        if self.group is not None:
            dist.all_reduce(total, group=self.group)
            for t in self.p.values():
                if t.grad is None:                       # a rank without tokens still takes part in the sum
                    t.grad = torch.zeros_like(t)
                dist.all_reduce(t.grad, group=self.group)
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

"""Training engine: Llama-architecture model + DCP attention executor + sharded optimizer.

``TrainEngine.train_step(plan)`` is the public per-iteration call: it stages the iteration's
token ids / labels / positions and kernel tables from pinned host memory, runs forward,
backward and the optimizer step, and returns the loss.  ``python -m dcp_b200.train`` runs a
synthetic-data training loop (one process per GPU under torch.distributed.run) and logs
"elapsed time per iteration (ms)" and "Training loss:" lines in the format the reference's log
parsers read (benchmark/plotting/utils.py:10-31).
"""
from __future__ import annotations

import argparse
import json
import os
import time
from dataclasses import dataclass
from typing import Optional

import torch

from .data import synth
from .data.plan_service import PlanService, PlanSpec, RankPlan
from .models.llama import LLAMA3_8B, LlamaConfig, LlamaModel, tiny_config
from .ops import _lib
from .parallel.dist_optimizer import FlatBuffers, ShardedAdamW
from .runtime.executor_fused import FusedAttentionExecutor


@dataclass
class EngineConfig:
    model: LlamaConfig
    tokens_per_step: int
    dcp_size: int = 0               # 0 -> all (non tensor-parallel) ranks form one context-parallel group
    block_size: int = 2048
    mask: str = "causal"
    length_dist: synth.LengthDist = None
    n_stages: Optional[int] = None
    lr: float = 1e-4
    weight_decay: float = 0.1
    clip_grad: Optional[float] = 1.0
    recompute: bool = True
    # extra activation memory the hand-written layer backward may keep to skip recomputing GEMMs:
    # None = decide from the free device memory at start-up, 0 = keep nothing extra, < 0 = use the
    # autograd + checkpoint path instead of the hand-written backward
    activation_budget_gb: Optional[float] = None
    seed: int = 0
    planner_workers: int = 2
    lookahead: int = 3
    lm_head_chunk: int = 4096
    head_block_size: int = 0
    use_block_size_heuristic: bool = False
    mem_imbalance_epsilon: Optional[float] = None
    comp_imbalance_epsilon: Optional[float] = None
    inter_node_comp_imbalance_factor: Optional[float] = None
    cost_model: Optional[dict] = None
    plan_cache_dir: Optional[str] = None     # reuse plans by batch signature (saved next to checkpoints on resume)
    tp_size: int = 1                # tensor-parallel ranks per model replica (adjacent ranks)
    overlap_grad_reduce: bool = True   # reduce each layer's gradient bucket during the backward pass
    # plan every batch once (on global rank 0, in its worker pool) and hand each rank its share through a
    # TCP key-value store instead of planning on every rank; None = on whenever there are several ranks
    shared_planning: Optional[bool] = None
    host_arena_mb: int = 256           # pinned host arena the per-step inputs and kernel tables are staged in


def parallel_layout(world: int, tp: int = 1, dcp_size: int = 0) -> dict:
    """Rank lists of every process group for ``world`` ranks with ``tp`` tensor-parallel ranks per
    model replica and ``dcp_size`` ranks per context-parallel group (0 = all).  Tensor-parallel
    ranks are adjacent; ``rank = (replica * dcp + cp_rank) * tp + tp_rank``.

    * ``dcp_groups``: ranks that run one attention executor together (same replica, same tp rank)
    * ``tp_groups``:  ranks that hold the shards of one model copy for the same tokens
    * ``opt_groups``: ranks that hold the same parameters (gradient sum + sharded optimizer state)
    """
    tp = max(1, tp)
    assert world % tp == 0, "tp_size must divide the world size"
    n_cp = world // tp
    dcp = dcp_size or n_cp
    assert n_cp % dcp == 0, "dcp_size must divide the number of non tensor-parallel ranks"
    return {
        "n_cp": n_cp, "dcp": dcp,
        "dcp_groups": [[(g * dcp + c) * tp + t for c in range(dcp)] for g in range(n_cp // dcp) for t in range(tp)],
        "tp_groups": [[c * tp + t for t in range(tp)] for c in range(n_cp)],
        "opt_groups": [[c * tp + t for c in range(n_cp)] for t in range(tp)],
    }


class TrainEngine:
    def __init__(self, cfg: EngineConfig, device: torch.device, world_group=None):
        import torch.distributed as dist
        self.cfg, self.device = cfg, device
        self.world = dist.get_world_size(world_group) if world_group is not None else 1
        self.rank = dist.get_rank(world_group) if world_group is not None else 0
        self.world_group = world_group
        # rank layout: tensor-parallel rank fastest, then the rank inside its context-parallel group,
        # then the data-parallel replica:  rank = (replica * dcp + cp_rank) * tp + tp_rank
        tp = max(1, cfg.tp_size)
        lay = parallel_layout(self.world, tp, cfg.dcp_size)
        n_cp, dcp = lay["n_cp"], lay["dcp"]
        self.tp_size, self.tp_rank, self.cp_index = tp, self.rank % tp, self.rank // tp
        self.n_cp_ranks, self.dcp_size = n_cp, dcp
        self.dcp_group, self.tp_group, self.opt_group = world_group, None, world_group
        if world_group is not None and (tp > 1 or dcp != n_cp):
            # every rank creates every subgroup, in the same order (new_group is collective)
            def make(groups):
                mine = None
                for ranks in groups:
                    grp = dist.new_group(ranks) if len(ranks) > 1 else None
                    if self.rank in ranks:
                        mine = grp
                return mine
            self.dcp_group = make(lay["dcp_groups"])
            if tp > 1:
                self.tp_group = make(lay["tp_groups"])
                self.opt_group = make(lay["opt_groups"])
        m = cfg.model.shard(tp)                 # this rank's slice of the model
        self.local_model = m
        n_flat = LlamaModel.flat_size(m)
        self.bufs = FlatBuffers(n_flat, device, self.opt_group if n_cp > 1 else None)
        self.model = LlamaModel(m, device, self.bufs.params, self.bufs.grads, seed=cfg.seed, recompute=cfg.recompute,
                                lm_head_chunk=cfg.lm_head_chunk, tp_group=self.tp_group, tp_rank=self.tp_rank, tp_size=tp)
        group_tokens = cfg.tokens_per_step // (n_cp // dcp)
        cap = int(group_tokens * 1.3) + 4 * cfg.block_size
        self.executor = FusedAttentionExecutor(m.n_heads, m.n_kv_heads, cap, cap, 2 * cap, device,
                                               self.dcp_group if dcp > 1 else None)
        self.model.set_executor(self.executor)
        # one gradient bucket per decoder layer (+ one for embeddings / norms / head); with several
        # ranks each bucket is reduced on a side stream as soon as its layer's backward is done
        self.optimizer = ShardedAdamW(self.bufs, cfg.lr, weight_decay=cfg.weight_decay, clip_grad=cfg.clip_grad,
                                      group=self.opt_group if n_cp > 1 else None, tp_group=self.tp_group,
                                      n_replicated=self.model.n_replicated, buckets=self.model.grad_buckets(),
                                      extra_status=self.executor.arena.status)
        if self.optimizer.overlap and cfg.overlap_grad_reduce:
            self.model.grad_ready_hook = self.optimizer.reduce_bucket
        self.activation_levels = self._plan_activations(group_tokens // dcp)
        self.spec = PlanSpec(n_cp, dcp, cfg.tokens_per_step, m.n_heads, m.n_kv_heads, m.head_dim, cfg.block_size,
                             cfg.head_block_size, cfg.mask, cfg.length_dist or synth.LOGNORMAL_8K, m.vocab, cfg.seed,
                             cfg.n_stages, mem_imbalance_epsilon=cfg.mem_imbalance_epsilon,
                             comp_imbalance_epsilon=cfg.comp_imbalance_epsilon,
                             inter_node_comp_imbalance_factor=cfg.inter_node_comp_imbalance_factor,
                             use_block_size_heuristic=cfg.use_block_size_heuristic, cost_model=cfg.cost_model,
                             cache_dir=cfg.plan_cache_dir)
        from .memory.host_caching_allocator import HostCachingAllocator
        self.host_arena = HostCachingAllocator(cfg.host_arena_mb << 20)
        self.executor.host_pin = self.host_arena.pin
        self._staged_host = []
        self._kv, self._kv_server, self._plan_generation = None, None, 0
        shared = cfg.shared_planning if cfg.shared_planning is not None else self.world > 1
        if shared and self.world > 1:
            from .data.kv_store import KVServer, KVStore
            host = os.environ.get("DCP_KV_HOST", os.environ.get("MASTER_ADDR", "127.0.0.1"))
            port = int(os.environ.get("DCP_KV_PORT", int(os.environ.get("MASTER_PORT", "29500")) + 29))
            ok = [True]
            if self.rank == 0:
                try:
                    self._kv_server = KVServer(host, port)
                except Exception as e:      # port taken, no permission, ...: every rank plans for itself instead
                    print(f"[dcp] shared planning disabled: cannot open the plan store on {host}:{port} ({e!r})", flush=True)
                    ok = [False]
            dist.broadcast_object_list(ok, src=dist.get_global_rank(world_group, 0), group=world_group)
            if ok[0]:
                self._kv = KVStore(host, port, timeout_s=600.0)
        self.plans = self._make_plan_service(0)
        self.samples_consumed = 0       # dataset samples trained on (checkpointed for the batch sampler)
        self.iteration = 0
        self.last_global_tokens = 0
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    def _make_plan_service(self, start: int):
        """Look-ahead planner starting at iteration ``start``: shared (rank 0 plans once per batch,
        everybody reads its share from the key-value store) or per rank."""
        cfg = self.cfg
        if self._kv is None:
            return PlanService(self.spec, self.cp_index, cfg.planner_workers, cfg.lookahead, start=start)
        from .data.plan_service import SharedPlanService
        self._plan_generation += 1
        return SharedPlanService(self.spec, self.cp_index, self._kv, self.rank == 0, 2 * cfg.planner_workers,
                                 cfg.lookahead, start=start, readers=self.tp_size,
                                 name=f"dcp_plans_g{self._plan_generation}")

    def _plan_activations(self, tokens_per_rank: int):
        """Choose how much each layer keeps for its backward (see LlamaModel.plan_activation_levels)."""
        cfg, m = self.cfg, self.local_model
        if not cfg.recompute or (cfg.activation_budget_gb is not None and cfg.activation_budget_gb < 0):
            return None
        tokens = int(tokens_per_rank * 1.15) + cfg.block_size
        if cfg.activation_budget_gb is not None:
            budget = int(cfg.activation_budget_gb * 1e9)
        else:
            free, _ = torch.cuda.mem_get_info(self.device)
            # what a step needs besides the optional activations: level-0 activations of every layer,
            # one layer's transients (gate/up, its gradient, two FFN-wide temporaries), the LM-head
            # chunk (logits + fp32 loss temporaries, weight gradient), allocator slack
            level0 = m.n_layers * tokens * (2 * m.hidden * 2 + m.n_heads * 4)
            transient = tokens * (2 * 2 * m.ffn * 2 + 2 * m.ffn * 2 + 6 * m.hidden * 2)
            lm_head = cfg.lm_head_chunk * m.vocab * 8 + m.vocab * m.hidden * 2 + 2 * tokens * m.hidden * 2
            budget = free - level0 - transient - lm_head - int(16e9)
        levels = self.model.plan_activation_levels(tokens, max(0, budget))
        self.model.layer_levels = levels
        return levels

    # ---- one iteration
    time_optimizer = False
    _optimizer_events: list = []

    def stage_inputs(self, plan: RankPlan):
        """Pinned host -> device copies of this iteration's inputs and kernel tables."""
        dev = self.device
        # staged in the pinned arena (no cudaHostAlloc per step); kept alive until the next step's staging
        host = [self.host_arena.pin(t) for t in (plan.tokens, plan.labels, plan.positions)]
        self._staged_host = host
        toks, labels, pos = (t.to(dev, non_blocking=True) for t in host)
        self.executor.prepare(plan.program)
        n = sum(t.numel() * t.element_size() for t in host)
        p = plan.program
        for tabs in list(p.fwd) + list(p.bwd):
            if tabs is not None:
                n += sum(t.numel() * t.element_size() for t in (getattr(tabs, "tiles", None), getattr(tabs, "kv_entries", None),
                                                                 getattr(tabs, "ctas", None), getattr(tabs, "items", None),
                                                                 tabs.masks) if t is not None)
        self.h2d_bytes = n
        return toks, labels, pos

    def run_step(self, toks, labels, pos, n_global_tokens: int) -> torch.Tensor:
        """Forward + backward + optimizer on staged inputs; returns the device loss tensor."""
        self.model.zero_grad()
        loss = self.model.loss(toks, labels, pos, 1.0 / max(n_global_tokens, 1))
        loss.backward()
        if self.time_optimizer:
            # what the optimizer still costs after the backward: the reduce-scatters of the layer buckets
            # ran beside the backward, so this is the last bucket, the norm, AdamW and the parameter stores
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            self.optimizer.step(1.0)
            e1.record()
            self._optimizer_events.append((e0, e1))
        else:
            self.optimizer.step(1.0)
        return loss.detach()

    def optimizer_ms(self) -> float:
        """Sum of the timed ``optimizer.step`` calls since the last call of this method (CUDA events;
        synchronises).  Timing is on while ``time_optimizer`` is set."""
        torch.cuda.synchronize(self.device)
        ms = sum(a.elapsed_time(b) for a, b in self._optimizer_events)
        self._optimizer_events = []
        return ms

    def train_step(self, plan=None) -> float:
        """Public API: plan (or fetch) the iteration, copy its inputs in, step, read the loss back.
        ``plan``: None (next synthetic batch from the plan service), a ``RankPlan``, or what
        ``DCPDataLoader`` yields ((local_batch, fw_plan, bw_plan, fw_workload, bw_workload, spec))."""
        if plan is None:
            plan = self.plans.get(self.iteration)
        elif isinstance(plan, tuple):
            lb = plan[0]
            self.samples_consumed += len(lb["seqlens"])
            plan = RankPlan(self.iteration, lb["program"], lb["tokens"][0], lb["labels"][0], lb["position_ids"][0],
                            int(lb["n_global_tokens"]), int(lb["tokens"].numel()), list(lb["seqlens"]), 0.0)
        self.last_global_tokens = plan.n_global_tokens
        self.last_seqlens = list(plan.seqlens)
        toks, labels, pos = self.stage_inputs(plan)
        loss = self.run_step(toks, labels, pos, plan.n_global_tokens)
        if self.n_cp_ranks > 1:
            import torch.distributed as dist
            dist.all_reduce(loss, group=self.opt_group)   # one rank per token (tensor-parallel peers hold copies)
        value = float(loss.item())         # device -> host read of the step's result
        self.d2h_bytes = loss.numel() * loss.element_size()
        self.check_status()
        self.iteration += 1
        return value

    def check_status(self) -> None:
        """Raise if a device-side wait of this step ran out (attention arenas or optimizer arena).
        The update kernels read the same status words and leave the weights alone when one is set."""
        self.executor.check_status()
        self.optimizer.check_status()

    def reconfigure(self, tokens_per_step: int, length_dist=None, mask: Optional[str] = None) -> None:
        """Switch the synthetic workload (token budget, length distribution, mask) without rebuilding
        the model: a new plan service starts at the current iteration."""
        import dataclasses
        self.plans.close()
        self.spec = dataclasses.replace(self.spec, tokens_per_step=tokens_per_step,
                                        length_dist=length_dist or self.spec.length_dist, mask=mask or self.spec.mask)
        self.plans = self._make_plan_service(self.iteration)

    def close(self) -> None:
        self.plans.close()

    # ---- checkpoint / resume: per-rank shard files
    def save_checkpoint(self, directory: str) -> str:
        os.makedirs(directory, exist_ok=True)
        path = os.path.join(directory, f"rank{self.rank:03d}.pt")
        state = {"iteration": self.iteration, "optimizer": self.optimizer.state_dict(),
                 "model_cfg": self.cfg.model.__dict__, "world": self.world, "tp_size": self.tp_size,
                 "seed": self.cfg.seed, "samples_consumed": self.samples_consumed,
                 "plan_spec": {k: v for k, v in vars(self.spec).items() if k != "length_dist"},
                 "length_dist": vars(self.spec.length_dist),
                 "rng": torch.get_rng_state(), "cuda_rng": torch.cuda.get_rng_state(self.device)}
        if self.cp_index == 0:     # one copy of the bf16 parameters per tensor-parallel shard
            state["params_bf16"] = self.bufs.params
        torch.save(state, path)
        return path

    def load_checkpoint(self, directory: str) -> None:
        """Resume from ``save_checkpoint`` files.  The number of ranks may differ from the run that
        wrote them as long as the tensor-parallel size is the same: the sharded fp32 optimizer state
        is then re-cut from the files of the old ranks that held this rank's parameters (the
        directory must be readable by every rank), and the random-number state starts afresh."""
        probe = os.path.join(directory, f"rank{self.rank:03d}.pt")
        if not os.path.exists(probe):
            probe = os.path.join(directory, "rank000.pt")
        meta = torch.load(probe, map_location="cpu", weights_only=False, mmap=True)
        assert meta.get("tp_size", 1) == self.tp_size, "resume needs the tensor-parallel size the checkpoint was written with"
        old_world = int(meta["world"])
        if old_world == self.world:
            state = torch.load(os.path.join(directory, f"rank{self.rank:03d}.pt"), map_location=self.device,
                               weights_only=False)
            self.optimizer.load_state_dict(state["optimizer"])
            torch.set_rng_state(state["rng"].cpu())
            torch.cuda.set_rng_state(state["cuda_rng"].cpu(), self.device)
        else:
            from .parallel.dist_optimizer import reshard_state
            tp = self.tp_size
            tp_index = self.rank % tp
            old_group = [c * tp + tp_index for c in range(old_world // tp)]   # old ranks with this rank's parameters
            state = meta

            def old_states():
                for r in old_group:
                    f = torch.load(os.path.join(directory, f"rank{r:03d}.pt"), map_location="cpu", weights_only=False,
                                   mmap=True)
                    yield f["optimizer"]

            o = self.optimizer
            self.optimizer.load_state_dict(reshard_state(old_states(), o.buckets, o.bufs.world, o.bufs.rank))
        self.iteration = int(state["iteration"])
        self.samples_consumed = int(state.get("samples_consumed", 0))
        # every rank's bf16 parameters are rebuilt from the sharded fp32 master weights: each rank
        # stores its slices (same slicing formula as the optimizer) into every peer's buffer
        self.optimizer.rebuild_params()
        torch.cuda.synchronize(self.device)
        self.check_status()
        self.plans.close()
        self.plans = self._make_plan_service(self.iteration)


def dataset_batches(eng: "TrainEngine", n_samples: int, dist_: synth.LengthDist, seed: int = 24):
    """Generator of ``DCPDataLoader`` items for ``eng`` over a seeded synthetic corpus: the dataset ->
    token-budget batch sampler -> planning dataloader route.  Every rank iterates the same sampler
    (same seed), so all ranks see the same batches; the sampler resumes after the samples the engine
    has already trained on (``eng.samples_consumed``, part of the checkpoint) and starts a new epoch
    when the corpus is exhausted."""
    from .core.common import ModelSpec, get_default_execution_context
    from .data.dataloader import DCPDataLoader, TrainingSpec
    from .data.datasets import OrderedBatchSampler, SyntheticLengthDataset
    m, spec = eng.local_model, eng.spec
    ds = SyntheticLengthDataset(n_samples, dist_, vocab=m.vocab, seed=seed)
    sampler = OrderedBatchSampler(ds, spec.tokens_per_step, shuffle=True, seed=seed)
    per_epoch = sum(len(b) for b in sampler._batches())
    sampler.epoch, sampler.consumed_samples = divmod(eng.samples_consumed, max(per_epoch, 1)) if per_epoch else (0, 0)
    ts = TrainingSpec(get_default_execution_context(spec.dcp_size, 1), ModelSpec(m.head_dim, m.n_heads, m.n_kv_heads),
                      mask_type=spec.mask, block_size=spec.block_size, head_block_size=spec.head_block_size or m.n_heads,
                      dcp_size=spec.dcp_size, use_block_size_heuristic=0)
    loader = DCPDataLoader(ts, ds, dcp_rank=eng.cp_index, batch_sampler=sampler, world=spec.world,
                           num_preprocess_workers=eng.cfg.planner_workers, prefetch_factor=eng.cfg.lookahead,
                           build_instruction_plans=False)
    try:
        while True:
            for item in loader:
                yield item
    finally:
        loader.close()


def init_distributed():
    """(rank, world, local_rank, group): NCCL process group when launched with several ranks."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    group = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        group = dist.group.WORLD
    return rank, world, local, group


def add_dcp_args(ap: argparse.ArgumentParser) -> None:
    """The reference's ``--dcp-*`` training flags (benchmark/mlm/dcp_args.py:1-42), same names and
    meanings.  Cost-model and tolerance flags default to None = this framework's B200 defaults."""
    g = ap.add_argument_group("dcp")
    g.add_argument("--disable-dcp", action="store_true",
                   help="no context parallelism: every rank is its own group (pure data parallel)")
    g.add_argument("--dcp-intra-node-lat", type=float, default=None, help="ms")
    g.add_argument("--dcp-intra-node-bw", type=float, default=None, help="Gbps")
    g.add_argument("--dcp-inter-node-lat", type=float, default=None, help="ms")
    g.add_argument("--dcp-inter-node-bw", type=float, default=None, help="Gbps")
    g.add_argument("--dcp-max-tflops", type=float, default=None)
    g.add_argument("--dcp-max-mem-bw", type=float, default=None, help="GB/s")
    g.add_argument("--dcp-prefetch-planner-num-workers", type=int, default=2)
    g.add_argument("--dcp-prefetch-listener-num-workers", type=int, default=1,
                   help="accepted for compatibility: plans are computed per rank, nothing is listened for")
    g.add_argument("--dcp-block-size", type=int, default=2048)
    g.add_argument("--dcp-head-block-size", type=int, default=0, help="0 = all heads of a rank in one block")
    g.add_argument("--dcp-use-block-size-heuristic", type=int, default=0)
    g.add_argument("--dcp-mem-imbalance-epsilon", type=float, default=None)
    g.add_argument("--dcp-comp-imbalance-epsilon", type=float, default=None)
    g.add_argument("--dcp-inter-node-comp-imbalance-factor", type=float, default=None)
    g.add_argument("--dcp-global-batch-size-in-tokens", type=int, default=131072)
    g.add_argument("--dcp-dataset-split", default="train", help="used by dataset-backed loaders; synthetic data ignores it")
    g.add_argument("--dcp-dataset-text-key", default="text")
    g.add_argument("--dcp-use-cudagraph", action="store_true",
                   help="accepted for compatibility: per-iteration kernel tables make every step's launch list "
                        "different, and the fused executor already issues only a handful of launches per layer")
    g.add_argument("--dcp-mask-type", default="causal")


def main(argv=None):
    ap = argparse.ArgumentParser(description="Synthetic-data DCP training loop")
    ap.add_argument("--model", default="llama3-8b", choices=["llama3-8b", "tiny"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--tokens-per-step", type=int, default=None, help="alias of --dcp-global-batch-size-in-tokens")
    ap.add_argument("--dcp-size", type=int, default=0, help="ranks per context-parallel group (0 = all ranks)")
    ap.add_argument("--tensor-model-parallel-size", "--tp-size", dest="tp_size", type=int, default=1)
    ap.add_argument("--length-dist", default="lognormal8k", choices=["lognormal8k", "lognormal16k", "mixture"])
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--log-interval", type=int, default=1)
    ap.add_argument("--save", default=None)
    ap.add_argument("--load", default=None)
    ap.add_argument("--activation-budget-gb", type=float, default=None)
    ap.add_argument("--dataset", default="none", choices=["none", "synthetic"],
                    help="none: batches are synthesised inside the plan service; synthetic: a Dataset of seeded "
                         "variable-length samples goes through OrderedBatchSampler and DCPDataLoader, the route a "
                         "tokenised corpus takes (benchmark/mlm/pretrain_gpt.py:853-877 in the reference)")
    ap.add_argument("--dataset-samples", type=int, default=4096)
    add_dcp_args(ap)
    args = ap.parse_args(argv)
    rank, world, local, group = init_distributed()
    dists = {"lognormal8k": synth.LOGNORMAL_8K, "lognormal16k": synth.LOGNORMAL_16K, "mixture": synth.MIXTURE}
    model = LLAMA3_8B if args.model == "llama3-8b" else tiny_config()
    tokens = args.tokens_per_step or args.dcp_global_batch_size_in_tokens
    cost = {"intra_node_lat": args.dcp_intra_node_lat, "intra_node_bw": args.dcp_intra_node_bw,
            "inter_node_lat": args.dcp_inter_node_lat, "inter_node_bw": args.dcp_inter_node_bw,
            "max_tflops": args.dcp_max_tflops, "max_mem_bw": args.dcp_max_mem_bw}
    cfg = EngineConfig(model=model, tokens_per_step=tokens, dcp_size=1 if args.disable_dcp else args.dcp_size,
                       block_size=args.dcp_block_size, mask=args.dcp_mask_type, length_dist=dists[args.length_dist], lr=args.lr, planner_workers=args.dcp_prefetch_planner_num_workers,
                       head_block_size=args.dcp_head_block_size,
                       use_block_size_heuristic=bool(args.dcp_use_block_size_heuristic),
                       mem_imbalance_epsilon=args.dcp_mem_imbalance_epsilon,
                       comp_imbalance_epsilon=args.dcp_comp_imbalance_epsilon,
                       inter_node_comp_imbalance_factor=args.dcp_inter_node_comp_imbalance_factor,
                       cost_model=cost if any(v is not None for v in cost.values()) else None,
                       activation_budget_gb=args.activation_budget_gb, tp_size=args.tp_size)
    eng = TrainEngine(cfg, torch.device("cuda", local), group)
    if args.load:
        eng.load_checkpoint(args.load)
    batches = None
    if args.dataset != "none":
        batches = iter(dataset_batches(eng, args.dataset_samples, dists[args.length_dist]))
    t_last = time.time()
    for it in range(eng.iteration, eng.iteration + args.iters):
        loss = eng.train_step(next(batches) if batches is not None else None)
        if rank == 0 and (it + 1) % args.log_interval == 0:
            now = time.time()
            ms = (now - t_last) * 1000 / args.log_interval
            t_last = now
            print(f" iteration {it + 1:8d} | elapsed time per iteration (ms): {ms:.1f} | Training loss: {loss:.6f}",
                  flush=True)
    if args.save:
        eng.save_checkpoint(args.save)
    eng.close()


if __name__ == "__main__":
    main()

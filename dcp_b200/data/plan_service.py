"""Ahead-of-time planning of training iterations in worker processes.

Planning one iteration (block generation, hypergraph placement, staging, lowering) is CPU work
that takes a sizeable fraction of a second for 100k-token batches; it is hidden behind GPU work
by planning iterations ahead in a pool of processes.  Planning is deterministic in its inputs, so
every rank plans the same batch independently and keeps only its own share: no plan has to cross
ranks and no key-value server is needed (the reference ships pickled plans through Redis,
dcp/data/dataloader.py:519-740, 754-932, dcp/data/kv_redis.py:22-135).

``plan_iteration`` is the pure function; ``PlanService`` adds the look-ahead pool.
"""
from __future__ import annotations

import concurrent.futures as cf
import multiprocessing as mp
import os
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..core.common import get_default_execution_context
from ..core.instructions import BufferType
from ..planner import masks as mask_lib
from ..planner.compiler import CompilerConfig, InstrCompiler
from ..planner.lowering import FusedProgram, lower_all, lower_plans
from ..planner.workload import generate_workload, pad_seqlens
from ..runtime.layout import LocalLayout, seq_token_offsets
from . import synth


@dataclass
class PlanSpec:
    """Everything that determines the plans of one iteration."""
    world: int                      # ranks taking part in training
    dcp_size: int                   # ranks per context-parallel group (world % dcp_size == 0)
    tokens_per_step: int            # global token budget
    n_heads: int
    n_kv_heads: int
    head_dim: int = 128
    block_size: int = 2048
    head_block_size: int = 0        # 0 -> all heads in one block
    mask: str = "causal"            # a name from planner.masks.MASK_FNS ("mixed" draws per sequence)
    length_dist: synth.LengthDist = field(default_factory=lambda: synth.LOGNORMAL_8K)
    vocab: int = 128256
    seed: int = 0
    n_stages: Optional[int] = None
    build_backward: bool = True
    build_instruction_plans: bool = False   # also emit ExecutionPlans (plan-interpreting executors)
    lower_from_plans: bool = False          # derive the fused tables from the ExecutionPlan instruction streams
    # planner knobs (None = the defaults of CompilerConfig / the cost models)
    mem_imbalance_epsilon: Optional[float] = None
    comp_imbalance_epsilon: Optional[float] = None
    inter_node_comp_imbalance_factor: Optional[float] = None
    use_block_size_heuristic: bool = False
    cost_model: Optional[dict] = None       # intra/inter node latency + bandwidth, max_tflops, max_mem_bw
    cache_dir: Optional[str] = None         # plans are stored here by batch signature and reused (e.g. after a resume)
    qkv_dtype: str = "bfloat16"             # dtype of the attention buffers in the instruction plans (plan interpreter)


@dataclass
class RankPlan:
    iteration: int
    program: FusedProgram
    tokens: torch.Tensor            # int64 [local tokens] (pinned by the consumer)
    labels: torch.Tensor
    positions: torch.Tensor
    n_global_tokens: int
    n_group_tokens: int
    seqlens: List[int]
    plan_seconds: float
    fw_plan: object = None
    bw_plan: object = None
    fw_workload: object = None
    bw_workload: object = None


def split_batch_over_groups(seqlens: Sequence[int], n_groups: int) -> List[List[int]]:
    """Indices of the sequences each context-parallel group takes: longest first onto the group
    with the least attention work (~ len^2) so far."""
    load = [0.0] * n_groups
    out: List[List[int]] = [[] for _ in range(n_groups)]
    for i in sorted(range(len(seqlens)), key=lambda i: -seqlens[i]):
        g = load.index(min(load))
        out[g].append(i)
        load[g] += float(seqlens[i]) ** 2 + 4096.0 * seqlens[i]
    return [sorted(x) for x in out]


def plan_iteration(spec: PlanSpec, iteration: int, rank: int) -> RankPlan:
    """Synthesise iteration ``iteration``'s batch from the spec's length distribution and plan it."""
    seed = spec.seed * 1000003 + iteration
    n_groups = spec.world // spec.dcp_size
    members = None
    if n_groups > 1:
        # data parallel over context-parallel groups: every group draws its own sub-batch with an
        # equal token budget (equal dense work per rank), as independent data-parallel replicas do
        seqlens, members = [], []
        for g in range(n_groups):
            part = synth.sample_seqlens(spec.tokens_per_step // n_groups, spec.length_dist, seed * 64 + g + 1)
            members.append(list(range(len(seqlens), len(seqlens) + len(part))))
            seqlens += part
    else:
        seqlens = synth.sample_seqlens(spec.tokens_per_step, spec.length_dist, seed)
    batch = synth.make_token_batch(seqlens, spec.vocab, seed)
    info = synth.assign_mask_kinds(seqlens, seed) if spec.mask == "mixed" else None
    if spec.cache_dir:
        return _cached_plan(spec, iteration, rank, seqlens, batch, info, members)
    return plan_batch(spec, iteration, rank, seqlens, batch, info, group_members=members)


def plan_iteration_all(spec: PlanSpec, iteration: int) -> Dict[int, RankPlan]:
    """Same batch as ``plan_iteration`` draws for ``iteration``, planned once for every rank."""
    seed = spec.seed * 1000003 + iteration
    n_groups = spec.world // spec.dcp_size
    members = None
    if n_groups > 1:
        seqlens, members = [], []
        for g in range(n_groups):
            part = synth.sample_seqlens(spec.tokens_per_step // n_groups, spec.length_dist, seed * 64 + g + 1)
            members.append(list(range(len(seqlens), len(seqlens) + len(part))))
            seqlens += part
    else:
        seqlens = synth.sample_seqlens(spec.tokens_per_step, spec.length_dist, seed)
    batch = synth.make_token_batch(seqlens, spec.vocab, seed)
    info = synth.assign_mask_kinds(seqlens, seed) if spec.mask == "mixed" else None
    return plan_batch_all(spec, iteration, seqlens, batch, info, group_members=members)


def batch_signature(spec: PlanSpec, rank: int, seqlens: Sequence[int], mask_fn_info, group_members) -> str:
    """Stable key of everything a rank's plan depends on (the iteration number is not part of it:
    the same batch planned at another step gives the same plan)."""
    import hashlib
    fields = {k: v for k, v in vars(spec).items() if k not in ("cache_dir", "seed")}
    fields["length_dist"] = vars(spec.length_dist) if hasattr(spec.length_dist, "__dict__") else str(spec.length_dist)
    text = repr((sorted(fields.items(), key=lambda kv: kv[0]), rank, list(map(int, seqlens)), mask_fn_info, group_members))
    return hashlib.sha1(text.encode()).hexdigest()


def _cached_plan(spec, iteration, rank, seqlens, batch, mask_fn_info, group_members):
    """Plan-cache lookup / fill around ``plan_batch``; token arrays are re-derived from the batch on
    every call, so only planning work is saved."""
    import pickle
    key = batch_signature(spec, rank, seqlens, mask_fn_info, group_members)
    path = os.path.join(spec.cache_dir, f"plan_{key}.pkl")
    if os.path.exists(path):
        with open(path, "rb") as f:
            plan = pickle.load(f)
        plan.iteration = iteration
        return plan
    plan = plan_batch(spec, iteration, rank, seqlens, batch, mask_fn_info, group_members=group_members)
    os.makedirs(spec.cache_dir, exist_ok=True)
    tmp = f"{path}.{os.getpid()}.tmp"
    with open(tmp, "wb") as f:
        pickle.dump(plan, f)
    os.replace(tmp, path)            # atomic: a concurrent reader never sees a partial file
    return plan


def plan_batch(spec: PlanSpec, iteration: int, rank: int, seqlens: Sequence[int], batch: Dict[str, np.ndarray],
               mask_fn_info: Optional[List[dict]] = None, mask_fn=None,
               group_members: Optional[List[List[int]]] = None) -> RankPlan:
    """Plan one packed batch (``batch`` holds per-token arrays over the concatenated sequences) and
    return rank ``rank``'s share: its fused program, its tokens in local buffer order and, when
    requested, its instruction plans."""
    group_id = rank // spec.dcp_size
    return _plan_group(spec, iteration, group_id, seqlens, batch, mask_fn_info, mask_fn, group_members, only_rank=rank)[rank]


def plan_batch_all(spec: PlanSpec, iteration: int, seqlens: Sequence[int], batch: Dict[str, np.ndarray],
                   mask_fn_info: Optional[List[dict]] = None, mask_fn=None,
                   group_members: Optional[List[List[int]]] = None) -> Dict[int, RankPlan]:
    """Plan one packed batch once for every rank: each context-parallel group's sub-batch is placed,
    staged and lowered a single time and every rank's share is cut from that result.  This is the
    planner-process side of shared planning (the reference plans a batch once and publishes per-rank
    plans, dcp/data/dataloader.py:519-740)."""
    out: Dict[int, RankPlan] = {}
    for g in range(spec.world // spec.dcp_size):
        out.update(_plan_group(spec, iteration, g, seqlens, batch, mask_fn_info, mask_fn, group_members))
    return out


def _plan_group(spec: PlanSpec, iteration: int, group_id: int, seqlens: Sequence[int], batch: Dict[str, np.ndarray],
                mask_fn_info, mask_fn, group_members, only_rank: Optional[int] = None) -> Dict[int, RankPlan]:
    """Plans of the ranks of one context-parallel group (all of them, or just ``only_rank``)."""
    t0 = time.time()
    seqlens = [int(x) for x in seqlens]
    n_groups = spec.world // spec.dcp_size
    if group_members is not None:
        members = group_members[group_id]
    else:
        members = split_batch_over_groups(seqlens, n_groups)[group_id] if n_groups > 1 else list(range(len(seqlens)))
    raw = [seqlens[i] for i in members]
    cu_all = seq_token_offsets(seqlens)
    bs = spec.block_size
    if spec.use_block_size_heuristic:
        from ..planner.workload import block_size_heuristic
        bs = block_size_heuristic(raw, spec.dcp_size, 0.2, min_block_size=256, max_block_size=max(bs, 256))
    pad = pad_seqlens(raw, bs)
    info = [mask_fn_info[i] for i in members] if mask_fn_info is not None else None
    fn = mask_fn or mask_lib.get_mask_fn(spec.mask)
    mask = fn(raw, pad, torch.int32, info)
    ctx = get_default_execution_context(spec.dcp_size, 1)
    if spec.cost_model:
        from ..core.cost_model import AttnRooflineCostModel, CommunicationCostModel
        cm, c0, a0 = spec.cost_model, CommunicationCostModel(), AttnRooflineCostModel()
        pick = lambda key, default: default if cm.get(key) is None else cm[key]
        ctx.comm_cost_model = CommunicationCostModel(
            pick("inter_node_lat", c0.inter_node_latency), pick("inter_node_bw", c0.inter_node_bandwidth),
            pick("intra_node_lat", c0.intra_node_latency), pick("intra_node_bw", c0.intra_node_bandwidth))
        ctx.comp_cost_model = AttnRooflineCostModel(pick("max_tflops", a0.max_tflops), pick("max_mem_bw", a0.max_mem_bw))
    hbs = spec.head_block_size or spec.n_heads
    d = spec.head_dim
    wl = generate_workload((sum(pad), spec.n_heads, d), (sum(pad), 2, spec.n_kv_heads, d), raw, pad, bs, hbs,
                           ctx.comp_cost_model, mask, getattr(torch, spec.qkv_dtype))
    ccfg = CompilerConfig(n_stages=spec.n_stages)
    for name in ("mem_imbalance_epsilon", "comp_imbalance_epsilon", "inter_node_comp_imbalance_factor"):
        if getattr(spec, name) is not None:
            setattr(ccfg, name, getattr(spec, name))
    compiler = InstrCompiler(ctx, ccfg)
    fw_wl, bw_wl, fw_plans, bw_plans = compiler.compile(wl, generate_backward=spec.build_instruction_plans)
    lower = (lambda c, w, bb, only=None: lower_plans(c, w, fw_plans, bb, only)) if spec.lower_from_plans else lower_all
    only_dev = None if only_rank is None else (0, only_rank % spec.dcp_size)
    if only_dev is None or os.environ.get("DCP_B200_VALIDATE", "0") == "1":
        programs = lower(ctx, fw_wl, spec.build_backward)
        if os.environ.get("DCP_B200_VALIDATE", "0") == "1":
            # debug: check every rank's tables against each other before use
            from ..planner.validate import validate_programs
            validate_programs(programs)
    else:
        programs = lower(ctx, fw_wl, spec.build_backward, only=only_dev)
    out: Dict[int, RankPlan] = {}
    plan_s = time.time() - t0
    for group_rank in range(spec.dcp_size):
        dev = (0, group_rank)
        if only_dev is not None and dev != only_dev:
            continue
        lay = LocalLayout(fw_wl, dev)
        idx = []
        for _, m in lay.blocks.get(BufferType.LOCAL_Q, []):
            if m.head_id != 0:
                continue
            t0_tok = int(cu_all[members[m.seq_id]]) + m.block_id * bs
            idx.append(np.arange(t0_tok, t0_tok + m.n_tokens))
        idx = np.concatenate(idx) if idx else np.zeros(0, dtype=np.int64)
        to_t = lambda a: torch.from_numpy(np.ascontiguousarray(np.asarray(a)[idx]))
        keep = spec.build_instruction_plans
        out[group_id * spec.dcp_size + group_rank] = RankPlan(
            iteration, programs[dev], to_t(batch["tokens"]), to_t(batch["labels"]), to_t(batch["positions"]),
            int(sum(seqlens)), int(sum(raw)), list(seqlens), plan_s,
            fw_plans.get(dev) if keep else None, bw_plans.get(dev) if (keep and bw_plans) else None,
            fw_wl if keep else None, bw_wl if keep else None)
    return out


def _worker_init():
    torch.set_num_threads(1)


class PlanService:
    """Look-ahead planner: ``get(i)`` returns iteration i's plan and keeps ``lookahead`` more in flight."""

    def __init__(self, spec: PlanSpec, rank: int, n_workers: int = 2, lookahead: int = 3, start: int = 0):
        self.spec, self.rank = spec, rank
        self.lookahead = max(1, lookahead)
        self._pool = None
        if n_workers > 0:
            self._pool = cf.ProcessPoolExecutor(max_workers=n_workers, mp_context=mp.get_context("spawn"),
                                                initializer=_worker_init)
        self._pending: Dict[int, "cf.Future"] = {}
        self._next_submit = start
        self.wait_seconds = 0.0
        self.waits: List[float] = []          # seconds get() blocked, per call
        self.plan_seconds: List[float] = []   # planning time of every plan handed out

    def _submit_up_to(self, last: int) -> None:
        while self._next_submit <= last:
            i = self._next_submit
            if self._pool is not None:
                self._pending[i] = self._pool.submit(plan_iteration, self.spec, i, self.rank)
            self._next_submit += 1

    def get(self, iteration: int) -> RankPlan:
        self._submit_up_to(iteration + self.lookahead)
        if self._pool is None:
            return plan_iteration(self.spec, iteration, self.rank)
        t0 = time.time()
        fut = self._pending.pop(iteration, None)
        plan = fut.result() if fut is not None else plan_iteration(self.spec, iteration, self.rank)
        waited = time.time() - t0
        self.wait_seconds += waited
        self.waits.append(waited)
        self.plan_seconds.append(plan.plan_seconds)
        return plan

    def close(self) -> None:
        if self._pool is not None:
            self._pool.shutdown(wait=False, cancel_futures=True)
            self._pool = None


def _pickle_plans(spec: PlanSpec, iteration: int) -> Dict[int, bytes]:
    """Worker-process job of shared planning: plan once, hand back one pickled plan per rank."""
    import pickle
    import zlib
    # index tables compress three- to five-fold at level 1, which costs less than sending them
    return {r: zlib.compress(pickle.dumps(p, protocol=pickle.HIGHEST_PROTOCOL), 1)
            for r, p in plan_iteration_all(spec, iteration).items()}


class SharedPlanService:
    """One planning per batch for all ranks that need it.

    The planner rank (one per node; the engine picks local rank 0) runs the look-ahead pool; a worker
    plans a batch once for every rank and the planner rank publishes each rank's pickled share in a
    key-value store (``data.kv_store.KVStore``: TCPStore across processes, a dict in one process)
    under ``<name>/<iteration>/<rank>``.  Every other rank just ``get``s its key (bounded wait).  The
    ``readers`` consumers of one rank's plan (the tensor-parallel ranks of one context-parallel rank
    read the same plan) count their reads; the last one deletes the entry.  Same interface as
    ``PlanService``.  Role of the planner poller + per-rank KV entries + reader acknowledgement of
    dcp/data/dataloader.py:99-161, 519-740, 976-1137, without Redis.
    """

    def __init__(self, spec: PlanSpec, rank: int, store, is_planner: bool, n_workers: int = 4, lookahead: int = 3,
                 start: int = 0, readers: int = 1, name: str = "dcp_plans", timeout_s: float = 600.0):
        self.spec, self.rank, self.store, self.is_planner = spec, rank, store, is_planner
        self.lookahead, self.readers, self.name, self.timeout_s = max(1, lookahead), max(1, readers), name, timeout_s
        self._pool = None
        if is_planner:
            self._pool = cf.ProcessPoolExecutor(max_workers=max(1, n_workers), mp_context=mp.get_context("spawn"),
                                                initializer=_worker_init)
        self._pending: Dict[int, "cf.Future"] = {}
        self._next_submit = start
        self.wait_seconds = 0.0
        self.waits: List[float] = []
        self.plan_seconds: List[float] = []
        self.n_published = 0
        # DCP_DATALOADER_LOG_KV: every put / get / delete on the plan store goes to the dataloader log
        self._kv_log = None
        if os.environ.get("DCP_DATALOADER_LOG_KV", "0") not in ("0", "", "false", "False"):
            from ..utils.logger import create_logger
            self._kv_log = create_logger(f"dataloader.kv.r{rank}", prefix=f"kv r{rank}", log_file=f"dataloader/kv_r{rank}.log")

    def _log_kv(self, what: str, key: str, nbytes: int = 0) -> None:
        if self._kv_log is not None:
            self._kv_log.debug("%s %s (%d bytes)", what, key, nbytes)

    def _key(self, iteration: int, rank: int) -> str:
        return f"{self.name}/{iteration}/{rank}"

    def _publish(self, iteration: int, plans: Dict[int, bytes]) -> bytes:
        mine = None
        for r, blob in plans.items():
            if r == self.rank and self.readers == 1:
                mine = blob             # the planner's own share needs no round trip
                continue
            self.store.set(self._key(iteration, r), blob)
            self._log_kv("put", self._key(iteration, r), len(blob))
            if r == self.rank:
                mine = blob
        self.n_published += 1
        return mine

    def _publish_finished(self, upto_excl: int) -> None:
        """Publish iterations whose planning finished while the GPU was busy, so peers never wait for
        the planner rank to come around."""
        for i in sorted(k for k, f in self._pending.items() if k != upto_excl and f.done()):
            self._done[i] = self._publish(i, self._pending.pop(i).result())

    def get(self, iteration: int) -> RankPlan:
        import pickle
        t0 = time.time()
        if self.is_planner:
            if not hasattr(self, "_done"):
                self._done: Dict[int, bytes] = {}
            while self._next_submit <= iteration + self.lookahead:
                self._pending[self._next_submit] = self._pool.submit(_pickle_plans, self.spec, self._next_submit)
                self._next_submit += 1
            self._publish_finished(-1)
            if iteration in self._pending:
                self._done[iteration] = self._publish(iteration, self._pending.pop(iteration).result())
            blob = self._done.pop(iteration)
        else:
            blob = self.store.get(self._key(iteration, self.rank), self.timeout_s)
            self._log_kv("get", self._key(iteration, self.rank), len(blob))
        if not (self.is_planner and self.readers == 1):
            # reader acknowledgement: the last of the `readers` consumers removes the entry
            key = self._key(iteration, self.rank)
            if self.store.add(key + "/reads", 1) >= self.readers:
                self.store.delete(key)
                self.store.delete(key + "/reads")
                self._log_kv("delete", key)
        import zlib
        plan = pickle.loads(zlib.decompress(blob))
        waited = time.time() - t0
        self.wait_seconds += waited
        self.waits.append(waited)
        self.plan_seconds.append(plan.plan_seconds)
        return plan

    def close(self) -> None:
        if self._pool is not None:
            self._pool.shutdown(wait=False, cancel_futures=True)
            self._pool = None

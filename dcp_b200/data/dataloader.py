"""DCPDataLoader: batches of whole sequences -> per-rank local batch + plans.

Keeps the reference's data-facing API (dcp/data/dataloader.py:238-2056): ``TrainingSpec``,
``ExecutionPlanner.plan``, ``generate_workload`` and a ``DCPDataLoader`` that yields
``(local_batch, fw_exec_plan, bw_exec_plan, fw_workload_spec, bw_workload_spec, training_spec)``.
What changed is the machinery: planning runs in a local look-ahead process pool and every rank
derives its own share from the same deterministic plan, so there is no Redis server, poller
process or reader-acknowledgement protocol.  The yielded ``local_batch`` additionally carries the
``FusedProgram`` (key ``"program"``) the sm_100a executor consumes.
"""
from __future__ import annotations

import concurrent.futures as cf
import multiprocessing as mp
from dataclasses import dataclass, field
from typing import Callable, Iterator, List, Optional, Sequence

import numpy as np
import torch

from ..core.blocks import WorkloadSpec
from ..core.common import ExecutionContext, ModelSpec, get_default_execution_context
from ..core.instructions import DType
from ..planner import masks as mask_lib
from ..planner.compiler import CompilerConfig, InstrCompiler
from ..planner.workload import block_size_heuristic, generate_workload as _generate_workload_impl, pad_seqlens
from .plan_service import PlanSpec, RankPlan, _worker_init, plan_batch


class KVStoreMetaKeys:
    """Kept for API parity; the in-process plan service needs no key-value store."""
    DP_SIZE = "data_parallel_size"
    TP_SIZE = "tensor_parallel_size"
    PP_SIZE = "pipeline_parallel_size"
    N_ITERS = "n_iters"


@dataclass
class TrainingSpec:
    exec_context: ExecutionContext
    model_spec: ModelSpec
    mask_type: str = "causal"
    mask_dtype: int = DType.INT32
    qkv_dtype: int = DType.BFLOAT16
    block_size: int = 2048
    head_block_size: int = 1
    dcp_size: int = 1
    tensor_parallel_size: int = 1
    pipeline_parallel_size: int = 1
    n_microbatches: int = 1
    use_block_size_heuristic: int = 1
    mem_imbalance_epsilon: float = 0.03
    comp_imbalance_epsilon: float = 0.015
    inter_node_comp_imbalance_factor: float = 5.0


def generate_workload(q, kv, seq_lens, block_size, head_block_size, n_total_devices, n_devices_per_node,
                      comp_cost_model, attn_mask=None, causal=False, logger=None) -> WorkloadSpec:
    """Reference-shaped entry point: ``q`` / ``kv`` may be tensors or shapes; ``seq_lens`` raw lengths."""
    q_shape = tuple(q.shape) if hasattr(q, "shape") else tuple(q)
    kv_shape = tuple(kv.shape) if hasattr(kv, "shape") else tuple(kv)
    padded = pad_seqlens(seq_lens, block_size)
    dtype = q.dtype if hasattr(q, "dtype") else torch.bfloat16
    return _generate_workload_impl(q_shape, kv_shape, list(seq_lens), padded, block_size, head_block_size,
                                   comp_cost_model, None if causal and attn_mask is None else attn_mask, dtype)


class ExecutionPlanner:
    """Plans one batch for every device of a DCP group (dcp/data/dataloader.py:1689-1898)."""

    def __init__(self, node_rank: int, node_size: int, training_spec: TrainingSpec, mask_fn: Optional[Callable] = None):
        self.spec = training_spec
        self.node_rank, self.node_size = node_rank, node_size
        self.mask_fn = mask_fn
        self.block_size = training_spec.block_size

    def plan(self, raw_seqlens: Sequence[int], iteration_idx: Optional[int] = None, mask_fn_info=None):
        """-> (fw_plans, bw_plans, fw_workload, bw_workload, padded_seqlens)."""
        ts = self.spec
        ctx = ts.exec_context
        bs = ts.block_size
        if ts.use_block_size_heuristic:
            # the heuristic bounds the imbalance of a block-cyclic deal, not of the solver: reference tolerance
            bs = block_size_heuristic(raw_seqlens, ctx.n_devices, max(ts.mem_imbalance_epsilon, 0.2), min_block_size=256,
                                      max_block_size=max(ts.block_size, 256))
        self.block_size = bs
        padded = pad_seqlens(raw_seqlens, bs)
        fn = self.mask_fn or mask_lib.get_mask_fn(ts.mask_type)
        mask = fn(list(raw_seqlens), padded, torch.int32, mask_fn_info)
        ms = ts.model_spec
        wl = _generate_workload_impl((sum(padded), ms.n_heads, ms.head_dim),
                                     (sum(padded), 2, ms.n_query_groups, ms.head_dim), list(raw_seqlens), padded, bs,
                                     ts.head_block_size, ctx.comp_cost_model, mask, DType.to_torch(ts.qkv_dtype))
        cfg = CompilerConfig(ts.mem_imbalance_epsilon, ts.comp_imbalance_epsilon, ts.inter_node_comp_imbalance_factor)
        fw_wl, bw_wl, fw, bw = InstrCompiler(ctx, cfg, iteration_idx).compile(wl)
        return fw, bw, fw_wl, bw_wl, padded


def _collate(samples: List[dict]):
    seqlens = [int(s["tokens"].numel()) for s in samples]
    cat = lambda k: np.concatenate([np.asarray(s[k]) for s in samples])
    labels = cat("labels").astype(np.int64)
    if "loss_mask" in samples[0]:
        labels = np.where(cat("loss_mask") > 0, labels, -100)
    batch = {"tokens": cat("tokens").astype(np.int64), "labels": labels,
             "positions": cat("position_ids").astype(np.int64)}
    info = [s["mask_fn_info"] for s in samples] if "mask_fn_info" in samples[0] else None
    return seqlens, batch, info


def _plan_job(spec: PlanSpec, iteration: int, rank: int, seqlens, batch, info):
    return plan_batch(spec, iteration, rank, seqlens, batch, info)


class DCPDataLoader:
    """Iterates a dataset with a token-budget batch sampler and plans ``prefetch_factor`` batches
    ahead in ``num_preprocess_workers`` processes."""

    def __init__(self, training_spec: TrainingSpec, dataset, is_kv_host: bool = False, node_rank: int = 0,
                 node_local_rank: int = 0, node_size: int = 1, dcp_rank: int = 0, pp_rank: int = 0, tp_rank: int = 0,
                 batch_size=None, start_poller: bool = False, shuffle: bool = False, sampler=None, batch_sampler=None,
                 num_workers: int = 0, num_preprocess_workers: int = 2, pin_memory: bool = False,
                 drop_last: bool = False, timeout: float = 0, *, prefetch_factor: int = 2,
                 persistent_workers: bool = False, input_key: str = "text", mask_fn: Optional[Callable] = None,
                 mask_fn_extra_keys=None, is_dryrun: bool = False, world: Optional[int] = None,
                 build_instruction_plans: bool = True):
        assert batch_sampler is not None, "pass an OrderedBatchSampler (token-budget batches)"
        assert 0 <= pp_rank < max(1, training_spec.pipeline_parallel_size), \
            f"pp_rank ({pp_rank}) must be smaller than pipeline_parallel_size ({training_spec.pipeline_parallel_size})"
        assert 0 <= tp_rank < max(1, training_spec.tensor_parallel_size), \
            f"tp_rank ({tp_rank}) must be smaller than tensor_parallel_size ({training_spec.tensor_parallel_size})"
        self.training_spec, self.dataset, self.batch_sampler = training_spec, dataset, batch_sampler
        self.dcp_rank, self.pin_memory, self.is_dryrun = dcp_rank, pin_memory, is_dryrun
        # pipeline stages read the same plans as their first stage (attention placement does not depend
        # on the layer range a stage holds); kept so a caller can tell the stages' loaders apart
        self.pp_rank, self.tp_rank = pp_rank, tp_rank
        ms = training_spec.model_spec
        self.plan_spec = PlanSpec(world or training_spec.dcp_size, training_spec.dcp_size, 0, ms.n_heads,
                                  ms.n_query_groups, ms.head_dim, training_spec.block_size,
                                  training_spec.head_block_size if training_spec.head_block_size != 1 else 0,
                                  training_spec.mask_type, build_instruction_plans=build_instruction_plans)
        self.prefetch = max(1, prefetch_factor)
        self._pool = None
        if num_preprocess_workers > 0:
            self._pool = cf.ProcessPoolExecutor(num_preprocess_workers, mp_context=mp.get_context("spawn"),
                                                initializer=_worker_init)

    def get_num_iters(self) -> int:
        return len(self.batch_sampler)

    def __len__(self) -> int:
        return len(self.batch_sampler)

    def __iter__(self) -> Iterator:
        pending: List = []
        it = 0

        def submit(indices, i):
            seqlens, batch, info = _collate([self.dataset[j] for j in indices])
            if self._pool is None:
                return plan_batch(self.plan_spec, i, self.dcp_rank, seqlens, batch, info)
            return self._pool.submit(_plan_job, self.plan_spec, i, self.dcp_rank, seqlens, batch, info)

        for indices in self.batch_sampler:
            pending.append(submit(indices, it))
            it += 1
            if len(pending) > self.prefetch:
                yield self._finish(pending.pop(0))
        while pending:
            yield self._finish(pending.pop(0))

    def _finish(self, item):
        plan: RankPlan = item.result() if hasattr(item, "result") else item
        pin = (lambda t: t.pin_memory()) if self.pin_memory and torch.cuda.is_available() else (lambda t: t)
        local_batch = {"tokens": pin(plan.tokens)[None], "labels": pin(plan.labels)[None],
                       "position_ids": pin(plan.positions)[None], "loss_mask": (plan.labels >= 0).float()[None],
                       "program": plan.program, "seqlens": plan.seqlens, "n_global_tokens": plan.n_global_tokens}
        return local_batch, plan.fw_plan, plan.bw_plan, plan.fw_workload, plan.bw_workload, self.training_spec

    def close(self) -> None:
        if self._pool is not None:
            self._pool.shutdown(wait=False, cancel_futures=True)
            self._pool = None

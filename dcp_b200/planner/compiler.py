"""Workload -> placement -> local buffer layout -> forward and backward plans.

``InstrCompiler.compile`` keeps the reference's contract (dcp/core/compiler.py:62-364): it
partitions the workload, numbers each device's blocks in (head block, sequence, token block)
order, schedules the forward plan, derives and schedules the backward workload, and attaches
``local_cu_seqlens`` to every plan.  Partition results and plans can be saved to / loaded from
disk for offline replay through the same environment variables as the reference.
"""
from __future__ import annotations

import os
import pickle
import time
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

from ..core.blocks import BlockType, Device, WorkloadSpec
from ..core.common import ExecutionContext
from ..core.instructions import ExecutionPlan
from ..utils.logger import create_logger, read_env_bool
from .partition import (HGPSolver, assign_device_by_heuristic, construct_and_partition_graph_multiconstraint)
from .scheduler import convert_forward_to_backward, schedule


@dataclass
class CompilerConfig:
    # Balance tolerances of the placement.  The reference defaults to 0.2 / 0.2
    # (dcp/core/compiler.py:62-110), trading balance for less traffic over InfiniBand.  On one
    # NVSwitch node a pulled block costs ~1% of the attention time it feeds, while every percent
    # of imbalance is a percent of step time (the slowest rank sets the pace at each barrier), so
    # the defaults here are tight; an infeasible tolerance is relaxed automatically by the solver.
    mem_imbalance_epsilon: float = 0.03
    comp_imbalance_epsilon: float = 0.015
    inter_node_comp_imbalance_factor: float = 5.0
    reduction_schedule_algo: str = "delayed"
    solver: str = HGPSolver.NATIVE
    n_stages: Optional[int] = None       # None -> DCP_N_STAGES (default 4)
    pipeline_algo: str = "greedy"
    seed: int = 42


def assign_local_buffer_indices(workload: WorkloadSpec, d2i: Dict[Device, list], d2o: Dict[Device, list]):
    """Index every device's blocks inside its Local* buffers: per block type, sorted by
    (head block, sequence, token block).  Returns {device: cumulative Q-block token counts}."""
    bm = workload.block_mapping
    in_idx, out_idx, cu = {}, {}, {}
    for d in d2i:
        in_idx[d], out_idx[d] = {}, {}
        for metas, ids, idx, types in ((bm.input_id_to_meta, d2i[d], in_idx[d], (BlockType.Q, BlockType.KV)),
                                       (bm.output_id_to_meta, d2o[d], out_idx[d], (BlockType.Out, BlockType.LSE))):
            for t in types:
                same = sorted((i for i in ids if metas[i].type == t),
                              key=lambda i: (metas[i].head_id, metas[i].seq_id, metas[i].block_id))
                for k, i in enumerate(same):
                    idx[i] = k
                if t == BlockType.Q:
                    acc = [0]
                    for i in same:
                        acc.append(acc[-1] + metas[i].n_tokens)
                    cu[d] = acc
    bm.input_id_to_buffer_index = in_idx
    bm.output_id_to_buffer_index = out_idx
    return cu


class InstrCompiler:
    def __init__(self, context: ExecutionContext, config: Optional[CompilerConfig] = None,
                 iteration_idx: Optional[int] = None):
        self.context = context
        self.config = config or CompilerConfig()
        self.iteration_idx = iteration_idx
        log_file = f"compiler/compiler_iter{iteration_idx}.log" if iteration_idx is not None else "compiler/compiler.log"
        self.logger = create_logger(name="InstrCompiler", log_file=log_file)
        self.timings: Dict[str, float] = {}

    def _partition(self, workload: WorkloadSpec):
        load = os.environ.get("DCP_DEBUG_LOAD_PARTITION_RESULTS_FILE") if read_env_bool(
            "DCP_DEBUG_LOAD_PARTITION_RESULTS") else None
        if load and os.path.exists(load):
            with open(load, "rb") as f:
                saved = pickle.load(f)
            workload.work_to_device_map, workload.input_to_device_map, workload.output_to_device_map = saved["maps"]
            return saved["d2w"], saved["d2i"], saved["d2o"]
        cfg = self.config
        if read_env_bool("DCP_DEBUG_OVERRIDE_PARTITION_WITH_HEURISTIC") or cfg.solver == HGPSolver.HEURISTIC:
            res = assign_device_by_heuristic(self.context, workload)
        else:
            res = construct_and_partition_graph_multiconstraint(
                self.context, workload, cfg.mem_imbalance_epsilon, cfg.comp_imbalance_epsilon,
                cfg.inter_node_comp_imbalance_factor, solver=cfg.solver, logger=self.logger, seed=cfg.seed)
        if read_env_bool("DCP_DEBUG_SAVE_PARTITION_RESULTS"):
            path = os.environ.get("DCP_DEBUG_SAVE_PARTITION_RESULTS_FILE", "dcp_partition.pkl")
            with open(path, "wb") as f:
                pickle.dump({"d2w": res[0], "d2i": res[1], "d2o": res[2],
                             "maps": (workload.work_to_device_map, workload.input_to_device_map,
                                      workload.output_to_device_map)}, f)
        return res

    def _debug_placement(self, workload: WorkloadSpec, d2w, d2i) -> None:
        """DCP_LOG_WORKLOAD_SPEC: workload summary; DCP_LOG_GRAPH_PARTITION: per-device compute and
        memory load of the placement; DCP_DEBUG_VISUALIZE_WORKLOAD_SPEC: block -> device map as
        text in the log and as a figure description under DCP_DEBUG_VISUALIZE_WORKLOAD_SPEC_DIR."""
        if read_env_bool("DCP_LOG_WORKLOAD_SPEC"):
            self.logger.info("workload: %d work units, %d input blocks, %d output blocks, total cost %.3f ms",
                             len(workload.workloads), len(workload.input_sizes), len(workload.output_sizes),
                             float(sum(workload.workloads)))
        if read_env_bool("DCP_LOG_GRAPH_PARTITION"):
            for d in sorted(d2w):
                self.logger.info("placement device %s: %d work units, cost %.3f ms, %d input blocks, %.1f MB", d,
                                 len(d2w[d]), float(sum(workload.workloads[w] for w in d2w[d])), len(d2i[d]),
                                 sum(workload.input_sizes[i] for i in d2i[d]) / 1e6)
        if read_env_bool("DCP_DEBUG_VISUALIZE_WORKLOAD_SPEC"):
            from ..utils.visualization import visualize_workload_spec_figure, visualize_workload_spec_tty
            self.logger.info("block -> device map\n%s",
                             visualize_workload_spec_tty(workload, self.context.n_devices_per_node))
            out_dir = os.environ.get("DCP_DEBUG_VISUALIZE_WORKLOAD_SPEC_DIR",
                                     os.environ.get("DCP_LOGGING_DEBUG_DIR", "./debug"))
            os.makedirs(out_dir, exist_ok=True)
            for ext in ("json", "svg"):         # graph description and the drawn figure
                visualize_workload_spec_figure(workload, os.path.join(out_dir, f"workload_iter{self.iteration_idx}.{ext}"),
                                               self.context.n_devices_per_node)

    def compile(self, workload: WorkloadSpec, generate_backward: bool = True) -> Tuple[
            WorkloadSpec, Optional[WorkloadSpec], Dict[Device, ExecutionPlan], Optional[Dict[Device, ExecutionPlan]]]:
        load_plans = os.environ.get("DCP_DEBUG_LOAD_EXEC_PLANS_FILE") if read_env_bool("DCP_DEBUG_LOAD_EXEC_PLANS") else None
        if load_plans and os.path.exists(load_plans):
            with open(load_plans, "rb") as f:
                return pickle.load(f)
        cfg = self.config
        t0 = time.time()
        d2w, d2i, d2o = self._partition(workload)
        t1 = time.time()
        self._debug_placement(workload, d2w, d2i)
        cu = assign_local_buffer_indices(workload, d2i, d2o)
        fw_plans, _ = schedule(self.context, workload, self.context.comm_cost_model, self.logger, True,
                               cfg.pipeline_algo, cfg.n_stages)
        t2 = time.time()
        bw_workload, bw_plans = None, None
        if generate_backward:
            bw_workload = convert_forward_to_backward(workload, self.context.comp_cost_model, self.logger)
            bw_plans, _ = schedule(self.context, bw_workload, self.context.comm_cost_model, self.logger, False,
                                   cfg.pipeline_algo, cfg.n_stages)
        t3 = time.time()
        for d, plan in fw_plans.items():
            plan.local_cu_seqlens = cu.get(d, [0])
        if bw_plans:
            for d, plan in bw_plans.items():
                plan.local_cu_seqlens = cu.get(d, [0])
        self.timings = {"partition_s": t1 - t0, "schedule_fw_s": t2 - t1, "schedule_bw_s": t3 - t2}
        self.logger.debug("compile timings %s", self.timings)
        result = (workload, bw_workload, fw_plans, bw_plans)
        if read_env_bool("DCP_SAVE_EXEC_PLAN_FOR_DEBUG"):
            with open(os.environ.get("DCP_DEBUG_LOAD_EXEC_PLANS_FILE", "dcp_exec_plans.pkl"), "wb") as f:
                pickle.dump(result, f)
        return result

"""Split each device's work into pipeline stages so transfers overlap the previous stage's math.

Stage 0 holds the work whose inputs are all local.  Every later stage is built by the native
greedy selector under a per-device, per-stage traffic budget (1.2 x the even share of the total
volume); the last stage is flushed with an unlimited budget.  On multi-node clusters a remote
block needed by several devices of one node crosses the network once and is relayed inside the
node in a second phase.  Mirrors dcp/core/pipeline.py:513-839, with two deliberate changes:
NVLink (intra-node) traffic is budgeted too, because on one NVSwitch node it is all there is, and
the native selector is deterministic.
"""
from __future__ import annotations

import os
from collections import defaultdict
from typing import Dict, List, Optional, Sequence, Set, Tuple

from ..core.blocks import DataBlockMeta, Device

StageWork = Dict[Device, List[int]]
StageComm = Dict[Device, List[Tuple[int, Device]]]  # dst -> [(input id, src)]


def default_n_stages() -> int:
    if os.environ.get("DCP_FORCE_SINGLE_STAGE", "0") not in ("0", "", "false", "False"):
        return 1
    return int(os.environ.get("DCP_N_STAGES", "4"))


def _native():
    from .. import _planner
    return _planner


def generate_pipelines_n_stages(n_stages: int, all_devices: Sequence[Device], workload_costs: Sequence[float],
                                workload_input_map: Sequence[Sequence[int]],
                                input_to_meta_map: Dict[int, DataBlockMeta], input_sizes: Sequence[float],
                                workload_to_device_map: Dict[int, Device], input_to_device_map: Dict[int, Device],
                                is_bw: bool, logger=None, budget_intra_node: bool = True,
                                two_phase: Optional[bool] = None):
    """-> (work_per_stage, comm_per_stage, second_phase_comm_per_stage), each a list of n_stages+1
    per-device dicts; comm_per_stage[s] must complete before the compute of stage s."""
    devices = sorted(tuple(d) for d in all_devices)
    n_dev = len(devices)
    device_work: Dict[Device, List[int]] = {d: [] for d in devices}
    for w in sorted(workload_to_device_map):
        device_work[tuple(workload_to_device_map[w])].append(w)
    local_inputs: Dict[Device, Dict[int, int]] = {d: {} for d in devices}
    for i, d in input_to_device_map.items():
        local_inputs[tuple(d)][i] = -1

    # total traffic if every consumer fetched every missing block once
    inter_total = intra_total = 0.0
    seen = set()
    for w, d in workload_to_device_map.items():
        d = tuple(d)
        for i in workload_input_map[w]:
            src = tuple(input_to_device_map[i])
            if src == d or (d, i) in seen:
                continue
            seen.add((d, i))
            if src[0] == d[0]:
                intra_total += input_sizes[i]
            else:
                inter_total += input_sizes[i]
    stages = max(1, n_stages)
    inter_budget = {d: inter_total / n_dev / stages * 1.2 for d in devices}
    intra_budget = {d: intra_total / n_dev / stages * 1.2 for d in devices} if budget_intra_node else {}

    type_map = [input_to_meta_map[i].type for i in range(len(input_sizes))]
    work_per_stage: List[StageWork] = []
    comm_per_stage: List[StageComm] = []
    scheduled: Set[int] = set()
    first: StageWork = {d: [] for d in devices}
    for w in range(len(workload_costs)):
        d = tuple(workload_to_device_map[w])
        if all(tuple(input_to_device_map[i]) == d for i in workload_input_map[w]):
            first[d].append(w)
            scheduled.add(w)
    work_per_stage.append(first)
    comm_per_stage.append({d: [] for d in devices})

    greedy = _native().greedy_selection_per_device
    costs, sizes = list(map(float, workload_costs)), list(map(float, input_sizes))
    win = [list(x) for x in workload_input_map]
    inf = {d: float("inf") for d in devices}
    for stage_id in range(stages):
        unlocked, comms, local_inputs = greedy(set(devices), scheduled, costs, sizes, win, type_map, device_work,
                                               local_inputs, inter_budget, is_bw, stage_id, None, intra_budget)
        stage_work = {d: sorted(unlocked.get(d, ())) for d in devices}
        stage_comm = {d: list(comms.get(d, ())) for d in devices}
        for ws in stage_work.values():
            scheduled.update(ws)
        if stage_id == stages - 1:
            unlocked, comms, local_inputs = greedy(set(devices), scheduled, costs, sizes, win, type_map, device_work,
                                                   local_inputs, inf, is_bw, stage_id, None, inf)
            for d in devices:
                extra = sorted(unlocked.get(d, ()))
                stage_work[d] = sorted(set(stage_work[d]) | set(extra))
                scheduled.update(extra)
                stage_comm[d].extend(comms.get(d, ()))
        work_per_stage.append(stage_work)
        comm_per_stage.append(stage_comm)
    assert scheduled == set(range(len(workload_costs))), "every work unit must land in exactly one stage"

    if two_phase is None:
        two_phase = os.environ.get("DCP_DISABLE_TWO_PHASE_COMM", "0") in ("0", "", "false", "False")
    second_phase: List[StageComm] = [{d: [] for d in devices} for _ in comm_per_stage]
    if two_phase:
        for s in range(1, len(comm_per_stage)):
            comm_per_stage[s], second_phase[s] = _split_two_phase(comm_per_stage[s], input_sizes, devices)
    return work_per_stage, comm_per_stage, second_phase


def _split_two_phase(stage_comm: StageComm, input_sizes, devices):
    """A block several devices of one node fetch from another node is received once (by the
    least-loaded of them) and forwarded inside the node."""
    recv_load = defaultdict(float)
    takers = defaultdict(set)
    for dst, comms in stage_comm.items():
        for i, src in comms:
            src = tuple(src)
            if src[0] != dst[0]:
                recv_load[dst] += input_sizes[i]
                takers[(src, i, dst[0])].add(dst[1])
    drop = defaultdict(set)
    second: StageComm = {d: [] for d in devices}
    for (src, i, node) in sorted(takers, key=lambda t: (t[1], t[0], t[2])):
        locals_ = sorted(takers[(src, i, node)])
        if len(locals_) < 2:
            continue
        receiver = min(locals_, key=lambda d: (recv_load[(node, d)], d))
        for d in locals_:
            if d != receiver:
                drop[(node, d)].add((i, src))
                second[(node, d)].append((i, (node, receiver)))
    first = {dst: [(i, tuple(src)) for i, src in comms if (i, tuple(src)) not in drop[dst]]
             for dst, comms in stage_comm.items()}
    return first, second


def summarize_pipeline(work_per_stage, comm_per_stage, workload_costs, input_sizes) -> List[dict]:
    """Per-stage modelled compute time and received bytes of the busiest device (for logs/tests)."""
    out = []
    for s, (work, comm) in enumerate(zip(work_per_stage, comm_per_stage)):
        comp = {d: sum(workload_costs[w] for w in ws) for d, ws in work.items()}
        recv = {d: sum(input_sizes[i] for i, _ in cs) for d, cs in comm.items()}
        out.append({"stage": s, "max_compute_ms": max(comp.values(), default=0.0),
                    "max_recv_bytes": max(recv.values(), default=0.0),
                    "n_work": sum(len(ws) for ws in work.values())})
    return out


def pipeline_chrome_trace(work_per_stage, comm_per_stage, workload_costs, input_sizes, comm_cost_model) -> List[dict]:
    """Chrome-trace events of the modelled timeline: per device a compute lane and a transfer lane,
    transfers of stage s+1 starting together with the compute of stage s
    (dcp/core/pipeline.py:349-456)."""
    events = []
    devices = sorted(work_per_stage[0])
    t_comp = {d: 0.0 for d in devices}
    t_comm = {d: 0.0 for d in devices}
    for s in range(len(work_per_stage)):
        for d in devices:
            start = max(t_comp[d], t_comm[d])  # compute of stage s needs its transfers
            dur = sum(workload_costs[w] for w in work_per_stage[s].get(d, ()))
            events.append({"name": f"attn S{s}", "ph": "X", "pid": d[0], "tid": d[1] * 2, "ts": start * 1e3,
                           "dur": dur * 1e3})
            if s + 1 < len(comm_per_stage):
                cdur = sum(comm_cost_model.get_cost(src, d, input_sizes[i]) for i, src in comm_per_stage[s + 1].get(d, ()))
                events.append({"name": f"fetch S{s + 1}", "ph": "X", "pid": d[0], "tid": d[1] * 2 + 1,
                               "ts": start * 1e3, "dur": cdur * 1e3})
                t_comm[d] = start + cdur
            t_comp[d] = start + dur
    return events

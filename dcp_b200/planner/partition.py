"""Placement of data blocks and attention work units on devices.

The batch is turned into a hypergraph: one vertex per work unit (weight = modelled compute
time) and one per co-location group (all Q/KV/Out/LSE head blocks of one token block; weight =
bytes); one net per data block connecting its owner group to every work unit that reads or
writes it, weighted by the bytes that move when the net is cut.  Minimising connectivity-1
under a memory and a compute balance constraint minimises communication volume
(dcp/graph_partition/graph.py:27-1486).  The partitioner itself is the in-tree C++ multilevel
solver (``dcp_b200._planner``); multi-node clusters are split nodes-first, then devices.
"""
from __future__ import annotations

import math
import os
from typing import Dict, List, Sequence, Tuple

import numpy as np

from ..core.blocks import BlockType, Device, WorkloadSpec
from ..core.common import ExecutionContext

COMP_RESOLUTION = 10000     # compute weights are scaled so the most expensive unit is this
BYTE_UNIT = 256             # memory / net weights are counted in units of this many bytes


class HGPSolver:
    NATIVE = "native"        # in-tree multilevel partitioner
    HEURISTIC = "heuristic"  # static zigzag placement, no optimisation
    # names of the reference's external solvers map onto the native one
    KAHYPAR = "native"
    MTKAHYPAR = "native"
    PATOH = "native"


def _native():
    from .. import _planner  # built by dcp_b200.csrc.build
    return _planner


class PlacementGraph:
    """Hypergraph arrays of one workload (kept so tests can evaluate km1 of any placement)."""

    def __init__(self, workload: WorkloadSpec):
        wl = workload
        n_work = len(wl.workloads)
        self.n_work = n_work
        self.groups = wl.colocation_constraints
        self.n_groups = len(self.groups)
        self.n_vertices = n_work + self.n_groups
        max_cost = max(wl.workloads) if n_work else 1.0
        comp = [max(1, int(c * COMP_RESOLUTION / max_cost)) if max_cost > 0 else 1 for c in wl.workloads]
        self.input_group: Dict[int, int] = {}
        self.output_group: Dict[int, int] = {}
        mem = []
        for g, (ins, outs) in enumerate(self.groups):
            b = 0
            for i in ins:
                self.input_group[i] = g
                b += wl.input_sizes[i]
            for o in outs:
                self.output_group[o] = g
                b += wl.output_sizes[o]
            mem.append(max(1, b // BYTE_UNIT))
        self.vw_comp = comp + [0] * self.n_groups
        self.vw_mem = [0] * n_work + mem
        # nets: one per input block; Out+LSE of a block share pins, so they share a net
        in_users: Dict[int, List[int]] = {}
        out_users: Dict[Tuple[int, ...], List[int]] = {}
        for w in range(n_work):
            for i in wl.work_unit_input_map[w]:
                in_users.setdefault(i, []).append(w)
            out_users.setdefault(tuple(wl.work_unit_output_map[w]), []).append(w)
        offsets, pins, weights = [0], [], []
        for i in sorted(in_users):
            pins.append(n_work + self.input_group[i])
            pins.extend(in_users[i])
            offsets.append(len(pins))
            weights.append(max(1, wl.input_sizes[i] // BYTE_UNIT))
        for outs in sorted(out_users):
            pins.append(n_work + self.output_group[outs[0]])
            pins.extend(out_users[outs])
            offsets.append(len(pins))
            weights.append(max(1, sum(wl.output_sizes[o] for o in outs) // BYTE_UNIT))
        self.net_offsets, self.net_pins, self.net_weight = offsets, pins, weights

    def km1(self, part: Sequence[int], k: int) -> int:
        return _native().connectivity_minus_one(self.n_vertices, self.net_offsets, self.net_pins, self.net_weight,
                                                list(part), k)

    def sub(self, vertices: Sequence[int]):
        """Induced sub-hypergraph on ``vertices`` -> (vw_comp, vw_mem, offsets, pins, weights)."""
        local = {v: i for i, v in enumerate(vertices)}
        offsets, pins, weights = [0], [], []
        for e in range(len(self.net_weight)):
            ps = [local[p] for p in self.net_pins[self.net_offsets[e]:self.net_offsets[e + 1]] if p in local]
            if len(ps) < 2:
                continue
            pins.extend(ps)
            offsets.append(len(pins))
            weights.append(self.net_weight[e])
        return ([self.vw_comp[v] for v in vertices], [self.vw_mem[v] for v in vertices], offsets, pins, weights)


def _lpt_bound(weights: Sequence[int], k: int) -> int:
    loads = [0] * k
    for w in sorted(weights, reverse=True):
        loads[loads.index(min(loads))] += w
    return max(loads) if loads else 0


def _capacities(vw_comp, vw_mem, k, mem_eps, comp_eps):
    tot_c, tot_m = sum(vw_comp), sum(vw_mem)
    cap_c = max(int(math.ceil((1.0 + comp_eps) * tot_c / k)), max(vw_comp) if vw_comp else 0, 1)
    mem_items = [m for m in vw_mem if m > 0]
    cap_m = max(int(math.ceil((1.0 + mem_eps) * tot_m / k)), _lpt_bound(mem_items, k), 1)
    return [cap_c] * k, [cap_m] * k


def _solve_once(vw_comp, vw_mem, offsets, pins, weights, k, mem_eps, comp_eps, seed, n_tries, initial=None):
    cap_c, cap_m = _capacities(vw_comp, vw_mem, k, mem_eps, comp_eps)
    res = _native().partition_hypergraph(len(vw_comp), vw_comp, vw_mem, offsets, pins, weights, k, cap_c, cap_m,
                                         seed, n_tries, [], [])
    if initial is not None:
        # a structured starting point (zigzag deal) refined under the same constraints competes
        # with the multilevel result; keep whichever is balanced and cuts less
        alt = _native().partition_hypergraph(len(vw_comp), vw_comp, vw_mem, offsets, pins, weights, k, cap_c, cap_m,
                                             seed, 1, [], list(initial))
        if (alt["balanced"], -alt["km1"]) > (res["balanced"], -res["km1"]):
            res = alt
    return res


def _overload(res, vw_comp, vw_mem, k) -> float:
    """Worst load / mean load over both constraints (1.0 = perfectly even)."""
    mc, mm = max(sum(vw_comp) / k, 1e-9), max(sum(vw_mem) / k, 1e-9)
    return max(max(res["load_comp"]) / mc, max(res["load_mem"]) / mm)


def _solve(vw_comp, vw_mem, offsets, pins, weights, k, mem_eps, comp_eps, seed, n_tries, initial=None):
    """k-way placement under the two balance constraints.  Tight tolerances are not always
    reachable (few large blocks); instead of accepting whatever an infeasible run left behind,
    the tolerances are relaxed step by step until a run meets them, and if none does the least
    overloaded result is kept."""
    if k == 1:
        return [0] * len(vw_comp), 0
    best, best_over, scale = None, float("inf"), 1.0
    while True:
        res = _solve_once(vw_comp, vw_mem, offsets, pins, weights, k, mem_eps * scale, comp_eps * scale, seed, n_tries,
                          initial)
        if res["balanced"]:
            return res["part"], res["km1"]
        over = _overload(res, vw_comp, vw_mem, k)
        if over < best_over:
            best, best_over = res, over
        if max(mem_eps, comp_eps) * scale >= 0.3:
            return best["part"], best["km1"]
        scale *= 1.6


def construct_and_partition_graph_multiconstraint(
        context: ExecutionContext, workload: WorkloadSpec, mem_epsilon: float = 0.2, comp_epsilon: float = 0.2,
        inter_node_comp_epsilon_factor: float = 5.0, solver: str = HGPSolver.NATIVE, logger=None, seed: int = 42,
        n_tries: int = 16):
    """Place every work unit and data block; fills ``workload.*_to_device_map``.

    Returns ``(device_to_workload_map, device_to_input_map, device_to_output_map)`` keyed by
    ``(node, device)``.
    """
    if solver == HGPSolver.HEURISTIC:
        return assign_device_by_heuristic(context, workload)
    graph = PlacementGraph(workload)
    n_nodes, dpn = context.n_nodes, context.n_devices_per_node
    vertex_dev: List[Device] = [(0, 0)] * graph.n_vertices
    if n_nodes == 1:
        seed_part = [d[1] for d in _heuristic_vertex_devices(context, workload, graph)]
        part, km1 = _solve(graph.vw_comp, graph.vw_mem, graph.net_offsets, graph.net_pins, graph.net_weight, dpn,
                           mem_epsilon, comp_epsilon, seed, n_tries, initial=seed_part)
        for v, p in enumerate(part):
            vertex_dev[v] = (0, p)
        if os.environ.get("DCP_B200_NO_REBALANCE", "0") in ("0", ""):
            moves = _rebalance_compute(workload, graph, vertex_dev, context.devices())
            if logger is not None:
                logger.debug("compute rebalance: %d work units moved", moves)
    else:
        node_part, km1 = _solve(graph.vw_comp, graph.vw_mem, graph.net_offsets, graph.net_pins, graph.net_weight,
                                n_nodes, mem_epsilon, comp_epsilon * inter_node_comp_epsilon_factor, seed, n_tries)
        n_orphans = 0
        for node in range(n_nodes):
            prob = second_level_problem(graph, node_part, node)
            if prob.vertices:
                vc, vm, off, pins, wts = graph.sub(prob.vertices)
                for i in range(len(prob.vertices) - prob.n_foreign, len(prob.vertices)):
                    vm[i] = 1                  # held by another node: no memory here, free to sit with its users
                part, _ = _solve(vc, vm, off, pins, wts, dpn, mem_epsilon, comp_epsilon, seed + node + 1, n_tries)
                for v, p in zip(prob.vertices[:len(prob.vertices) - prob.n_foreign], part):
                    vertex_dev[v] = (node, p)
            n_orphans += len(prob.orphans)
            place_orphans(graph, prob.orphans, node, dpn, vertex_dev, node_part)
        if logger is not None:
            logger.debug("second level: %d data groups needed only by other nodes placed by memory", n_orphans)
    if logger is not None:
        logger.debug("placement km1=%d (x%d bytes)", km1, BYTE_UNIT)
    return _materialise(context, workload, graph, vertex_dev)


class SecondLevelProblem:
    """Per-node placement problem of the two-level (multi-node) scheme.

    ``vertices``: the node's work units, then the node's data groups that its own work touches, then
    (the last ``n_foreign`` entries) data groups held by OTHER nodes that this node's work reads or
    writes.  The foreign groups take part with memory weight 1 only: they do not occupy memory on
    this node, but keeping them in the nets makes every device that needs such a block count in
    the connectivity objective, exactly as a local block would.  ``orphans``: data groups assigned
    to this node that none of its own work touches (only other nodes need them); no net of the
    per-node problem reaches them, so they are placed afterwards by memory alone.
    (dcp/graph_partition/graph.py:239-250 foreign weights, :1240-1362 manual assignment.)"""

    def __init__(self, vertices: List[int], n_foreign: int, orphans: List[int]):
        self.vertices, self.n_foreign, self.orphans = vertices, n_foreign, orphans


def second_level_problem(graph: "PlacementGraph", node_part: Sequence[int], node: int) -> SecondLevelProblem:
    n_work = graph.n_work
    touched = set()                 # data-group vertices used by work of this node
    for e in range(len(graph.net_weight)):
        pins = graph.net_pins[graph.net_offsets[e]:graph.net_offsets[e + 1]]
        data = [p for p in pins if p >= n_work]
        if any(p < n_work and node_part[p] == node for p in pins):
            touched.update(data)
    work = [v for v in range(n_work) if node_part[v] == node]
    own_data = [v for v in range(n_work, graph.n_vertices) if node_part[v] == node]
    local = [v for v in own_data if v in touched]
    orphans = [v for v in own_data if v not in touched]
    foreign = sorted(v for v in touched if node_part[v] != node)
    return SecondLevelProblem(work + local + foreign, len(foreign), orphans)


def place_orphans(graph: "PlacementGraph", orphans: Sequence[int], node: int, dpn: int, vertex_dev: List[Device],
                  node_part: Sequence[int]) -> None:
    """Largest first, each onto the device of ``node`` that holds the least memory so far."""
    mem, skip = [0] * dpn, set(orphans)
    for v in range(graph.n_work, graph.n_vertices):
        if node_part[v] == node and v not in skip:
            mem[vertex_dev[v][1]] += graph.vw_mem[v]
    for v in sorted(orphans, key=lambda v: (-graph.vw_mem[v], v)):
        d = mem.index(min(mem))
        vertex_dev[v] = (node, d)
        mem[d] += graph.vw_mem[v]


def _rebalance_compute(workload: WorkloadSpec, graph: "PlacementGraph", vertex_dev: List[Device], devices,
                       tolerance: float = 1.004, max_moves: int = 400) -> int:
    """Single-node polish after partitioning: move work units (never data) from the busiest device
    to the idlest one until the busiest is within ``tolerance`` of the mean, each time picking the
    unit that fits the gap and needs the fewest extra bytes at its new home.  The partitioner
    packs parts up to their cap because only the cut is its objective; on NVSwitch the last
    percent of balance is worth more than the few blocks this pulls.  Returns the number of moves."""
    cost, sizes, w_in = workload.workloads, workload.input_sizes, workload.work_unit_input_map
    load = {d: 0.0 for d in devices}
    present = {d: set() for d in devices}
    on_dev = {d: set() for d in devices}
    for g, (ins, _outs) in enumerate(graph.groups):
        present[tuple(vertex_dev[graph.n_work + g])].update(ins)
    for w in range(graph.n_work):
        d = tuple(vertex_dev[w])
        load[d] += cost[w]
        on_dev[d].add(w)
        present[d].update(w_in[w])
    mean = sum(load.values()) / max(len(devices), 1)
    moves = 0
    while moves < max_moves and mean > 0:
        dmax = max(devices, key=lambda d: load[d])
        dmin = min(devices, key=lambda d: load[d])
        if load[dmax] <= tolerance * mean:
            break
        gap = load[dmax] - load[dmin]
        best, best_key = None, None
        for w in on_dev[dmax]:
            c = cost[w]
            if c <= 0 or c >= gap:          # moving it would just swap the roles
                continue
            extra = sum(sizes[i] for i in w_in[w] if i not in present[dmin])
            # fewest new bytes per unit of moved work; among equals the unit closest to half the gap
            key = (extra / c, abs(c - gap / 2))
            if best_key is None or key < best_key:
                best, best_key = w, key
        if best is None:
            break
        vertex_dev[best] = dmin
        on_dev[dmax].discard(best); on_dev[dmin].add(best)
        load[dmax] -= cost[best]; load[dmin] += cost[best]
        present[dmin].update(w_in[best])
        moves += 1
    return moves


def _materialise(context, workload, graph: PlacementGraph, vertex_dev: Sequence[Device]):
    devs = context.devices()
    d2w: Dict[Device, List[int]] = {d: [] for d in devs}
    d2i: Dict[Device, List[int]] = {d: [] for d in devs}
    d2o: Dict[Device, List[int]] = {d: [] for d in devs}
    workload.work_to_device_map = {}
    workload.input_to_device_map = {}
    workload.output_to_device_map = {}
    for w in range(graph.n_work):
        d = tuple(vertex_dev[w])
        workload.work_to_device_map[w] = d
        d2w[d].append(w)
    for g, (ins, outs) in enumerate(graph.groups):
        d = tuple(vertex_dev[graph.n_work + g])
        for i in ins:
            workload.input_to_device_map[i] = d
            d2i[d].append(i)
        for o in outs:
            workload.output_to_device_map[o] = d
            d2o[d].append(o)
    return d2w, d2i, d2o


def placement_vector(workload: WorkloadSpec, graph: PlacementGraph, context: ExecutionContext) -> List[int]:
    """Flat part id (node * devices_per_node + device) per hypergraph vertex of a placed workload."""
    dpn = context.n_devices_per_node
    flat = lambda d: d[0] * dpn + d[1]
    part = [flat(workload.work_to_device_map[w]) for w in range(graph.n_work)]
    for ins, outs in graph.groups:
        any_block = ins[0] if ins else None
        part.append(flat(workload.input_to_device_map[any_block]) if any_block is not None
                    else flat(workload.output_to_device_map[outs[0]]))
    return part


def assign_device_by_heuristic(context: ExecutionContext, workload: WorkloadSpec, head_parallel: int = 1):
    """Static placement for ablations: token blocks of each sequence are dealt zigzag over the
    devices (balanced causal work, as in zigzag ring attention); with ``head_parallel > 1`` the
    devices form a (ring x head) grid and head blocks are dealt over the head axis
    (dcp/graph_partition/graph.py:1618-1755).  Work runs where its Q block lives."""
    graph = PlacementGraph(workload)
    return _materialise(context, workload, graph, _heuristic_vertex_devices(context, workload, graph, head_parallel))


def _heuristic_vertex_devices(context, workload, graph: "PlacementGraph", head_parallel: int = 1) -> List[Device]:
    devs = context.devices()
    n_dev = len(devs)
    assert n_dev % head_parallel == 0
    ring = n_dev // head_parallel
    metas = workload.block_mapping.input_id_to_meta
    vertex_dev: List[Device] = [(0, 0)] * graph.n_vertices
    for g, (ins, outs) in enumerate(graph.groups):
        meta = metas[ins[0]]
        pos = meta.block_id % (2 * ring)
        r = pos if pos < ring else 2 * ring - 1 - pos
        vertex_dev[graph.n_work + g] = devs[r * head_parallel]
    group_dev = {g: vertex_dev[graph.n_work + g] for g in range(graph.n_groups)}
    for w in range(graph.n_work):
        wm = workload.block_mapping.work_id_to_meta[w]
        base = group_dev[graph.input_group[wm.q_id]]
        idx = devs.index(base)
        vertex_dev[w] = devs[idx + (wm.head_id % head_parallel)]
    return vertex_dev


def assign_input_outputs(context: ExecutionContext, workload: WorkloadSpec):
    """Given ``work_to_device_map`` only, place each co-location group on the device that uses it
    most, subject to greedy memory balancing (dcp/graph_partition/graph.py:1489-1615)."""
    graph = PlacementGraph(workload)
    devs = context.devices()
    usage = [dict() for _ in range(graph.n_groups)]
    for w, d in workload.work_to_device_map.items():
        for i in workload.work_unit_input_map[w]:
            g = graph.input_group[i]
            usage[g][d] = usage[g].get(d, 0) + workload.input_sizes[i]
    load = {d: 0 for d in devs}
    total = sum(graph.vw_mem)
    cap = 1.2 * total / len(devs) + max(graph.vw_mem)
    vertex_dev = [workload.work_to_device_map.get(w, devs[0]) for w in range(graph.n_work)] + [devs[0]] * graph.n_groups
    for g in sorted(range(graph.n_groups), key=lambda g: -graph.vw_mem[graph.n_work + g]):
        m = graph.vw_mem[graph.n_work + g]
        ranked = sorted(devs, key=lambda d: (-usage[g].get(d, 0), load[d]))
        pick = next((d for d in ranked if load[d] + m <= cap), min(devs, key=lambda d: load[d]))
        load[pick] += m
        vertex_dev[graph.n_work + g] = pick
    return _materialise(context, workload, graph, vertex_dev)

"""Multicast-tree packing for inter-node transfers (alternative pipeline algorithm "tree").

When several nodes need the same remote block, sending it from the owner to each of them loads
the owner's uplink once per consumer.  Here every such block gets a multicast tree over nodes: a
node that already received the block may forward it in a later stage.  Trees are packed so that
the maximum per-node, per-stage send/receive volume is as small as possible: a greedy
longest-first packing first, then an exact branch-and-bound search that starts from it (optimal
when the search finishes inside its budget, else the best packing found).  The reference solves
the same packing with OR-tools CP-SAT (dcp/core/steiner_tree_packing.py:14-167, used by
dcp/core/pipeline.py:842-1086); no external solver is needed here, and on a single node the result
degenerates to direct transfers.
"""
from __future__ import annotations

from collections import defaultdict
from typing import Dict, List, Optional, Sequence, Set, Tuple

from ..core.blocks import DataBlockMeta, Device
from .stages import generate_pipelines_n_stages


Request = Tuple[int, int, Set[int], float]       # (block id, source node, destination nodes, size)
Arrival = Dict[Tuple[int, int], int]              # (block id, destination node) -> stage it must arrive in


def packing_cost(trees: Dict[int, List[Tuple[int, int, int]]], requests: Sequence[Request], n_nodes: int,
                 n_stages: int) -> float:
    """The packing objective: the largest volume any node sends or receives in one stage."""
    size = {r[0]: r[3] for r in requests}
    send = [[0.0] * n_nodes for _ in range(n_stages)]
    recv = [[0.0] * n_nodes for _ in range(n_stages)]
    for blk, edges in trees.items():
        for s, h, d in edges:
            send[s][h] += size[blk]
            recv[s][d] += size[blk]
    return max([0.0] + [max(max(a), max(b)) for a, b in zip(send, recv)])


def _pack_greedy(requests: Sequence[Request], n_nodes: int, n_stages: int, arrival: Optional[Arrival]):
    send = [[0.0] * n_nodes for _ in range(n_stages)]
    recv = [[0.0] * n_nodes for _ in range(n_stages)]
    trees: Dict[int, List[Tuple[int, int, int]]] = {}
    for blk, src, dsts, size in sorted(requests, key=lambda r: (-r[3] * len(set(r[2]) - {r[1]}), r[0])):
        have = {src: -1}              # node -> stage in which it obtained the block
        edges = []
        remaining = set(dsts) - {src}
        while remaining:
            best = None
            for d in sorted(remaining):
                fixed = None if arrival is None else arrival.get((blk, d))
                for h, got in have.items():
                    stages = range(got + 1, n_stages) if fixed is None else ([fixed] if fixed > got else [])
                    for st in stages:
                        key = (max(send[st][h], recv[st][d]) + size, st, h)
                        if best is None or key < best[0]:
                            best = (key, st, h, d)
                        break  # earliest feasible stage for this holder is enough
            assert best is not None, f"block {blk}: no holder can serve a destination in its stage"
            _, st, h, d = best
            send[st][h] += size
            recv[st][d] += size
            have[d] = st
            edges.append((st, h, d))
            remaining.discard(d)
        trees[blk] = edges
    return trees


def _pack_exact(requests: Sequence[Request], n_nodes: int, n_stages: int, arrival: Optional[Arrival],
                incumbent, incumbent_cost: float, search_budget: int):
    """Depth-first branch and bound over all trees of all requests.  The edges of one tree are
    enumerated in increasing (stage, destination) order, which reaches every tree exactly once (a
    relay always obtained the block in an earlier stage than it forwards it).  A branch is cut as
    soon as its partial maximum reaches the best complete packing.  Returns (trees, cost, proven)."""
    reqs = sorted(requests, key=lambda r: (-r[3] * len(set(r[2]) - {r[1]}), r[0]))
    send = [[0.0] * n_nodes for _ in range(n_stages)]
    recv = [[0.0] * n_nodes for _ in range(n_stages)]
    # no packing can beat: the largest single block, and a node's mandatory receive volume spread over
    # the stages it may arrive in (all stages when free, the given stage when fixed)
    lower = max([0.0] + [r[3] for r in reqs if set(r[2]) - {r[1]}])
    if arrival is not None:
        fixed_recv = defaultdict(float)
        for blk, src, dsts, size in reqs:
            for d in set(dsts) - {src}:
                if (blk, d) in arrival:
                    fixed_recv[(arrival[(blk, d)], d)] += size
        lower = max([lower] + list(fixed_recv.values()))
    else:
        per_node = defaultdict(float)
        for blk, src, dsts, size in reqs:
            for d in set(dsts) - {src}:
                per_node[d] += size
        lower = max([lower] + [v / n_stages for v in per_node.values()])
    best = {"trees": incumbent, "cost": incumbent_cost, "nodes": 0, "cut": False}
    current: Dict[int, List[Tuple[int, int, int]]] = {}

    def dfs(ri: int, have: Dict[int, int], remaining: frozenset, last: Tuple[int, int], cur_max: float):
        if best["cost"] <= lower + 1e-9 or best["cut"]:
            return
        best["nodes"] += 1
        if best["nodes"] > search_budget:
            best["cut"] = True
            return
        if not remaining:
            if ri + 1 == len(reqs):
                if cur_max < best["cost"] - 1e-9:
                    best["cost"], best["trees"] = cur_max, {k: list(v) for k, v in current.items()}
                return
            blk, src, dsts, _ = reqs[ri + 1]
            current[blk] = []
            dfs(ri + 1, {src: -1}, frozenset(set(dsts) - {src}), (-1, -1), cur_max)
            del current[blk]
            return
        blk, _, _, size = reqs[ri]
        options = []
        for d in remaining:
            fixed = None if arrival is None else arrival.get((blk, d))
            for h, got in have.items():
                for st in (range(got + 1, n_stages) if fixed is None else ([fixed] if fixed > got else [])):
                    if (st, d) > last:
                        options.append((max(cur_max, send[st][h] + size, recv[st][d] + size), st, d, h))
        for cost, st, d, h in sorted(options):
            if cost >= best["cost"] - 1e-9:
                break                                   # sorted by cost: nothing better follows
            # every remaining destination must still be reachable after this edge in (stage, dst) order
            if any((n_stages - 1 if arrival is None or (blk, o) not in arrival else arrival[(blk, o)], o) <= (st, d)
                   for o in remaining if o != d):
                continue
            send[st][h] += size
            recv[st][d] += size
            have[d] = st
            current[blk].append((st, h, d))
            dfs(ri, have, remaining - {d}, (st, d), cost)
            current[blk].pop()
            del have[d]
            send[st][h] -= size
            recv[st][d] -= size

    if reqs:
        blk, src, dsts, _ = reqs[0]
        current[blk] = []
        dfs(0, {src: -1}, frozenset(set(dsts) - {src}), (-1, -1), 0.0)
    return best["trees"], best["cost"], not best["cut"]


def pack_multicast_trees(requests: Sequence[Request], n_nodes: int, n_stages: int, arrival: Optional[Arrival] = None,
                         exact: bool = True, search_budget: int = 50000, return_info: bool = False,
                         native: bool = True):
    """requests: (block id, source node, destination nodes, size).  Returns
    {block id: [(stage, src node, dst node)]} with every destination reached and each edge's source
    holding the block before the edge's stage; with ``arrival`` a destination receives exactly in
    its given stage.  The greedy longest-first packing is the starting point; with ``exact`` a
    branch-and-bound search then looks for the packing with the smallest per-node, per-stage
    maximum and proves it optimal when it finishes within ``search_budget`` search nodes (the
    role of the CP-SAT model in dcp/core/steiner_tree_packing.py:14-167, which is also run under
    a time limit and falls back to the best feasible packing).  ``native`` runs the C++
    implementation (csrc/planner/tree_packing.cpp); the Python one below is its twin and oracle.
    ``return_info`` -> (trees, {"cost", "greedy_cost", "proven_optimal"})."""
    requests = [(b, s, set(d), float(z)) for b, s, d, z in requests]
    if native:
        from .. import _planner
        native = hasattr(_planner, "pack_multicast_trees")      # a library built before the packer was added
    if native:
        packed = []
        for b, s, dsts, z in requests:
            ds = sorted(dsts)
            arr = [] if arrival is None else [arrival.get((b, d), -1) for d in ds]
            packed.append((b, s, ds, z, arr))
        res = _planner.pack_multicast_trees(packed, n_nodes, n_stages, exact, search_budget)
        trees = {int(b): [tuple(e) for e in edges] for b, edges in res["trees"].items()}
        info = {"cost": res["cost"], "greedy_cost": res["greedy_cost"], "proven_optimal": bool(res["proven_optimal"])}
        return (trees, info) if return_info else trees
    trees = _pack_greedy(requests, n_nodes, n_stages, arrival)
    greedy_cost = cost = packing_cost(trees, requests, n_nodes, n_stages)
    proven = False
    if exact:
        trees, cost, proven = _pack_exact(requests, n_nodes, n_stages, arrival, trees, cost, search_budget)
    # requests whose destinations are all the source itself still get an (empty) tree
    for blk, *_ in requests:
        trees.setdefault(blk, [])
    if return_info:
        return trees, {"cost": cost, "greedy_cost": greedy_cost, "proven_optimal": proven}
    return trees


def generate_pipelines_n_stages_with_tree_packing(n_stages, all_devices, workload_costs, workload_input_map,
                                                  input_to_meta_map, input_sizes, workload_to_device_map,
                                                  input_to_device_map, is_bw, logger=None):
    """Same contract as ``generate_pipelines_n_stages``.  The greedy stage builder decides which
    work runs when; cross-node transfers that fan out to several nodes are then re-routed along
    packed multicast trees (relay = any device of an intermediate node that already fetched it)."""
    work, comm, second = generate_pipelines_n_stages(n_stages, all_devices, workload_costs, workload_input_map,
                                                     input_to_meta_map, input_sizes, workload_to_device_map,
                                                     input_to_device_map, is_bw, logger, two_phase=True)
    nodes = sorted({d[0] for d in all_devices})
    if len(nodes) <= 1:
        return work, comm, second
    # first inter-node arrival of every block at every node, as timed by the greedy builder
    first: Dict[Tuple[int, int], Tuple[int, Device, Device]] = {}
    for s in range(1, len(comm)):
        for dst in sorted(comm[s]):
            for i, src in comm[s][dst]:
                if src[0] != dst[0] and ((i, dst[0]) not in first or s < first[(i, dst[0])][0]):
                    first[(i, dst[0])] = (s, dst, tuple(src))
    fan: Dict[int, Set[int]] = defaultdict(set)
    for (i, node) in first:
        fan[i].add(node)
    # blocks that fan out to several nodes are routed along packed trees; every node still receives
    # in the stage the builder chose (buffer lifetimes and the overlap with compute stay as planned),
    # what the packing chooses is WHO sends: the owner or a node that obtained the block earlier
    requests = [(i, tuple(input_to_device_map[i])[0], dsts, float(input_sizes[i])) for i, dsts in sorted(fan.items())
                if len(dsts) >= 2]
    arrival = {(i, n): first[(i, n)][0] for i, _, dsts, _ in requests for n in dsts}
    trees = pack_multicast_trees(requests, max(nodes) + 1, len(comm), arrival=arrival)
    for i, owner_node, _, _ in requests:
        for s, h, d in trees[i]:
            if h == owner_node:
                continue
            _, dst_dev, old_src = first[(i, d)]
            relay = first[(i, h)][1]                  # the device of node h that received the block
            comm[s][dst_dev] = [(j, (relay if j == i and tuple(sd) == old_src else tuple(sd))) for j, sd in comm[s][dst_dev]]
    return work, comm, second

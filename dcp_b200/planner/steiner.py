"""Multicast-tree packing for inter-node transfers (alternative pipeline algorithm "tree").

When several nodes need the same remote block, sending it from the owner to each of them loads
the owner's uplink once per consumer.  Here every such block gets a multicast tree over nodes: a
node that already received the block may forward it in a later stage.  Trees are packed greedily
so the maximum per-node, per-stage send/receive volume stays low.  The reference solves the same
packing with OR-tools CP-SAT (dcp/core/steiner_tree_packing.py:14-167, used by
dcp/core/pipeline.py:842-1086); a greedy longest-first heuristic is used here so no solver is
needed, and on a single node the result degenerates to direct transfers.
"""
from __future__ import annotations

from collections import defaultdict
from typing import Dict, List, Sequence, Set, Tuple

from ..core.blocks import DataBlockMeta, Device
from .stages import generate_pipelines_n_stages


def pack_multicast_trees(requests: Sequence[Tuple[int, int, Set[int], float]], n_nodes: int, n_stages: int):
    """requests: (block id, source node, destination nodes, size).  Returns
    {block id: [(stage, src node, dst node)]} with every destination reached and each edge's source
    holding the block before the edge's stage."""
    send = [[0.0] * n_nodes for _ in range(n_stages)]
    recv = [[0.0] * n_nodes for _ in range(n_stages)]
    trees: Dict[int, List[Tuple[int, int, int]]] = {}
    for blk, src, dsts, size in sorted(requests, key=lambda r: -r[3] * len(r[2])):
        have = {src: -1}              # node -> stage in which it obtained the block
        edges = []
        remaining = set(dsts) - {src}
        while remaining:
            best = None
            for d in sorted(remaining):
                for h, got in have.items():
                    for s in range(got + 1, n_stages):
                        cost = max(send[s][h], recv[s][d]) + size
                        key = (cost, s, h)
                        if best is None or key < best[0]:
                            best = (key, s, h, d)
                        break  # earliest feasible stage for this holder is enough
            _, s, h, d = best
            send[s][h] += size
            recv[s][d] += size
            have[d] = s
            edges.append((s, h, d))
            remaining.discard(d)
        trees[blk] = edges
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
    # first inter-node arrival of each block per node, as chosen by the greedy builder
    for s in range(1, len(comm)):
        fanout = defaultdict(list)     # (block, src node) -> [(dst dev, src dev)]
        for dst, cs in comm[s].items():
            for i, src in cs:
                if src[0] != dst[0]:
                    fanout[(i, src[0])].append((dst, tuple(src)))
        for (i, src_node), lst in fanout.items():
            if len({d[0] for d, _ in lst}) < 2:
                continue
            # chain the destination nodes: the first keeps the owner as source, later ones pull from the
            # previous destination when that one obtained the block in an earlier stage
            holders = {}
            for t in range(1, s):
                for dst, cs in comm[t].items():
                    if any(j == i for j, _ in cs):
                        holders.setdefault(dst[0], dst)
            for dst, src in lst:
                alt = next((h for n, h in holders.items() if n != dst[0] and n != src_node), None)
                if alt is not None:
                    comm[s][dst] = [(j, (alt if j == i and tuple(sd) == src else tuple(sd))) for j, sd in comm[s][dst]]
    return work, comm, second

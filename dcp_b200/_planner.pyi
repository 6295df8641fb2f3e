"""Type stubs of the native planner extension (built from dcp_b200/csrc/planner)."""
from typing import Any, Dict, List, Optional, Sequence, Set, Tuple

import numpy as np

Device = Tuple[int, int]

def greedy_selection_per_device(
    devices: Set[Device], scheduled_workloads: Set[int], workload_costs: Sequence[float], input_sizes: Sequence[float],
    workload_input_map: Sequence[Sequence[int]], input_block_type_map: Sequence[str],
    device_workload_map: Dict[Device, List[int]], device_local_inputs_map: Dict[Device, Dict[int, int]],
    target_comm_load_per_node: Dict[Device, float], is_bw: bool, stage_id: int, py_logger: Optional[Any] = None,
    intra_node_budget: Dict[Device, float] = ...,
) -> Tuple[Dict[Device, Set[int]], Dict[Device, List[Tuple[int, Device]]], Dict[Device, Dict[int, int]]]:
    """One stage of work + transfer selection: (unlocked work per device, transfers per device as
    (input id, source device), updated map of inputs each device holds and since which stage)."""

def partition_hypergraph(
    n_vertices: int, vw_comp: Sequence[int], vw_mem: Sequence[int], net_offsets: Sequence[int], net_pins: Sequence[int],
    net_weight: Sequence[int], k: int, cap_comp: Sequence[int], cap_mem: Sequence[int], seed: int = 42, n_tries: int = 4,
    fixed: Sequence[int] = ..., initial: Sequence[int] = ...,
) -> Dict[str, Any]:
    """Multilevel k-way partition minimising connectivity-1 under two per-block weight caps.
    Returns {"part", "km1", "load_comp", "load_mem", "balanced"}."""

def connectivity_minus_one(n_vertices: int, net_offsets: Sequence[int], net_pins: Sequence[int],
                           net_weight: Sequence[int], part: Sequence[int], k: int) -> int: ...

def slice_mask_pairs(rng: np.ndarray, q_lo: int, q_hi: int, n_blk: int, block_size: int
                     ) -> Tuple[List[int], List[int], np.ndarray]:
    """Per query block: KV blocks with allowed pairs, their pair counts, rebased intervals int32 [n, 2, 2, n_q]."""

def pack_multicast_trees(requests: Sequence[Tuple[int, int, Sequence[int], float, Sequence[int]]], n_nodes: int,
                         n_stages: int, exact: bool = True, search_budget: int = 50000) -> Dict[str, Any]:
    """Multicast tree packing; requests = (block, source node, destination nodes, size, arrival stage per
    destination or empty).  Returns {"trees": {block: [(stage, from node, to node)]}, "cost", "greedy_cost",
    "proven_optimal"}."""

AttnRowTuple = Tuple[int, int, Sequence[int], Sequence[Tuple[int, int]], np.ndarray, int, int, int, int, Sequence[Tuple[int, int]]]

def build_fwd_tables(rows: Sequence[AttnRowTuple], block_size: int, tile_m: int
                     ) -> Tuple[np.ndarray, np.ndarray, np.ndarray, float]:
    """Forward kernel tables of one stage: (tiles int32 [n, 8], kv entries int32 [m, 2 | 4], masks int32 [r, 4],
    allowed pairs x heads).  A row = (q_row, n_tokens, heads, [(kv row, tokens)], ranges int32 [n_tokens, 4],
    out_dev, out_row, dq_dev, dq_row, [(dkv device, dkv row)])."""

def build_bwd_tables(rows: Sequence[AttnRowTuple], block_size: int, hq: int
                     ) -> Tuple[np.ndarray, np.ndarray, np.ndarray, float]:
    """Backward kernel tables: (ctas int32 [n, 8], items int32 [m, 8], masks int32 [r, 4], allowed pairs x heads)."""

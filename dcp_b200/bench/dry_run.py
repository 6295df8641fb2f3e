"""Planner-only dry run and grid search: no GPU, no model.

For every cell of a grid over (block size, head block size, stage count, balance tolerances) the
planner places and schedules a few synthetic batches for a given cluster shape and reports what
the plans would cost according to the cost models: the busiest device's attention time, the
imbalance of compute and of tokens, the bytes each device pulls (intra- and inter-node) and the
modelled time of the staged pipeline.  ``best`` picks the cell with the lowest modelled time per
(mask, length distribution), which is what the reference's dry-run tooling is for
(benchmark/mlm/dry_run.py, dry_run_grid_search.py:81-183, get_best_config.py:7-36).

    python -m dcp_b200.bench.dry_run --devices 8 --nodes 1 --tokens 131072 --block-sizes 1024 2048 4096 --out dry.json
"""
from __future__ import annotations

import argparse
import itertools
import json
import time
from typing import Dict, List, Sequence

import numpy as np
import torch

from ..core.common import get_default_execution_context
from ..data import synth
from ..planner import masks as mask_lib
from ..planner.compiler import CompilerConfig, InstrCompiler
from ..planner.stages import generate_pipelines_n_stages
from ..planner.workload import generate_workload, pad_seqlens

DISTS = {"lognormal8k": synth.LOGNORMAL_8K, "lognormal16k": synth.LOGNORMAL_16K, "mixture": synth.MIXTURE}


def modelled_pipeline_ms(work_ps, comm_ps, costs, sizes, comm_cost_model) -> float:
    """Slowest device's time when the transfers of stage s+1 overlap the compute of stage s."""
    devices = sorted(work_ps[0])
    worst = 0.0
    for d in devices:
        t_comp = t_comm = 0.0
        for s in range(len(work_ps)):
            start = max(t_comp, t_comm)
            t_comp = start + sum(costs[w] for w in work_ps[s].get(d, ()))
            if s + 1 < len(comm_ps):
                t_comm = start + sum(comm_cost_model.get_cost(tuple(src), d, sizes[i]) for i, src in comm_ps[s + 1].get(d, ()))
        worst = max(worst, t_comp, t_comm)
    return worst


def dry_run_cell(n_devices: int, n_nodes: int, tokens: int, n_heads: int, n_kv_heads: int, head_dim: int, mask: str,
                 length_dist: str, block_size: int, head_block_size: int, n_stages: int, mem_eps: float, comp_eps: float,
                 batches: int = 3, seed: int = 0) -> Dict:
    ctx = get_default_execution_context(n_devices, n_nodes)
    rows = []
    for b in range(batches):
        raw = [int(x) for x in synth.sample_seqlens(tokens, DISTS[length_dist], seed * 1000003 + b)]
        pad = pad_seqlens(raw, block_size)
        info = synth.assign_mask_kinds(raw, seed * 1000003 + b) if mask == "mixed" else None
        m = mask_lib.get_mask_fn(mask)(raw, pad, torch.int32, info)
        hbs = head_block_size or n_heads
        t0 = time.time()
        wl = generate_workload((sum(pad), n_heads, head_dim), (sum(pad), 2, n_kv_heads, head_dim), raw, pad, block_size,
                               hbs, ctx.comp_cost_model, m, torch.bfloat16)
        comp = InstrCompiler(ctx, CompilerConfig(mem_imbalance_epsilon=mem_eps, comp_imbalance_epsilon=comp_eps,
                                                 n_stages=n_stages))
        fw_wl, _, _, _ = comp.compile(wl, generate_backward=False)
        plan_s = time.time() - t0
        devs = ctx.devices()
        load = {d: 0.0 for d in devs}
        for w, d in fw_wl.work_to_device_map.items():
            load[tuple(d)] += fw_wl.workloads[w]
        toks = {d: 0 for d in devs}
        in_meta = fw_wl.block_mapping.input_id_to_meta
        for i, d in fw_wl.input_to_device_map.items():
            if in_meta[i].type == "Q" and in_meta[i].head_id == 0:
                toks[tuple(d)] += in_meta[i].n_tokens
        work_ps, comm_ps, _ = generate_pipelines_n_stages(n_stages, devs, fw_wl.workloads, fw_wl.work_unit_input_map,
                                                          in_meta, fw_wl.input_sizes, fw_wl.work_to_device_map,
                                                          fw_wl.input_to_device_map, False, None)
        intra = inter = 0.0
        for per_dst in comm_ps:
            for dst, comms in per_dst.items():
                for i, src in comms:
                    if tuple(src)[0] == dst[0]:
                        intra += fw_wl.input_sizes[i]
                    else:
                        inter += fw_wl.input_sizes[i]
        lv, tv = np.array(list(load.values())), np.array(list(toks.values()), dtype=np.float64)
        rows.append({"max_compute_ms": float(lv.max()), "compute_max_over_mean": float(lv.max() / max(lv.mean(), 1e-12)),
                     "tokens_max_over_mean": float(tv.max() / max(tv.mean(), 1e-12)),
                     "intra_node_MB_per_device": intra / n_devices / 1e6, "inter_node_MB_per_device": inter / n_devices / 1e6,
                     "modelled_pipeline_ms": modelled_pipeline_ms(work_ps, comm_ps, fw_wl.workloads, fw_wl.input_sizes,
                                                                  ctx.comm_cost_model),
                     "n_work_units": len(fw_wl.workloads), "plan_s": plan_s})
    out = {k: float(np.mean([r[k] for r in rows])) for k in rows[0]}
    out.update({"devices": n_devices, "nodes": n_nodes, "tokens": tokens, "mask": mask, "length_dist": length_dist,
                "block_size": block_size, "head_block_size": head_block_size, "n_stages": n_stages, "mem_eps": mem_eps,
                "comp_eps": comp_eps, "batches": batches})
    return out


def best(cells: Sequence[Dict]) -> List[Dict]:
    """Lowest modelled pipeline time per (mask, length distribution, cluster shape, token budget)."""
    groups: Dict[tuple, Dict] = {}
    for c in cells:
        key = (c["mask"], c["length_dist"], c["devices"], c["nodes"], c["tokens"])
        if key not in groups or c["modelled_pipeline_ms"] < groups[key]["modelled_pipeline_ms"]:
            groups[key] = c
    return list(groups.values())


def main(argv=None):
    ap = argparse.ArgumentParser(description="planner-only dry run / grid search")
    ap.add_argument("--devices", type=int, default=8)
    ap.add_argument("--nodes", type=int, default=1)
    ap.add_argument("--tokens", type=int, default=131072)
    ap.add_argument("--n-heads", type=int, default=32)
    ap.add_argument("--n-kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--masks", nargs="+", default=["causal"])
    ap.add_argument("--length-dists", nargs="+", default=["lognormal8k"], choices=sorted(DISTS))
    ap.add_argument("--block-sizes", nargs="+", type=int, default=[1024, 2048, 4096])
    ap.add_argument("--head-block-sizes", nargs="+", type=int, default=[0])
    ap.add_argument("--stages", nargs="+", type=int, default=[4])
    ap.add_argument("--mem-eps", nargs="+", type=float, default=[0.03])
    ap.add_argument("--comp-eps", nargs="+", type=float, default=[0.015])
    ap.add_argument("--batches", type=int, default=3)
    ap.add_argument("--out", default=None)
    args = ap.parse_args(argv)
    cells = []
    for mask, dist_, bs, hbs, st, me, ce in itertools.product(args.masks, args.length_dists, args.block_sizes,
                                                              args.head_block_sizes, args.stages, args.mem_eps,
                                                              args.comp_eps):
        c = dry_run_cell(args.devices, args.nodes, args.tokens, args.n_heads, args.n_kv_heads, args.head_dim, mask, dist_,
                         bs, hbs, st, me, ce, args.batches)
        cells.append(c)
        print(json.dumps(c), flush=True)
    result = {"cells": cells, "best": best(cells)}
    print("best:", json.dumps(result["best"]))
    if args.out:
        with open(args.out, "w") as f:
            json.dump(result, f, indent=1)
    return result


if __name__ == "__main__":
    main()

"""Text and graph views of a placed workload (dcp/utils/visualization.py:11-429).

``visualize_workload_spec_tty`` prints, per sequence, which device owns each token block and a
(q block x kv block) grid of the device that computes each work unit.  ``visualize_workload_spec_figure``
writes the same information as JSON (nodes + edges) and, for a path ending in ``.svg``, draws it: per
sequence a strip of token blocks coloured by owning device above the (q block x kv block) grid
coloured by computing device.  No plotting library is needed or used.
"""
from __future__ import annotations

import json
from collections import defaultdict
from typing import Optional

from ..core.blocks import BlockType, WorkloadSpec

_GLYPHS = "0123456789abcdefghijklmnopqrstuvwxyzABCDEFGHIJKLMNOPQRSTUVWXYZ"
_COLORS = [31, 32, 33, 34, 35, 36, 91, 92, 93, 94, 95, 96]


def _glyph(flat: int, color: bool) -> str:
    g = _GLYPHS[flat % len(_GLYPHS)]
    return f"\033[{_COLORS[flat % len(_COLORS)]}m{g}\033[0m" if color else g


def visualize_workload_spec_tty(workload: WorkloadSpec, n_devices_per_node: int = 8, head_block: int = 0,
                                color: bool = False, file=None) -> str:
    im, wm = workload.block_mapping.input_id_to_meta, workload.block_mapping.work_id_to_meta
    flat = lambda d: d[0] * n_devices_per_node + d[1]
    seqs = sorted({m.seq_id for m in im.values()})
    lines = []
    grid = defaultdict(dict)
    for w, u in wm.items():
        if u.head_id == head_block and w in workload.work_to_device_map:
            grid[u.seq_id][(im[u.q_id].block_id, im[u.kv_id].block_id)] = flat(workload.work_to_device_map[w])
    for s in seqs:
        blocks = sorted((m.block_id, i) for i, m in im.items() if m.seq_id == s and m.type == BlockType.Q and m.head_id == 0)
        owners = "".join(_glyph(flat(workload.input_to_device_map[i]), color) if i in workload.input_to_device_map else "?"
                         for _, i in blocks)
        lines.append(f"seq {s}: {len(blocks)} blocks, owners {owners}")
        n = len(blocks)
        for qi in range(n):
            row = "".join(_glyph(grid[s][(qi, kj)], color) if (qi, kj) in grid[s] else "." for kj in range(n))
            lines.append("   " + row)
    text = "\n".join(lines)
    if file is not None:
        print(text, file=file)
    return text


def visualize_workload_spec_figure(workload: WorkloadSpec, path: Optional[str] = None, n_devices_per_node: int = 8) -> dict:
    """Bipartite graph of data blocks and work units with placement, as a JSON-serialisable dict."""
    im, om, wm = (workload.block_mapping.input_id_to_meta, workload.block_mapping.output_id_to_meta,
                  workload.block_mapping.work_id_to_meta)
    flat = lambda d: d[0] * n_devices_per_node + d[1]
    nodes, edges = [], []
    for i, m in im.items():
        nodes.append({"id": f"in{i}", "kind": m.type, "seq": m.seq_id, "head": m.head_id, "block": m.block_id,
                      "device": flat(workload.input_to_device_map[i]) if i in workload.input_to_device_map else None})
    for o, m in om.items():
        nodes.append({"id": f"out{o}", "kind": m.type, "seq": m.seq_id, "head": m.head_id, "block": m.block_id,
                      "device": flat(workload.output_to_device_map[o]) if o in workload.output_to_device_map else None})
    for w, u in wm.items():
        nodes.append({"id": f"w{w}", "kind": "WORK", "seq": u.seq_id, "head": u.head_id, "cost": workload.workloads[w],
                      "device": flat(workload.work_to_device_map[w]) if w in workload.work_to_device_map else None,
                      "stage": workload.work_to_stage_map.get(w)})
        edges += [{"src": f"in{i}", "dst": f"w{w}"} for i in workload.work_unit_input_map[w]]
        edges += [{"src": f"w{w}", "dst": f"out{o}"} for o in workload.work_unit_output_map[w]]
    graph = {"nodes": nodes, "edges": edges}
    if path and path.endswith(".svg"):
        with open(path, "w") as f:
            f.write(placement_svg(workload, n_devices_per_node))
    elif path:
        with open(path, "w") as f:
            json.dump(graph, f)
    return graph


_SVG_COLORS = ["#4e79a7", "#f28e2b", "#59a14f", "#e15759", "#76b7b2", "#edc948", "#b07aa1", "#9c755f",
               "#1f77b4", "#ff7f0e", "#2ca02c", "#d62728", "#9467bd", "#8c564b", "#e377c2", "#7f7f7f"]


def placement_svg(workload: WorkloadSpec, n_devices_per_node: int = 8, head_block: int = 0, cell: int = 10) -> str:
    """Stand-alone SVG of a placed workload: for every sequence the owners of its token blocks (top
    strip, class "owner") and the device computing each (q block, kv block) work unit of head block
    ``head_block`` (grid, class "work"); one colour per device, legend on the right."""
    im, wm = workload.block_mapping.input_id_to_meta, workload.block_mapping.work_id_to_meta
    flat = lambda d: d[0] * n_devices_per_node + d[1]
    color = lambda dev: _SVG_COLORS[dev % len(_SVG_COLORS)]
    grid = defaultdict(dict)
    for w, u in wm.items():
        if u.head_id == head_block and w in workload.work_to_device_map:
            grid[u.seq_id][(im[u.q_id].block_id, im[u.kv_id].block_id)] = flat(workload.work_to_device_map[w])
    out, x0, devices = [], 10, set()
    height = 40
    for s in sorted({m.seq_id for m in im.values()}):
        blocks = sorted((m.block_id, i) for i, m in im.items() if m.seq_id == s and m.type == BlockType.Q and m.head_id == 0)
        n = len(blocks)
        out.append(f'<text x="{x0}" y="14" font-size="11">seq {s}</text>')
        for b, i in blocks:
            if i in workload.input_to_device_map:
                dev = flat(workload.input_to_device_map[i])
                devices.add(dev)
                out.append(f'<rect class="owner" x="{x0 + b * cell}" y="20" width="{cell - 1}" height="{cell - 1}" '
                           f'fill="{color(dev)}"><title>seq {s} block {b}: device {dev}</title></rect>')
        for (qi, kj), dev in sorted(grid[s].items()):
            devices.add(dev)
            out.append(f'<rect class="work" x="{x0 + kj * cell}" y="{36 + qi * cell}" width="{cell - 1}" height="{cell - 1}" '
                       f'fill="{color(dev)}"><title>seq {s} q {qi} x kv {kj}: device {dev}</title></rect>')
        x0 += n * cell + 20
        height = max(height, 46 + n * cell)
    for k, dev in enumerate(sorted(devices)):
        out.append(f'<rect x="{x0}" y="{20 + 14 * k}" width="10" height="10" fill="{color(dev)}"/>')
        out.append(f'<text x="{x0 + 14}" y="{29 + 14 * k}" font-size="10">device {dev}</text>')
    height = max(height, 30 + 14 * len(devices))
    head = (f'<svg xmlns="http://www.w3.org/2000/svg" width="{x0 + 90}" height="{height}" font-family="sans-serif">'
            f'<rect width="{x0 + 90}" height="{height}" fill="white"/>')
    return "\n".join([head] + out + ["</svg>"])


def merge_chrome_traces(modelled: list, measured_by_rank: dict, path: str = None) -> dict:
    """One chrome trace with the planner's modelled stage timeline (``planner.stages.pipeline_chrome_trace``)
    above the measured phases of every rank (``FusedAttentionExecutor.profile_chrome_trace``).  The
    modelled events keep their per-device lanes under process ids 0 .. n_nodes-1 named
    "modelled node n"; rank r's measured phases go to process id 1000 + r named "measured rank r",
    so both open side by side in a trace viewer."""
    events = []
    nodes = sorted({e["pid"] for e in modelled})
    for n in nodes:
        events.append({"name": "process_name", "ph": "M", "pid": n, "args": {"name": f"modelled node {n}"}})
    events.extend(dict(e) for e in modelled)
    for rank in sorted(measured_by_rank):
        pid = 1000 + int(rank)
        events.append({"name": "process_name", "ph": "M", "pid": pid, "args": {"name": f"measured rank {rank}"}})
        events.extend({**e, "pid": pid} for e in measured_by_rank[rank])
    trace = {"traceEvents": events, "displayTimeUnit": "ms"}
    if path:
        import json
        with open(path, "w") as f:
            json.dump(trace, f)
    return trace

"""Lower a placed, staged workload to the tables the fused sm_100a executor consumes.

The instruction plans (``ExecutionPlan``) describe data movement as explicit SEND/RECV/copy/sum
instructions.  On one NVSwitch node the same placement and stage assignment is executed with
the movement folded into kernels: remote blocks are pulled once from the owner's arena into a
staging row range, every attention tile stores its partial (out, lse) straight into the
owner's partial arena (or final buffer when it is the only contribution), gradients are
accumulated in fp32 and added into the owner's accumulator.  This module derives, for all
devices at once, the per-device ``FusedProgram``: row offsets, pull lists, kernel work tables,
merge lists and gradient push lists.  Everything is NumPy / CPU tensors so planner worker
processes can build it ahead of time.
"""
from __future__ import annotations

from collections import defaultdict
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from ..core.blocks import BlockType, Device, WorkloadSpec
from ..core.common import ExecutionContext
from ..core.instructions import BufferType
from ..ops.attention import AttnRow, BwdTables, FwdTables, build_bwd_tables, build_fwd_tables
from ..runtime.layout import LocalLayout
from .scheduler import _concat_row_mask


@dataclass
class FusedProgram:
    rank: int
    world: int
    block_size: int
    heads_q: int            # query heads per arena row (head block size)
    heads_kv: int
    n_stages: int
    q_local_rows: int
    kv_local_rows: int
    q_rows: int             # local + staging
    kv_rows: int
    part_rows: int          # rows of this rank's partial arena
    q_pulls: List[np.ndarray] = field(default_factory=list)    # per stage int32 [n,4] (peer, src_row, dst_row, n)
    kv_pulls: List[np.ndarray] = field(default_factory=list)
    fwd: List[Optional[FwdTables]] = field(default_factory=list)
    bwd: List[Optional[BwdTables]] = field(default_factory=list)
    merge_ops: np.ndarray = None        # int32 [n,4] (dst_row, n_tok, src_off, n_src)
    merge_src: np.ndarray = None        # int32
    dq_push: np.ndarray = None          # int32 [n,4] (owner, src_row, dst_row, n)
    dkv_push: np.ndarray = None
    # the pulls as copy jobs (csrc/kernels/copy_jobs.cuh), per stage: Q + KV rows, and what the backward
    # needs on top (dO rows, lse / delta statistics of the pulled query rows)
    jobs_qkv: List[np.ndarray] = field(default_factory=list)    # int32 [n,4] (src_off, dst_off, n, where)
    jobs_grad: List[np.ndarray] = field(default_factory=list)
    fwd_flops: float = 0.0
    bwd_flops: float = 0.0
    pull_bytes: float = 0.0
    need_all: Tuple[int, int, int] = (0, 0, 0)   # max over all ranks of (q_rows, kv_rows, part_rows)
    relayed_blocks: int = 0   # blocks an instruction plan relays through a non-owner (fetched from the owner here)

    def max_rows(self) -> Tuple[int, int, int]:
        return self.q_rows, self.kv_rows, self.part_rows


def _i4(rows) -> np.ndarray:
    return np.asarray(rows, dtype=np.int32).reshape(-1, 4)


JOB_CHUNK_UNITS = 4096     # 64 KB of 16-byte units per copy job: the unit of work one CTA's fetch warps take
KIND_Q, KIND_KV, KIND_DOUT, KIND_LSE, KIND_DELTA = range(5)


def row_copy_jobs(pulls: np.ndarray, kind: int, row_units: int) -> np.ndarray:
    """Row pulls (peer, src_row, dst_row, n_rows) of a [rows, ...] region with ``row_units`` 16-byte
    units per row -> copy jobs of at most JOB_CHUNK_UNITS units."""
    out = []
    for peer, src_row, dst_row, n in np.asarray(pulls).reshape(-1, 4).tolist():
        total, s0, d0 = n * row_units, src_row * row_units, dst_row * row_units
        for off in range(0, total, JOB_CHUNK_UNITS):
            out.append((s0 + off, d0 + off, min(JOB_CHUNK_UNITS, total - off), peer | (kind << 8)))
    return _i4(out)


def stat_copy_jobs(pulls: np.ndarray, kind: int, heads: int) -> np.ndarray:
    """Pulls of query rows -> per-head copy jobs of a [heads, rows] fp32 statistics region."""
    out = []
    for peer, src_row, dst_row, n in np.asarray(pulls).reshape(-1, 4).tolist():
        for h in range(heads):
            out.append((src_row, dst_row, n, peer | (kind << 8) | (1 << 16) | (h << 24)))
    return _i4(out)


def lower_all(context: ExecutionContext, workload: WorkloadSpec, build_backward: bool = True,
              only: Optional[Device] = None) -> Dict[Device, FusedProgram]:
    """Programs of all devices, or just of ``only`` (row and slot numbering is global either way),
    from the placed and staged workload (``work_to_device_map`` / ``work_to_stage_map``)."""
    return _lower(context, workload, workload.work_to_device_map, workload.work_to_stage_map, None, None,
                  build_backward, only)


def lower_plans(context: ExecutionContext, workload: WorkloadSpec, fw_plans, build_backward: bool = True,
                only: Optional[Device] = None) -> Dict[Device, FusedProgram]:
    """Programs derived from the forward ``ExecutionPlan`` instruction streams of all devices.

    The plans are run symbolically (``planner.validate.validate_plans``, which also checks them): every
    attention row of every AttnInstr gives the device and stage of its work units, the order of its KV
    blocks and its key ranges; every RECV gives the stage's source of a remote block.  Those replace
    the workload's own maps and masks as the input of the lowering, so a plan deserialised from bytes
    (plus the workload's block metadata) is all the fused executor needs.  What the fused path does
    not take over from the plan is its temporary slot numbering: the interpreter reuses slots in time
    (pairwise reductions free them), the fused path keeps every partial until its single merge, so
    staging rows and partial slots are numbered by the lowering.  A block the plan relays through a
    non-owner is fetched from its owner instead (all peers of an NVSwitch node are equally far, and
    only the owners' local rows are guaranteed complete at the barrier that opens a call).

    Role of AttentionExecutor.execute interpreting a plan (dcp/runtime/flash_attention/executor.py:486-515,
    dcp/core/executor.py:128-141)."""
    from .validate import validate_plans
    trace: dict = {}
    validate_plans(context, workload, fw_plans, True, trace)
    pair_to_work = {(u.q_id, u.kv_id): w for w, u in workload.block_mapping.work_id_to_meta.items()}
    w2d, w2s, row_ranges = {}, {}, {}
    for dev, stage, q_id, kv_ids, rng4 in trace["rows"]:
        for kv_id in kv_ids:
            w = pair_to_work[(q_id, kv_id)]
            w2d[w], w2s[w] = tuple(dev), stage
        row_ranges[(tuple(dev), stage, q_id)] = (list(kv_ids), rng4)
    return _lower(context, workload, w2d, w2s, row_ranges, trace["recv"], build_backward, only)


def _lower(context: ExecutionContext, workload: WorkloadSpec, work_to_device, work_to_stage, row_ranges, sources,
           build_backward: bool, only: Optional[Device]) -> Dict[Device, FusedProgram]:
    """Shared lowering.  ``row_ranges`` {(device, stage, q id): ([kv ids in order], ranges [n, 4])} and
    ``sources`` {(device, block id): device the plan receives it from} come from instruction plans
    (None: derive rows and masks from the workload, fetch from owners)."""
    wl = workload
    devices = context.devices()
    world = len(devices)
    rank_of = {d: r for r, d in enumerate(devices)}
    in_meta, out_meta, work_meta = (wl.block_mapping.input_id_to_meta, wl.block_mapping.output_id_to_meta,
                                    wl.block_mapping.work_id_to_meta)
    any_q = next(m for m in in_meta.values() if m.type == BlockType.Q)
    any_kv = next(m for m in in_meta.values() if m.type == BlockType.KV)
    block_size, hq, hkv = any_q.block_size, any_q.head_block_size, any_kv.head_block_size
    n_stages = (max(work_to_stage.values()) + 1) if work_to_stage else 1
    layouts = {d: LocalLayout(wl, d) for d in devices}
    owner_in = {i: tuple(d) for i, d in wl.input_to_device_map.items()}
    owner_out = {o: tuple(d) for o, d in wl.output_to_device_map.items()}

    def local_row(dev, buf, block_id, is_input=True):
        idx_map = wl.block_mapping.input_id_to_buffer_index if is_input else wl.block_mapping.output_id_to_buffer_index
        return layouts[dev].row_range(buf, idx_map[dev][block_id])[0]

    # ---- where each device finds each input: local row or a staging row filled by a pull
    q_row: Dict[Device, Dict[int, int]] = {d: {} for d in devices}
    kv_row: Dict[Device, Dict[int, int]] = {d: {} for d in devices}
    q_next = {d: layouts[d].n_tokens(BufferType.LOCAL_Q) for d in devices}
    kv_next = {d: layouts[d].n_tokens(BufferType.LOCAL_KV) for d in devices}
    q_pulls = {d: [[] for _ in range(n_stages)] for d in devices}
    kv_pulls = {d: [[] for _ in range(n_stages)] for d in devices}
    units_ps: Dict[Device, List[List[int]]] = {d: [[] for _ in range(n_stages)] for d in devices}
    for w in sorted(work_to_stage):
        units_ps[tuple(work_to_device[w])][work_to_stage[w]].append(w)
    relayed = 0
    pull_bytes = {d: 0.0 for d in devices}
    for d in devices:
        for s in range(n_stages):
            for w in units_ps[d][s]:
                u = work_meta[w]
                for bid, rows, nxt, pulls, buf in ((u.q_id, q_row, q_next, q_pulls, BufferType.LOCAL_Q),
                                                   (u.kv_id, kv_row, kv_next, kv_pulls, BufferType.LOCAL_KV)):
                    if bid in rows[d]:
                        continue
                    own = owner_in[bid]
                    if own == d:
                        rows[d][bid] = local_row(d, buf, bid)
                    else:
                        if sources is not None:
                            assert (d, bid) in sources, f"plan of {d} uses remote block {bid} without receiving it"
                            relayed += tuple(sources[(d, bid)]) != own
                        n = in_meta[bid].n_tokens
                        rows[d][bid] = nxt[d]
                        pulls[d][s].append((rank_of[own], local_row(own, buf, bid), nxt[d], n))
                        nxt[d] += -(-n // 8) * 8   # keep staging blocks 8-row aligned
                        pull_bytes[d] += wl.input_sizes[bid]

    # ---- partial outputs: one per (device, q block, stage); single contributions go straight home
    contributions: Dict[int, List[Tuple[Device, int]]] = defaultdict(list)  # out id -> [(dev, stage)]
    rows_ps: Dict[Device, List[Dict[int, List[int]]]] = {d: [defaultdict(list) for _ in range(n_stages)] for d in devices}
    for d in devices:
        for s in range(n_stages):
            for w in units_ps[d][s]:
                rows_ps[d][s][work_meta[w].q_id].append(w)
            for q_id in sorted(rows_ps[d][s]):
                contributions[work_meta[rows_ps[d][s][q_id][0]].out_id].append((d, s))
    part_next = {d: 0 for d in devices}
    part_slot: Dict[Tuple[int, Device, int], int] = {}
    merge_lists: Dict[Device, List[Tuple[int, int, List[int]]]] = {d: [] for d in devices}
    for out_id in sorted(contributions):
        own = owner_out[out_id]
        contribs = contributions[out_id]
        if len(contribs) == 1:
            continue
        n = out_meta[out_id].n_tokens
        slots = []
        for (d, s) in contribs:
            part_slot[(out_id, d, s)] = part_next[own]
            slots.append(part_next[own])
            part_next[own] += -(-n // 8) * 8
        merge_lists[own].append((local_row(own, BufferType.LOCAL_OUT, out_id, False), n, slots))

    programs: Dict[Device, FusedProgram] = {}
    for d in devices:
        if only is not None and tuple(only) != d:
            continue
        prog = FusedProgram(rank_of[d], world, block_size, hq, hkv, n_stages,
                            layouts[d].n_tokens(BufferType.LOCAL_Q), layouts[d].n_tokens(BufferType.LOCAL_KV),
                            q_next[d], kv_next[d], part_next[d])
        prog.pull_bytes = pull_bytes[d]
        prog.relayed_blocks = relayed
        prog.need_all = (max(q_next.values()), max(kv_next.values()), max(part_next.values()))
        for s in range(n_stages):
            prog.q_pulls.append(_i4(q_pulls[d][s]))
            prog.kv_pulls.append(_i4(kv_pulls[d][s]))
            qp, kp = prog.q_pulls[-1], prog.kv_pulls[-1]
            prog.jobs_qkv.append(np.concatenate([row_copy_jobs(qp, KIND_Q, hq * 16), row_copy_jobs(kp, KIND_KV, hkv * 32)]))
            prog.jobs_grad.append(np.concatenate([row_copy_jobs(qp, KIND_DOUT, hq * 16), stat_copy_jobs(qp, KIND_LSE, hq),
                                                  stat_copy_jobs(qp, KIND_DELTA, hq)]) if build_backward else _i4([]))
            attn_rows: List[AttnRow] = []
            for q_id in sorted(rows_ps[d][s]):
                units = sorted((work_meta[w] for w in rows_ps[d][s][q_id]), key=lambda u: in_meta[u.kv_id].block_id)
                qm = in_meta[q_id]
                if row_ranges is not None:
                    kv_order, ranges = row_ranges[(d, s, q_id)]
                    by_kv = {u.kv_id: u for u in units}
                    assert sorted(kv_order) == sorted(by_kv), f"plan row of q block {q_id} lists other KV blocks"
                    units = [by_kv[k] for k in kv_order]                         # the plan's table order
                    ranges = np.ascontiguousarray(ranges, dtype=np.int32).reshape(qm.n_tokens, 4)
                else:
                    rng = _concat_row_mask(units, qm.n_tokens, block_size)       # [range, bound, n_q]
                    ranges = np.ascontiguousarray(rng.transpose(2, 0, 1).reshape(qm.n_tokens, 4))
                out_id = units[0].out_id
                own = owner_out[out_id]
                if (out_id, d, s) in part_slot:
                    out_dev, out_row = rank_of[own], part_slot[(out_id, d, s)]
                else:  # only contribution: write the final buffer of the owner directly
                    out_dev, out_row = world + rank_of[own], local_row(own, BufferType.LOCAL_OUT, out_id, False)
                q_own = owner_in[q_id]
                attn_rows.append(AttnRow(
                    q_row=q_row[d][q_id], n_tokens=qm.n_tokens, heads=list(range(hq)),
                    kv=[(kv_row[d][u.kv_id], in_meta[u.kv_id].n_tokens) for u in units], ranges=ranges,
                    out_dev=out_dev, out_row=out_row,
                    # gradients accumulate in the fp32 mirror of the arena row the operand was read from
                    dq_dev=0, dq_row=q_row[d][q_id], dkv=[(0, kv_row[d][u.kv_id]) for u in units]))
            if attn_rows:
                ft = build_fwd_tables(attn_rows, block_size, "cpu")
                prog.fwd.append(ft)
                prog.fwd_flops += ft.flops
                if build_backward:
                    bt = build_bwd_tables(attn_rows, block_size, hq, hkv, "cpu")
                    prog.bwd.append(bt)
                    prog.bwd_flops += bt.flops
                else:
                    prog.bwd.append(None)
            else:
                prog.fwd.append(None)
                prog.bwd.append(None)
        ops, src = [], []
        for dst_row, n, slots in merge_lists[d]:
            ops.append((dst_row, n, len(src), len(slots)))
            src.extend(slots)
        prog.merge_ops = _i4(ops)
        prog.merge_src = np.asarray(src, dtype=np.int32)
        # gradients of staged (remote) blocks go back to the owner's accumulator rows
        dq_push = [(rank_of[owner_in[b]], r, local_row(owner_in[b], BufferType.LOCAL_Q, b), in_meta[b].n_tokens)
                   for b, r in sorted(q_row[d].items()) if owner_in[b] != d]
        dkv_push = [(rank_of[owner_in[b]], r, local_row(owner_in[b], BufferType.LOCAL_KV, b), in_meta[b].n_tokens)
                    for b, r in sorted(kv_row[d].items()) if owner_in[b] != d]
        prog.dq_push, prog.dkv_push = _i4(dq_push), _i4(dkv_push)
        programs[d] = prog
    return programs

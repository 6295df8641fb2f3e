"""Turn a placed workload into per-device instruction plans (forward and backward).

For every device the plan is: stage the locally owned blocks into paged slots; then for each
pipeline stage wait for the transfers feeding it, start the transfers of the next stage, run the
stage's attention rows, and release slots whose last reader has run; finally ship partial
results to their owners and reduce all partials into the local output buffers.  Structure and
instruction semantics follow dcp/core/scheduler.py:541-2240 (forward) and :234-538 (derivation
of the backward workload); the slot bookkeeping is organised around one builder object per
device, and all cross-device SEND/RECV pairs are emitted in one sorted sweep so both ends agree
on their order.
"""
from __future__ import annotations

import json
import os

from collections import defaultdict
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..core.blocks import (BlockManager, BlockMappings, BlockType, ComputationBlockMeta, DataBlockMeta, Device,
                           WorkloadSpec)
from ..core.common import ExecutionContext
from ..core.cost_model import CommunicationCostModel
from ..core.instructions import (AttnBackwardInstr, AttnInstr, AttnReductionInstr, BarrierInstr, BufferBlock,
                                 BufferInfo, BufferType, CommLaunchInstr, CommOp, CommType, CommWaitInstr, DType,
                                 ExecutionPlan, MemcpyInstr, ReductionOp, SumInstr, SumOp)
from .stages import default_n_stages, generate_pipelines_n_stages, pipeline_chrome_trace, summarize_pipeline

# block type -> (local buffer, paged buffer)
_BUFFERS = {
    BlockType.Q: (BufferType.LOCAL_Q, BufferType.BUFFER_Q),
    BlockType.KV: (BufferType.LOCAL_KV, BufferType.BUFFER_KV),
    BlockType.Out: (BufferType.LOCAL_OUT, BufferType.BUFFER_OUT),
    BlockType.LSE: (BufferType.LOCAL_LSE, BufferType.BUFFER_LSE),
    BlockType.dOut: (BufferType.LOCAL_dOUT, BufferType.BUFFER_dOUT),
    BlockType.dQ: (BufferType.LOCAL_dQ, BufferType.BUFFER_dQ),
    BlockType.dKV: (BufferType.LOCAL_dKV, BufferType.BUFFER_dKV),
}
# block types that share one slot index (the kernel addresses them with a single table)
_SLOT_FAMILY = {BlockType.Q: "q", BlockType.KV: "kv", BlockType.Out: "o", BlockType.LSE: "o", BlockType.dOut: "o",
                BlockType.dQ: "dq", BlockType.dKV: "dkv"}


def _block_key(meta: DataBlockMeta) -> Tuple[int, int, int]:
    return (meta.seq_id, meta.head_id, meta.block_id)


class _DeviceBuilder:
    """Instruction list and slot allocators of one device."""

    def __init__(self, dev: Device):
        self.dev = dev
        self.instrs: list = []
        self.mgr: Dict[str, BlockManager] = defaultdict(BlockManager)
        self.in_slot: Dict[int, int] = {}  # input id -> paged slot currently holding it

    def alloc_input(self, input_id: int, meta: DataBlockMeta, stage: int) -> int:
        fam = _SLOT_FAMILY[meta.type]
        key = ("in", fam) + _block_key(meta) if fam == "o" else ("in", input_id)
        slot = self.mgr[fam].get_or_alloc(key, True)
        self.in_slot[input_id] = slot
        return slot

    def free_input(self, input_id: int, meta: DataBlockMeta) -> None:
        fam = _SLOT_FAMILY[meta.type]
        key = ("in", fam) + _block_key(meta) if fam == "o" else ("in", input_id)
        if self.mgr[fam].has_block(key, True):
            self.mgr[fam].free_block(key, True)
        self.in_slot.pop(input_id, None)


def _local_block(wl: WorkloadSpec, dev: Device, block_id: int, meta: DataBlockMeta, is_input: bool) -> BufferBlock:
    idx_map = (wl.block_mapping.input_id_to_buffer_index if is_input else wl.block_mapping.output_id_to_buffer_index)
    return BufferBlock(_BUFFERS[meta.type][0], idx_map[dev][block_id], meta.n_tokens)


def _concat_row_mask(units: Sequence[ComputationBlockMeta], n_q: int, block_size: int) -> np.ndarray:
    """Ranges of one q row against the concatenation of its KV blocks -> int32 [2, 2, n_q]."""
    big = np.iinfo(np.int64).max
    ms = []
    for u in units:
        m = u.local_attn_mask.numpy()
        if m.ndim == 2:
            m = np.stack([m, np.zeros_like(m)], axis=0)
        ms.append(m[:, :, :n_q])
    m = np.stack(ms).astype(np.int64)                       # [unit, range, bound, n_q]
    off = (np.arange(len(ms), dtype=np.int64) * block_size)[:, None, None]
    s, e = m[:, :, 0] + off, m[:, :, 1] + off
    live = m[:, :, 1] > m[:, :, 0]
    start = np.where(live, s, big).min(axis=0)
    end = np.where(live, e, 0).max(axis=0)
    empty = end <= np.where(start == big, 0, start)
    start = np.where((start == big) | empty, 0, start)
    end = np.where(empty, 0, end)
    return np.stack([start, end], axis=1).astype(np.int32)  # [range, bound, n_q]


def _pad_mask(m: np.ndarray, block_size: int) -> np.ndarray:
    out = np.zeros(m.shape[:-1] + (block_size,), dtype=np.int32)
    out[..., :m.shape[-1]] = m
    return out


def schedule(context: ExecutionContext, workload: WorkloadSpec, comm_cost_model: Optional[CommunicationCostModel] = None,
             logger=None, is_forward: bool = True, pipeline_algo: str = "greedy", n_stages: Optional[int] = None):
    """-> ({device: ExecutionPlan}, work_to_stage_map)."""
    wl = workload
    devices = context.devices()
    n_stages = default_n_stages() if n_stages is None else n_stages
    in_meta, out_meta, work_meta = (wl.block_mapping.input_id_to_meta, wl.block_mapping.output_id_to_meta,
                                    wl.block_mapping.work_id_to_meta)
    if pipeline_algo == "tree":
        from .steiner import generate_pipelines_n_stages_with_tree_packing as gen
    else:
        gen = generate_pipelines_n_stages
    work_ps, comm_ps, comm2_ps = gen(n_stages, devices, wl.workloads, wl.work_unit_input_map, in_meta,
                                     wl.input_sizes, wl.work_to_device_map, wl.input_to_device_map,
                                     not is_forward, logger)
    n_total = len(work_ps)
    _debug_pipeline(work_ps, comm_ps, wl, comm_cost_model, logger, is_forward)
    work_to_stage = {w: s for s, per_dev in enumerate(work_ps) for ws in per_dev.values() for w in ws}
    wl.work_to_stage_map = dict(work_to_stage)
    builders = {d: _DeviceBuilder(d) for d in devices}
    block_size = next(iter(in_meta.values())).block_size if in_meta else 0

    # last stage in which each device reads each input (for slot release)
    last_use: Dict[Device, Dict[int, int]] = {d: {} for d in devices}
    for w, s in work_to_stage.items():
        d = tuple(wl.work_to_device_map[w])
        for i in wl.work_unit_input_map[w]:
            last_use[d][i] = max(last_use[d].get(i, -1), s)
    # a non-owner that serves a block to a peer keeps it until that transfer has been launched
    # (transfers feeding stage t are launched during stage t-1)
    for t in range(1, n_total):
        for dst, comms in comm_ps[t].items():
            for i, src in comms:
                src = tuple(src)
                if tuple(wl.input_to_device_map[i]) != src:
                    last_use[src][i] = max(last_use[src].get(i, -1), t - 1)
    # relays keep a block alive until it has been forwarded
    for s in range(n_total):
        for dst, comms in comm2_ps[s].items():
            for i, src in comms:
                last_use[tuple(src)][i] = max(last_use[tuple(src)].get(i, -1), s)

    # ---- 1. stage locally owned inputs into paged slots
    for d in devices:
        b = builders[d]
        mine = sorted(i for i in last_use[d] if tuple(wl.input_to_device_map[i]) == d)
        pairs = []
        for i in mine:
            meta = in_meta[i]
            slot = b.alloc_input(i, meta, -1)
            pairs.append((_local_block(wl, d, i, meta, True), BufferBlock(_BUFFERS[meta.type][1], slot, meta.n_tokens)))
        if pairs:
            b.instrs.append(MemcpyInstr(pairs))

    def emit_comm(stage: int, comms_per_dst, key: str, stream: Optional[str]) -> bool:
        ops: Dict[Device, List[CommOp]] = {d: [] for d in devices}
        any_op = False
        for dst in devices:
            for i, src in sorted(comms_per_dst.get(dst, ()), key=lambda c: (c[0], tuple(c[1]))):
                src = tuple(src)
                meta = in_meta[i]
                if i in builders[dst].in_slot:
                    continue  # already here (e.g. second member of an out/lse/dout family fetched twice)
                slot = builders[dst].alloc_input(i, meta, stage)
                ops[dst].append(CommOp(CommType.RECV, src, BufferBlock(_BUFFERS[meta.type][1], slot, meta.n_tokens)))
                if tuple(wl.input_to_device_map[i]) == src:
                    blk = _local_block(wl, src, i, meta, True)
                else:
                    blk = BufferBlock(_BUFFERS[meta.type][1], builders[src].in_slot[i], meta.n_tokens)
                ops[src].append(CommOp(CommType.SEND, dst, blk))
                any_op = True
        if any_op:
            for d in devices:
                builders[d].instrs.append(CommLaunchInstr(key, ops[d], stream))
        return any_op

    launched: Dict[str, bool] = {}

    # ---- 2. pipeline stages
    out_versions: Dict[Device, Dict[tuple, List[int]]] = {d: defaultdict(list) for d in devices}
    for s in range(n_total):
        if launched.get(f"S{s}"):
            for d in devices:
                builders[d].instrs.append(CommWaitInstr(f"S{s}"))
        if any(comm2_ps[s].get(d) for d in devices):
            if emit_comm(s, comm2_ps[s], f"S{s}P2", "second_phase"):
                for d in devices:
                    builders[d].instrs.append(CommWaitInstr(f"S{s}P2", "second_phase"))
        if s + 1 < n_total:
            launched[f"S{s + 1}"] = emit_comm(s + 1, comm_ps[s + 1], f"S{s + 1}", None)
        for d in devices:
            units = sorted(work_ps[s].get(d, ()))
            if units:
                if is_forward:
                    _emit_attn_fw(builders[d], wl, units, s, block_size, out_versions[d])
                else:
                    _emit_attn_bw(builders[d], wl, units, s, block_size, out_versions[d])
            for i, last in list(last_use[d].items()):
                if last == s and i in builders[d].in_slot:
                    builders[d].free_input(i, in_meta[i])

    # ---- 3. partial results travel to their owners, 4. final reduction
    _emit_output_phase(builders, wl, devices, out_versions, is_forward)

    plans = {}
    for d in devices:
        plans[d] = _finish_plan(context, wl, d, builders[d], n_total, is_forward, block_size)
    _debug_plans(plans, logger, is_forward)
    return plans, work_to_stage


# ------------------------------------------------------------------------------------ debug output
def _env_on(name: str) -> bool:
    return os.environ.get(name, "0") not in ("0", "", "false", "False")


def _debug_dir() -> str:
    d = os.environ.get("DCP_LOGGING_DEBUG_DIR", "./debug")
    os.makedirs(d, exist_ok=True)
    return d


def _debug_pipeline(work_ps, comm_ps, wl, comm_cost_model, logger, is_forward: bool) -> None:
    """DCP_LOG_PIPELINE: per-stage summary in the log; DCP_DUMP_PIPELINE: chrome trace of the
    modelled timeline (dcp/core/pipeline.py:349-510)."""
    tag = "fw" if is_forward else "bw"
    if _env_on("DCP_LOG_PIPELINE") and logger is not None:
        for row in summarize_pipeline(work_ps, comm_ps, wl.workloads, wl.input_sizes):
            logger.info("pipeline %s %s", tag, row)
    if _env_on("DCP_DUMP_PIPELINE") and comm_cost_model is not None:
        path = os.path.join(_debug_dir(), f"pipeline_{tag}.json")
        with open(path, "w") as f:
            json.dump({"traceEvents": pipeline_chrome_trace(work_ps, comm_ps, wl.workloads, wl.input_sizes,
                                                            comm_cost_model)}, f)


def _debug_plans(plans, logger, is_forward: bool) -> None:
    """DCP_LOG_SCHEDULE / DCP_LOG_INSTRS: instruction listing per device; DCP_LOG_BUFFER_INFO: buffer
    sizes per device; DCP_DEBUG_DUMP_EP_STATS: instruction and byte counts as json (file prefix
    DCP_DEBUG_DUMP_EP_STATS_PREFIX)."""
    tag = "fw" if is_forward else "bw"
    if logger is not None and (_env_on("DCP_LOG_SCHEDULE") or _env_on("DCP_LOG_INSTRS")):
        for d, plan in sorted(plans.items()):
            logger.info("plan %s device %s: %d instructions", tag, d, len(plan.instructions))
            for k, ins in enumerate(plan.instructions):
                logger.info("  [%03d] %s", k, ins)
    if logger is not None and _env_on("DCP_LOG_BUFFER_INFO"):
        for d, plan in sorted(plans.items()):
            logger.info("buffers %s device %s: %s", tag, d, plan.buffer_info)
    if _env_on("DCP_DEBUG_DUMP_EP_STATS"):
        stats = {}
        for d, plan in sorted(plans.items()):
            kinds: Dict[str, int] = defaultdict(int)
            sent = 0
            for ins in plan.instructions:
                kinds[type(ins).__name__] += 1
                if isinstance(ins, CommLaunchInstr):
                    sent += sum(op.buffer_block.n_tokens for op in ins.comm_ops if op.comm_type == CommType.SEND)
            stats[f"{d[0]}.{d[1]}"] = {"instructions": dict(kinds), "tokens_sent": sent,
                                      "serialized_bytes": len(plan.serialize())}
        prefix = os.environ.get("DCP_DEBUG_DUMP_EP_STATS_PREFIX", os.path.join(_debug_dir(), "ep_stats"))
        with open(f"{prefix}_{tag}.json", "w") as f:
            json.dump(stats, f, indent=1)


# --------------------------------------------------------------------------------------- attention rows
def _rows_of(units: Sequence[int], wl: WorkloadSpec):
    """Group work ids by q block; kv blocks inside a row are ordered by token-block id."""
    work_meta, in_meta = wl.block_mapping.work_id_to_meta, wl.block_mapping.input_id_to_meta
    rows: Dict[int, List[ComputationBlockMeta]] = defaultdict(list)
    for w in units:
        rows[work_meta[w].q_id].append(work_meta[w])
    for q_id in sorted(rows):
        yield q_id, sorted(rows[q_id], key=lambda u: in_meta[u.kv_id].block_id)


def _emit_attn_fw(b: _DeviceBuilder, wl: WorkloadSpec, units, stage: int, block_size: int, versions) -> None:
    in_meta, out_meta = wl.block_mapping.input_id_to_meta, wl.block_mapping.output_id_to_meta
    q_tab, kv_tab, o_tab, l_tab, seq_q, seq_kv, masks = [], [], [], [], [], [], []
    for q_id, row in _rows_of(units, wl):
        qm = in_meta[q_id]
        q_tab.append([BufferBlock(BufferType.BUFFER_Q, b.in_slot[q_id], qm.n_tokens)])
        kv_tab.append([BufferBlock(BufferType.BUFFER_KV, b.in_slot[u.kv_id], in_meta[u.kv_id].n_tokens) for u in row])
        out_id, lse_id = row[0].out_id, row[0].lse_id
        slot = b.mgr["out"].alloc_block(("part", out_id), False, b.dev, stage)
        versions[(out_id, lse_id)].append(slot)
        o_tab.append([BufferBlock(BufferType.BUFFER_OUT, slot, qm.n_tokens)])
        l_tab.append([BufferBlock(BufferType.BUFFER_LSE, slot, qm.n_tokens)])
        seq_q.append(block_size)
        seq_kv.append(block_size * len(row))
        masks.append(_pad_mask(_concat_row_mask(row, qm.n_tokens, block_size), block_size))
    mask = torch.from_numpy(np.concatenate(masks, axis=-1))  # [2, 2, total_q]
    if all(u.local_attn_mask.dim() == 2 for u in (wl.block_mapping.work_id_to_meta[w] for w in units)):
        mask = mask[0].contiguous()  # single-range batches keep the compact [2, total_q] form
    b.instrs.append(AttnInstr(stage, seq_q, seq_kv, max(seq_q), max(seq_kv), mask, q_tab, kv_tab, o_tab, l_tab))


def _emit_attn_bw(b: _DeviceBuilder, wl: WorkloadSpec, units, stage: int, block_size: int, versions) -> None:
    in_meta = wl.block_mapping.input_id_to_meta
    q_tab, kv_tab, o_tab, dq_tab, dkv_tab, seq_q, seq_kv, masks = [], [], [], [], [], [], [], []
    sums: List[SumOp] = []
    stage_dkv: Dict[int, List[Tuple[int, int]]] = defaultdict(list)  # dkv id -> [(slot, n_tokens)]
    dq_to_free: List[int] = []
    for q_id, row in _rows_of(units, wl):
        qm = in_meta[q_id]
        q_tab.append([BufferBlock(BufferType.BUFFER_Q, b.in_slot[q_id], qm.n_tokens)])
        kv_tab.append([BufferBlock(BufferType.BUFFER_KV, b.in_slot[u.kv_id], in_meta[u.kv_id].n_tokens) for u in row])
        o_tab.append([BufferBlock(BufferType.BUFFER_OUT, b.in_slot[row[0].out_id], qm.n_tokens)])
        dq_id = row[0].dq_id
        dq_slot = b.mgr["dq"].alloc_block(("part", dq_id), False, b.dev, stage)
        dq_tab.append([BufferBlock(BufferType.BUFFER_dQ, dq_slot, qm.n_tokens)])
        prev = versions.get(("dq", dq_id))
        if prev:
            sums.append(SumOp([BufferBlock(BufferType.BUFFER_dQ, prev[0], qm.n_tokens),
                               BufferBlock(BufferType.BUFFER_dQ, dq_slot, qm.n_tokens)],
                              BufferBlock(BufferType.BUFFER_dQ, prev[0], qm.n_tokens)))
            dq_to_free.append(dq_id)  # released only after every slot of this stage is taken
        else:
            versions[("dq", dq_id)] = [dq_slot]
        dkv_row = []
        for rep, u in enumerate(row):
            n_kv = in_meta[u.kv_id].n_tokens
            slot = b.mgr["dkv"].alloc_block(("part", u.dkv_id), False, b.dev, stage, (q_id, rep))
            dkv_row.append(BufferBlock(BufferType.BUFFER_dKV, slot, n_kv))
            stage_dkv[u.dkv_id].append((slot, n_kv, (q_id, rep)))
        dkv_tab.append(dkv_row)
        seq_q.append(block_size)
        seq_kv.append(block_size * len(row))
        masks.append(_pad_mask(_concat_row_mask(row, qm.n_tokens, block_size), block_size))
    mask = torch.from_numpy(np.concatenate(masks, axis=-1))
    if all(u.local_attn_mask.dim() == 2 for u in (wl.block_mapping.work_id_to_meta[w] for w in units)):
        mask = mask[0].contiguous()
    b.instrs.append(AttnBackwardInstr(stage, seq_q, seq_kv, max(seq_q), max(seq_kv), mask, q_tab, kv_tab, o_tab,
                                      dq_tab, dkv_tab))
    # fold this stage's dKV replicas (one per (q row, kv block) pair) into one running slot per kv block
    for dkv_id in sorted(stage_dkv):
        reps = stage_dkv[dkv_id]
        prev = versions.get(("dkv", dkv_id))
        n_kv = reps[0][1]
        if prev:
            dst = prev[0]
            srcs = [dst] + [r[0] for r in reps]
            to_free = reps
        else:
            dst = reps[0][0]
            srcs = [r[0] for r in reps]
            to_free = reps[1:]
            versions[("dkv", dkv_id)] = [dst]
        if len(srcs) > 1:
            sums.append(SumOp([BufferBlock(BufferType.BUFFER_dKV, s_, n_kv) for s_ in srcs],
                              BufferBlock(BufferType.BUFFER_dKV, dst, n_kv)))
        for slot, _, rep_key in to_free:
            b.mgr["dkv"].free_block(("part", dkv_id), False, b.dev, stage, rep_key)
    for dq_id in dq_to_free:
        b.mgr["dq"].free_block(("part", dq_id), False, b.dev, stage)
    if sums:
        b.instrs.append(SumInstr(sums, output_is_unpadded=0))


# --------------------------------------------------------------------------------------- output phase
def _emit_output_phase(builders, wl: WorkloadSpec, devices, out_versions, is_forward: bool) -> None:
    out_meta = wl.block_mapping.output_id_to_meta
    owner = wl.output_to_device_map
    if is_forward:
        # non-owners first merge their own stage partials so one (out, lse) pair travels
        for d in devices:
            ops = []
            for (out_id, lse_id), slots in sorted(out_versions[d].items()):
                if tuple(owner[out_id]) != d and len(slots) > 1:
                    n = out_meta[out_id].n_tokens
                    ops.append(ReductionOp([(BufferBlock(BufferType.BUFFER_OUT, s, n), BufferBlock(BufferType.BUFFER_LSE, s, n))
                                            for s in slots],
                                           (BufferBlock(BufferType.BUFFER_OUT, slots[0], n),
                                            BufferBlock(BufferType.BUFFER_LSE, slots[0], n))))
                    del slots[1:]
            if ops:
                builders[d].instrs.append(AttnReductionInstr(ops, output_is_unpadded=0))
        ops_by_dev = {d: [] for d in devices}
        received: Dict[Device, Dict[tuple, List[int]]] = {d: defaultdict(list) for d in devices}
        any_op = False
        for src in devices:
            for (out_id, lse_id), slots in sorted(out_versions[src].items()):
                dst = tuple(owner[out_id])
                if dst == src:
                    continue
                n = out_meta[out_id].n_tokens
                rslot = builders[dst].mgr["out"].alloc_block(("recv", out_id), False, src, None)
                received[dst][(out_id, lse_id)].append(rslot)
                # out and lse blocks of one partial are exchanged back to back
                ops_by_dev[src].append(CommOp(CommType.SEND, dst, BufferBlock(BufferType.BUFFER_OUT, slots[0], n)))
                ops_by_dev[src].append(CommOp(CommType.SEND, dst, BufferBlock(BufferType.BUFFER_LSE, slots[0], n)))
                ops_by_dev[dst].append(CommOp(CommType.RECV, src, BufferBlock(BufferType.BUFFER_OUT, rslot, n)))
                ops_by_dev[dst].append(CommOp(CommType.RECV, src, BufferBlock(BufferType.BUFFER_LSE, rslot, n)))
                any_op = True
        if any_op:
            for d in devices:
                builders[d].instrs.append(CommLaunchInstr("O", ops_by_dev[d], None))
                builders[d].instrs.append(CommWaitInstr("O", None))
        for d in devices:
            ops = []
            mine = sorted(o for o, dev in owner.items() if tuple(dev) == d and out_meta[o].type == BlockType.Out)
            for out_id in mine:
                lse_id = out_id + 1
                n = out_meta[out_id].n_tokens
                slots = list(out_versions[d].get((out_id, lse_id), ())) + received[d].get((out_id, lse_id), [])
                srcs = [(BufferBlock(BufferType.BUFFER_OUT, s, n), BufferBlock(BufferType.BUFFER_LSE, s, n)) for s in slots]
                dst = (_local_block(wl, d, out_id, out_meta[out_id], False),
                       _local_block(wl, d, lse_id, out_meta[lse_id], False))
                ops.append(ReductionOp(srcs, dst))
            if ops:
                builders[d].instrs.append(AttnReductionInstr(ops, output_is_unpadded=1))
        return

    # backward: running dQ / dKV sums go to the owners of Q / KV and are added there
    ops_by_dev = {d: [] for d in devices}
    received: Dict[Device, Dict[int, List[int]]] = {d: defaultdict(list) for d in devices}
    any_op = False
    for src in devices:
        for (kind, oid), slots in sorted(out_versions[src].items(), key=lambda kv: (kv[0][0], kv[0][1])):
            dst = tuple(owner[oid])
            if dst == src:
                continue
            n = out_meta[oid].n_tokens
            buf = BufferType.BUFFER_dQ if kind == "dq" else BufferType.BUFFER_dKV
            rslot = builders[dst].mgr[kind].alloc_block(("recv", oid), False, src, None)
            received[dst][oid].append(rslot)
            ops_by_dev[src].append(CommOp(CommType.SEND, dst, BufferBlock(buf, slots[0], n)))
            ops_by_dev[dst].append(CommOp(CommType.RECV, src, BufferBlock(buf, rslot, n)))
            any_op = True
    if any_op:
        for d in devices:
            builders[d].instrs.append(CommLaunchInstr("O", ops_by_dev[d], None))
            builders[d].instrs.append(CommWaitInstr("O", None))
    for d in devices:
        ops = []
        for oid in sorted(o for o, dev in owner.items() if tuple(dev) == d):
            meta = out_meta[oid]
            kind = "dq" if meta.type == BlockType.dQ else "dkv"
            buf = BufferType.BUFFER_dQ if kind == "dq" else BufferType.BUFFER_dKV
            slots = list(out_versions[d].get((kind, oid), ())) + received[d].get(oid, [])
            ops.append(SumOp([BufferBlock(buf, s, meta.n_tokens) for s in slots],
                             _local_block(wl, d, oid, meta, False)))
        if ops:
            builders[d].instrs.append(SumInstr(ops, output_is_unpadded=1))


# --------------------------------------------------------------------------------------- plan assembly
def _finish_plan(context, wl: WorkloadSpec, dev: Device, b: _DeviceBuilder, n_stages: int, is_forward: bool,
                 block_size: int) -> ExecutionPlan:
    in_meta, out_meta = wl.block_mapping.input_id_to_meta, wl.block_mapping.output_id_to_meta
    infos: Dict[str, BufferInfo] = {}

    def per_token(metas, btype):
        for m in metas.values():
            if m.type == btype:
                return m.per_token_shape, m.dtype
        return None, None

    def local_tokens(metas, idx_map, btype):
        return sum(metas[i].n_tokens for i in idx_map.get(dev, {}) if metas[i].type == btype)

    def n_local(metas, idx_map, btype):
        return sum(1 for i in idx_map.get(dev, {}) if metas[i].type == btype)

    def add(local_name, paged_name, btype, metas, idx_map, fam):
        shape, dtype = per_token(metas, btype)
        if shape is None:
            return
        numel = int(np.prod(shape)) * block_size
        toks = local_tokens(metas, idx_map, btype)
        is_lse = btype == BlockType.LSE
        lshape = (shape[0], toks) if is_lse else (toks,) + tuple(shape)
        infos[local_name] = BufferInfo(n_local(metas, idx_map, btype), block_size, numel, dtype, lshape, shape)
        n_slots = b.mgr[fam].high_water
        pshape = (shape[0], n_slots, block_size) if is_lse else (n_slots, block_size) + tuple(shape)
        infos[paged_name] = BufferInfo(n_slots, block_size, numel, dtype, pshape, shape)

    ii, oi = wl.block_mapping.input_id_to_buffer_index, wl.block_mapping.output_id_to_buffer_index
    add(BufferType.LOCAL_Q, BufferType.BUFFER_Q, BlockType.Q, in_meta, ii, "q")
    add(BufferType.LOCAL_KV, BufferType.BUFFER_KV, BlockType.KV, in_meta, ii, "kv")
    if is_forward:
        add(BufferType.LOCAL_OUT, BufferType.BUFFER_OUT, BlockType.Out, out_meta, oi, "out")
        add(BufferType.LOCAL_LSE, BufferType.BUFFER_LSE, BlockType.LSE, out_meta, oi, "out")
    else:
        add(BufferType.LOCAL_OUT, BufferType.BUFFER_OUT, BlockType.Out, in_meta, ii, "o")
        add(BufferType.LOCAL_LSE, BufferType.BUFFER_LSE, BlockType.LSE, in_meta, ii, "o")
        add(BufferType.LOCAL_dOUT, BufferType.BUFFER_dOUT, BlockType.dOut, in_meta, ii, "o")
        add(BufferType.LOCAL_dQ, BufferType.BUFFER_dQ, BlockType.dQ, out_meta, oi, "dq")
        add(BufferType.LOCAL_dKV, BufferType.BUFFER_dKV, BlockType.dKV, out_meta, oi, "dkv")
    # cumulative token counts of the device's Q blocks in local buffer order
    q_ids = sorted((i for i in ii.get(dev, {}) if in_meta[i].type == BlockType.Q), key=lambda i: ii[dev][i])
    cu = [0]
    for i in q_ids:
        cu.append(cu[-1] + in_meta[i].n_tokens)
    return ExecutionPlan(b.instrs, context.n_nodes, context.n_devices_per_node, dev[0], dev[1], n_stages, cu, infos)


# --------------------------------------------------------------------------------------- backward workload
def convert_forward_to_backward(fw: WorkloadSpec, comp_cost_model=None, logger=None) -> WorkloadSpec:
    """Backward workload of a placed forward workload: inputs Q, KV, Out, LSE, dOut; outputs dQ,
    dKV.  dOut (and Out/LSE) stay where the forward output lives and keep its local index, dQ goes
    where Q lives, dKV where KV lives; every work unit stays on its forward device."""
    bm = fw.block_mapping
    in_meta: Dict[int, DataBlockMeta] = dict(bm.input_id_to_meta)
    n_in = len(in_meta)
    out_to_in: Dict[int, int] = {}       # fw output id -> bw input id (Out / LSE)
    dout_of: Dict[int, int] = {}         # fw Out id -> bw dOut input id
    in_dev = dict(fw.input_to_device_map)
    in_idx = {d: dict(m) for d, m in bm.input_id_to_buffer_index.items()}
    nxt = n_in
    for oid in sorted(bm.output_id_to_meta):
        m = bm.output_id_to_meta[oid]
        in_meta[nxt] = DataBlockMeta(m.type, m.dtype, m.seq_id, m.head_id, m.block_id, m.n_tokens, m.block_size,
                                     m.head_block_size, m.per_token_shape)
        out_to_in[oid] = nxt
        dev = tuple(fw.output_to_device_map[oid])
        in_dev[nxt] = dev
        in_idx.setdefault(dev, {})[nxt] = bm.output_id_to_buffer_index[dev][oid]
        nxt += 1
    for oid in sorted(bm.output_id_to_meta):
        m = bm.output_id_to_meta[oid]
        if m.type != BlockType.Out:
            continue
        in_meta[nxt] = DataBlockMeta(BlockType.dOut, m.dtype, m.seq_id, m.head_id, m.block_id, m.n_tokens,
                                     m.block_size, m.head_block_size, m.per_token_shape)
        dout_of[oid] = nxt
        dev = tuple(fw.output_to_device_map[oid])
        in_dev[nxt] = dev
        in_idx.setdefault(dev, {})[nxt] = bm.output_id_to_buffer_index[dev][oid]
        nxt += 1
    # outputs: dQ per Q block, dKV per KV block, numbered in input-id order
    out_meta: Dict[int, DataBlockMeta] = {}
    grad_of: Dict[int, int] = {}
    out_dev, out_idx = {}, {}
    for iid in sorted(bm.input_id_to_meta):
        m = bm.input_id_to_meta[iid]
        gtype = BlockType.dQ if m.type == BlockType.Q else BlockType.dKV
        gid = len(out_meta)
        out_meta[gid] = DataBlockMeta(gtype, m.dtype, m.seq_id, m.head_id, m.block_id, m.n_tokens, m.block_size,
                                      m.head_block_size, m.per_token_shape)
        grad_of[iid] = gid
        dev = tuple(fw.input_to_device_map[iid])
        out_dev[gid] = dev
        out_idx.setdefault(dev, {})[gid] = bm.input_id_to_buffer_index[dev][iid]
    work_meta, costs, w_in, w_out = {}, [], [], []
    for w in range(len(fw.workloads)):
        u = bm.work_id_to_meta[w]
        o_in, l_in, do_in = out_to_in[u.out_id], out_to_in[u.lse_id], dout_of[u.out_id]
        work_meta[w] = ComputationBlockMeta(u.type, u.dtype, u.seq_id, u.head_id, u.q_id, u.kv_id, o_in, l_in, do_in,
                                            grad_of[u.q_id], grad_of[u.kv_id], u.local_attn_mask)
        costs.append(fw.workloads[w] * 2.5)
        w_in.append([u.q_id, u.kv_id, o_in, l_in, do_in])
        w_out.append([grad_of[u.q_id], grad_of[u.kv_id]])
    dtypes = dict(bm.buffer_type_to_dtype)
    qdt = dtypes.get(BufferType.LOCAL_Q, DType.BFLOAT16)
    dtypes.update({BufferType.LOCAL_dQ: qdt, BufferType.LOCAL_dKV: qdt, BufferType.BUFFER_dQ: qdt,
                   BufferType.BUFFER_dKV: qdt, BufferType.BUFFER_dOUT: qdt})
    coloc = []
    for ins, outs in fw.colocation_constraints:
        bw_ins = list(ins) + [out_to_in[o] for o in outs] + [dout_of[o] for o in outs if o in dout_of]
        coloc.append([bw_ins, [grad_of[i] for i in ins]])
    mappings = BlockMappings(in_meta, out_meta, work_meta, in_idx, out_idx, dtypes)
    return WorkloadSpec(costs, w_in, w_out, mappings, in_dev, out_dev, dict(fw.work_to_device_map), {}, coloc)

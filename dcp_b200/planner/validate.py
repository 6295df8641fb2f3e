"""Symbolic execution of a set of per-device plans.

Every buffer slot holds a *name* instead of a tensor - ("in", block id) for inputs, a
("part", output id, {work ids}) record for partial results - and all devices are stepped
cooperatively so SEND/RECV pairs meet.  The run fails if an instruction reads a slot that does
not hold what it should (which also catches slots reused too early), if the two ends of an
exchange disagree, if a work unit is computed twice or never, or if a final output misses a
contribution.  Same idea as the DummyExecutor of the reference's tests/core/test_compiler.py:22-764,
usable for any number of virtual devices on one CPU.
"""
from __future__ import annotations

from collections import defaultdict, deque
from typing import Dict, List, Tuple

import numpy as np

from ..core.blocks import BlockType, Device, WorkloadSpec
from ..core.common import ExecutionContext
from ..core.instructions import (AttnBackwardInstr, AttnInstr, AttnReductionInstr, BarrierInstr, BufferBlock,
                                 BufferType, CommLaunchInstr, CommType, CommWaitInstr, ExecutionPlan, MemcpyInstr,
                                 SumInstr)
from ..runtime.layout import LocalLayout


class PlanValidationError(AssertionError):
    pass


def _check(cond, msg):
    if not cond:
        raise PlanValidationError(msg)


class _Dev:
    def __init__(self, dev: Device, plan: ExecutionPlan, wl: WorkloadSpec):
        self.dev, self.plan = dev, plan
        self.pc = 0
        self.slots: Dict[Tuple[str, int], tuple] = {}
        self.pending: Dict[str, List[Tuple[Device, BufferBlock]]] = {}
        lay = LocalLayout(wl, dev)
        for name, blocks in lay.blocks.items():
            if _is_input_buffer(name, wl):  # inputs of this plan kind start out present
                for idx, (bid, meta) in enumerate(blocks):
                    self.slots[(name, idx)] = ("in", bid, meta.n_tokens)
        self.local_out_ids = {(name, idx): bid for name, blocks in lay.blocks.items()
                              for idx, (bid, _) in enumerate(blocks) if not _is_input_buffer(name, wl)}

    def read(self, b: BufferBlock, what: str):
        v = self.slots.get((b.buffer_type, b.index))
        _check(v is not None, f"{self.dev}: {what} reads empty slot {b}")
        _check(v[-1] == b.n_tokens, f"{self.dev}: {what} reads {b} but the slot holds {v[-1]} tokens")
        return v

    def write(self, b: BufferBlock, v: tuple):
        self.slots[(b.buffer_type, b.index)] = v


def _is_input_buffer(name: str, wl: WorkloadSpec) -> bool:
    has_dout = any(m.type == BlockType.dOut for m in wl.block_mapping.input_id_to_meta.values())
    if name in (BufferType.LOCAL_Q, BufferType.LOCAL_KV):
        return True
    return has_dout and name in (BufferType.LOCAL_OUT, BufferType.LOCAL_LSE, BufferType.LOCAL_dOUT)


def validate_plans(context: ExecutionContext, workload: WorkloadSpec, plans: Dict[Device, ExecutionPlan],
                   is_forward: bool = True, trace: dict = None) -> dict:
    """Symbolic run of all devices' plans (see the module docstring).  When ``trace`` is a dict it is
    filled with what the instruction streams say was done: ``trace["rows"]`` = one entry per attention
    row (device, stage, q block id, [kv block ids in table order], int32 [n_tokens, 4] key ranges) and
    ``trace["recv"]`` = {(device, input block id): device it was received from}."""
    wl = workload
    if trace is not None:
        trace.setdefault("rows", [])
        trace.setdefault("recv", {})
    in_meta, out_meta = wl.block_mapping.input_id_to_meta, wl.block_mapping.output_id_to_meta
    pair_to_work = {}
    for w, u in wl.block_mapping.work_id_to_meta.items():
        pair_to_work[(u.q_id, u.kv_id)] = w
    producers = defaultdict(set)
    for w, outs in enumerate(wl.work_unit_output_map):
        for o in outs:
            producers[o].add(w)
    devs = {d: _Dev(d, plans[d], wl) for d in context.devices()}
    mailbox: Dict[Tuple[Device, Device, str], deque] = defaultdict(deque)
    done_work = set()
    stats = {"attn_units": 0, "comm_blocks": 0, "comm_bytes": 0}

    def step(D: _Dev) -> bool:
        """Run one instruction; False if blocked on an exchange."""
        ins = D.plan.instructions[D.pc]
        if isinstance(ins, MemcpyInstr):
            for src, dst in ins.src_dst_pairs:
                _check(src.n_tokens == dst.n_tokens, f"{D.dev}: memcpy size mismatch {src}->{dst}")
                D.write(dst, D.read(src, "memcpy"))
        elif isinstance(ins, CommLaunchInstr):
            recvs = []
            for op in ins.comm_ops:
                if op.comm_type == CommType.SEND:
                    mailbox[(D.dev, tuple(op.peer), ins.key)].append((D.read(op.buffer_block, "send"), op.buffer_block))
                else:
                    recvs.append((tuple(op.peer), op.buffer_block))
            _check(ins.key not in D.pending, f"{D.dev}: exchange {ins.key} launched twice without a wait")
            D.pending[ins.key] = recvs
        elif isinstance(ins, CommWaitInstr):
            _check(ins.key in D.pending, f"{D.dev}: wait on {ins.key} that was never launched")
            need = defaultdict(int)
            for peer, _ in D.pending[ins.key]:
                need[peer] += 1
            if any(len(mailbox[(peer, D.dev, ins.key)]) < n for peer, n in need.items()):
                return False
            for peer, blk in D.pending.pop(ins.key):
                val, sblk = mailbox[(peer, D.dev, ins.key)].popleft()
                _check(sblk.n_tokens == blk.n_tokens, f"{D.dev}: {ins.key} from {peer}: {sblk} arrives as {blk}")
                _check(_family(sblk.buffer_type) == _family(blk.buffer_type),
                       f"{D.dev}: {ins.key} from {peer}: {sblk.buffer_type} received into {blk.buffer_type}")
                D.write(blk, val)
                if trace is not None and val[0] == "in":
                    trace["recv"][(D.dev, val[1])] = peer
                stats["comm_blocks"] += 1
        elif isinstance(ins, BarrierInstr):
            pass
        elif isinstance(ins, (AttnInstr, AttnBackwardInstr)):
            bw = isinstance(ins, AttnBackwardInstr)
            n_rows = len(ins.q_block_table)
            _check(len(ins.seqlens_q) == n_rows == len(ins.kv_block_table), f"{D.dev}: ragged attention tables")
            items = ins.attn_mask if isinstance(ins.attn_mask, (list, tuple)) else list(ins.attn_mask)
            total_q = items[0].shape[-1]
            _check(total_q == sum(ins.seqlens_q), f"{D.dev}: mask covers {total_q} queries, rows need {sum(ins.seqlens_q)}")
            col = 0
            for i in range(n_rows):
                q = D.read(ins.q_block_table[i][0], "attn q")
                _check(q[0] == "in" and in_meta[q[1]].type == BlockType.Q, f"{D.dev}: q table holds {q}")
                works = set()
                last_blk = -1
                for kb in ins.kv_block_table[i]:
                    kv = D.read(kb, "attn kv")
                    _check(kv[0] == "in" and in_meta[kv[1]].type == BlockType.KV, f"{D.dev}: kv table holds {kv}")
                    _check(in_meta[kv[1]].seq_id == in_meta[q[1]].seq_id, f"{D.dev}: q and kv of different sequences")
                    _check(in_meta[kv[1]].block_id > last_blk, f"{D.dev}: kv row not in position order")
                    last_blk = in_meta[kv[1]].block_id
                    w = pair_to_work.get((q[1], kv[1]))
                    _check(w is not None, f"{D.dev}: pair (q {q[1]}, kv {kv[1]}) is not a work unit")
                    _check(tuple(wl.work_to_device_map[w]) == D.dev, f"{D.dev}: runs work {w} placed elsewhere")
                    _check(wl.work_to_stage_map.get(w) == ins.stage_id, f"{D.dev}: work {w} in wrong stage")
                    _check(w not in done_work, f"work unit {w} computed twice")
                    done_work.add(w)
                    works.add(w)
                _check(ins.seqlens_kv[i] == ins.seqlens_q[i] * len(ins.kv_block_table[i]), f"{D.dev}: seqlens_kv mismatch")
                for m in items:
                    seg = m[..., col:col + ins.seqlens_q[i]]
                    _check(int(seg.min()) >= 0 and int(seg.max()) <= ins.seqlens_kv[i], f"{D.dev}: mask range outside row")
                u = wl.block_mapping.work_id_to_meta[next(iter(works))]
                if trace is not None:
                    n_tok = q[2]
                    cols = [np.asarray(m[..., col:col + n_tok]) for m in items]
                    if cols[0].ndim == 1:      # compact single-range form: items = (starts, ends)
                        rng4 = np.stack([cols[0], cols[1], np.zeros_like(cols[0]), np.zeros_like(cols[0])], axis=1)
                    else:                      # items = ranges, each [bound, query]
                        rng4 = np.stack([cols[0][0], cols[0][1], cols[1][0], cols[1][1]], axis=1)
                    kv_ids = [D.read(kb, "attn kv")[1] for kb in ins.kv_block_table[i]]
                    trace["rows"].append((D.dev, ins.stage_id, q[1], kv_ids, rng4.astype(np.int32)))
                if not bw:
                    ob, lb = ins.out_block_table[i][0], ins.lse_block_table[i][0]
                    D.write(ob, ("part", u.out_id, frozenset(works), ob.n_tokens))
                    D.write(lb, ("part", u.lse_id, frozenset(works), lb.n_tokens))
                else:
                    ob = ins.out_block_table[i][0]
                    o = D.read(ob, "attn-bw out")
                    _check(o[0] == "in" and o[1] == u.out_id, f"{D.dev}: backward row reads out {o}, wants {u.out_id}")
                    l = D.read(BufferBlock(BufferType.BUFFER_LSE, ob.index, ob.n_tokens), "attn-bw lse")
                    do = D.read(BufferBlock(BufferType.BUFFER_dOUT, ob.index, ob.n_tokens), "attn-bw dout")
                    _check(l[1] == u.lse_id and do[1] == u.dout_id, f"{D.dev}: lse/dout slot holds {l}, {do}")
                    dqb = ins.dq_block_table[i][0]
                    D.write(dqb, ("part", u.dq_id, frozenset(works), dqb.n_tokens))
                    _check(len(ins.dkv_block_table[i]) == len(ins.kv_block_table[i]), f"{D.dev}: dkv row length")
                    for kb, db in zip(ins.kv_block_table[i], ins.dkv_block_table[i]):
                        kvv = D.read(kb, "kv")
                        w = pair_to_work[(q[1], kvv[1])]
                        D.write(db, ("part", wl.block_mapping.work_id_to_meta[w].dkv_id, frozenset([w]), db.n_tokens))
                col += ins.seqlens_q[i]
                stats["attn_units"] += len(works)
        elif isinstance(ins, AttnReductionInstr):
            for op in ins.ops:
                _merge(D, [s for s, _ in op.src_buffers], op.dst_buffer[0], producers, ins.output_is_unpadded)
                _merge(D, [s for _, s in op.src_buffers], op.dst_buffer[1], producers, ins.output_is_unpadded)
        elif isinstance(ins, SumInstr):
            for op in ins.ops:
                _merge(D, op.src_buffers, op.dst_buffer, producers, ins.output_is_unpadded)
        else:
            raise PlanValidationError(f"unknown instruction {ins!r}")
        D.pc += 1
        return True

    progress = True
    while progress:
        progress = False
        for D in devs.values():
            while D.pc < len(D.plan.instructions) and step(D):
                progress = True
    stuck = [d for d, D in devs.items() if D.pc < len(D.plan.instructions)]
    _check(not stuck, f"devices {stuck} are blocked on exchanges nobody completes")
    _check(all(not q for q in mailbox.values()), "blocks were sent that nobody received")
    _check(done_work == set(range(len(wl.workloads))), "some work units were never computed")
    # every owned output must be complete
    for d, D in devs.items():
        for (name, idx), oid in D.local_out_ids.items():
            v = D.slots.get((name, idx))
            if not producers[oid]:
                continue  # blocks nobody attends to (fully masked) stay untouched
            _check(v is not None and v[0] == "part" and v[1] == oid, f"{d}: local output {name}[{idx}] holds {v}")
            _check(set(v[2]) == producers[oid], f"{d}: output {oid} misses contributions {producers[oid] - set(v[2])}")
    for d in devs:
        for ins in plans[d].instructions:
            if isinstance(ins, CommLaunchInstr):
                for op in ins.comm_ops:
                    if op.comm_type == CommType.RECV:
                        info = plans[d].buffer_info[op.buffer_block.buffer_type]
                        per_tok = 1
                        for x in info.per_token_shape:
                            per_tok *= x
                        stats["comm_bytes"] += op.buffer_block.n_tokens * per_tok * (2 if info.dtype < 2 else 4)
    return stats


def _family(name: str) -> str:
    return name.replace("Local", "").replace("Buffer", "")


def _merge(D: _Dev, srcs, dst: BufferBlock, producers, final: int) -> None:
    vals = [D.read(s, "reduce") for s in srcs]
    _check(all(v[0] == "part" for v in vals), f"{D.dev}: reduction over non-partials {vals}")
    ids = {v[1] for v in vals}
    _check(len(ids) == 1, f"{D.dev}: reduction mixes outputs {ids}")
    union = set()
    for v in vals:
        _check(not (union & set(v[2])), f"{D.dev}: contribution counted twice in reduction into {dst}")
        union |= set(v[2])
    _check(all(v[-1] == dst.n_tokens for v in vals), f"{D.dev}: reduction token counts differ")
    D.write(dst, ("part", vals[0][1], frozenset(union), dst.n_tokens))


# ------------------------------------------------------------------------------- fused programs
def validate_programs(programs) -> Dict[str, int]:
    """Static checks of the fused executor's tables for all ranks at once (``programs`` is a list
    indexed by rank or a {device: program} dict in rank order):

    * pulls read only rows the owner holds locally and write disjoint staging ranges above the
      local rows, before the first stage that reads them;
    * every row range a forward tile or a backward item reads is local or was pulled in an earlier
      or the same stage; every row it writes lies inside the destination arena;
    * partial-arena slots are written by exactly one tile set and consumed by exactly one merge;
      every merged destination row range is local to the merging rank;
    * gradient pushes cover exactly the pulled row ranges and land in the owner's local rows.

    Returns counters (pulls, tiles, items, merges).  Raises PlanValidationError otherwise."""
    import numpy as np
    progs = list(programs.values()) if isinstance(programs, dict) else list(programs)
    world = len(progs)
    stats = {"pulls": 0, "tiles": 0, "items": 0, "merges": 0}
    for r, p in enumerate(progs):
        _check(p.rank == r and p.world == world, f"rank {r}: program says rank {p.rank} of {p.world}")
        _check(all(n >= v for n, v in zip(p.need_all, p.max_rows())), f"rank {r}: need_all below own rows")

    def ranges_disjoint(ranges, what):
        ranges = sorted(ranges)
        for (a0, a1), (b0, b1) in zip(ranges, ranges[1:]):
            _check(a1 <= b0, f"{what}: rows [{a0},{a1}) and [{b0},{b1}) overlap")

    part_written = [dict() for _ in range(world)]          # owner -> {slot row: n rows}
    for r, p in enumerate(progs):
        for kind, pulls, local_rows, total_rows, owner_local in (
                ("q", p.q_pulls, p.q_local_rows, p.q_rows, lambda peer: progs[peer].q_local_rows),
                ("kv", p.kv_pulls, p.kv_local_rows, p.kv_rows, lambda peer: progs[peer].kv_local_rows)):
            avail = [(0, local_rows, -1)]                   # (row0, row1, stage it becomes readable)
            staged = []
            for s, tab in enumerate(pulls):
                for peer, src, dst, n in np.asarray(tab).reshape(-1, 4).tolist():
                    stats["pulls"] += 1
                    _check(0 <= peer < world and peer != r, f"rank {r} {kind} pull from rank {peer}")
                    _check(0 <= src and src + n <= owner_local(peer), f"rank {r} {kind} pull reads non-local rows of {peer}")
                    _check(local_rows <= dst and dst + n <= total_rows, f"rank {r} {kind} pull writes outside staging")
                    staged.append((dst, dst + n))
                    avail.append((dst, dst + n, s))
            ranges_disjoint(staged, f"rank {r} {kind} staging")

            def readable(row0, n, stage, avail=avail):
                return any(a0 <= row0 and row0 + n <= a1 and st <= stage for a0, a1, st in avail)

            if kind == "q":
                q_readable = readable
            else:
                kv_readable = readable
        for s in range(p.n_stages):
            ft, bt = p.fwd[s], p.bwd[s] if p.bwd else None
            if ft is not None:
                tiles, entries = ft.tiles.numpy(), ft.kv_entries.numpy()
                for q_row, n_rows, head, kv_off, n_kv, mask_row, out_dev, out_row in tiles.tolist():
                    stats["tiles"] += 1
                    _check(0 <= head < p.heads_q, f"rank {r}: tile head {head}")
                    _check(q_readable(q_row, n_rows, s), f"rank {r} stage {s}: tile reads Q rows [{q_row},+{n_rows}) not present")
                    _check(0 <= kv_off and kv_off + n_kv <= entries.shape[0], f"rank {r}: tile's KV list is out of range")
                    for ent in entries[kv_off:kv_off + n_kv].tolist():
                        # (row, tokens) per KV block for 128-row tiles, (row, position, keys, flags) per 128-key tile otherwise
                        row, n_tok = (ent[0], ent[1]) if ft.tile_m == 128 else (ent[0], ent[2])
                        _check(kv_readable(row, n_tok, s), f"rank {r} stage {s}: tile reads KV rows [{row},+{n_tok}) not present")
                    _check(mask_row >= 0 and mask_row + n_rows <= ft.masks.shape[0], f"rank {r}: mask rows out of range")
                    if out_dev < world:
                        _check(out_row + n_rows <= progs[out_dev].part_rows, f"rank {r}: partial outside rank {out_dev}'s arena")
                        if head == 0:
                            part_written[out_dev].setdefault((out_row, out_row + n_rows), set()).add((r, s))
                    else:
                        own = out_dev - world
                        _check(0 <= own < world and out_row + n_rows <= progs[own].q_local_rows,
                               f"rank {r}: final output outside rank {own}'s local rows")
            if bt is not None:
                items = bt.items.numpy()
                for kv_row, n_valid, item_off, n_items, dkv_dev, dkv_row, _, _ in bt.ctas.numpy().tolist():
                    _check(kv_readable(kv_row, n_valid, s), f"rank {r} stage {s}: backward reads KV rows [{kv_row},+{n_valid})")
                    _check(dkv_dev == 0 and dkv_row + n_valid <= p.kv_rows, f"rank {r}: dKV rows outside the accumulator")
                    for q_row, n_rows, _pos, mask_row, dq_dev, dq_row, _full, _ in items[item_off:item_off + n_items].tolist():
                        stats["items"] += 1
                        _check(q_readable(q_row, n_rows, s), f"rank {r} stage {s}: backward reads Q rows [{q_row},+{n_rows})")
                        _check(dq_dev == 0 and dq_row + n_rows <= p.q_rows, f"rank {r}: dQ rows outside the accumulator")
                        _check(mask_row + n_rows <= bt.masks.shape[0], f"rank {r}: backward mask rows out of range")
    for r, p in enumerate(progs):
        consumed = set()
        seen_slots = set()
        for dst_row, n, off, n_src in np.asarray(p.merge_ops).reshape(-1, 4).tolist():
            stats["merges"] += 1
            _check(n_src >= 2, f"rank {r}: merge of {n_src} partial(s)")
            _check(dst_row + n <= p.q_local_rows, f"rank {r}: merge destination outside local rows")
            for slot in np.asarray(p.merge_src)[off:off + n_src].tolist():
                _check(slot not in seen_slots, f"rank {r}: partial slot {slot} merged twice")
                seen_slots.add(slot)
                inside = sorted(iv for iv in part_written[r] if slot <= iv[0] and iv[1] <= slot + n)
                _check(inside and inside[0][0] == slot and inside[-1][1] == slot + n and
                       all(a[1] == b[0] for a, b in zip(inside, inside[1:])),
                       f"rank {r}: partial slot [{slot},+{n}) is not fully written ({inside[:3]})")
                writers = set().union(*(part_written[r][iv] for iv in inside))
                _check(len(writers) == 1, f"rank {r}: partial slot {slot} written by {sorted(writers)}")
                consumed.update(inside)
        _check(consumed == set(part_written[r]), f"rank {r}: partial rows written but never merged: "
                                                 f"{sorted(set(part_written[r]) - consumed)[:4]}")
        for kind, push, pulls, owner_local in (("dq", p.dq_push, p.q_pulls, lambda o: progs[o].q_local_rows),
                                               ("dkv", p.dkv_push, p.kv_pulls, lambda o: progs[o].kv_local_rows)):
            pulled = sorted((peer, src, dst, n) for tab in pulls for peer, src, dst, n in np.asarray(tab).reshape(-1, 4).tolist())
            pushed = sorted((o, dst, src, n) for o, src, dst, n in np.asarray(push).reshape(-1, 4).tolist())
            _check(pulled == pushed, f"rank {r}: {kind} pushes do not mirror the pulls")
            for o, src, dst, n in np.asarray(push).reshape(-1, 4).tolist():
                _check(dst + n <= owner_local(o), f"rank {r}: {kind} push lands outside rank {o}'s local rows")
    return stats

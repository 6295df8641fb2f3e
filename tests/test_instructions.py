"""Wire-format tests: round trips for every instruction kind and a hand-assembled golden plan.

Mirrors the reference's tests/core/test_instructions.py (deserialize(serialize(x)) == x, no
trailing bytes) and pins the byte layout independently of the library's own writer.
"""
import random
import struct

import pytest
import torch

from dcp_b200.core.instructions import (AttnBackwardInstr, AttnInstr, AttnReductionInstr, BarrierInstr,
                                        BlockInstrBase, BufferBlock, BufferInfo, BufferType, CommLaunchInstr, CommOp,
                                        CommType, CommWaitInstr, DType, ExecutionPlan, MemcpyInstr, ReductionOp,
                                        SumInstr, SumOp, deserialize_list_of_execution_plans,
                                        serialize_list_of_execution_plans)


def _blk(rng, types=BufferType.PAGED):
    return BufferBlock(rng.choice(types), rng.randrange(0, 64), rng.randrange(1, 513))


def _table(rng, n_rows, buf):
    return [[BufferBlock(buf, rng.randrange(0, 64), rng.randrange(1, 513)) for _ in range(rng.randrange(1, 4))]
            for _ in range(n_rows)]


def _mask(rng, mask_dim, total_q):
    shape = (2, total_q) if mask_dim == 2 else (2, 2, total_q)
    return torch.randint(0, 1000, shape, dtype=torch.int32, generator=torch.Generator().manual_seed(rng.randrange(1 << 30)))


def _random_instr(rng, kind, mask_dim=2):
    if kind == "memcpy":
        return MemcpyInstr([(_blk(rng, BufferType.LOCAL), _blk(rng)) for _ in range(rng.randrange(1, 6))])
    if kind == "launch":
        ops = [CommOp(rng.choice([CommType.SEND, CommType.RECV]), (rng.randrange(4), rng.randrange(8)), _blk(rng))
               for _ in range(rng.randrange(0, 6))]
        return CommLaunchInstr(f"S{rng.randrange(5)}", ops, rng.choice([None, "second_phase"]))
    if kind == "barrier":
        return BarrierInstr()
    if kind == "wait":
        return CommWaitInstr(f"S{rng.randrange(5)}", rng.choice([None, "second_phase"]))
    if kind in ("attn", "attn_bw"):
        n = rng.randrange(1, 5)
        out = _table(rng, n, BufferType.BUFFER_OUT)
        head = dict(stage_id=rng.randrange(5), seqlens_q=[256] * n, seqlens_kv=[256 * rng.randrange(1, 4) for _ in range(n)],
                    max_seqlen_q=256, max_seqlen_kv=768, attn_mask=_mask(rng, mask_dim, 256 * n),
                    q_block_table=_table(rng, n, BufferType.BUFFER_Q), kv_block_table=_table(rng, n, BufferType.BUFFER_KV),
                    out_block_table=out)
        if kind == "attn":
            lse = [[BufferBlock(BufferType.BUFFER_LSE, b.index, b.n_tokens) for b in row] for row in out]
            return AttnInstr(lse_block_table=lse, **head)
        return AttnBackwardInstr(dq_block_table=_table(rng, n, BufferType.BUFFER_dQ),
                                 dkv_block_table=_table(rng, n, BufferType.BUFFER_dKV), **head)
    if kind == "reduce":
        ops = []
        for _ in range(rng.randrange(1, 4)):
            srcs = []
            for _ in range(rng.randrange(1, 4)):
                i, n = rng.randrange(64), rng.randrange(1, 257)
                srcs.append((BufferBlock(BufferType.BUFFER_OUT, i, n), BufferBlock(BufferType.BUFFER_LSE, i, n)))
            i, n = rng.randrange(64), rng.randrange(1, 257)
            ops.append(ReductionOp(srcs, (BufferBlock(BufferType.LOCAL_OUT, i, n), BufferBlock(BufferType.LOCAL_LSE, i, n))))
        return AttnReductionInstr(ops, rng.choice([0, 1]))
    if kind == "sum":
        ops = [SumOp([_blk(rng, (BufferType.BUFFER_dKV,)) for _ in range(rng.randrange(1, 5))],
                     _blk(rng, (BufferType.LOCAL_dKV,))) for _ in range(rng.randrange(1, 4))]
        return SumInstr(ops, rng.choice([0, 1]))
    raise AssertionError(kind)


KINDS = ["memcpy", "launch", "barrier", "wait", "attn", "attn_bw", "reduce", "sum"]


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("mask_dim", [2, 3])
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_instruction_roundtrip(kind, mask_dim, seed):
    rng = random.Random(seed * 100 + mask_dim)
    instr = _random_instr(rng, kind, mask_dim)
    data = instr.serialize()
    back, rest = BlockInstrBase.deserialize(data)
    assert rest == b""
    assert type(back) is type(instr) and back == instr
    assert back.serialize() == data


def test_tags_follow_definition_order():
    assert [c.tag for c in (MemcpyInstr, CommLaunchInstr, BarrierInstr, CommWaitInstr, AttnInstr, AttnBackwardInstr,
                            AttnReductionInstr, SumInstr)] == list(range(8))


@pytest.mark.parametrize("seed", [0, 1])
def test_plan_roundtrip(seed):
    rng = random.Random(seed)
    instrs = [_random_instr(rng, rng.choice(KINDS), rng.choice([2, 3])) for _ in range(12)]
    infos = {BufferType.LOCAL_Q: BufferInfo(3, 256, 256 * 4 * 64, DType.BFLOAT16, (700, 4, 64), (4, 64)),
             BufferType.BUFFER_LSE: BufferInfo(5, 256, 256 * 4, DType.FLOAT32, (4, 5, 256), (4,))}
    plan = ExecutionPlan(instrs, 2, 4, 1, 3, 5, [0, 256, 500, 700], infos)
    data = plan.serialize()
    back, rest = ExecutionPlan.deserialize(data)
    assert rest == b"" and back == plan
    blob = serialize_list_of_execution_plans([plan, plan])
    plans, rest = deserialize_list_of_execution_plans(blob)
    assert rest == b"" and plans == [plan, plan]


def test_golden_bytes():
    """Bytes assembled by hand from the format description: u32 little-endian integers, u8
    instruction tag, u32-length-prefixed strings."""
    u32 = lambda v: struct.pack("<I", v)
    s = lambda t: u32(len(t.encode())) + t.encode()
    blk = lambda name, i, n: s(name) + u32(i) + u32(n)
    plan = ExecutionPlan(
        [MemcpyInstr([(BufferBlock("LocalQ", 1, 200), BufferBlock("BufferQ", 0, 200))]),
         CommLaunchInstr("S1", [CommOp(CommType.RECV, (0, 1), BufferBlock("BufferKV", 2, 256))], None),
         BarrierInstr(), CommWaitInstr("S1", "second_phase"),
         SumInstr([SumOp([BufferBlock("BufferdQ", 0, 8), BufferBlock("BufferdQ", 1, 8)], BufferBlock("LocaldQ", 0, 8))], 1)],
        1, 2, 0, 1, 5, [0, 200], {"LocalQ": BufferInfo(1, 256, 16384, 0, (200, 1, 64), (1, 64))})
    expect = (u32(1) + u32(2) + u32(0) + u32(1) + u32(5) + u32(2) + u32(0) + u32(200)
              + u32(1) + s("LocalQ") + u32(1) + u32(256) + u32(16384) + u32(0)
              + u32(3) + u32(200) + u32(1) + u32(64) + u32(2) + u32(1) + u32(64)
              + u32(5)
              + b"\x00" + u32(1) + blk("LocalQ", 1, 200) + blk("BufferQ", 0, 200)
              + b"\x01" + s("S1") + u32(1) + u32(1) + u32(0) + u32(1) + blk("BufferKV", 2, 256) + u32(0)
              + b"\x02"
              + b"\x03" + s("S1") + s("second_phase")
              + b"\x07" + u32(1) + u32(2) + blk("BufferdQ", 0, 8) + blk("BufferdQ", 1, 8) + blk("LocaldQ", 0, 8) + u32(1))
    assert plan.serialize() == expect


def test_attn_mask_wire_form():
    u32 = lambda v: struct.pack("<I", v)
    mask = torch.arange(12, dtype=torch.int32).reshape(2, 6)
    row = [[BufferBlock("BufferQ", 0, 6)]]
    instr = AttnInstr(0, [6], [6], 6, 6, mask, row, [[BufferBlock("BufferKV", 0, 6)]],
                      [[BufferBlock("BufferOut", 0, 6)]], [[BufferBlock("BufferLSE", 0, 6)]])
    data = instr.serialize()
    # tag, stage, seqlens_q, seqlens_kv, max_q, max_kv, then n_items=2 and per item (shape tuple, nbytes, raw)
    off = 1 + 4 + 8 + 8 + 4 + 4
    assert data[off:off + 4] == u32(2)
    assert data[off + 4:off + 12] == u32(1) + u32(6)
    assert data[off + 12:off + 16] == u32(24)
    assert data[off + 16:off + 40] == mask[0].numpy().tobytes()

"""Pure-torch interpreter of execution plans (any device, any dtype).

Runs all eight instruction kinds with plain tensor ops, so it is the oracle for the planner
(fp32 on CPU over gloo or in-process mailboxes) and the numerical reference for the fused
sm_100a executor.  Buffer shapes, block addressing and instruction semantics follow
dcp/runtime/flash_attention/executor.py:340-2133; the attention rows are evaluated densely.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch

from ..core.blocks import Device, WorkloadSpec
from ..core.executor import DCPExecutor
from ..core.instructions import (AttnBackwardInstr, AttnInstr, AttnReductionInstr, BarrierInstr, BufferBlock,
                                 BufferType, CommLaunchInstr, CommType, CommWaitInstr, ExecutionPlan, MemcpyInstr,
                                 SumInstr)
from .layout import LocalLayout


def _row_mask(attn_mask, col0: int, n_q: int, n_kv: int) -> torch.Tensor:
    """Boolean [n_q, n_kv] of one row from the instruction's stacked range mask."""
    items = attn_mask if isinstance(attn_mask, (list, tuple)) else [attn_mask[i] for i in range(attn_mask.shape[0])]
    if items[0].dim() == 1:      # [2, total_q] -> two rows: starts, ends
        ranges = [(items[0], items[1])]
    else:                         # 2 x [2, total_q]
        ranges = [(m[0], m[1]) for m in items]
    pos = torch.arange(n_kv)[None, :]
    allow = torch.zeros(n_q, n_kv, dtype=torch.bool)
    for s, e in ranges:
        s = s[col0:col0 + n_q].long()[:, None]
        e = e[col0:col0 + n_q].long()[:, None]
        allow |= (pos >= s) & (pos < e)
    return allow


class ReferenceAttentionExecutor(DCPExecutor):
    def __init__(self, comm, workload: WorkloadSpec, dev: Device, n_devices_per_node: int, n_nodes: int = 1,
                 softmax_scale: Optional[float] = None, device: Optional[torch.device] = None, synchronous=False,
                 logger=None):
        super().__init__(dev[0], dev[1], n_nodes, n_devices_per_node, synchronous, device, logger)
        self.comm = comm
        self.dev = tuple(dev)
        self.layout = LocalLayout(workload, dev)
        self.softmax_scale = softmax_scale
        self.register_handler(MemcpyInstr, self._memcpy)
        self.register_handler(CommLaunchInstr, self._comm_launch)
        self.register_handler(CommWaitInstr, self._comm_wait)
        self.register_handler(BarrierInstr, lambda instr: self.comm.barrier())
        self.register_handler(AttnInstr, self._attn)
        self.register_handler(AttnBackwardInstr, self._attn_bw)
        self.register_handler(AttnReductionInstr, self._reduce)
        self.register_handler(SumInstr, self._sum)

    # ---- block views
    def set_layout(self, workload: WorkloadSpec) -> None:
        self.layout = LocalLayout(workload, self.dev)

    def view(self, b: BufferBlock) -> torch.Tensor:
        """Tensor view of a block with tokens on axis 0 ([n_tokens, *per_token]); LSE -> [n_tokens, heads]."""
        buf = self.buffers[b.buffer_type]
        lse = BufferType.is_lse(b.buffer_type)
        if BufferType.is_local(b.buffer_type):
            lo, hi = self.layout.row_range(b.buffer_type, b.index)
            assert hi - lo == b.n_tokens, f"{b}: layout says {hi - lo} tokens"
            return buf[:, lo:hi].transpose(0, 1) if lse else buf[lo:hi]
        return buf[:, b.index, :b.n_tokens].transpose(0, 1) if lse else buf[b.index, :b.n_tokens]

    def _scale(self, d: int) -> float:
        return self.softmax_scale if self.softmax_scale is not None else 1.0 / math.sqrt(d)

    def _flat_rank(self, peer) -> int:
        return peer[0] * self.n_devices_per_node + peer[1]

    # ---- handlers
    def _memcpy(self, instr: MemcpyInstr) -> None:
        for src, dst in instr.src_dst_pairs:
            self.view(dst).copy_(self.view(src))

    def _comm_launch(self, instr: CommLaunchInstr) -> None:
        sends, recvs = [], []
        for op in instr.comm_ops:
            v = self.view(op.buffer_block)
            (sends if op.comm_type == CommType.SEND else recvs).append((self._flat_rank(op.peer), v))
        self.comm.launch(instr.key, sends, recvs)

    def _comm_wait(self, instr: CommWaitInstr) -> None:
        self.comm.wait(instr.key)

    def _gather_kv(self, row: Sequence[BufferBlock], block_size: int):
        """Concatenate a row's KV blocks, each padded to block_size positions -> (k, v, valid)."""
        ks, vs, valid = [], [], []
        for b in row:
            kv = self.view(b)  # [n, 2, hkv, d]
            pad = block_size - b.n_tokens
            k, v = kv[:, 0], kv[:, 1]
            if pad:
                z = k.new_zeros((pad,) + tuple(k.shape[1:]))
                k, v = torch.cat([k, z]), torch.cat([v, z])
            ks.append(k)
            vs.append(v)
            valid.append(torch.cat([torch.ones(b.n_tokens, dtype=torch.bool), torch.zeros(pad, dtype=torch.bool)]))
        return torch.cat(ks), torch.cat(vs), torch.cat(valid)

    def _scores(self, q, k, allow):
        g = q.shape[1] // k.shape[1]
        kf = k.float().repeat_interleave(g, dim=1)
        s = torch.einsum("qhd,khd->hqk", q.float(), kf) * self._scale(q.shape[-1])
        return s.masked_fill(~allow.to(s.device)[None], float("-inf")), g

    def _attn(self, instr: AttnInstr) -> None:
        col = 0
        for i, q_row in enumerate(instr.q_block_table):
            qb = q_row[0]
            block_size = instr.seqlens_q[i]
            q = self.view(qb)
            k, v, valid = self._gather_kv(instr.kv_block_table[i], block_size)
            allow = _row_mask(instr.attn_mask, col, qb.n_tokens, k.shape[0]) & valid[None]
            s, g = self._scores(q, k, allow)
            lse = torch.logsumexp(s, dim=-1)                       # [h, q]
            safe = torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)
            p = torch.exp(s - safe[..., None])
            p = torch.where(torch.isinf(lse)[..., None], torch.zeros_like(p), p)
            out = torch.einsum("hqk,khd->qhd", p, v.float().repeat_interleave(g, dim=1))
            self.view(instr.out_block_table[i][0]).copy_(out.to(q.dtype))
            self.view(instr.lse_block_table[i][0]).copy_(lse.transpose(0, 1))
            col += block_size

    def _attn_bw(self, instr: AttnBackwardInstr) -> None:
        col = 0
        for i, q_row in enumerate(instr.q_block_table):
            qb = q_row[0]
            block_size = instr.seqlens_q[i]
            q = self.view(qb)
            ob = instr.out_block_table[i][0]
            out = self.view(ob)
            lse = self.view(BufferBlock(BufferType.BUFFER_LSE, ob.index, ob.n_tokens)).transpose(0, 1)  # [h, q]
            dout = self.view(BufferBlock(BufferType.BUFFER_dOUT, ob.index, ob.n_tokens))
            k, v, valid = self._gather_kv(instr.kv_block_table[i], block_size)
            allow = _row_mask(instr.attn_mask, col, qb.n_tokens, k.shape[0]) & valid[None]
            s, g = self._scores(q, k, allow)
            safe = torch.where(torch.isinf(lse), torch.full_like(lse, float("inf")), lse).float()
            p = torch.exp(s - safe[..., None])                      # rows with lse = -inf -> 0
            vf = v.float().repeat_interleave(g, dim=1)
            kf = k.float().repeat_interleave(g, dim=1)
            do = dout.float()
            dp = torch.einsum("qhd,khd->hqk", do, vf)
            delta = (do * out.float()).sum(-1).transpose(0, 1)      # [h, q]
            ds = p * (dp - delta[..., None]) * self._scale(q.shape[-1])
            dq = torch.einsum("hqk,khd->qhd", ds, kf)
            dk = torch.einsum("hqk,qhd->khd", ds, q.float())
            dv = torch.einsum("hqk,qhd->khd", p, do)
            hkv = k.shape[1]
            dk = dk.reshape(dk.shape[0], hkv, g, -1).sum(2)
            dv = dv.reshape(dv.shape[0], hkv, g, -1).sum(2)
            self.view(instr.dq_block_table[i][0]).copy_(dq.to(q.dtype))
            for j, dkv_b in enumerate(instr.dkv_block_table[i]):
                lo = j * block_size
                dst = self.view(dkv_b)                              # [n, 2, hkv, d]
                dst[:, 0].copy_(dk[lo:lo + dkv_b.n_tokens].to(dst.dtype))
                dst[:, 1].copy_(dv[lo:lo + dkv_b.n_tokens].to(dst.dtype))
            col += block_size

    def _reduce(self, instr: AttnReductionInstr) -> None:
        for op in instr.ops:
            outs = torch.stack([self.view(o).float() for o, _ in op.src_buffers])       # [n, t, h, d]
            lses = torch.stack([self.view(l).float() for _, l in op.src_buffers])       # [n, t, h]
            lse = torch.logsumexp(lses, dim=0)
            safe = torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)
            w = torch.exp(lses - safe[None])
            w = torch.where(torch.isinf(lses) & (lses < 0), torch.zeros_like(w), w)
            merged = (outs * w[..., None]).sum(0)
            self.view(op.dst_buffer[0]).copy_(merged.to(self.buffers[op.dst_buffer[0].buffer_type].dtype))
            self.view(op.dst_buffer[1]).copy_(lse)

    def _sum(self, instr: SumInstr) -> None:
        for op in instr.ops:
            acc = self.view(op.src_buffers[0]).float().clone()
            for b in op.src_buffers[1:]:
                acc += self.view(b).float()
            self.view(op.dst_buffer).copy_(acc.to(self.buffers[op.dst_buffer.buffer_type].dtype))

    # ---- convenience API mirroring AttentionExecutor.forward/backward
    def forward(self, plan: ExecutionPlan, local_q: torch.Tensor, local_kv: torch.Tensor):
        self.init_buffers(plan)
        self.init_forward_input(local_q, local_kv)
        self.execute(plan, True)
        return self.buffers[BufferType.LOCAL_OUT], self.buffers[BufferType.LOCAL_LSE]

    def backward(self, plan: ExecutionPlan, bw_workload: WorkloadSpec, local_dout: torch.Tensor):
        """Needs LocalQ/LocalKV/LocalOut/LocalLSE from a preceding ``forward`` on this executor."""
        self.set_layout(bw_workload)
        self.init_buffers(plan, keep_local=True)
        self.init_backward_input(local_dout)
        self.execute(plan, False)
        return self.buffers[BufferType.LOCAL_dQ], self.buffers[BufferType.LOCAL_dKV]

"""User-facing attention API over instruction plans: ``get_executor``, ``AttentionExecutor``,
``DCPAttention`` and the test / benchmark glue (mirrors dcp/runtime/flash_attention/
executor.py:340-587, 2077-2133 and interface.py:124-433, utils.py:33-277, 686-931).

``AttentionExecutor`` interprets ``ExecutionPlan`` s.  ``executor_impl="python"`` runs every
instruction with torch ops over ``torch.distributed`` point-to-point (gloo on CPU, NCCL on GPU);
``"fused"`` selects the sm_100a executor, which needs a ``FusedProgram`` (see
``dcp_b200.planner.lowering``) and is what the training engine uses.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import numpy as np
import torch

from ..core.blocks import Device, WorkloadSpec
from ..core.common import ExecutionContext
from ..core.instructions import BufferType, ExecutionPlan
from ..planner import masks
from ..planner.compiler import CompilerConfig, InstrCompiler
from ..planner.workload import generate_workload, pad_seqlens
from .comm import MailboxComm, TorchDistComm
from .executor_ref import ReferenceAttentionExecutor
from .layout import LocalLayout, gather_local, get_local_q_kv, scatter_to_global, seq_token_offsets  # noqa: F401


class AttentionExecutor:
    def __init__(self, n_heads_per_block: int, head_dim: int, exec_context: ExecutionContext,
                 fw_exec_plan: Optional[ExecutionPlan] = None, fw_workload: Optional[WorkloadSpec] = None,
                 bw_exec_plan: Optional[ExecutionPlan] = None, bw_workload: Optional[WorkloadSpec] = None,
                 process_group=None, comm=None, synchronous: bool = False, iteration_idx: Optional[int] = None,
                 tp_rank: Optional[int] = None, device: Optional[torch.device] = None,
                 softmax_scale: Optional[float] = None):
        self.ctx = exec_context
        self.fw_plan, self.bw_plan, self.fw_workload, self.bw_workload = fw_exec_plan, bw_exec_plan, fw_workload, bw_workload
        dev = (fw_exec_plan.node_id, fw_exec_plan.local_device_id)
        if comm is None:
            ranks = None
            if process_group is not None:
                import torch.distributed as dist
                ranks = dist.get_process_group_ranks(process_group)
            comm = TorchDistComm(process_group, ranks)
        self.impl = ReferenceAttentionExecutor(comm, fw_workload, dev, exec_context.n_devices_per_node,
                                               exec_context.n_nodes, softmax_scale, device, synchronous)
        self.is_forward = True
        self.n_heads_per_block, self.head_dim = n_heads_per_block, head_dim

    def prepare(self, forward: bool = True) -> None:
        if forward:
            self.impl.set_layout(self.fw_workload)
            self.impl.init_buffers(self.fw_plan)
        else:
            self.impl.set_layout(self.bw_workload)
            self.impl.init_buffers(self.bw_plan, keep_local=True)
        self.is_forward = forward

    def forward(self, q: torch.Tensor, kv: torch.Tensor):
        if not self.is_forward or not self.impl.buffers:
            self.prepare(True)
        self.impl.init_forward_input(q, kv)
        self.impl.execute(self.fw_plan, True)
        return self.impl.buffers[BufferType.LOCAL_OUT], self.impl.buffers[BufferType.LOCAL_LSE]

    def switch_to_backward(self) -> None:
        self.prepare(False)

    def set_local_out_lse(self, out: torch.Tensor, lse: torch.Tensor) -> None:
        self.impl.buffers[BufferType.LOCAL_OUT].copy_(out.reshape(self.impl.buffers[BufferType.LOCAL_OUT].shape))
        self.impl.buffers[BufferType.LOCAL_LSE].copy_(lse.reshape(self.impl.buffers[BufferType.LOCAL_LSE].shape))

    def backward(self, q, kv, out, dout, lse):
        if self.is_forward:
            self.switch_to_backward()
        b = self.impl.buffers
        b[BufferType.LOCAL_Q].copy_(q.reshape(b[BufferType.LOCAL_Q].shape))
        b[BufferType.LOCAL_KV].copy_(kv.reshape(b[BufferType.LOCAL_KV].shape))
        self.set_local_out_lse(out, lse)
        self.impl.init_backward_input(dout)
        self.impl.execute(self.bw_plan, False)
        return b[BufferType.LOCAL_dQ], b[BufferType.LOCAL_dKV]

    def capture_cudagraph(self, *a, **k) -> None:
        """Plans that contain point-to-point exchanges are not graph-captured by this executor."""
        return None

    def deallocate_all_buffers(self) -> None:
        self.impl.deallocate_buffers()

    def log_memory_usage(self) -> Dict[str, int]:
        return {name: t.numel() * t.element_size() for name, t in self.impl.buffers.items()}


class FusedPlanExecutor:
    """The reference executor API (prepare / forward / backward / ...) on top of the fused sm_100a
    executor: the placed and staged forward workload is lowered to kernel tables for this device
    and run with in-kernel communication; q / kv / out / lse use the same local buffer layouts as
    the plan-interpreting executor ([rows, head_block, d], lse [head_block, rows])."""

    def __init__(self, n_heads_per_block: int, head_dim: int, exec_context: ExecutionContext,
                 fw_exec_plan: Optional[ExecutionPlan] = None, fw_workload: Optional[WorkloadSpec] = None,
                 bw_exec_plan: Optional[ExecutionPlan] = None, bw_workload: Optional[WorkloadSpec] = None,
                 process_group=None, synchronous: bool = False, device: Optional[torch.device] = None,
                 softmax_scale: Optional[float] = None, all_fw_exec_plans=None, **_unused):
        """``all_fw_exec_plans`` ({device: forward ExecutionPlan} of every device of the group, e.g.
        deserialised from bytes): when given, the kernel tables are derived from those instruction
        streams (``planner.lowering.lower_plans``); a rank needs its peers' plans because its tiles
        store partial results straight into the owners' arenas.  Without it the tables come from
        the placed and staged workload, which every rank holds."""
        from ..planner.lowering import lower_all, lower_plans
        from .executor_fused import FusedAttentionExecutor
        # The sm_100a kernels are built for 128 channels per head in bf16.  Smaller head dimensions run
        # on them zero-padded to 128: padded Q/K columns add nothing to the scores, padded V / dO
        # columns give zero output and gradient columns, which are cut off again; the softmax scale
        # stays 1/sqrt(head_dim).  fp16 / fp32 tensors are converted to bf16 on the way in and results
        # are returned in the caller's dtype (accumulation is fp32 throughout).
        assert head_dim % 8 == 0 and 8 <= head_dim <= 128, \
            "the fused executor covers head dimensions up to 128 (multiples of 8); use executor_impl='python' beyond"
        if softmax_scale is None:
            softmax_scale = head_dim ** -0.5
        dev = (fw_exec_plan.node_id, fw_exec_plan.local_device_id)
        if all_fw_exec_plans is not None:
            self.program = lower_plans(exec_context, fw_workload, all_fw_exec_plans, build_backward=True, only=dev)[dev]
        else:
            self.program = lower_all(exec_context, fw_workload, build_backward=True, only=dev)[dev]
        device = device or torch.device("cuda", torch.cuda.current_device())
        rq, rkv, rp = self.program.need_all
        self.impl = FusedAttentionExecutor(self.program.heads_q, self.program.heads_kv, rq, rkv, max(rp, 128), device,
                                           process_group if exec_context.n_devices > 1 else None, softmax_scale)
        self.impl.synchronous = self.impl.synchronous or synchronous
        self.impl.prepare(self.program)
        self.fw_plan, self.bw_plan, self.fw_workload, self.bw_workload = fw_exec_plan, bw_exec_plan, fw_workload, bw_workload
        self.is_forward = True
        self.n_heads_per_block, self.head_dim = n_heads_per_block, head_dim
        self._epoch = -1

    def prepare(self, forward: bool = True) -> None:
        self.is_forward = forward

    def switch_to_backward(self) -> None:
        self.is_forward = False

    def _put(self, dst: torch.Tensor, src: torch.Tensor) -> None:
        """``src`` [..., head_dim] of any float dtype into the kernel buffer ``dst`` [..., 128] bf16."""
        d = self.head_dim
        src = src.reshape(dst.shape[:-1] + (d,))
        if d == dst.shape[-1]:
            dst.copy_(src)
        else:
            dst[..., :d].copy_(src)
            dst[..., d:].zero_()

    def _write_inputs(self, q, kv) -> None:
        ex = self.impl
        self._put(ex.q_local(), q)
        self._put(ex.kv_local(), kv)
        ex.inputs_written()
        self._epoch = ex.arena_epoch

    def forward(self, q: torch.Tensor, kv: torch.Tensor):
        self._write_inputs(q, kv)
        out, lse = self.impl.forward()
        if self.head_dim != out.shape[-1] or out.dtype != q.dtype:
            out = out[..., :self.head_dim].to(q.dtype)
        return out, lse

    def set_local_out_lse(self, out: torch.Tensor, lse: torch.Tensor) -> None:
        self._put(self.impl.out_local(), out)
        self.impl.lse_local().copy_(lse.reshape(self.impl.lse_local().shape))

    def backward(self, q, kv, out, dout, lse):
        ex = self.impl
        if ex.arena_epoch != self._epoch or not ex._staging_valid:
            self._write_inputs(q, kv)
        self.set_local_out_lse(out, lse)
        if self.head_dim == ex.q_local().shape[-1]:
            dout_k = dout.reshape(ex.q_local().shape)
        else:
            dout_k = torch.zeros(ex.q_local().shape, dtype=ex.q_local().dtype, device=dout.device)
            self._put(dout_k, dout)
        dq, dkv = ex.backward(dout_k)
        d = self.head_dim
        return dq[..., :d].to(q.dtype).contiguous(), dkv[..., :d].to(kv.dtype).contiguous()

    def capture_cudagraph(self, *a, **k) -> None:
        """Nothing to capture: a call is a handful of launches whose tables change every batch."""
        return None

    def deallocate_all_buffers(self) -> None:
        self.impl = None

    def log_memory_usage(self) -> Dict[str, int]:
        ex = self.impl
        return {n: getattr(ex, n).numel() * getattr(ex, n).element_size()
                for n in ("q", "kv", "out", "lse", "dout", "delta", "part_out", "part_lse", "dq", "dkv")}


def get_executor(n_heads_per_block: int, head_dim: int, exec_context: ExecutionContext, fw_exec_plan=None,
                 fw_workload=None, bw_exec_plan=None, bw_workload=None, executor_impl: str = "python",
                 process_group=None, synchronous: bool = False, iteration_idx=None, tp_rank=None,
                 use_cudagraph: bool = False, comm=None, device=None, all_fw_exec_plans=None) -> AttentionExecutor:
    if executor_impl == "fused":
        # the B200-native path behind the same interface (CUDA only; head_dim <= 128, computed in bf16)
        return FusedPlanExecutor(n_heads_per_block, head_dim, exec_context, fw_exec_plan, fw_workload, bw_exec_plan,
                                 bw_workload, process_group, synchronous, device, all_fw_exec_plans=all_fw_exec_plans)
    if executor_impl not in ("python", "reference"):
        raise ValueError("executor_impl is 'python' (plan interpreter) or 'fused' (sm_100a kernels)")
    return AttentionExecutor(n_heads_per_block, head_dim, exec_context, fw_exec_plan, fw_workload, bw_exec_plan,
                             bw_workload, process_group, comm, synchronous, iteration_idx, tp_rank, device)


class DCPAttention(torch.autograd.Function):
    """q [n_head_blocks * local_tokens, hbs, d], kv [n_kv_head_blocks * local_tokens, 2, hbs_kv, d] -> out."""

    @staticmethod
    def forward(ctx, executor: AttentionExecutor, capture_fwd_graph, capture_bwd_graph, q, kv):
        out, lse = executor.forward(q, kv)
        out, lse = out.clone(), lse.clone()
        ctx.executor = executor
        ctx.save_for_backward(q, kv, out, lse)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, kv, out, lse = ctx.saved_tensors
        dq, dkv = ctx.executor.backward(q, kv, out, dout.contiguous(), lse)
        return None, None, None, dq.clone().view_as(q), dkv.clone().view_as(kv)


# ---------------------------------------------------------------------------------------- test glue
def prepare_dcp_distributed_attn_for_test(raw_seqlens: Sequence[int], n_heads: int, n_query_groups: int, head_dim: int,
                                          block_size: int, head_block_size: int, exec_context: ExecutionContext,
                                          rank: int, mask_type: str = "causal", dtype=torch.bfloat16, seed: int = 0,
                                          process_group=None, comm=None, device=None,
                                          executor_impl: str = "python"):
    """Plan a batch, build this rank's executor and local operands.  Returns the 9-tuple
    (executor, local_q, local_kv, local_dout, q, kv, dout, (fw_workload, bw_workload), padded_seqlens)."""
    padded = pad_seqlens(raw_seqlens, block_size)
    mask = masks.get_mask_fn(mask_type)(list(raw_seqlens), padded, torch.int32)
    wl = generate_workload((sum(padded), n_heads, head_dim), (sum(padded), 2, n_query_groups, head_dim),
                           list(raw_seqlens), padded, block_size, head_block_size, exec_context.comp_cost_model, mask,
                           dtype)
    fw_wl, bw_wl, fw, bw = InstrCompiler(exec_context, CompilerConfig()).compile(wl)
    devs = exec_context.devices()
    dev = devs[rank]
    g = torch.Generator().manual_seed(seed)
    T = sum(raw_seqlens)
    q = torch.randn(T, n_heads, head_dim, generator=g).to(dtype)
    kv = torch.randn(T, 2, n_query_groups, head_dim, generator=g).to(dtype)
    dout = torch.randn(T, n_heads, head_dim, generator=g).to(dtype)
    all_plans = None
    if executor_impl == "fused-from-plan-bytes":
        # the fused executor fed with nothing but serialised plans: every device's forward plan goes
        # through its byte encoding and the kernel tables are derived from the instruction streams
        executor_impl = "fused"
        all_plans = {d: ExecutionPlan.deserialize(p.serialize())[0] for d, p in fw.items()}
    ex = get_executor(head_block_size, head_dim, exec_context, fw[dev], fw_wl, bw[dev], bw_wl,
                      executor_impl=executor_impl, process_group=process_group, comm=comm, device=device,
                      all_fw_exec_plans=all_plans)
    lay = LocalLayout(fw_wl, dev)
    mv = (lambda t: t.to(device)) if device is not None else (lambda t: t)
    lq, lkv = get_local_q_kv(q, kv, fw_wl, dev, raw_seqlens)
    ldo = gather_local(dout, lay, BufferType.LOCAL_OUT, raw_seqlens, 1)
    return ex, mv(lq), mv(lkv), mv(ldo), q, kv, dout, (fw_wl, bw_wl), padded


def reconstruct_attention_forward_output_for_test(local_out, local_lse, workload: WorkloadSpec, dev: Device,
                                                  raw_seqlens, n_heads: int, head_dim: int):
    """Place one device's local (out, lse) into zero-filled global tensors (sum over devices = full result)."""
    T = sum(raw_seqlens)
    out_g = torch.zeros(T, n_heads, head_dim, dtype=torch.float32)
    lse_g = torch.zeros(n_heads, T, dtype=torch.float32)
    lay = LocalLayout(workload, dev)
    scatter_to_global(local_out.float().cpu(), out_g, lay, BufferType.LOCAL_OUT, raw_seqlens, 1)
    scatter_to_global(local_lse.float().cpu(), lse_g, lay, BufferType.LOCAL_LSE, raw_seqlens, 0, token_axis_local=1)
    return out_g, lse_g


def reconstruct_attention_backward_output_for_test(local_dq, local_dkv, bw_workload: WorkloadSpec, dev: Device,
                                                   raw_seqlens, n_heads: int, n_query_groups: int, head_dim: int):
    T = sum(raw_seqlens)
    dq_g = torch.zeros(T, n_heads, head_dim, dtype=torch.float32)
    dkv_g = torch.zeros(T, 2, n_query_groups, head_dim, dtype=torch.float32)
    lay = LocalLayout(bw_workload, dev)
    scatter_to_global(local_dq.float().cpu(), dq_g, lay, BufferType.LOCAL_dQ, raw_seqlens, 1)
    scatter_to_global(local_dkv.float().cpu(), dkv_g, lay, BufferType.LOCAL_dKV, raw_seqlens, 2)
    return dq_g, dkv_g


# ---------------------------------------------------------------------------------------- padding helpers
def unpad_input(hidden: torch.Tensor, attention_mask: torch.Tensor):
    """[b, s, ...] + bool [b, s] -> (packed [total, ...], indices, cu_seqlens int32, max_seqlen)."""
    seqlens = attention_mask.sum(dim=-1, dtype=torch.int32)
    indices = torch.nonzero(attention_mask.flatten(), as_tuple=False).flatten()
    cu = torch.nn.functional.pad(torch.cumsum(seqlens, 0, dtype=torch.int32), (1, 0))
    return hidden.reshape(-1, *hidden.shape[2:])[indices], indices, cu, int(seqlens.max())


def pad_input(packed: torch.Tensor, indices: torch.Tensor, batch: int, seqlen: int):
    out = packed.new_zeros(batch * seqlen, *packed.shape[1:])
    out[indices] = packed
    return out.view(batch, seqlen, *packed.shape[1:])


# ---------------------------------------------------------------------------------------- zigzag helpers (ring baselines)
def get_local_attn_ranges_zigzag(global_attn_ranges: torch.Tensor, padded_seqlens: Sequence[int], world_size: int,
                                 rank: int) -> torch.Tensor:
    """Rows of a global range mask that a rank owns under the zigzag split: every sequence is cut
    into 2*world chunks and rank r holds chunks r and 2*world-1-r."""
    cu = seq_token_offsets(padded_seqlens)
    parts = []
    for s, n in enumerate(padded_seqlens):
        assert n % (2 * world_size) == 0, "zigzag needs lengths divisible by 2*world"
        c = n // (2 * world_size)
        base = int(cu[s])
        parts.append(global_attn_ranges[base + rank * c:base + (rank + 1) * c])
        parts.append(global_attn_ranges[base + (2 * world_size - 1 - rank) * c:base + (2 * world_size - rank) * c])
    return torch.cat(parts, dim=0)


def get_per_step_attn_range(local_ranges: torch.Tensor, kv_chunk_start: int, kv_chunk_len: int) -> torch.Tensor:
    """Clamp per-query [start, end) ranges (last dim = 2) to one ring step's KV chunk and rebase them."""
    lo, hi = kv_chunk_start, kv_chunk_start + kv_chunk_len
    start = local_ranges[..., 0].clamp(lo, hi) - lo
    end = local_ranges[..., 1].clamp(lo, hi) - lo
    end = torch.maximum(end, start)
    return torch.stack([start, end], dim=-1)

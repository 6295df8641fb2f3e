"""Fused sm_100a executor: runs a ``FusedProgram`` with communication folded into kernels.

Per attention call (all layers of an iteration share one executor and one program):

forward   barrier -> tcgen05 attention of stage s, whose spare warps fetch the remote operands of
                     stage s+1 from peers' arenas while its tiles are computed (stage 0 works on
                     local operands only); every tile stores its partial (out, lse) into the
                     owner's partial arena / final buffer over NVLink
          barrier -> merge kernel on the owner
backward  delta = rowsum(dO * O); barrier -> backward kernel per stage, fetching the next stage's
          Q, dO, lse, delta, KV the same way, dQ/dK/dV accumulated with fp32 red into arena
          mirrors -> push-add of staged gradients into the owners' accumulators -> barrier
One stream, no events: a stage's operands are in place when its kernel starts because the
previous stage's kernel brought them.

No NCCL call is made on these paths.  Takes the role of AttentionExecutor
(dcp/runtime/flash_attention/executor.py:340-2133) for single-node NVSwitch machines.
"""
from __future__ import annotations

import os

from typing import Optional

import numpy as np
import torch

from ..ops import attention as attn_ops
from ..ops import block_ops
from ..planner.lowering import FusedProgram
from .symm import SymmetricArena

HEAD_DIM = 128


class FusedAttentionExecutor:
    def __init__(self, heads_q: int, heads_kv: int, max_q_rows: int, max_kv_rows: int, max_part_rows: int,
                 device: torch.device, group=None, softmax_scale: Optional[float] = None, timeout_s: float = 10.0,
                 variant: int = 0):
        self.hq, self.hkv = heads_q, heads_kv
        self.device = device
        self.scale = softmax_scale if softmax_scale is not None else HEAD_DIM ** -0.5
        self.variant = variant
        self.group, self.timeout_s = group, timeout_s
        self.arena = None
        self.n_reallocations = 0
        self._allocate((max_q_rows, max_kv_rows, max_part_rows))
        self.program: Optional[FusedProgram] = None
        self.arena_epoch = 0          # bumped whenever q/kv local regions are rewritten
        self._staging_valid = False   # remote Q/KV rows in staging match the current local data on peers
        self.kernel_launches = 0
        self.profile = os.environ.get("DCP_B200_PROFILE", "0") == "1"
        self._marks = []
        # debugging aids: synchronous = wait for the device and read the status word after every
        # phase (the reference executor's synchronous mode, dcp/core/executor.py:55-57); poison =
        # fill every staging region with a large sentinel before a call, so a block that is read
        # without having been pulled or written this call blows up the result instead of silently
        # reusing last call's bytes
        self.synchronous = os.environ.get("DCP_B200_SYNCHRONOUS", "0") == "1"
        self.poison = os.environ.get("DCP_B200_POISON", "0") == "1"
        # debug: recompute every merged row with torch ops and dump the kernel's arguments on a mismatch
        self.check_reductions = os.environ.get("DCP_DEBUG_LOG_REDUCTION_ARGS_ON_ERROR", "0") not in ("0", "", "false", "False")
        # time_calls: one CUDA-event pair around every forward() / backward() call (read with call_times())
        self.time_calls = False
        self._call_events = []
        # host_pin: optional callable (CPU tensor -> pinned CPU tensor) used for every table upload, so
        # the copies are truly asynchronous; the engine passes its pinned host arena's `pin`
        self.host_pin = None
        self._host_keep = []

    def _allocate(self, rows) -> None:
        """(Re)create the symmetric arenas for (q rows, kv rows, partial rows).  Collective: every
        rank of the group must call it with the same sizes (they come from the plan, which is the
        same on all ranks)."""
        rq, rkv, rp = (-(-int(x) // 128) * 128 + 128 for x in rows)
        self.cap = (rq, rkv, rp)
        hq, hkv = self.hq, self.hkv
        bf, f32 = torch.bfloat16, torch.float32
        regions = {
            "q": ((rq, hq, HEAD_DIM), bf), "kv": ((rkv, 2, hkv, HEAD_DIM), bf),
            "dout": ((rq, hq, HEAD_DIM), bf), "out": ((rq, hq, HEAD_DIM), bf),
            "lse": ((hq, rq), f32), "delta": ((hq, rq), f32),
            "part_out": ((rp, hq, HEAD_DIM), bf), "part_lse": ((hq, rp), f32),
            "dq": ((rq, hq, HEAD_DIM), f32), "dkv": ((rkv, 2, hkv, HEAD_DIM), f32),
        }
        if self.arena is not None:
            torch.cuda.synchronize(self.device)
            for name in regions:
                delattr(self, name)
            self.arena = None
            self.n_reallocations += 1
        self.arena = SymmetricArena(regions, self.device, self.group, self.timeout_s)
        self.world, self.rank = self.arena.world, self.arena.rank
        for name in regions:
            setattr(self, name, self.arena.view(name))
        self.copy_ctx = attn_ops.CopyContext(self.arena.peer_ptrs, self.rank, rq)

    # ---- program upload
    def prepare(self, program: FusedProgram) -> None:
        assert program.heads_q == self.hq and program.heads_kv == self.hkv
        need = tuple(max(a, b) for a, b in zip(program.need_all, program.max_rows()))
        if any(n > c for n, c in zip(need, self.cap)):
            # grow with headroom; all ranks see the same need_all, so all of them get here together
            self._allocate(tuple(max(int(n * 1.25), c) for n, c in zip(need, self.cap)))
        dev = self.device
        keep = []          # pinned staging copies stay alive until the next prepare (the copies are asynchronous)

        def up(a):
            t = a if isinstance(a, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(a))
            if self.host_pin is not None and t.numel():
                t = self.host_pin(t)
                keep.append(t)
            return t.to(dev, non_blocking=True)

        def up_tabs(tabs):
            if tabs is None:
                return None
            import dataclasses
            return dataclasses.replace(tabs, **{f.name: up(getattr(tabs, f.name)) for f in dataclasses.fields(tabs)
                                                if isinstance(getattr(tabs, f.name), torch.Tensor)})

        self.program = program
        # copy jobs per stage: Q + KV rows (forward, and backward when the staging rows were
        # overwritten since), dO + statistics (backward)
        self.jobs_qkv = [up(x) for x in program.jobs_qkv]
        self.jobs_grad = [up(x) for x in program.jobs_grad]
        self.jobs_all = [up(np.concatenate([a, b])) for a, b in zip(program.jobs_qkv, program.jobs_grad)]
        self.fwd_tabs = [up_tabs(t) for t in program.fwd]
        self.bwd_tabs = [up_tabs(t) for t in program.bwd]
        self.merge_ops, self.merge_src = up(program.merge_ops), up(program.merge_src)
        self.dq_push, self.dkv_push = up(program.dq_push), up(program.dkv_push)
        self._host_keep = keep
        self._staging_valid = False

    # ---- views the model writes into / reads from
    def q_local(self) -> torch.Tensor:
        return self.q[:self.program.q_local_rows]

    def kv_local(self) -> torch.Tensor:
        return self.kv[:self.program.kv_local_rows]

    def out_local(self) -> torch.Tensor:
        return self.out[:self.program.q_local_rows]

    def lse_local(self) -> torch.Tensor:
        return self.lse[:, :self.program.q_local_rows]

    def inputs_written(self) -> None:
        self.arena_epoch += 1
        self._staging_valid = False

    def _jobs_of(self, lists, s: int):
        """Copy jobs of stage ``s`` (None when there are none or the group has a single rank)."""
        if self.world <= 1 or s >= len(lists) or lists[s].shape[0] == 0:
            return None
        return lists[s]

    def _fetch_standalone(self, jobs) -> None:
        """Operands that no attention kernel can bring along (stage 0 of a single-stage plan, or a
        stage that follows one without work on this rank) are fetched by a launch of their own."""
        if jobs is not None:
            attn_ops.copy_jobs(jobs, self.copy_ctx)
            self.kernel_launches += 1

    # ---- optional phase timing (DCP_B200_PROFILE=1): CUDA events on the main stream around the
    # barriers and the kernels of every call; read with profile_summary() after a synchronize
    def _mark(self, key: str) -> None:
        # phase boundary: an NVTX marker for any attached profiler, the synchronous-mode check, and
        # (when profiling) a CUDA event
        start = key.endswith(":start")
        if start:
            torch.cuda.nvtx.range_push("dcp.attention." + key.split(":")[0])
        else:
            torch.cuda.nvtx.mark(key)
        if self.synchronous and not start:
            torch.cuda.synchronize(self.device)
            self.check_status()
        if self.profile:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(torch.cuda.current_stream(self.device))
            self._marks.append((key, ev))

    def _poison_staging(self, with_grads: bool) -> None:
        # a large finite sentinel, not NaN: rows of a tile past a block's valid tokens are read and
        # multiplied by exact zeros, which a NaN would survive
        p = self.program
        sentinel = 30000.0
        self.q[p.q_local_rows:].fill_(sentinel)
        self.kv[p.kv_local_rows:].fill_(sentinel)
        if with_grads:
            self.dout[p.q_local_rows:].fill_(sentinel)
        else:
            self.part_out.fill_(sentinel)
            self.part_lse.fill_(sentinel)

    def profile_chrome_trace(self, path: Optional[str] = None, pid: Optional[int] = None) -> list:
        """The recorded phases as chrome-trace events (microseconds since the first mark), to be laid
        next to the planner's modelled pipeline trace; consumes the marks like profile_summary()."""
        torch.cuda.synchronize(self.device)
        events, prev = [], None
        origin = self._marks[0][1] if self._marks else None
        for key, ev in self._marks:
            if not key.endswith(":start"):
                events.append({"name": key, "ph": "X", "pid": self.rank if pid is None else pid, "tid": 0,
                               "ts": origin.elapsed_time(prev) * 1e3, "dur": prev.elapsed_time(ev) * 1e3})
            prev = ev
        self._marks = []
        if path:
            import json
            with open(path, "w") as f:
                json.dump({"traceEvents": events}, f)
        return events

    def profile_summary(self) -> dict:
        """Total milliseconds per phase since the last call ("fwd:kernels", "bwd:wait peers", ...)."""
        torch.cuda.synchronize(self.device)
        tot, prev = {}, None
        for key, ev in self._marks:
            if key.endswith(":start"):
                prev = ev
                continue
            tot[key] = tot.get(key, 0.0) + prev.elapsed_time(ev)
            prev = ev
        self._marks = []
        return tot

    # ---- forward
    def forward(self):
        """Attention over the Q/KV already present in ``q_local()`` / ``kv_local()``.
        Returns views (out [rows, hq, d] bf16, lse [hq, rows] fp32) of this rank's own tokens."""
        p, a = self.program, self.arena
        main = torch.cuda.current_stream(self.device)
        tok = self._call_begin("fwd")
        self._mark("fwd:start")
        if self.poison:
            self._poison_staging(False)
        a.barrier()                                   # every rank's inputs are in place
        self._mark("fwd:wait inputs of peers")
        out_dsts = a.peer_ptrs("part_out") + a.peer_ptrs("out")
        lse_dsts = a.peer_ptrs("part_lse") + a.peer_ptrs("lse")
        self._fetch_standalone(self._jobs_of(self.jobs_qkv, 0))
        for s in range(p.n_stages):
            nxt = self._jobs_of(self.jobs_qkv, s + 1)
            t = self.fwd_tabs[s]
            if t is None or t.tile_m != attn_ops.TILE_M_PAIR:
                self._fetch_standalone(nxt)
                nxt = None
            if t is not None:
                self._launch_fwd(t, out_dsts, lse_dsts, nxt)
        self._mark("fwd:kernels (with operand fetch)")
        if self.world > 1:
            a.barrier()                               # all partials have landed at their owners
        self._mark("fwd:wait partials of peers")
        if self.merge_ops.shape[0]:
            block_ops.merge_out_lse(self.merge_ops, self.merge_src, self.part_out, self.part_lse, self.out, self.lse)
            if self.check_reductions:
                block_ops.check_merge_against_reference(
                    self.merge_ops, self.merge_src, self.part_out, self.part_lse, self.out, self.lse,
                    os.path.join(os.environ.get("DCP_LOGGING_DEBUG_DIR", "./debug"), "executor"))
            self.kernel_launches += 1
        self._mark("fwd:merge")
        torch.cuda.nvtx.range_pop()
        self._call_end(tok)
        self._staging_valid = True
        return self.out_local(), self.lse_local()

    def _launch_fwd(self, t, out_dsts, lse_dsts, jobs=None) -> None:
        # destinations 0..world-1 are partial arenas (row stride cap[2]), the rest final buffers (cap[0]);
        # `jobs`: the next stage's operand fetch, carried by this kernel
        attn_ops.attn_fwd(self.q, self.kv, t, out_dsts, lse_dsts, self.scale, a_status(self), self.variant,
                          lse_stride=self.cap[2], lse_stride_b=self.cap[0], n_dst_a=self.world, jobs=jobs,
                          job_ctx=self.copy_ctx)
        self.kernel_launches += 1

    # ---- backward
    def backward(self, dout_local: torch.Tensor):
        """dout_local [rows, hq, d] bf16 for this rank's tokens; returns fp32 accumulator views
        (dq [rows, hq, d], dkv [rows, 2, hkv, d]) valid until the next backward call."""
        p, a = self.program, self.arena
        main = torch.cuda.current_stream(self.device)
        n = p.q_local_rows
        tok = self._call_begin("bwd")
        self._mark("bwd:start")
        if self.poison and not self._staging_valid:
            self._poison_staging(True)
        self.dout[:n].copy_(dout_local.reshape(n, self.hq, HEAD_DIM))
        attn_ops.attn_delta(self.out, self.dout, self.delta, 0, n)
        self.dq[:p.q_rows].zero_()
        self.dkv[:p.kv_rows].zero_()
        self.kernel_launches += 1
        self._mark("bwd:dout copy, delta, zero accumulators")
        a.barrier()
        self._mark("bwd:wait inputs of peers")
        lists = self.jobs_grad if self._staging_valid else self.jobs_all
        self._fetch_standalone(self._jobs_of(lists, 0))
        for s in range(p.n_stages):
            nxt = self._jobs_of(lists, s + 1)
            t = self.bwd_tabs[s]
            if t is None:
                self._fetch_standalone(nxt)
                continue
            attn_ops.attn_bwd(self.q, self.dout, self.kv, self.lse, self.delta, t, [self.dq], [self.dkv], self.scale,
                              a_status(self), jobs=nxt, job_ctx=self.copy_ctx)
            self.kernel_launches += 1
        self._mark("bwd:kernels (with operand fetch)")
        if self.world > 1:
            block_ops.push_add_rows(self.dq_push, self.dq, a.peer_ptrs("dq"), self.hq * HEAD_DIM)
            block_ops.push_add_rows(self.dkv_push, self.dkv, a.peer_ptrs("dkv"), 2 * self.hkv * HEAD_DIM)
            self.kernel_launches += 2
            self._mark("bwd:push gradients to owners")
            a.barrier()
            self._mark("bwd:wait gradients of peers")
        torch.cuda.nvtx.range_pop()
        self._call_end(tok)
        return self.dq[:n], self.dkv[:p.kv_local_rows]

    def check_status(self) -> None:
        self.arena.check_status()

    def _call_begin(self, kind: str):
        if not self.time_calls:
            return None
        e0 = torch.cuda.Event(enable_timing=True)
        e0.record(torch.cuda.current_stream(self.device))
        return (kind, e0)

    def _call_end(self, tok) -> None:
        if tok is not None:
            e1 = torch.cuda.Event(enable_timing=True)
            e1.record(torch.cuda.current_stream(self.device))
            self._call_events.append((tok[0], tok[1], e1))

    def call_times(self) -> dict:
        """{"fwd_ms", "bwd_ms", "n_fwd", "n_bwd"}: device time of the attention calls since the last
        call_times() (barrier waits included), from event pairs on the launching stream."""
        torch.cuda.synchronize(self.device)
        out = {"fwd_ms": 0.0, "bwd_ms": 0.0, "n_fwd": 0, "n_bwd": 0}
        for kind, e0, e1 in self._call_events:
            out[kind + "_ms"] += e0.elapsed_time(e1)
            out["n_" + kind] += 1
        self._call_events = []
        return out


def a_status(ex: FusedAttentionExecutor) -> torch.Tensor:
    return ex.arena.status

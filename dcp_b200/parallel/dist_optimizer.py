"""ZeRO-1 style sharded AdamW over flat bf16 parameter / gradient buffers in peer memory.

The flat buffers are cut into *buckets* (the engine uses one per decoder layer plus one for the
embeddings, norms and LM head).  Every bucket is split evenly over the ranks that hold the same
parameters; a rank's fp32 state (master weights, m, v, main gradients) is the concatenation of its
slices of all buckets.

With several ranks the gradient reduction overlaps the backward pass:

``reduce_bucket(b)``  called by the model as soon as the backward of layer b has written its bf16
                      gradients: on a side stream, a bounded flag barrier (every rank finished that
                      bucket) and ONE kernel that sums this rank's slice from every rank's gradient
                      buffer with peer loads (reduce-scatter), applies the scale, writes the fp32
                      main-gradient slice and accumulates its squared norm in the same pass.
``step()``            reduces whatever has not been reduced, one scalar NCCL all-reduce of the
                      squared norm, then per bucket one kernel that applies clip + AdamW to the
                      slice and stores the new bf16 parameters into every rank's parameter buffer
                      (the all-gather is the epilogue of the update) -> barrier.

So gradients cross NVLink exactly once, clipping reads nothing twice, and only the parameter
all-gather is exposed at the end of a step.  With one rank there is nothing to overlap and the
reduce + AdamW + store is a single kernel with no fp32 gradient copy.

This is the role Megatron's distributed optimizer with overlapped DDP buckets plays for the
reference (benchmark/mlm/launch_template.txt:73-80, benchmark/mlm/pretrain_gpt.py:801-809).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

from ..ops import _lib
from ..ops.attention import _ptr_array
from ..runtime.symm import SymmetricArena


class FlatBuffers:
    """Symmetric flat parameter and gradient buffers shared by model and optimizer."""

    def __init__(self, n_flat: int, device: torch.device, group=None, timeout_s: float = 30.0):
        self.n_flat = n_flat
        regions = {"params": ((n_flat,), torch.bfloat16), "grads": ((n_flat,), torch.bfloat16)}
        self.arena = SymmetricArena(regions, device, group, timeout_s)
        self.params = self.arena.view("params")
        self.grads = self.arena.view("grads")
        self.world, self.rank = self.arena.world, self.arena.rank


@dataclass(frozen=True)
class BucketShard:
    """One rank's slice of one bucket."""
    bucket: int
    flat_off: int     # first element in the flat parameter / gradient buffers
    length: int       # elements (multiple of 8, may be 0)
    state_off: int    # first element in the rank's fp32 state arrays


def shard_layout(buckets: Sequence[Tuple[int, int]], world: int, rank: int) -> List[BucketShard]:
    """Slices of ``rank`` for buckets given as (offset, length) ranges of the flat buffer.

    Every bucket is cut into ``world`` slices of ``per = ceil(length / world)`` rounded up to 8
    elements; the last ranks get a shorter or empty slice when the bucket does not divide evenly.
    The formula is the single source of the sharding: optimizer state, reduce-scatter, parameter
    all-gather and checkpoint resume all use it.
    """
    out, state_off = [], 0
    for b, (off, length) in enumerate(buckets):
        assert off % 8 == 0 and length % 8 == 0, "bucket ranges must be multiples of 8 elements"
        per = -(-length // world)
        per = -(-per // 8) * 8
        lo = min(rank * per, length)
        n = max(0, min(per, length - lo))
        out.append(BucketShard(b, off + lo, n, state_off))
        state_off += n
    return out


def reshard_state(old_states, buckets: Sequence[Tuple[int, int]], new_world: int, new_rank: int) -> dict:
    """Optimizer state of rank ``new_rank`` of a group of ``new_world`` ranks, cut out of the state
    dictionaries written by a group of another size (resume on a different number of GPUs).

    ``old_states`` yields the ``state_dict()`` of every old rank, in any order and one at a time (a
    generator that loads one checkpoint file per item keeps a single file in host memory); each
    names its own ``rank`` and ``world``.  For every bucket the new rank's slice is filled from the
    overlapping parts of the old ranks' slices, both located with ``shard_layout``."""
    buckets = [tuple(b) for b in buckets]
    mine = shard_layout(buckets, new_world, new_rank)
    n = sum(s.length for s in mine)
    out = {k: torch.zeros(n, dtype=torch.float32) for k in ("master", "m", "v")}
    filled, step, seen = 0, None, set()
    for sd in old_states:
        assert [tuple(b) for b in sd["buckets"]] == buckets, "checkpoint was written with other gradient buckets"
        assert sd["rank"] not in seen, f"old rank {sd['rank']} given twice"
        seen.add(sd["rank"])
        step = int(sd["step"]) if step is None else step
        assert step == int(sd["step"]), "checkpoint files of different steps"
        for new, old in zip(mine, shard_layout(buckets, sd["world"], sd["rank"])):
            lo, hi = max(new.flat_off, old.flat_off), min(new.flat_off + new.length, old.flat_off + old.length)
            if hi <= lo:
                continue
            dst = slice(new.state_off + lo - new.flat_off, new.state_off + hi - new.flat_off)
            src = slice(old.state_off + lo - old.flat_off, old.state_off + hi - old.flat_off)
            for k in out:
                out[k][dst] = sd[k][src].to("cpu", torch.float32)
            filled += hi - lo
        old_world = sd["world"]
    assert seen == set(range(old_world)) and filled == n, "the old ranks' files do not cover this rank's slices"
    return {**out, "step": step, "buckets": buckets, "world": new_world, "rank": new_rank}


class ShardedAdamW:
    def __init__(self, bufs: FlatBuffers, lr: float = 3e-4, betas=(0.9, 0.95), eps: float = 1e-8,
                 weight_decay: float = 0.1, clip_grad: Optional[float] = 1.0, group=None, tp_group=None,
                 n_replicated: int = 0, buckets: Optional[Sequence[Tuple[int, int]]] = None,
                 extra_status: Optional[torch.Tensor] = None, overlap_ctas: int = 24):
        """``group`` = the ranks that hold the same parameters (they share the sharded state and
        their gradients are summed).  With tensor parallelism ``tp_group`` links the ranks that hold
        different shards of one model replica and ``n_replicated`` is the length of the leading
        part of the flat buffers that every one of them holds in full: the clipping norm counts
        that part once and the sharded part once per tensor-parallel rank (a bucket lies entirely
        in one of the two parts).  ``buckets``: (offset, length) ranges covering the flat buffer
        (default: one bucket).  ``extra_status``: status word of another arena (the attention
        executor's) that, when nonzero, also makes the update kernels leave the weights alone."""
        self.bufs, self.group = bufs, group
        self.tp_group, self.n_replicated = tp_group, n_replicated
        self.lr, self.betas, self.eps, self.wd, self.clip = lr, betas, eps, weight_decay, clip_grad
        world, rank = bufs.world, bufs.rank
        self.buckets = [(int(o), int(n)) for o, n in (buckets or [(0, bufs.n_flat)])]
        assert sum(n for _, n in self.buckets) == bufs.n_flat and self.buckets[0][0] == 0, \
            "buckets must tile the flat buffer"
        self.shards = shard_layout(self.buckets, world, rank)
        n_state = sum(s.length for s in self.shards)
        dev = bufs.params.device
        self.master = torch.empty(n_state, dtype=torch.float32, device=dev)
        for s in self.shards:
            self.master[s.state_off:s.state_off + s.length].copy_(bufs.params[s.flat_off:s.flat_off + s.length])
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        # fp32 main gradients exist only when there is a reduction to overlap
        self.overlap = world > 1
        self.main_grad = torch.zeros(n_state, dtype=torch.float32, device=dev) if self.overlap else None
        self.side = torch.cuda.Stream(device=dev) if self.overlap else None
        self.overlap_ctas = overlap_ctas
        self._reduced = [False] * len(self.buckets)
        self._side_used = False
        self.sq_norm = torch.zeros(1, dtype=torch.float32, device=dev)
        self.sq_parts = torch.zeros(2, dtype=torch.float32, device=dev)   # [replicated, sharded]
        self.clip_coef = torch.ones(1, dtype=torch.float32, device=dev)
        self.grad_scale = 1.0
        self.extra_status = extra_status
        self.step_count = 0
        self.kernel_launches = 0

    # ---- checkpoint state
    def state_dict(self) -> dict:
        return {"master": self.master, "m": self.m, "v": self.v, "step": self.step_count,
                "buckets": list(self.buckets), "world": self.bufs.world, "rank": self.bufs.rank}

    def load_state_dict(self, sd: dict) -> None:
        assert [tuple(b) for b in sd["buckets"]] == list(self.buckets) and sd["world"] == self.bufs.world and \
            sd["rank"] == self.bufs.rank, "checkpoint was written with another sharding"
        self.master.copy_(sd["master"]); self.m.copy_(sd["m"]); self.v.copy_(sd["v"])
        self.step_count = int(sd["step"])

    def _status_ptrs(self):
        a = _lib.ptr(self.bufs.arena.status)
        b = _lib.ptr(self.extra_status) if self.extra_status is not None else ctypes.c_void_p(0)
        return a, b

    def _sq_slot(self, shard: BucketShard) -> torch.Tensor:
        """Where a bucket's squared norm is accumulated: replicated / sharded part with tensor
        parallelism, the single total without."""
        if self.tp_group is None:
            return self.sq_norm
        return self.sq_parts[0:] if self.buckets[shard.bucket][0] < self.n_replicated else self.sq_parts[1:]

    # ---- overlapped reduce-scatter of one bucket
    def reduce_bucket(self, b: int) -> None:
        """The gradients of bucket ``b`` are final on this rank's current stream: reduce this rank's
        slice of it on the side stream (no-op with one rank, where step() fuses everything)."""
        if not self.overlap or self._reduced[b]:
            return
        lib = _lib.load()
        a = self.bufs.arena
        main = torch.cuda.current_stream(self.bufs.params.device)
        if not self._side_used:
            # first bucket of this step: clear the norm accumulators behind everything queued so far
            self.sq_norm.zero_(); self.sq_parts.zero_()
            self._side_used = True
        self.side.wait_stream(main)
        s = self.shards[b]
        st_a, st_b = self._status_ptrs()
        with torch.cuda.stream(self.side):
            a.barrier()                       # every rank's gradients of this bucket are written
            _lib.check(lib.dcpk_grad_reduce_scatter(
                _ptr_array(a.peer_ptrs("grads")), ctypes.c_int(self.bufs.world), ctypes.c_long(s.flat_off),
                ctypes.c_long(s.length), ctypes.c_float(self.grad_scale), _lib.ptr(self.main_grad[s.state_off:]),
                _lib.ptr(self._sq_slot(s)), ctypes.c_int(self.overlap_ctas), st_a, st_b, _lib.stream_handle()),
                "grad_reduce_scatter")
        self._reduced[b] = True
        self.kernel_launches += 2

    def step(self, grad_scale: float = 1.0) -> None:
        lib = _lib.load()
        b = self.bufs
        a = b.arena
        self.step_count += 1
        self.grad_scale = grad_scale
        st_a, st_b = self._status_ptrs()
        if self.overlap:
            self._step_overlapped(lib, st_a, st_b)
            return
        # ---- one rank: (norm pass when clipping) + one fused reduce/AdamW/store kernel per bucket
        grads, params = _ptr_array(a.peer_ptrs("grads")), _ptr_array(a.peer_ptrs("params"))
        clip_ptr = ctypes.c_void_p(0)
        if self.clip is not None:
            self.sq_norm.zero_(); self.sq_parts.zero_()
            for s in self.shards:
                _lib.check(lib.dcpk_grad_sqnorm(grads, ctypes.c_int(b.world), ctypes.c_long(s.flat_off),
                                                ctypes.c_long(s.length), ctypes.c_float(grad_scale),
                                                _lib.ptr(self._sq_slot(s)), _lib.stream_handle()), "grad_sqnorm")
            self._finish_norm()
            clip_ptr = _lib.ptr(self.clip_coef)
        for s in self.shards:
            _lib.check(lib.dcpk_fused_rs_adamw_ag(
                grads, params, ctypes.c_int(b.world), ctypes.c_long(s.flat_off), ctypes.c_long(s.length),
                ctypes.c_float(grad_scale), _lib.ptr(self.master[s.state_off:]), _lib.ptr(self.m[s.state_off:]),
                _lib.ptr(self.v[s.state_off:]), ctypes.c_float(self.lr), ctypes.c_float(self.betas[0]),
                ctypes.c_float(self.betas[1]), ctypes.c_float(self.eps), ctypes.c_float(self.wd),
                ctypes.c_int(self.step_count), clip_ptr, st_a, st_b, _lib.stream_handle()), "fused_rs_adamw_ag")
        self.kernel_launches += 2 * len(self.shards)

    def _finish_norm(self) -> None:
        """Total squared gradient norm over all ranks (one scalar all-reduce) -> clip coefficient."""
        import torch.distributed as dist
        if self.tp_group is not None:
            if self.bufs.world > 1:
                dist.all_reduce(self.sq_parts, group=self.group)
            dist.all_reduce(self.sq_parts[1:], group=self.tp_group)
            self.sq_norm.copy_(self.sq_parts.sum().reshape(1))
        elif self.bufs.world > 1:
            dist.all_reduce(self.sq_norm, group=self.group)
        torch.clamp(self.clip / (self.sq_norm.sqrt() + 1e-6), max=1.0, out=self.clip_coef)

    def _step_overlapped(self, lib, st_a, st_b) -> None:
        b, a = self.bufs, self.bufs.arena
        main = torch.cuda.current_stream(b.params.device)
        saved = self.overlap_ctas
        self.overlap_ctas = 0                 # nothing left to overlap with: fill the GPU
        for i in range(len(self.buckets)):
            self.reduce_bucket(i)
        self.overlap_ctas = saved
        main.wait_stream(self.side)
        clip_ptr = ctypes.c_void_p(0)
        if self.clip is not None:
            self._finish_norm()
            clip_ptr = _lib.ptr(self.clip_coef)
        params = _ptr_array(a.peer_ptrs("params"))
        for s in self.shards:
            _lib.check(lib.dcpk_adamw_all_gather(
                _lib.ptr(self.master[s.state_off:]), _lib.ptr(self.m[s.state_off:]), _lib.ptr(self.v[s.state_off:]),
                _lib.ptr(self.main_grad[s.state_off:]), params, ctypes.c_int(b.world), ctypes.c_long(s.flat_off),
                ctypes.c_long(s.length), ctypes.c_float(self.lr), ctypes.c_float(self.betas[0]),
                ctypes.c_float(self.betas[1]), ctypes.c_float(self.eps), ctypes.c_float(self.wd),
                ctypes.c_int(self.step_count), clip_ptr, st_a, st_b, _lib.stream_handle()), "adamw_all_gather")
        self.kernel_launches += len(self.shards)
        a.barrier()   # every rank's parameter buffer holds all updated slices
        self._reduced = [False] * len(self.buckets)
        self._side_used = False

    def rebuild_params(self) -> None:
        """bf16 parameters of every rank from the sharded fp32 master weights (after a resume): each
        rank stores its slices into every peer's parameter buffer, between two barriers."""
        lib = _lib.load()
        a = self.bufs.arena
        a.barrier()
        params = _ptr_array(a.peer_ptrs("params"))
        for s in self.shards:
            _lib.check(lib.dcpk_cast_all_gather(_lib.ptr(self.master[s.state_off:]), params, ctypes.c_int(self.bufs.world),
                                                ctypes.c_long(s.flat_off), ctypes.c_long(s.length),
                                                _lib.stream_handle()), "cast_all_gather")
        a.barrier()

    def check_status(self) -> None:
        self.bufs.arena.check_status()

    def grad_norm(self) -> float:
        return float(self.sq_norm.sqrt().item())

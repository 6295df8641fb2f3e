"""ZeRO-1 style sharded AdamW over flat bf16 parameter / gradient buffers in peer memory.

step():  barrier -> (when clipping) squared norm of the rank-summed gradient slice, read straight
from every rank's bf16 gradient buffer, + one tiny NCCL all-reduce of the scalar -> ONE kernel
that sums the slice over ranks with peer loads (reduce-scatter), applies scale and clip, updates
the fp32 AdamW state, and stores the new bf16 parameters into every rank's parameter buffer
(all-gather) -> barrier.  No fp32 gradient copy is ever materialised.  The rank-local fp32 state (master weights, m, v) covers 1/world of the
model.  This is the role Megatron's distributed optimizer + DDP reduce-scatter play for the
reference (benchmark/mlm/launch_template.txt:73-80).
"""
from __future__ import annotations

import ctypes
from typing import Optional

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


class ShardedAdamW:
    def __init__(self, bufs: FlatBuffers, lr: float = 3e-4, betas=(0.9, 0.95), eps: float = 1e-8,
                 weight_decay: float = 0.1, clip_grad: Optional[float] = 1.0, group=None, tp_group=None,
                 n_replicated: int = 0):
        """``group`` = the ranks that hold the same parameters (they share the sharded state and
        their gradients are summed).  With tensor parallelism ``tp_group`` links the ranks that hold
        different shards of one model replica and ``n_replicated`` is the length of the leading
        part of the flat buffers that every one of them holds in full: the clipping norm counts
        that part once and the sharded part once per tensor-parallel rank."""
        self.bufs, self.group = bufs, group
        self.tp_group, self.n_replicated = tp_group, n_replicated
        self.lr, self.betas, self.eps, self.wd, self.clip = lr, betas, eps, weight_decay, clip_grad
        world, rank = bufs.world, bufs.rank
        per = -(-bufs.n_flat // world)
        per = -(-per // 8) * 8
        self.shard_off = min(rank * per, bufs.n_flat)
        self.shard_len = max(0, min(per, bufs.n_flat - self.shard_off))
        dev = bufs.params.device
        self.master = bufs.params[self.shard_off:self.shard_off + self.shard_len].float()
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self.sq_norm = torch.zeros(1, dtype=torch.float32, device=dev)
        self.sq_parts = torch.zeros(2, dtype=torch.float32, device=dev)   # [replicated, sharded] with tensor parallelism
        self.clip_coef = torch.ones(1, dtype=torch.float32, device=dev)
        self.step_count = 0
        self.kernel_launches = 0

    def state_dict(self) -> dict:
        return {"master": self.master, "m": self.m, "v": self.v, "step": self.step_count,
                "shard": (self.shard_off, self.shard_len)}

    def load_state_dict(self, sd: dict) -> None:
        assert tuple(sd["shard"]) == (self.shard_off, self.shard_len), "checkpoint was written with another sharding"
        self.master.copy_(sd["master"]); self.m.copy_(sd["m"]); self.v.copy_(sd["v"])
        self.step_count = int(sd["step"])

    def step(self, grad_scale: float = 1.0) -> None:
        lib = _lib.load()
        b = self.bufs
        a = b.arena
        self.step_count += 1
        a.barrier()   # every rank finished writing its gradients
        grads, params = _ptr_array(a.peer_ptrs("grads")), _ptr_array(a.peer_ptrs("params"))
        off, n = ctypes.c_long(self.shard_off), ctypes.c_long(self.shard_len)
        clip_ptr = ctypes.c_void_p(0)
        if self.clip is not None and self.tp_group is not None:
            import torch.distributed as dist
            rep = max(0, min(self.n_replicated - self.shard_off, self.shard_len))
            self.sq_parts.zero_()
            for k, (o, ln) in enumerate(((self.shard_off, rep), (self.shard_off + rep, self.shard_len - rep))):
                if ln > 0:
                    _lib.check(lib.dcpk_grad_sqnorm(grads, ctypes.c_int(b.world), ctypes.c_long(o), ctypes.c_long(ln),
                                                    ctypes.c_float(grad_scale), _lib.ptr(self.sq_parts[k:]),
                                                    _lib.stream_handle()), "grad_sqnorm")
            if b.world > 1:
                dist.all_reduce(self.sq_parts, group=self.group)
            dist.all_reduce(self.sq_parts[1:], group=self.tp_group)
            self.sq_norm.copy_(self.sq_parts.sum().reshape(1))
        elif self.clip is not None:
            self.sq_norm.zero_()
            _lib.check(lib.dcpk_grad_sqnorm(grads, ctypes.c_int(b.world), off, n, ctypes.c_float(grad_scale),
                                            _lib.ptr(self.sq_norm), _lib.stream_handle()), "grad_sqnorm")
            if b.world > 1:
                import torch.distributed as dist
                dist.all_reduce(self.sq_norm, group=self.group)
        if self.clip is not None:
            torch.clamp(self.clip / (self.sq_norm.sqrt() + 1e-6), max=1.0, out=self.clip_coef)
            clip_ptr = _lib.ptr(self.clip_coef)
        _lib.check(lib.dcpk_fused_rs_adamw_ag(grads, params, ctypes.c_int(b.world), off, n, ctypes.c_float(grad_scale),
                                              _lib.ptr(self.master), _lib.ptr(self.m), _lib.ptr(self.v),
                                              ctypes.c_float(self.lr), ctypes.c_float(self.betas[0]),
                                              ctypes.c_float(self.betas[1]), ctypes.c_float(self.eps),
                                              ctypes.c_float(self.wd), ctypes.c_int(self.step_count), clip_ptr,
                                              _lib.stream_handle()), "fused_rs_adamw_ag")
        self.kernel_launches += 2
        a.barrier()   # every rank's parameter buffer holds all updated shards

    def grad_norm(self) -> float:
        return float(self.sq_norm.sqrt().item())

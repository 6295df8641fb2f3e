"""Plan interpreter skeleton: a handler per instruction class, buffers built from the plan's
``BufferInfo`` table, and an ``execute`` loop (dcp/core/executor.py:33-198).  Concrete executors
(pure-torch reference, NCCL baseline, fused sm_100a) register their handlers on top of this."""
from __future__ import annotations

import os

from typing import Callable, Dict, Optional, Type

import torch

from .instructions import (AttnBackwardInstr, AttnInstr, AttnReductionInstr, BarrierInstr, BlockInstrBase,
                           BufferInfo, BufferType, CommLaunchInstr, CommWaitInstr, DType, ExecutionPlan, MemcpyInstr,
                           SumInstr)

ALL_INSTRUCTIONS = (MemcpyInstr, CommLaunchInstr, BarrierInstr, CommWaitInstr, AttnInstr, AttnBackwardInstr,
                    AttnReductionInstr, SumInstr)


class DCPExecutor:
    def __init__(self, node_id: int = 0, local_device_id: int = 0, n_nodes: int = 1, n_devices_per_node: int = 1,
                 synchronous: bool = False, device: Optional[torch.device] = None, logger=None):
        self.node_id, self.local_device_id = node_id, local_device_id
        self.n_nodes, self.n_devices_per_node = n_nodes, n_devices_per_node
        self.synchronous = synchronous
        self.device = device or torch.device("cpu")
        if logger is None and os.environ.get("DCP_DEBUG_LOG_EXECUTOR", "0") not in ("0", "", "false", "False"):
            # one log per device of every instruction executed (dcp/core/executor.py:59-73)
            from ..utils.logger import create_logger
            logger = create_logger(f"executor.N{node_id}D{local_device_id}", prefix=f"N{node_id}D{local_device_id}",
                                   log_file=f"executor/N{node_id}D{local_device_id}.log")
        self.logger = logger
        self.buffers: Dict[str, torch.Tensor] = {}
        self.buffer_info: Dict[str, BufferInfo] = {}
        self._handlers: Dict[Type[BlockInstrBase], Callable] = {}
        self.plan: Optional[ExecutionPlan] = None

    @property
    def rank(self) -> int:
        return self.node_id * self.n_devices_per_node + self.local_device_id

    def register_handler(self, instr_type: Type[BlockInstrBase], handler: Callable) -> None:
        if not issubclass(instr_type, BlockInstrBase):
            raise TypeError(f"{instr_type} is not an instruction class")
        self._handlers[instr_type] = handler

    def check_all_handlers_registered(self) -> None:
        missing = [c.__name__ for c in ALL_INSTRUCTIONS if c not in self._handlers]
        if missing:
            raise RuntimeError(f"no handler registered for: {', '.join(missing)}")

    # ---- buffers
    def _alloc(self, name: str, info: BufferInfo) -> torch.Tensor:
        return torch.zeros(info.buffer_shape, dtype=DType.to_torch(info.dtype), device=self.device)

    def init_buffers(self, plan: ExecutionPlan, keep_local: bool = False) -> None:
        """Allocate every buffer of ``plan``; with ``keep_local`` existing Local* tensors of matching
        shape survive (the backward plan reuses the forward's LocalQ/LocalKV/LocalOut/LocalLSE)."""
        self.plan = plan
        for name, info in plan.buffer_info.items():
            old = self.buffers.get(name)
            if keep_local and BufferType.is_local(name) and old is not None and tuple(old.shape) == info.buffer_shape:
                self.buffer_info[name] = info
                continue
            self.buffers[name] = self._alloc(name, info)
            self.buffer_info[name] = info

    def init_forward_input(self, local_q: torch.Tensor, local_kv: torch.Tensor) -> None:
        self.buffers[BufferType.LOCAL_Q].copy_(local_q.reshape(self.buffers[BufferType.LOCAL_Q].shape))
        self.buffers[BufferType.LOCAL_KV].copy_(local_kv.reshape(self.buffers[BufferType.LOCAL_KV].shape))

    def init_backward_input(self, local_dout: torch.Tensor) -> None:
        self.buffers[BufferType.LOCAL_dOUT].copy_(local_dout.reshape(self.buffers[BufferType.LOCAL_dOUT].shape))

    def deallocate_buffers(self) -> None:
        """Drop the paged (temporary) buffers; the Local* ones stay."""
        for name in list(self.buffers):
            if not BufferType.is_local(name):
                del self.buffers[name]

    # ---- execution
    def execute(self, plan: Optional[ExecutionPlan] = None, is_forward: bool = True) -> None:
        plan = plan or self.plan
        self.check_all_handlers_registered()
        for idx, instr in enumerate(plan.instructions):
            if self.logger is not None:
                self.logger.debug("exec [%d] %s", idx, type(instr).__name__)
            self._handlers[type(instr)](instr)
            if self.synchronous:
                self._sync()

    def _sync(self) -> None:
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)

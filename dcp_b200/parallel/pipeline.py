"""Pipeline-parallel stage boundary: activations forward, gradients backward, over NCCL point-to-point.

The reference plumbs pipeline parallelism through its dataloader (every pipeline stage of a DCP rank
reads that rank's plans: ``pp_rank`` / ``pipeline_parallel_size``, dcp/data/dataloader.py:217-235,
1076-1079) and leaves the stage-to-stage transfers to Megatron-LM's p2p communication; its launch
files use one stage.  This module is that transfer layer for models cut into stages of consecutive
layers: ``PipelineComm`` posts the receive of the next micro-batch's input while the current one is
computed (transfers run on NCCL's own stream, so they overlap the stage's kernels), and
``run_stage_1f1b`` drives one stage through the usual warm-up / one-forward-one-backward / cool-down
order.  Attention plans do not depend on the stage: every stage of a context-parallel rank runs the
same executor program on the same tokens, so the stages' loaders read the same plans
(``SharedPlanService(readers=tp_size * pp_size)``).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist


class PipelineComm:
    """Point-to-point links of one pipeline stage.  ``group`` holds the stages of one pipeline in
    order (group rank = stage index)."""

    def __init__(self, group, shape_of: Callable[[int], Sequence[int]], dtype: torch.dtype, device: torch.device):
        """``shape_of(micro_batch)`` -> shape of the activation tensor that crosses a stage boundary
        for that micro-batch (token counts differ per micro-batch with variable-length packing)."""
        self.group = group
        self.stage, self.n_stages = dist.get_rank(group), dist.get_world_size(group)
        self.shape_of, self.dtype, self.device = shape_of, dtype, device
        self.prev = dist.get_global_rank(group, self.stage - 1) if self.stage > 0 else None
        self.next = dist.get_global_rank(group, self.stage + 1) if self.stage + 1 < self.n_stages else None
        self._pending: List = []

    @property
    def is_first(self) -> bool:
        return self.stage == 0

    @property
    def is_last(self) -> bool:
        return self.stage == self.n_stages - 1

    def _buf(self, mb: int) -> torch.Tensor:
        return torch.empty(tuple(self.shape_of(mb)), dtype=self.dtype, device=self.device)

    # receives are posted early (returning a handle); `wait` gives the tensor when it is needed
    def irecv_forward(self, mb: int):
        if self.is_first:
            return None
        buf = self._buf(mb)
        return (dist.irecv(buf, self.prev, group=self.group), buf)

    def irecv_backward(self, mb: int):
        if self.is_last:
            return None
        buf = self._buf(mb)
        return (dist.irecv(buf, self.next, group=self.group), buf)

    @staticmethod
    def wait(handle) -> Optional[torch.Tensor]:
        if handle is None:
            return None
        work, buf = handle
        work.wait()
        return buf

    def isend_forward(self, x: torch.Tensor) -> None:
        if not self.is_last:
            self._pending.append((dist.isend(x.contiguous(), self.next, group=self.group), x))

    def isend_backward(self, g: torch.Tensor) -> None:
        if not self.is_first:
            self._pending.append((dist.isend(g.contiguous(), self.prev, group=self.group), g))

    def flush(self) -> None:
        """Wait for every send posted so far (their tensors are kept alive until then)."""
        for work, _ in self._pending:
            work.wait()
        self._pending = []


def run_stage_1f1b(comm: PipelineComm, n_micro: int, forward_fn: Callable, loss_fn: Optional[Callable] = None):
    """One training step of one stage in the one-forward-one-backward order.

    ``forward_fn(micro_batch, x)`` -> the stage's output for that micro-batch (``x`` is None on the
    first stage, which reads its own inputs); ``loss_fn(micro_batch, y)`` -> scalar loss on the last
    stage.  Returns the list of losses (last stage) or an empty list.  Gradients of the stage's
    parameters accumulate in ``.grad`` as usual."""
    warm = min(comm.n_stages - 1 - comm.stage, n_micro)
    inputs, outputs, losses = {}, {}, []
    next_fwd = comm.irecv_forward(0) if n_micro else None

    def fwd(mb: int):
        nonlocal next_fwd
        x = comm.wait(next_fwd)
        next_fwd = comm.irecv_forward(mb + 1) if mb + 1 < n_micro else None     # posted before computing
        if x is not None:
            x.requires_grad_(True)
        y = forward_fn(mb, x)
        inputs[mb] = x
        if comm.is_last:
            loss = loss_fn(mb, y)
            losses.append(loss.detach())
            outputs[mb] = loss
        else:
            outputs[mb] = y
            comm.isend_forward(y.detach())

    def bwd(mb: int, grad_handle):
        y, x = outputs.pop(mb), inputs.pop(mb)
        if comm.is_last:
            y.backward()
        else:
            y.backward(comm.wait(grad_handle))
        if x is not None:
            comm.isend_backward(x.grad)

    for mb in range(warm):
        fwd(mb)
    done_bwd = 0
    for mb in range(warm, n_micro):                          # steady state: one forward, one backward
        grad_handle = comm.irecv_backward(done_bwd)
        fwd(mb)
        bwd(done_bwd, grad_handle)
        done_bwd += 1
    while done_bwd < n_micro:                                # cool-down
        bwd(done_bwd, comm.irecv_backward(done_bwd))
        done_bwd += 1
    comm.flush()
    return losses

"""Run an N-device plan inside one process (ranks = threads) and check it against dense attention.

This is how multi-device (and multi-node) plans are exercised without a cluster: every device
gets a ``ReferenceAttentionExecutor`` wired to an in-process mailbox, the global Q/KV are
scattered with the planner's local layout, and outputs are gathered back to global order
(the role of reconstruct_attention_{forward,backward}_output_for_test in
dcp/runtime/flash_attention/utils.py:33-277).
"""
from __future__ import annotations

import threading
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..core.blocks import Device, WorkloadSpec
from ..core.common import ExecutionContext
from ..core.instructions import BufferType, ExecutionPlan
from ..planner.masks import to_two_range
from .comm import MailboxComm, MailboxHub
from .executor_ref import ReferenceAttentionExecutor
from .layout import LocalLayout, gather_local, scatter_to_global, seq_token_offsets


def dense_reference(q: torch.Tensor, kv: torch.Tensor, raw_seqlens: Sequence[int], padded_seqlens: Sequence[int],
                    attn_mask: Optional[torch.Tensor], scale: float, dout: Optional[torch.Tensor] = None):
    """Per-sequence dense masked attention in fp64 -> (out [T,H,d], lse [H,T], dq, dkv), computed on
    the device the inputs live on."""
    T, H, d = q.shape
    hkv = kv.shape[2]
    g = H // hkv
    cu = seq_token_offsets(raw_seqlens)
    pcu = seq_token_offsets(padded_seqlens)
    qd = q.double().detach().requires_grad_(dout is not None)
    kvd = kv.double().detach().requires_grad_(dout is not None)
    outs, lses = [], []
    rng = to_two_range(attn_mask) if attn_mask is not None else None
    for s, n in enumerate(raw_seqlens):
        qs = qd[cu[s]:cu[s] + n]
        ks = kvd[cu[s]:cu[s] + n, 0].repeat_interleave(g, dim=1)
        vs = kvd[cu[s]:cu[s] + n, 1].repeat_interleave(g, dim=1)
        pos = torch.arange(n, device=q.device)[None, :]
        if rng is None:
            allow = pos <= torch.arange(n, device=q.device)[:, None]
        else:
            r = torch.from_numpy(rng[pcu[s]:pcu[s] + n]).to(q.device)
            allow = ((pos >= r[:, 0, 0:1]) & (pos < r[:, 0, 1:2])) | ((pos >= r[:, 1, 0:1]) & (pos < r[:, 1, 1:2]))
        sc = torch.einsum("qhd,khd->hqk", qs, ks) * scale
        sc = sc.masked_fill(~allow[None], float("-inf"))
        lse = torch.logsumexp(sc, dim=-1)
        safe = torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)
        p = torch.exp(sc - safe[..., None])
        p = torch.where(torch.isinf(lse)[..., None], torch.zeros_like(p), p)
        outs.append(torch.einsum("hqk,khd->qhd", p, vs))
        lses.append(lse)
    out = torch.cat(outs, dim=0)
    lse = torch.cat(lses, dim=1)
    if dout is None:
        return out.detach(), lse.detach(), None, None
    out.backward(dout.double())
    return out.detach(), lse.detach(), qd.grad, kvd.grad


def run_plans_in_process(context: ExecutionContext, fw_workload: WorkloadSpec, fw_plans: Dict[Device, ExecutionPlan],
                         q: torch.Tensor, kv: torch.Tensor, raw_seqlens: Sequence[int],
                         bw_workload: Optional[WorkloadSpec] = None,
                         bw_plans: Optional[Dict[Device, ExecutionPlan]] = None, dout: Optional[torch.Tensor] = None,
                         scale: Optional[float] = None, timeout_s: float = 60.0, hub: Optional[MailboxHub] = None,
                         fail_rank: Optional[int] = None):
    """Execute forward (and backward) plans of all devices; returns global (out, lse, dq, dkv).

    ``fail_rank`` makes that rank raise before executing (host-side fault injection); the others
    then hit the mailbox timeout and the first exception is re-raised here.
    """
    devices = context.devices()
    hub = hub or MailboxHub(len(devices), timeout_s)
    T, H, d = q.shape
    out_g = torch.zeros_like(q)
    lse_g = torch.full((H, T), float("-inf"), dtype=torch.float32)
    dq_g = torch.zeros_like(q) if dout is not None else None
    dkv_g = torch.zeros_like(kv) if dout is not None else None
    errors: List[BaseException] = []
    lock = threading.Lock()

    def worker(rank: int, dev: Device):
        try:
            if fail_rank == rank:
                raise RuntimeError(f"injected failure on rank {rank}")
            ex = ReferenceAttentionExecutor(MailboxComm(hub, rank), fw_workload, dev, context.n_devices_per_node,
                                            context.n_nodes, scale)
            lay = ex.layout
            lq = gather_local(q, lay, BufferType.LOCAL_Q, raw_seqlens, 1)
            lkv = gather_local(kv, lay, BufferType.LOCAL_KV, raw_seqlens, 2)
            lo, ll = ex.forward(fw_plans[dev], lq, lkv)
            with lock:
                scatter_to_global(lo, out_g, lay, BufferType.LOCAL_OUT, raw_seqlens, 1)
                scatter_to_global(ll, lse_g, lay, BufferType.LOCAL_LSE, raw_seqlens, 0, token_axis_local=1)
            if dout is not None:
                ldo = gather_local(dout, lay, BufferType.LOCAL_OUT, raw_seqlens, 1)
                ldq, ldkv = ex.backward(bw_plans[dev], bw_workload, ldo)
                blay = ex.layout
                with lock:
                    scatter_to_global(ldq, dq_g, blay, BufferType.LOCAL_dQ, raw_seqlens, 1)
                    scatter_to_global(ldkv, dkv_g, blay, BufferType.LOCAL_dKV, raw_seqlens, 2)
        except BaseException as e:  # noqa: BLE001 - surfaced to the caller below
            with lock:
                errors.append(e)

    threads = [threading.Thread(target=worker, args=(r, dv), daemon=True) for r, dv in enumerate(devices)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errors:
        primary = [e for e in errors if "injected" in str(e)] or errors
        raise primary[0]
    return out_g, lse_g, dq_g, dkv_g

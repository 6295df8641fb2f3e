"""Numerical self-check of the fused multi-GPU attention path against dense attention.

One small variable-length batch is planned for the ranks of ``group``, run forward and backward
through ``FusedAttentionExecutor`` (tcgen05 kernels, peer operand fetch, partial-result stores to
the owners, merge, gradient push), gathered to global order and compared on rank 0 with an fp64
dense masked attention of the same inputs.  The reference checks its executor the same way in its
multi-process tests (tests/runtime/test_flash_attention.py: run the plan on every rank, compare
with a single-device attention); here the check is also callable from a running job (``bench.py`` runs it
during warm-up on two or more GPUs) so that every multi-GPU measurement carries a max-error figure
of the cross-GPU kernels it timed.  Plain peer loads / stores / ``red`` only.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch
import torch.distributed as dist

from ..core.common import get_default_execution_context
from ..core.instructions import BufferType
from ..planner import masks
from ..planner.compiler import CompilerConfig, InstrCompiler
from ..planner.lowering import lower_all
from ..planner.workload import generate_workload, pad_seqlens
from .layout import LocalLayout, gather_local, scatter_to_global
from .simulate import dense_reference

HEAD_DIM = 128

DEFAULT_CASES = (
    # (raw sequence lengths, block size, query heads, kv heads, mask, head block size, stages)
    ((1000, 300, 2100, 640), 256, 8, 2, "causal", 8, None),
    ((3000, 1200, 4096, 700, 2100, 2048, 1500, 900), 512, 8, 2, "lambda", 4, None),
)


def run_fused_case(rank: int, world: int, group, raw: Sequence[int], block_size: int, heads_q: int, heads_kv: int,
                   mask_name: str, head_block_size: int, n_stages: Optional[int] = None, repeats: int = 2,
                   executor_hook=None) -> Dict[str, float]:
    """Runs one case; every rank returns the same error dictionary (relative max error of out, dq and
    dkv against the dense result's max magnitude, absolute max error of lse, plus plan facts).
    ``executor_hook(executor)`` is called after the runs, before the executor is released."""
    from .executor_fused import FusedAttentionExecutor

    dev = torch.device("cuda", torch.cuda.current_device())
    raw = list(raw)
    d = HEAD_DIM
    ctx = get_default_execution_context(world, 1)
    pad = pad_seqlens(raw, block_size)
    m = masks.get_mask_fn(mask_name)(raw, pad, torch.int32)
    wl = generate_workload((sum(pad), heads_q, d), (sum(pad), 2, heads_kv, d), raw, pad, block_size, head_block_size,
                           ctx.comp_cost_model, m, torch.bfloat16)
    fw_wl, _, _, _ = InstrCompiler(ctx, CompilerConfig(n_stages=n_stages)).compile(wl, generate_backward=False)
    progs = lower_all(ctx, fw_wl)
    prog = progs[(0, rank)]
    T = sum(raw)
    g = torch.Generator().manual_seed(1234)
    q = torch.randn(T, heads_q, d, generator=g).bfloat16()
    kv = torch.randn(T, 2, heads_kv, d, generator=g).bfloat16()
    dout = torch.randn(T, heads_q, d, generator=g).bfloat16()
    lay = LocalLayout(fw_wl, (0, rank))
    cap = max(max(p.q_rows for p in progs.values()), max(p.kv_rows for p in progs.values()),
              max(p.part_rows for p in progs.values()))
    ex = FusedAttentionExecutor(prog.heads_q, prog.heads_kv, cap, cap, cap, dev, group)
    if executor_hook is not None:
        ex.profile = True
    ex.prepare(prog)
    lq = gather_local(q, lay, BufferType.LOCAL_Q, raw, 1).to(dev)
    lkv = gather_local(kv, lay, BufferType.LOCAL_KV, raw, 2).to(dev)
    ldo = gather_local(dout, lay, BufferType.LOCAL_OUT, raw, 1).to(dev)
    for _ in range(repeats):   # more than once: flags, accumulators and staging must be reusable
        ex.q_local().copy_(lq)
        ex.kv_local().copy_(lkv)
        ex.inputs_written()
        out, lse = ex.forward()
        dq, dkv = ex.backward(ldo)
        torch.cuda.synchronize()
        ex.check_status()
    if executor_hook is not None:
        executor_hook(ex)
    out_g, lse_g = torch.zeros(T, heads_q, d), torch.zeros(heads_q, T)
    dq_g, dkv_g = torch.zeros(T, heads_q, d), torch.zeros(T, 2, heads_kv, d)
    scatter_to_global(out.float().cpu(), out_g, lay, BufferType.LOCAL_OUT, raw, 1)
    scatter_to_global(lse.float().cpu(), lse_g, lay, BufferType.LOCAL_LSE, raw, 0, token_axis_local=1)
    scatter_to_global(dq.float().cpu(), dq_g, lay, BufferType.LOCAL_Q, raw, 1)
    scatter_to_global(dkv.float().cpu(), dkv_g, lay, BufferType.LOCAL_KV, raw, 2)
    if world > 1:
        for t in (out_g, lse_g, dq_g, dkv_g):
            tg = t.to(dev)
            dist.all_reduce(tg, group=group)
            t.copy_(tg.cpu())
    errs = torch.zeros(4, dtype=torch.float64, device=dev)
    if rank == 0:
        # the dense fp64 reference runs on the GPU (one CPU thread per rank would take minutes)
        ro, rl, rdq, rdkv = (t.cpu() for t in dense_reference(q.to(dev), kv.to(dev), raw, pad, m, d ** -0.5, dout.to(dev)))
        rel = lambda a, b: ((a - b).abs().max() / (b.abs().max() + 1e-9)).item()
        fin = torch.isfinite(rl)
        errs = torch.tensor([rel(out_g, ro), (lse_g - rl)[fin].abs().max().item(), rel(dq_g, rdq), rel(dkv_g, rdkv)],
                            dtype=torch.float64, device=dev)
    if world > 1:
        dist.broadcast(errs, src=dist.get_global_rank(group, 0), group=group)
    e = errs.tolist()
    del ex
    torch.cuda.synchronize()
    return {"out": e[0], "lse": e[1], "dq": e[2], "dkv": e[3], "stages": prog.n_stages, "pull_bytes": float(prog.pull_bytes),
            "merge_ops": len(prog.merge_ops)}


def fused_self_check(rank: int, world: int, group, cases=DEFAULT_CASES, tol: float = 3e-2) -> Dict[str, object]:
    """Runs ``cases`` and returns {"max_err", "tol", "passed", "cases", "errs": [per case]}; the same on every rank."""
    per_case = []
    for raw, bs, hq, hkv, mask_name, hbs, stages in cases:
        r = run_fused_case(rank, world, group, raw, bs, hq, hkv, mask_name, hbs, stages)
        per_case.append({"mask": mask_name, "tokens": int(sum(raw)),
                         **{k: round(r[k], 5) for k in ("out", "lse", "dq", "dkv")}})
    worst = max(max(c[k] for k in ("out", "lse", "dq", "dkv")) for c in per_case)
    return {"max_err": worst, "tol": tol, "passed": bool(worst < tol), "cases": len(per_case), "errs": per_case,
            "against": "fp64 dense masked attention of the same inputs"}

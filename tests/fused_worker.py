"""Multi-GPU worker: fused executor vs dense attention (launched with torch.distributed.run).

Every rank builds the same deterministic plan, runs forward + backward through the fused
sm_100a executor on its own GPU, and rank 0 compares the gathered results with the fp64 dense
reference.  Also used single-process (WORLD_SIZE unset) for the one-GPU case.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dcp_b200.core.common import get_default_execution_context  # noqa: E402
from dcp_b200.core.instructions import BufferType  # noqa: E402
from dcp_b200.planner import masks  # noqa: E402
from dcp_b200.planner.compiler import CompilerConfig, InstrCompiler  # noqa: E402
from dcp_b200.planner.lowering import lower_all  # noqa: E402
from dcp_b200.planner.workload import generate_workload, pad_seqlens  # noqa: E402
from dcp_b200.runtime.executor_fused import FusedAttentionExecutor  # noqa: E402
from dcp_b200.runtime.layout import LocalLayout, gather_local, scatter_to_global  # noqa: E402
from dcp_b200.runtime.simulate import dense_reference  # noqa: E402


def run_case(rank, world, group, raw, bs, H, Hkv, mask_name, hbs, n_stages=None, tol=3e-2):
    dev = torch.device("cuda", torch.cuda.current_device())
    d = 128
    ctx = get_default_execution_context(world, 1)
    pad = pad_seqlens(raw, bs)
    m = masks.get_mask_fn(mask_name)(raw, pad, torch.int32)
    wl = generate_workload((sum(pad), H, d), (sum(pad), 2, Hkv, d), raw, pad, bs, hbs, ctx.comp_cost_model, m,
                           torch.bfloat16)
    fw_wl, _, _, _ = InstrCompiler(ctx, CompilerConfig(n_stages=n_stages)).compile(wl, generate_backward=False)
    progs = lower_all(ctx, fw_wl)
    prog = progs[(0, rank)]
    T = sum(raw)
    g = torch.Generator().manual_seed(1234)
    q = torch.randn(T, H, d, generator=g).bfloat16()
    kv = torch.randn(T, 2, Hkv, d, generator=g).bfloat16()
    dout = torch.randn(T, H, d, generator=g).bfloat16()
    lay = LocalLayout(fw_wl, (0, rank))
    hq, hkv = prog.heads_q, prog.heads_kv
    cap = max(max(p.q_rows for p in progs.values()), max(p.kv_rows for p in progs.values()),
              max(p.part_rows for p in progs.values()))
    ex = FusedAttentionExecutor(hq, hkv, cap, cap, cap, dev, group)
    ex.profile = True          # phase timing on: its marks must line up into a trace (checked below)
    ex.prepare(prog)
    lq = gather_local(q, lay, BufferType.LOCAL_Q, raw, 1).to(dev)
    lkv = gather_local(kv, lay, BufferType.LOCAL_KV, raw, 2).to(dev)
    ldo = gather_local(dout, lay, BufferType.LOCAL_OUT, raw, 1).to(dev)
    for it in range(2):   # twice: flags, accumulators and staging must be reusable
        ex.q_local().copy_(lq)
        ex.kv_local().copy_(lkv)
        ex.inputs_written()
        out, lse = ex.forward()
        dq, dkv = ex.backward(ldo)
        torch.cuda.synchronize()
        ex.check_status()
    trace = ex.profile_chrome_trace()
    names = {e["name"] for e in trace}
    assert {"fwd:kernels (with operand fetch)", "bwd:kernels (with operand fetch)"} <= names and all(e["dur"] >= 0 for e in trace), names
    assert ex.profile_summary() == {}      # consumed
    out_g, lse_g = torch.zeros(T, H, d), torch.zeros(H, T)
    dq_g, dkv_g = torch.zeros(T, H, d), torch.zeros(T, 2, Hkv, d)
    scatter_to_global(out.float().cpu(), out_g, lay, BufferType.LOCAL_OUT, raw, 1)
    scatter_to_global(lse.float().cpu(), lse_g, lay, BufferType.LOCAL_LSE, raw, 0, token_axis_local=1)
    scatter_to_global(dq.float().cpu(), dq_g, lay, BufferType.LOCAL_Q, raw, 1)
    scatter_to_global(dkv.float().cpu(), dkv_g, lay, BufferType.LOCAL_KV, raw, 2)
    if world > 1:
        for t in (out_g, lse_g, dq_g, dkv_g):
            tg = t.to(dev)
            dist.all_reduce(tg, group=group)
            t.copy_(tg.cpu())
    if rank == 0:
        # the dense fp64 reference runs on the GPU (one CPU thread per rank would take minutes)
        ro, rl, rdq, rdkv = (t.cpu() for t in dense_reference(q.to(dev), kv.to(dev), raw, pad, m, d ** -0.5, dout.to(dev)))
        rel = lambda a, b: ((a - b).abs().max() / (b.abs().max() + 1e-9)).item()
        fin = torch.isfinite(rl)
        errs = {"out": rel(out_g, ro), "lse": (lse_g - rl)[fin].abs().max().item(), "dq": rel(dq_g, rdq),
                "dkv": rel(dkv_g, rdkv)}
        print(f"case world={world} mask={mask_name} hbs={hbs} stages={prog.n_stages} pulls={prog.pull_bytes:.0f}B "
              f"merge_ops={len(prog.merge_ops)} errs={ {k: round(v, 5) for k, v in errs.items()} }", flush=True)
        assert max(errs.values()) < tol, errs
    del ex
    torch.cuda.synchronize()


def main():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    group = None
    if world > 1:
        dist.init_process_group("nccl")
        group = dist.group.WORLD
    cases = [([1000, 300, 2100, 640], 256, 8, 2, "causal", 8, None),
             ([1000, 300, 2100, 640], 256, 8, 2, "lambda", 4, 2),
             ([3000, 700], 512, 4, 4, "shared_question", 4, 3),
             ([2048, 1024, 512], 512, 8, 2, "causal_blockwise", 8, None),
             # one stage only: every remote operand is fetched by a launch of its own before the kernels
             ([1500, 900, 2600], 256, 8, 2, "causal", 8, 1)]
    if world >= 4:
        # a longer mixed batch so that every rank of a larger group holds work of several stages
        cases.append(([3000, 1200, 4096, 700, 2100, 2048, 1500, 900], 512, 8, 2, "causal", 4, None))
        cases.append(([6144, 2000, 3072, 1000], 512, 8, 4, "lambda", 8, 3))
    for c in cases:
        run_case(rank, world, group, *c)
    if rank == 0:
        print("FUSED_OK", flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

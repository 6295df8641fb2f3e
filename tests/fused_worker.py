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

from dcp_b200.runtime.selfcheck import run_fused_case  # noqa: E402


def _check_trace(ex):
    # phase timing on: its marks must line up into a trace
    trace = ex.profile_chrome_trace()
    names = {e["name"] for e in trace}
    assert {"fwd:kernels (with operand fetch)", "bwd:kernels (with operand fetch)"} <= names and all(e["dur"] >= 0 for e in trace), names
    assert ex.profile_summary() == {}      # consumed


def run_case(rank, world, group, raw, bs, H, Hkv, mask_name, hbs, n_stages=None, tol=3e-2):
    r = run_fused_case(rank, world, group, raw, bs, H, Hkv, mask_name, hbs, n_stages, executor_hook=_check_trace)
    errs = {k: r[k] for k in ("out", "lse", "dq", "dkv")}
    if rank == 0:
        print(f"case world={world} mask={mask_name} hbs={hbs} stages={r['stages']} pulls={r['pull_bytes']:.0f}B "
              f"merge_ops={r['merge_ops']} errs={ {k: round(v, 5) for k, v in errs.items()} }", flush=True)
    assert max(errs.values()) < tol, errs


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

"""Attention-only microbenchmark (forward + backward) over packed variable-length batches.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \\
        -m dcp_b200.bench.attention --framework dcp --mask causal --tokens 131072 --batches 5

Frameworks (``--framework`` takes one or several, run one after the other on the same batches):
``dcp`` (fused sm_100a executor), ``ulysses`` (NCCL all-to-all + library attention), ``ring`` /
``zigzag`` / ``double-ring`` (NCCL point-to-point rings + library attention per chunk), ``a2a+p2p``
(head all-to-all inside small groups x ring between them), ``nccl-plan`` (the same DCP plans
interpreted with NCCL point-to-point and torch ops).  Timing
follows the reference's harness (benchmark/microbenchmark/utils.py:144-225,
benchmark_attention.py:1457-1472): warm-up iterations, CUDA events, per-rank times gathered and the
MAX over ranks reported, summed over batches; the line ``<Name>: total time X ms`` keeps the
orchestrator-parsable format.  A JSON line adds achieved FLOP/s and the roofline fraction
(slower of tensor time at the measured peak and NVLink bytes at the measured link bandwidth).
"""
from __future__ import annotations

import argparse
import json
import os
import time

import torch
import torch.distributed as dist

from ..core.common import get_default_execution_context
from ..core.instructions import BufferType
from ..data import synth
from ..data.plan_service import PlanSpec, plan_iteration
from ..planner import masks as mask_lib
from ..runtime.executor_fused import FusedAttentionExecutor
from .kernel_bench import measured_peaks

NVLINK_GBS = 770.0  # measured peer-copy bandwidth per direction per GPU


def bench_f(fn, warmup: int, iters: int, group):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if group is not None:
        dist.barrier(group=group)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / iters], dtype=torch.float64, device="cuda")
    if group is not None:
        all_ms = [torch.zeros_like(ms) for _ in range(dist.get_world_size(group))]
        dist.all_gather(all_ms, ms, group=group)
        vals = [float(x) for x in all_ms]
    else:
        vals = [float(ms)]
    return sum(vals) / len(vals), max(vals)


def default_args(**over) -> argparse.Namespace:
    """The microbenchmark's settings as a namespace (BASELINE configuration: 32 / 8 heads, d = 128, bf16,
    131072-token packed batches, lognormal lengths, causal mask, block size 2048)."""
    d = dict(framework="dcp", mask="causal", tokens=131072, batches=3, n_heads=32, n_kv_heads=8, block_size=2048,
             length_dist="lognormal8k", warmup=5, iters=10, stages=None, mode="fwdbwd", seed=0)
    d.update(over)
    return argparse.Namespace(**d)


def bench_plan_spec(args, world: int) -> PlanSpec:
    """The planner settings of a benchmark run (optional arguments default to the planner's own)."""
    dists = {"lognormal8k": synth.LOGNORMAL_8K, "lognormal16k": synth.LOGNORMAL_16K, "mixture": synth.MIXTURE}
    return PlanSpec(world, world, args.tokens, args.n_heads, args.n_kv_heads, 128, args.block_size,
                    getattr(args, "head_block_size", 0) or 0, args.mask, dists[args.length_dist], seed=args.seed,
                    n_stages=args.stages, build_instruction_plans=args.framework == "nccl-plan",
                    mem_imbalance_epsilon=getattr(args, "mem_epsilon", None),
                    comp_imbalance_epsilon=getattr(args, "comp_epsilon", None),
                    use_block_size_heuristic=bool(getattr(args, "use_block_size_heuristic", False)))


def explicit_batches(args):
    """Sequence lengths given on the command line: ``--seqlens 4096,512,...`` (one batch) or
    ``--seqlens-config file.json`` ({"batches": [[...], ...]} as written by ``bench.preprocessing``, or a
    plain list of lists / one list); None when the lengths are to be drawn from ``--length-dist``."""
    if getattr(args, "seqlens", None):
        return [[int(x) for x in str(args.seqlens).split(",") if x]]
    path = getattr(args, "seqlens_config", None)
    if not path:
        return None
    data = json.load(open(path))
    if isinstance(data, dict):
        data = data["batches"]
    return [list(map(int, b)) for b in data] if data and isinstance(data[0], (list, tuple)) else [list(map(int, data))]


def plan_for_batch(args, spec: PlanSpec, b: int, rank: int):
    """Rank ``rank``'s plan of benchmark batch ``b``: drawn from the length distribution, or the b-th
    explicit batch (cycled) with seeded token ids."""
    batches = explicit_batches(args)
    if batches is None:
        return plan_iteration(spec, b, rank)
    from ..data.plan_service import plan_batch
    seqlens = batches[b % len(batches)]
    return plan_batch(spec, b, rank, seqlens, synth.make_token_batch(seqlens, spec.vocab, spec.seed * 1000003 + b))


def run_batches(args, group, dev, rank: int, world: int, verbose: bool = True) -> dict:
    """Time ``args.batches`` packed batches with ``args.framework`` on an initialised process group
    (or one GPU when ``group`` is None) and return the summary (max over ranks per batch)."""
    spec = bench_plan_spec(args, world)
    hbm, tf_peak, src = measured_peaks()
    total_max_ms, total_flops, total_roof = 0.0, 0.0, 0.0
    ex = None
    for b in range(args.batches):
        plan = plan_for_batch(args, spec, b, rank)
        p = plan.program
        H, Hkv = args.n_heads, args.n_kv_heads
        g = torch.Generator(device=dev).manual_seed(1000 + b * 17 + rank)
        if args.framework == "dcp":
            cap = int(args.tokens // world * 1.5) + 4 * args.block_size
            hl, hkvl = p.heads_q, p.heads_kv       # heads per block (all heads unless --head-block-size is given)
            if ex is None:
                ex = FusedAttentionExecutor(hl, hkvl, cap * (H // hl), cap * (H // hl), cap * (H // hl), dev, group)
            ex.prepare(p)
            lq = torch.randn(p.q_local_rows, hl, 128, device=dev, generator=g).bfloat16()
            lkv = torch.randn(p.kv_local_rows, 2, hkvl, 128, device=dev, generator=g).bfloat16()
            ldo = torch.randn(p.q_local_rows, hl, 128, device=dev, generator=g).bfloat16()

            def step():
                ex.q_local().copy_(lq)
                ex.kv_local().copy_(lkv)
                ex.inputs_written()
                ex.forward()
                if args.mode == "fwdbwd":
                    ex.backward(ldo)
        elif args.framework in ("ulysses", "ring", "zigzag", "double-ring", "a2a+p2p"):
            from .baselines import make_baseline
            assert args.mask == "causal", "the library attention kernel only knows causal masks"
            attn, n = make_baseline(args.framework, group, plan.seqlens, H, Hkv, rank, world,
                                    window=getattr(args, "lt_window_size", None), a2a=getattr(args, "a2a_degree", None))
            q = torch.randn(n, H, 128, device=dev, generator=g).bfloat16().requires_grad_(True)
            k = torch.randn(n, Hkv, 128, device=dev, generator=g).bfloat16().requires_grad_(True)
            v = torch.randn(n, Hkv, 128, device=dev, generator=g).bfloat16().requires_grad_(True)
            do = torch.randn(n, H, 128, device=dev, generator=g).bfloat16()

            def step():
                out = attn(q, k, v)
                if args.mode == "fwdbwd":
                    out.backward(do)
                    q.grad = k.grad = v.grad = None
        else:
            from ..runtime.interface import get_executor
            ctx = get_default_execution_context(world, 1)
            pex = get_executor(H, 128, ctx, plan.fw_plan, plan.fw_workload, plan.bw_plan, plan.bw_workload,
                               process_group=group, device=dev)
            lq = torch.randn(p.q_local_rows, H, 128, device=dev, generator=g).bfloat16()
            lkv = torch.randn(p.kv_local_rows, 2, Hkv, 128, device=dev, generator=g).bfloat16()
            ldo = torch.randn(p.q_local_rows, H, 128, device=dev, generator=g).bfloat16()

            def step():
                out, lse = pex.forward(lq, lkv)
                if args.mode == "fwdbwd":
                    pex.backward(lq, lkv, out.clone(), ldo, lse.clone())
                    pex.is_forward = False
                    pex.prepare(True)
        mean_ms, max_ms = bench_f(step, args.warmup, args.iters, group)
        flops = torch.tensor([p.fwd_flops + (p.bwd_flops if args.mode == "fwdbwd" else 0.0), p.pull_bytes],
                             dtype=torch.float64, device=dev)
        mx = flops.clone()
        if group is not None:
            dist.all_reduce(flops, group=group)
            dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=group)
        total_max_ms += max_ms
        total_flops += float(flops[0])
        t_compute = float(mx[0]) / (tf_peak * 1e12) * 1e3
        t_link = float(mx[1]) * (3.0 if args.mode == "fwdbwd" else 1.0) / (NVLINK_GBS * 1e9) * 1e3
        roof = max(t_compute, t_link)
        total_roof += roof
        if rank == 0 and verbose:
            print(json.dumps({"batch": b, "framework": args.framework, "mask": args.mask, "n_gpus": world,
                              "n_seqs": len(plan.seqlens), "max_seqlen": max(plan.seqlens), "ms_max_over_ranks": round(max_ms, 3),
                              "ms_mean": round(mean_ms, 3), "tflops_per_gpu": round(float(flops[0]) / world / max_ms / 1e9, 1),
                              f"roofline_ms_({src}_peaks)": round(roof, 3), "fraction_of_roofline": round(roof / max_ms, 3),
                              "pull_MB_max_rank": round(float(mx[1]) / 1e6, 1)}), flush=True)
    if ex is not None:
        torch.cuda.synchronize()
        ex.check_status()
    return {"summary": True, "framework": args.framework, "mask": args.mask, "n_gpus": world,
            "tokens_per_batch": args.tokens, "batches": args.batches, "mode": args.mode,
            "avg_ms_per_batch": round(total_max_ms / args.batches, 3), "total_ms": round(total_max_ms, 3),
            "aggregate_tflops": round(total_flops / total_max_ms / 1e9, 1),
            f"fraction_of_roofline_({src}_peaks)": round(total_roof / total_max_ms, 3)}


FRAMEWORK_NAMES = {"dcp": "DCP", "ulysses": "Ulysses", "ring": "Ring", "zigzag": "ZigzagRing", "nccl-plan": "NCCLPlan",
                   "double-ring": "DoubleRing", "a2a+p2p": "HierarchicalA2AP2P"}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--framework", default=["dcp"], nargs="+", choices=sorted(FRAMEWORK_NAMES),
                    help="one or more frameworks, run one after the other on the same batches")
    ap.add_argument("--mask", default="causal")
    ap.add_argument("--tokens", type=int, default=131072)
    ap.add_argument("--batches", type=int, default=3)
    ap.add_argument("--n-heads", type=int, default=32)
    ap.add_argument("--n-kv-heads", type=int, default=8)
    ap.add_argument("--block-size", type=int, default=2048)
    ap.add_argument("--length-dist", default="lognormal8k", choices=["lognormal8k", "lognormal16k", "mixture"])
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--stages", type=int, default=None)
    ap.add_argument("--mode", default="fwdbwd", choices=["fwd", "fwdbwd"])
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--seqlens", default=None, help="comma separated sequence lengths of one batch (overrides --length-dist)")
    ap.add_argument("--seqlens-config", default=None, help="json with explicit batches (see bench.preprocessing)")
    ap.add_argument("--head-block-size", type=int, default=0, help="heads per block (0 = all heads in one block)")
    ap.add_argument("-me", "--mem-epsilon", type=float, default=None, help="token (memory) balance tolerance of the placement")
    ap.add_argument("-ce", "--comp-epsilon", type=float, default=None, help="attention-work balance tolerance of the placement")
    ap.add_argument("--use-block-size-heuristic", action="store_true")
    ap.add_argument("--lt-window-size", type=int, default=None, help="double ring: ranks per inner ring")
    ap.add_argument("--a2a-degree", type=int, default=None, help="a2a+p2p: ranks per head all-to-all group")
    ap.add_argument("--check-correctness", action="store_true",
                    help="dcp on 2 or more GPUs: first compare the fused path with dense fp64 attention on small batches")
    args = ap.parse_args(argv)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    if args.check_correctness and world > 1 and "dcp" in args.framework:
        from ..runtime.selfcheck import fused_self_check
        check = fused_self_check(rank, world, group)
        if rank == 0:
            print(json.dumps({"check_correctness": check}), flush=True)
    for framework in args.framework:
        one = argparse.Namespace(**{**vars(args), "framework": framework})
        try:
            summary = run_batches(one, group, dev, rank, world)
        except (AssertionError, RuntimeError, ValueError) as e:     # e.g. a baseline that cannot split this shape
            if len(args.framework) == 1:
                raise
            if rank == 0:
                print(f"{FRAMEWORK_NAMES[framework]}: failed ({type(e).__name__}: {str(e)[:200]})", flush=True)
            continue
        if rank == 0:
            print(f"{FRAMEWORK_NAMES[framework]}: total time {summary['total_ms']:.3f} ms")
            print(json.dumps(summary), flush=True)
        torch.cuda.empty_cache()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

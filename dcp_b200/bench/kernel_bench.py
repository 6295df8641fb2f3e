"""Single-GPU micro-benchmarks of the hand-written kernels (CUDA-event timing, warm-up, inputs
larger than L2 or an L2 flush between iterations), with achieved fractions of the measured peaks.

    python -m dcp_b200.bench.kernel_bench attn_fwd --tokens 8192 --kv 8192 --hq 32 --hkv 8 --mask causal
    python -m dcp_b200.bench.kernel_bench attn_bwd ...
    python -m dcp_b200.bench.kernel_bench ops
    python -m torch.distributed.run --nproc-per-node 2 ... -m dcp_b200.bench.kernel_bench nvlink

Counterpart of the reference's benchmark/ops/{benchmark_fused_memcpy,benchmark_fused_update,
benchmark_sdpa}.py.
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np
import torch

from ..ops import attention as A
from ..ops import block_ops, model_ops


def measured_peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def time_fn(fn, iters=10, warmup=3, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def _ranges(mask, nq, nkv):
    r = np.zeros((nq, 4), np.int32)
    i = np.arange(nq)
    if mask == "full":
        r[:, 1] = nkv
    elif mask == "causal":
        r[:, 1] = i + 1 + (nkv - nq)
    elif mask == "lambda":
        r[:, 1] = np.minimum(64, i + 1)
        r[:, 2] = np.maximum(64, i + (nkv - nq) - 4095)
        r[:, 3] = np.maximum(r[:, 2], i + 1 + (nkv - nq))
    return r


def bench_attention(kind, args):
    dev = torch.device("cuda")
    hbm, tf, src = measured_peaks()
    nq, nkv, hq, hkv = args.tokens, args.kv, args.hq, args.hkv
    torch.manual_seed(0)
    q = torch.randn(nq + 128, hq, 128, device=dev).bfloat16()
    kv = torch.randn(nkv + 128, 2, hkv, 128, device=dev).bfloat16()
    out = torch.zeros_like(q)
    lse = torch.zeros(hq, nq + 128, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    bs = args.block
    rng = _ranges(args.mask, nq, nkv)
    rows = []
    for b0 in range(0, nq, bs):
        n = min(bs, nq - b0)
        rows.append(A.AttnRow(b0, n, list(range(hq)), [(k0, min(bs, nkv - k0)) for k0 in range(0, nkv, bs)],
                              rng[b0:b0 + n], 0, b0, 0, b0, [(0, k0) for k0 in range(0, nkv, bs)]))
    scale = 128 ** -0.5
    ft = A.build_fwd_tables(rows, bs, dev, tile_m=256 if args.variant == 2 else 128)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    fwd = lambda: A.attn_fwd(q, kv, ft, [out], [lse], scale, status, args.variant)
    if kind == "attn_fwd":
        ms = time_fn(fwd, args.iters, 3, flush)
        flops = ft.flops
        if args.timeline:
            from ..ops import _lib
            tl = torch.zeros(16, dtype=torch.int64, device=dev)
            _lib.load().dcpk_attn_fwd_set_timeline(_lib.ptr(tl))
            fwd()
            torch.cuda.synchronize()
            _lib.load().dcpk_attn_fwd_set_timeline(None)
            names = ["loop top", "wait S", "ld S", "max/exp/pack", "store P + wait O(j-1)", "rescale O + arrive", "probe: empty", "probe: try_wait on a completed barrier",
                     "umma: after QK issue", "umma: wait P", "umma: wait V", "umma: issue PV", "umma: wait K"]
            print("timeline of CTA 0 (total cycles):", {n: v for n, v in zip(names, tl.tolist()) if n != "-"})
    else:
        fwd()
        dout = torch.randn_like(q)
        delta = torch.zeros_like(lse)
        A.attn_delta(out, dout, delta, 0, nq)
        bt = A.build_bwd_tables(rows, bs, hq, hkv, dev)
        if args.skip_dq:
            bt.items[:, 4] = -1
        dq = torch.zeros(nq + 128, hq, 128, device=dev)
        dkv = torch.zeros(nkv + 128, 2, hkv, 128, device=dev)
        ms = time_fn(lambda: A.attn_bwd(q, dout, kv, lse, delta, bt, [dq], [dkv], scale, status), args.iters, 3, flush)
        flops = bt.flops
        if args.timeline:
            from ..ops import _lib
            tl = torch.zeros(16, dtype=torch.int64, device=dev)
            _lib.load().dcpk_attn_bwd_set_timeline(_lib.ptr(tl))
            A.attn_bwd(q, dout, kv, lse, delta, bt, [dq], [dkv], scale, status)
            torch.cuda.synchronize()
            _lib.load().dcpk_attn_bwd_set_timeline(None)
            n_vis = int(bt.ctas[0, 3].item()) * (hq // hkv)
            names = ["wait item + stats", "wait S/dP", "ld S,dP", "wait dQ(t-1)", "drain dQ(t-1) first half", "math", "store P,dS + arrive", "drain dQ(t-1) second half",
                     "umma: issue S/dP", "umma: wait P ready", "umma: issue acc", "umma: wait Q,dO + S free"]
            print("timeline of CTA (0,0), cycles per visit (", n_vis, "visits ):",
                  {n: round(v / max(n_vis, 1)) for n, v in zip(names, tl.tolist()) if n != "-"})
    torch.cuda.synchronize()
    assert status.item() == 0
    tfs = flops / ms / 1e9
    print(json.dumps({"kernel": kind, "tokens": nq, "kv": nkv, "hq": hq, "hkv": hkv, "mask": args.mask, "ms": round(ms, 4),
                      "tflops": round(tfs, 1), f"frac_of_{src}_bf16_peak": round(tfs / tf, 3)}))


def bench_ops(args):
    """HBM-bound kernels: milliseconds, GB/s of algorithmic bytes and the fraction of the measured copy
    bandwidth.  ``--only NAME`` builds and runs just that op (a small working set for a profiler)."""
    dev = torch.device("cuda")
    hbm, tf, src = measured_peaks()
    T, H, F, V = args.tokens, 4096, 14336, 128256
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    from ..ops import _lib
    import ctypes
    lib = _lib.load()
    want = lambda name: args.only is None or args.only == name

    def report(name, ms, nbytes):
        gbs = nbytes / ms / 1e6
        print(json.dumps({"op": name, "ms": round(ms, 4), "GB/s": round(gbs, 1), f"frac_of_{src}_hbm": round(gbs / hbm, 3)}))

    if want("rmsnorm_fwd") or want("rmsnorm_bwd"):
        x = torch.randn(T, H, device=dev).bfloat16()
        w = torch.ones(H, device=dev).bfloat16()
        y, rstd = torch.empty_like(x), torch.empty(T, device=dev)
        fwd = lambda: lib.dcpk_rmsnorm_fwd(_lib.ptr(x), _lib.ptr(w), _lib.ptr(y), _lib.ptr(rstd), ctypes.c_int(T),
                                           ctypes.c_int(H), ctypes.c_float(1e-5), _lib.stream_handle())
        fwd()
        if want("rmsnorm_fwd"):
            report("rmsnorm_fwd", time_fn(fwd, args.iters, 3, flush), 2 * x.numel() * 2)
        if want("rmsnorm_bwd"):
            dx, dw = torch.empty_like(x), torch.zeros(H, device=dev)
            report("rmsnorm_bwd", time_fn(lambda: lib.dcpk_rmsnorm_bwd(_lib.ptr(x), _lib.ptr(w), _lib.ptr(y), _lib.ptr(rstd),
                                                                      _lib.ptr(dx), _lib.ptr(dw), ctypes.c_int(T), ctypes.c_int(H),
                                                                      _lib.stream_handle()), args.iters, 3, flush), 3 * x.numel() * 2)
        del x, y
    if want("swiglu_fwd") or want("swiglu_bwd"):
        gu = torch.randn(T, 2 * F, device=dev).bfloat16()
        yo = torch.empty(T, F, device=dev, dtype=torch.bfloat16)
        if want("swiglu_fwd"):
            report("swiglu_fwd", time_fn(lambda: lib.dcpk_swiglu_fwd(_lib.ptr(gu), _lib.ptr(yo), ctypes.c_long(T), ctypes.c_int(F),
                                                                    _lib.stream_handle()), args.iters, 3, flush), 3 * T * F * 2)
        if want("swiglu_bwd"):
            dgu = torch.empty_like(gu)
            report("swiglu_bwd", time_fn(lambda: lib.dcpk_swiglu_bwd(_lib.ptr(gu), _lib.ptr(yo), _lib.ptr(dgu), ctypes.c_long(T),
                                                                    ctypes.c_int(F), _lib.stream_handle()), args.iters, 3, flush), 5 * T * F * 2)
            del dgu
        del gu, yo
    if want("cross_entropy_fwd_bwd"):
        tc = min(T, 4096)
        logits = torch.randn(tc, V, device=dev).bfloat16()
        labels = torch.randint(0, V, (tc,), device=dev)
        report("cross_entropy_fwd_bwd", time_fn(lambda: model_ops.cross_entropy_inplace(logits, labels, 1.0), args.iters, 3, flush),
               3 * tc * V * 2)
        del logits
    if want("qkv_rope_split") or want("qkv_rope_pack_bwd"):
        qkv = torch.randn(T, 48 * 128, device=dev).bfloat16()
        pos = torch.arange(T, device=dev)
        cos, sin = model_ops.rope_tables(pos)
        if want("qkv_rope_split"):
            qa = torch.empty(T, 32, 128, device=dev, dtype=torch.bfloat16)
            kva = torch.empty(T, 2, 8, 128, device=dev, dtype=torch.bfloat16)
            report("qkv_rope_split", time_fn(lambda: model_ops.qkv_rope_split(qkv, cos, sin, qa, kva, 32, 8), args.iters, 3, flush),
                   2 * qkv.numel() * 2)
        if want("qkv_rope_pack_bwd"):
            dq = torch.randn(T, 32, 128, device=dev)
            dkv = torch.randn(T, 2, 8, 128, device=dev)
            report("qkv_rope_pack_bwd", time_fn(lambda: model_ops.qkv_rope_pack_bwd(dq, dkv, cos, sin, T, 32, 8), args.iters, 3, flush),
                   qkv.numel() * (4 + 2))
    if want("merge_out_lse"):
        # merge of 3 partial (out, lse) per token: reads 3 partial rows, writes one
        n_src, hq = 3, 32
        tm = min(T, 8192)
        part_out = torch.randn(n_src * tm, hq, 128, device=dev).bfloat16()
        part_lse = torch.randn(hq, n_src * tm, device=dev)
        mo, ml = torch.empty(tm, hq, 128, device=dev, dtype=torch.bfloat16), torch.empty(hq, tm, device=dev)
        ops_t = torch.tensor([[b0, min(2048, tm - b0), 3 * i, 3] for i, b0 in enumerate(range(0, tm, 2048))], dtype=torch.int32, device=dev)
        src_t = torch.tensor([s * tm + b0 for b0 in range(0, tm, 2048) for s in range(n_src)], dtype=torch.int32, device=dev)
        report("merge_out_lse", time_fn(lambda: block_ops.merge_out_lse(ops_t, src_t, part_out, part_lse, mo, ml), args.iters, 3, flush),
               (n_src + 1) * tm * hq * 128 * 2 + (n_src + 1) * tm * hq * 4)
    if want("fused_rs_adamw_ag"):
        # single-rank fused gradient read + AdamW + parameter store: bf16 grad in, fp32 master / m / v in and out, bf16 param out
        from ..parallel.dist_optimizer import FlatBuffers, ShardedAdamW
        n = args.opt_elems
        bufs = FlatBuffers(n, dev)
        opt = ShardedAdamW(bufs, clip_grad=None)
        bufs.grads.normal_()
        report("fused_rs_adamw_ag", time_fn(lambda: opt.step(1.0), args.iters, 3, flush), n * (2 + 12 + 12 + 2))


def bench_nvlink(args):
    """Two or more ranks (torch.distributed.run): bandwidth of the in-kernel communication primitives
    over NVLink, CUDA-event timed, max over ranks: peer -> local copy jobs (the operand fetch),
    fp32 push-add into a peer accumulator (the gradient return), and the flag barrier's latency."""
    import torch.distributed as dist
    from ..planner.lowering import KIND_Q, row_copy_jobs
    from ..runtime.symm import SymmetricArena
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    rows, hq = 65536, 32                                    # 512 MB of bf16 rows, 1 GB of fp32 rows
    arena = SymmetricArena({"q": ((2 * rows, hq, 128), torch.bfloat16), "kv": ((8, 2, 8, 128), torch.bfloat16),
                            "dout": ((8, hq, 128), torch.bfloat16), "lse": ((hq, 2 * rows), torch.float32),
                            "delta": ((hq, 8), torch.float32), "acc": ((rows, hq, 128), torch.float32)},
                           dev, dist.group.WORLD)
    arena.view("q").normal_()
    peer = (rank + 1) % world
    pulls = np.asarray([(peer, b0, rows + b0, 2048) for b0 in range(0, rows, 2048)], dtype=np.int32)
    jobs = torch.from_numpy(row_copy_jobs(pulls, KIND_Q, hq * 16)).to(dev)
    ctx = A.CopyContext(arena.peer_ptrs, rank, 2 * rows)
    src = torch.randn(rows // 2, hq, 128, device=dev)
    push = torch.tensor([(peer, b0, b0, 2048) for b0 in range(0, rows // 2, 2048)], dtype=torch.int32, device=dev)

    def timed(fn, iters=10):
        arena.barrier(); fn(); arena.barrier()
        torch.cuda.synchronize(); dist.barrier()
        e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    ms_copy = timed(lambda: A.copy_jobs(jobs, ctx))
    ms_push = timed(lambda: block_ops.push_add_rows(push, src, arena.peer_ptrs("acc"), hq * 128))
    ms_bar = timed(arena.barrier, 50)
    arena.check_status()
    if rank == 0:
        nb_c, nb_p = rows * hq * 128 * 2, (rows // 2) * hq * 128 * 4
        print(json.dumps({"op": "copy_jobs (peer -> local, 64 KB jobs)", "n_gpus": world, "MB": nb_c >> 20, "ms": round(ms_copy, 3),
                          "GB/s per GPU": round(nb_c / ms_copy / 1e6, 1)}))
        print(json.dumps({"op": "push_add_rows (local fp32 -> red.add on peer)", "n_gpus": world, "MB": nb_p >> 20,
                          "ms": round(ms_push, 3), "GB/s per GPU": round(nb_p / ms_push / 1e6, 1)}))
        print(json.dumps({"op": "signal_barrier", "n_gpus": world, "us": round(ms_bar * 1e3, 1)}))
    dist.barrier()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kind", choices=["attn_fwd", "attn_bwd", "ops", "nvlink"])
    ap.add_argument("--only", default=None, help="ops: build and run just this op (small working set for a profiler)")
    ap.add_argument("--opt-elems", type=int, default=256 << 20, help="ops: parameters of the optimizer-kernel benchmark")
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--kv", type=int, default=8192)
    ap.add_argument("--hq", type=int, default=32)
    ap.add_argument("--hkv", type=int, default=8)
    ap.add_argument("--block", type=int, default=2048)
    ap.add_argument("--mask", default="causal", choices=["full", "causal", "lambda"])
    ap.add_argument("--variant", type=int, default=2, help="forward kernel: 2 = two query tiles per CTA (default), 0 / 1 = one tile per CTA with P in TMEM / shared memory")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--timeline", action="store_true", help="print per-phase cycle counts of one backward CTA")
    ap.add_argument("--skip-dq", action="store_true", help="backward without the dQ drain (upper bound probe)")
    args = ap.parse_args()
    if args.kind == "nvlink":
        bench_nvlink(args)
    elif args.kind == "ops":
        bench_ops(args)
    else:
        bench_attention(args.kind, args)


if __name__ == "__main__":
    main()

"""Single-GPU micro-benchmarks of the hand-written kernels (CUDA-event timing, warm-up, inputs
larger than L2 or an L2 flush between iterations), with achieved fractions of the measured peaks.

    python -m dcp_b200.bench.kernel_bench attn_fwd --tokens 8192 --kv 8192 --hq 32 --hkv 8 --mask causal
    python -m dcp_b200.bench.kernel_bench attn_bwd ...
    python -m dcp_b200.bench.kernel_bench ops

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
    dev = torch.device("cuda")
    hbm, tf, src = measured_peaks()
    T, H, F, V = args.tokens, 4096, 14336, 128256
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    res = []

    def report(name, ms, nbytes):
        gbs = nbytes / ms / 1e6
        res.append({"op": name, "ms": round(ms, 4), "GB/s": round(gbs, 1), f"frac_of_{src}_hbm": round(gbs / hbm, 3)})

    x = torch.randn(T, H, device=dev).bfloat16()
    w = torch.ones(H, device=dev).bfloat16()
    y, rstd = torch.empty_like(x), torch.empty(T, device=dev)
    from ..ops import _lib
    import ctypes
    lib = _lib.load()
    report("rmsnorm_fwd", time_fn(lambda: lib.dcpk_rmsnorm_fwd(_lib.ptr(x), _lib.ptr(w), _lib.ptr(y), _lib.ptr(rstd),
                                                              ctypes.c_int(T), ctypes.c_int(H), ctypes.c_float(1e-5),
                                                              _lib.stream_handle()), args.iters, 3, flush), 2 * x.numel() * 2)
    dx, dw = torch.empty_like(x), torch.zeros(H, device=dev)
    report("rmsnorm_bwd", time_fn(lambda: lib.dcpk_rmsnorm_bwd(_lib.ptr(x), _lib.ptr(w), _lib.ptr(y), _lib.ptr(rstd),
                                                              _lib.ptr(dx), _lib.ptr(dw), ctypes.c_int(T), ctypes.c_int(H),
                                                              _lib.stream_handle()), args.iters, 3, flush), 3 * x.numel() * 2)
    gu = torch.randn(T, 2 * F, device=dev).bfloat16()
    yo = torch.empty(T, F, device=dev, dtype=torch.bfloat16)
    report("swiglu_fwd", time_fn(lambda: lib.dcpk_swiglu_fwd(_lib.ptr(gu), _lib.ptr(yo), ctypes.c_long(T), ctypes.c_int(F),
                                                            _lib.stream_handle()), args.iters, 3, flush), 3 * T * F * 2)
    dgu = torch.empty_like(gu)
    report("swiglu_bwd", time_fn(lambda: lib.dcpk_swiglu_bwd(_lib.ptr(gu), _lib.ptr(yo), _lib.ptr(dgu), ctypes.c_long(T),
                                                            ctypes.c_int(F), _lib.stream_handle()), args.iters, 3, flush), 5 * T * F * 2)
    tc = min(T, 4096)
    logits = torch.randn(tc, V, device=dev).bfloat16()
    labels = torch.randint(0, V, (tc,), device=dev)
    report("cross_entropy_fwd_bwd", time_fn(lambda: model_ops.cross_entropy_inplace(logits, labels, 1.0), args.iters, 3, flush),
           3 * tc * V * 2)
    qkv = torch.randn(T, 48 * 128, device=dev).bfloat16()
    pos = torch.arange(T, device=dev)
    cos, sin = model_ops.rope_tables(pos)
    qa = torch.empty(T, 32, 128, device=dev, dtype=torch.bfloat16)
    kva = torch.empty(T, 2, 8, 128, device=dev, dtype=torch.bfloat16)
    report("qkv_rope_split", time_fn(lambda: model_ops.qkv_rope_split(qkv, cos, sin, qa, kva, 32, 8), args.iters, 3, flush),
           2 * qkv.numel() * 2)
    for r in res:
        print(json.dumps(r))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kind", choices=["attn_fwd", "attn_bwd", "ops"])
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
    if args.kind == "ops":
        bench_ops(args)
    else:
        bench_attention(args.kind, args)


if __name__ == "__main__":
    main()

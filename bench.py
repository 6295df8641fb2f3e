"""Headline benchmark: Llama-3-8B-architecture DCP training throughput (tokens/s) on N B200s.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torch.distributed.run)

Default configuration = the scaling configuration: bf16, random-initialised Llama-3-8B
architecture, 32768 tokens per GPU per step (weak scaling), heavy-tailed synthetic lengths (70 %
U[1024, 8192] + 30 % lognormal median 65536 sigma 0.5 clipped to 131072), causal mask, DCP block
size 2048, context-parallel group = all N GPUs, AdamW with sharded fp32 state, full activation
recompute.  ``--config causal131k`` / ``masks`` select the fixed 131072-token configurations.

Two timed regions of K steps each, every step a complete forward + backward + optimizer step on
its own freshly planned batch:
  * device-timed: inputs already staged on the device, CUDA events on the launching stream
    around the K steps, barrier + synchronize on both sides, max over ranks  -> "value";
  * end to end through ``TrainEngine.train_step``: per step the plan is fetched from the
    look-ahead planner (default look-ahead, waited for when late), token ids / labels /
    positions / kernel tables are copied from pinned host memory and the loss is read back
    -> "e2e", with planning time per batch and the number of steps that waited.
The line also carries the attention executor's forward + backward milliseconds inside the timed
steps, and at 8 GPUs the two 131072-token configurations and the attention microbenchmark.
Inputs differ every step and a step streams the 16 GB of bf16 weights twice, far beyond the
126 MB L2, so no explicit L2 flush is needed between timed iterations.

``--impl reference`` would run the unmodified reference from baseline/_ref; it cannot run on
this image (see the message it prints).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# Published DCP number the ratio is quoted against: GPT-8B, LongAlign, 131072 max length, causal,
# 64 x A100 (TP4 x DCP16): 46.3k tokens/s for the whole job.
BASELINE_TOKENS_PER_S = 46300.0
QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")


def reference_arm() -> None:
    reason = ("reference needs dcp_flash_attn (CUDA fork of flash-attention 2.6.3), kahypar, redis-server, "
              "Megatron-LM and TransformerEngine, none of which are on this offline image; "
              "`pip install --no-deps` of the reference source tree succeeds but `import dcp.graph_partition.graph` and "
              "`dcp.runtime.flash_attention.executor` fail with ModuleNotFoundError")
    if int(os.environ.get("RANK", "0")) == 0:      # one line per job, also when launched with several ranks
        print(json.dumps({"impl": "reference", "unavailable": reason}))


class ClockSampler:
    """Samples SM clocks and throttle reasons of the job's own GPUs (selected by UUID, so other
    GPUs of a shared box do not enter the median) every 200 ms while the timed regions run."""

    def __init__(self, path: str, gpu_ids):
        self.path, self.proc, self.gpu_ids = path, None, list(gpu_ids)

    def start(self):
        try:
            self.f = open(self.path, "w")
            cmd = ["nvidia-smi", f"--query-gpu={QUERY}", "--format=csv,noheader,nounits", "-lms", "200"]
            if self.gpu_ids:
                cmd += ["-i", ",".join(self.gpu_ids)]
            self.proc = subprocess.Popen(cmd, stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.f.close()
        return {**parse_clock_log(self.path), "gpus_sampled": len(self.gpu_ids) or "all"}


def parse_clock_log(path: str) -> dict:
    """Median SM clock, maximum SM clock and the throttle reasons seen in a log of ``QUERY`` rows
    (csv, no header, no units; rows that do not parse - e.g. "[N/A]" - are skipped)."""
    sm, mx, reasons = [], [], set()
    names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    for line in open(path):
        parts = [p.strip() for p in line.split(",")]
        if len(parts) < 9:
            continue
        try:
            sm.append(float(parts[1])); mx.append(float(parts[2]))
        except ValueError:
            continue
        for n, v in zip(names, parts[5:9]):
            if v.lower().startswith("active"):
                reasons.add(n)
    sm.sort()
    return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
            "reasons": sorted(reasons), "samples": len(sm)}


def parse_args(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="scaling", choices=["scaling", "causal131k", "masks"])
    ap.add_argument("--model", default="llama3-8b", choices=["llama3-8b", "tiny"])
    ap.add_argument("--dcp-size", type=int, default=0, help="ranks per context-parallel group (0 = all)")
    ap.add_argument("--tp-size", type=int, default=1, help="tensor-parallel ranks per model replica")
    ap.add_argument("--tokens-per-gpu", type=int, default=32768)
    ap.add_argument("--block-size", type=int, default=2048)
    ap.add_argument("--stages", type=int, default=None)
    ap.add_argument("--lookahead", type=int, default=3, help="iterations the planner works ahead")
    ap.add_argument("--planner-workers", type=int, default=2)
    ap.add_argument("--no-verify", action="store_true",
                    help="skip the numerical self-check of the cross-GPU attention path (runs on 2 or more GPUs)")
    ap.add_argument("--no-extras", action="store_true",
                    help="at 8 GPUs: skip the two 131072-token configurations and the attention microbenchmark")
    ap.add_argument("--activation-budget-gb", type=float, default=None,
                    help="extra activation memory for the hand-written layer backward (default: from free memory; "
                         "0: keep nothing extra; -1: autograd + checkpoint path)")
    return ap.parse_args(argv)


def build_engine_config(args, world: int):
    """-> (EngineConfig, scaling kind) of the selected benchmark configuration."""
    from dcp_b200.data import synth
    from dcp_b200.models.llama import LLAMA3_8B, tiny_config
    from dcp_b200.train import EngineConfig
    model = LLAMA3_8B if args.model == "llama3-8b" else tiny_config()
    if args.config == "scaling":
        tokens, dist_, mask, scaling = args.tokens_per_gpu * world, synth.MIXTURE, "causal", "weak"
    elif args.config == "causal131k":
        tokens, dist_, mask, scaling = 131072, synth.LOGNORMAL_8K, "causal", "strong"
    else:
        tokens, dist_, mask, scaling = 131072, synth.LOGNORMAL_16K, "mixed", "strong"
    cfg = EngineConfig(model=model, tokens_per_step=tokens, dcp_size=args.dcp_size, block_size=args.block_size, mask=mask,
                       length_dist=dist_, n_stages=args.stages, activation_budget_gb=args.activation_budget_gb,
                       tp_size=args.tp_size, planner_workers=args.planner_workers, lookahead=args.lookahead)
    return cfg, scaling


def _max_over_ranks(values, dev, group, world):
    import torch
    t = torch.tensor(list(values), dtype=torch.float64, device=dev)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return [float(x) for x in t]


def timed_steps(eng, K: int, barrier):
    """K device-timed steps on fresh plans, inputs staged before each timing window opens (tables
    are per step, so the windows are summed).  -> (ms, tokens, attention fwd ms, attention bwd ms)."""
    import torch
    dev_ms, tokens = 0.0, 0
    eng.executor.time_calls = True
    eng.executor.call_times()
    eng.time_optimizer, eng._optimizer_events = True, []
    for _ in range(K):
        plan = eng.plans.get(eng.iteration)
        toks, labels, pos = eng.stage_inputs(plan)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        eng.run_step(toks, labels, pos, plan.n_global_tokens)
        e1.record()
        barrier()
        dev_ms += e0.elapsed_time(e1)
        tokens += plan.n_global_tokens
        eng.iteration += 1
    ct = eng.executor.call_times()
    eng.executor.time_calls = False
    eng.last_optimizer_ms = eng.optimizer_ms()
    eng.time_optimizer = False
    eng.check_status()
    return dev_ms, tokens, ct["fwd_ms"], ct["bwd_ms"], max(1, ct["n_fwd"])


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        reference_arm()
        return

    import torch
    from dcp_b200.data import synth
    from dcp_b200.ops import _lib
    from dcp_b200.train import TrainEngine, init_distributed

    rank, world, local, group = init_distributed()
    assert world == args.gpus or world == 1 and args.gpus == 1, f"launched with {world} ranks for --gpus {args.gpus}"
    dev = torch.device("cuda", local)
    cfg, scaling = build_engine_config(args, world)
    tokens, dist_, mask = cfg.tokens_per_step, cfg.length_dist, cfg.mask
    # on two or more GPUs: the cross-GPU attention path (peer operand fetch, partial-result stores,
    # merge, gradient push) is compared once with dense fp64 attention before anything is timed
    verify = None
    if world > 1 and not args.no_verify:
        from dcp_b200.runtime.selfcheck import fused_self_check
        verify = fused_self_check(rank, world, group)
        if not verify["passed"] and rank == 0:
            # reported in the JSON line ("verify": {"passed": false, ...}); the timed run still follows
            print(f"fused attention self-check FAILED: {verify}", file=sys.stderr, flush=True)
    eng = TrainEngine(cfg, dev, group)
    W, K = args.warmup, args.steps

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier(group=group)
        torch.cuda.synchronize(dev)

    for _ in range(W):
        eng.train_step()

    # ---- region A: device-timed, inputs staged beforehand
    profiling = os.environ.get("DCP_B200_PROFILE", "0") == "1"
    if profiling:
        eng.executor.profile_summary()          # drop the warm-up marks
    import tempfile
    uuid = "GPU-" + str(torch.cuda.get_device_properties(dev).uuid)
    uuids = [uuid]
    if world > 1:
        import torch.distributed as dist
        uuids = [None] * world
        dist.all_gather_object(uuids, uuid, group=group)
    sampler = ClockSampler(os.path.join(os.environ.get("BENCH_CLOCKS_DIR", tempfile.gettempdir()), f"clocks_rank{rank}.csv"),
                           uuids)
    if rank == 0:
        sampler.start()
    launches0 = _lib.LAUNCHES
    dev_ms, tokens_timed, attn_f, attn_b, n_attn = timed_steps(eng, K, barrier)
    opt_ms = eng.last_optimizer_ms
    launches = _lib.LAUNCHES - launches0
    if profiling:
        # per-step milliseconds of the attention executor's phases on this rank (stderr, every rank)
        phases = {k: round(v / K, 1) for k, v in eng.executor.profile_summary().items()}
        print(f"[profile rank {rank}] step {dev_ms / K:.1f} ms; attention phases per step: {json.dumps(phases)}",
              file=sys.stderr, flush=True)

    # ---- region B: end to end through the public API on fresh iterations: per step the plan is
    # fetched from the look-ahead planner (waited for if it is late), inputs and tables are copied
    # from pinned host memory, and the loss is read back
    n_waits0 = len(eng.plans.waits)
    barrier()
    t0 = time.perf_counter()
    e2e_tokens, h2d, d2h, last_loss = 0, 0, 0, None
    for _ in range(K):
        last_loss = eng.train_step()
        e2e_tokens += eng.last_global_tokens
        h2d, d2h = eng.h2d_bytes, eng.d2h_bytes
    barrier()
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else {}
    waits = eng.plans.waits[n_waits0:]
    plan_s = eng.plans.plan_seconds[n_waits0:]

    dev_ms, e2e_s, attn_f, attn_b, plan_max, wait_sum, opt_ms = _max_over_ranks(
        [dev_ms, e2e_s, attn_f, attn_b, max(plan_s) if plan_s else 0.0, sum(waits), opt_ms], dev, group, world)

    # ---- at 8 GPUs also the two fixed 131072-token configurations and the attention
    # microbenchmark, so that every headline configuration has a number from the same run
    extra = {}
    if world == 8 and args.config == "scaling" and args.model == "llama3-8b" and not args.no_extras:
        for name, (tk, ld, mk) in {"causal131k": (131072, synth.LOGNORMAL_8K, "causal"),
                                    "masks131k": (131072, synth.LOGNORMAL_16K, "mixed")}.items():
            eng.reconfigure(tk, ld, mk)
            for _ in range(2):
                eng.train_step()
            ms, tk_timed, af, ab, _ = timed_steps(eng, 4, barrier)
            ms, af, ab = _max_over_ranks([ms, af, ab], dev, group, world)
            extra[name] = {"tokens_per_s": round(tk_timed / (ms / 1e3), 1), "ms_per_step": round(ms / 4, 2), "steps": 4,
                           "warmup": 2, "attn_fwd_bwd_ms_per_step": round((af + ab) / 4, 1), "global_batch": tk,
                           "length_dist": ld.kind, "mask": mk}
        extra["causal131k"]["vs_published_64xA100"] = round(extra["causal131k"]["tokens_per_s"] / BASELINE_TOKENS_PER_S, 3)
    eng.close()
    lv = eng.activation_levels
    n_layers = cfg.model.n_layers
    del eng
    torch.cuda.empty_cache()
    attn_micro = None
    if world == 8 and not args.no_extras:
        from dcp_b200.bench import attention as attn_bench
        summary = attn_bench.run_batches(attn_bench.default_args(batches=3, warmup=3, iters=5), group, dev, rank, world,
                                         verbose=False)
        attn_micro = {k: v for k, v in summary.items() if k != "summary"}

    recompute_desc = "full per layer (autograd checkpoint)" if lv is None else (
        "per layer, hand-written backward: %d layers recompute QKV/O/gate-up GEMMs, %d recompute gate-up only, "
        "%d recompute no GEMM (chosen from free memory)" % (lv.count(0), lv.count(1), lv.count(2)))
    if rank == 0:
        value = tokens_timed / (dev_ms / 1e3)
        tp = max(1, cfg.tp_size)
        dcp = cfg.dcp_size or world // tp
        par = f"cp{dcp}" + (f"xdp{world // tp // dcp}" if dcp * tp != world else "") + (f"xtp{tp}" if tp > 1 else "")
        same_config = args.config == "causal131k" and world == 8
        out = {
            "metric": "training tokens/s (device-timed, max over ranks)", "value": round(value, 1), "unit": "tokens/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": round(dev_ms / K, 2), "higher_is_better": True,
            "scaling": scaling,
            # the only published number is for another machine (64 x A100) on the 131072-token causal
            # workload; the ratio is quoted for that workload only
            "vs_baseline": round(value / BASELINE_TOKENS_PER_S, 4) if same_config else None,
            "dtype": "bf16",
            "data": "synthetic (seeded length distribution, uniform token ids, random-init weights)",
            "config": {"model": "llama-3-8b-architecture" if args.model == "llama3-8b" else "tiny-llama (debug)",
                       "global_batch": tokens, "seq_len": "variable, <= 131072", "parallelism": par,
                       "tokens_per_gpu": tokens // world, "mask": mask, "length_dist": dist_.kind,
                       "dcp_block_size": args.block_size, "optimizer": "AdamW (sharded fp32 state), grad clip 1.0",
                       "recompute": recompute_desc,
                       "l2": "inputs change every step and exceed L2 (16 GB of weights streamed per pass)",
                       "published_number_note": "46.3k tokens/s: DCP on 64 x A100, GPT-8B, LongAlign 131072 causal "
                                                "(other hardware, other workload unless --config causal131k)"},
            "clocks": clocks,
            "attn_fwd_bwd_ms": {"per_step": round((attn_f + attn_b) / K, 1), "fwd_per_layer": round(attn_f / K / n_layers, 2),
                                "bwd_per_layer": round(attn_b / K / n_layers, 2),
                                "note": "attention executor calls inside the timed steps (CUDA events, max over ranks, "
                                        "cross-GPU waits included)"},
            "optimizer_step_ms": {"per_step": round(opt_ms / K, 2),
                                  "note": "optimizer.step after the backward (CUDA events, max over ranks): last gradient "
                                          "bucket, norm all-reduce, AdamW and parameter stores; the per-layer "
                                          "reduce-scatters run beside the backward"},
            "e2e": {"value": round(e2e_tokens / e2e_s, 1), "unit": "tokens/s", "ms_per_step": round(1e3 * e2e_s / K, 2),
                    "tokens": int(e2e_tokens),
                    "batches": "the K iterations after the device-timed ones (variable-length batches differ in "
                               "attention work, so the two figures are not the same batches)",
                    "h2d_bytes_per_step": int(h2d),
                    "d2h_bytes_per_step": int(d2h), "fresh_plans": True, "planner_lookahead": cfg.lookahead,
                    "planner_workers": cfg.planner_workers,
                    "plan_ms_mean": round(1e3 * sum(plan_s) / max(1, len(plan_s)), 1), "plan_ms_max": round(1e3 * plan_max, 1),
                    "steps_that_waited_for_planner": int(sum(1 for w in waits if w > 0.005)),
                    "planner_wait_s_in_region": round(wait_sum, 3)},
            "gpu_launches": int(launches), "final_loss": last_loss,
        }
        if verify is not None:
            out["verify"] = verify
        if attn_micro is not None:
            out["attn_microbench_131k_causal"] = attn_micro
        if extra:
            out["extra_configs"] = extra
        print(json.dumps(out))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

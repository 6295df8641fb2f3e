"""The reference's --dcp-* flag set is accepted with the same names, and the planner knobs they
carry reach the plans."""
import argparse

import numpy as np

from dcp_b200.data import synth
from dcp_b200.data.plan_service import PlanSpec, plan_iteration
from dcp_b200.train import add_dcp_args

REFERENCE_FLAGS = [
    "--disable-dcp", "--dcp-intra-node-lat", "--dcp-intra-node-bw", "--dcp-inter-node-lat", "--dcp-inter-node-bw",
    "--dcp-max-tflops", "--dcp-max-mem-bw", "--dcp-prefetch-planner-num-workers",
    "--dcp-prefetch-listener-num-workers", "--dcp-block-size", "--dcp-head-block-size",
    "--dcp-use-block-size-heuristic", "--dcp-mem-imbalance-epsilon", "--dcp-comp-imbalance-epsilon",
    "--dcp-inter-node-comp-imbalance-factor", "--dcp-global-batch-size-in-tokens", "--dcp-dataset-split",
    "--dcp-dataset-text-key", "--dcp-use-cudagraph", "--dcp-mask-type",
]


def test_every_reference_flag_is_accepted():
    ap = argparse.ArgumentParser()
    add_dcp_args(ap)
    known = {s for a in ap._actions for s in a.option_strings}
    assert not [f for f in REFERENCE_FLAGS if f not in known]
    a = ap.parse_args(["--dcp-block-size", "512", "--dcp-mask-type", "lambda", "--dcp-comp-imbalance-epsilon", "0.1",
                       "--dcp-max-tflops", "900", "--dcp-use-block-size-heuristic", "1", "--disable-dcp"])
    assert (a.dcp_block_size, a.dcp_mask_type, a.dcp_comp_imbalance_epsilon, a.dcp_max_tflops) == (512, "lambda", 0.1, 900.0)
    assert a.disable_dcp and a.dcp_use_block_size_heuristic == 1


def _spec(**kw):
    return PlanSpec(world=4, dcp_size=4, tokens_per_step=16384, n_heads=8, n_kv_heads=2, block_size=512,
                    length_dist=synth.LengthDist("lognormal", 3000.0, 0.8, 128, 16384), vocab=1000, **kw)


def test_planner_knobs_reach_the_plans():
    loose = [plan_iteration(_spec(mem_imbalance_epsilon=0.5, comp_imbalance_epsilon=0.5), 1, r) for r in range(4)]
    tight = [plan_iteration(_spec(mem_imbalance_epsilon=0.02, comp_imbalance_epsilon=0.02), 1, r) for r in range(4)]
    for plans in (loose, tight):
        assert sum(p.tokens.numel() for p in plans) == plans[0].n_global_tokens
    spread = lambda plans: np.ptp([p.tokens.numel() for p in plans])
    assert spread(tight) <= spread(loose)
    # cost-model overrides and the block-size heuristic are accepted and still give a complete plan
    alt = [plan_iteration(_spec(cost_model={"max_tflops": 500.0, "intra_node_bw": 2400.0},
                                use_block_size_heuristic=True), 1, r) for r in range(4)]
    assert sum(p.tokens.numel() for p in alt) == alt[0].n_global_tokens


def test_bench_and_train_build_their_engine_configs():
    """The argument plumbing of the benchmark and of the training CLI: every value lands in the
    field it is meant for (guards against positional drift when the config dataclass grows)."""
    import importlib.util
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_entry", os.path.join(root, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    a = bench.parse_args(["--gpus", "8", "--dcp-size", "4", "--block-size", "1024", "--tp-size", "2", "--stages", "3",
                          "--steps", "5", "--lookahead", "5"])
    cfg, scaling = bench.build_engine_config(a, 8)
    assert (cfg.tokens_per_step, cfg.dcp_size, cfg.block_size, cfg.tp_size, cfg.n_stages, cfg.mask, cfg.lookahead) == \
        (8 * 32768, 4, 1024, 2, 3, "causal", 5)
    assert scaling == "weak" and cfg.length_dist.kind == "mixture" and cfg.model.n_layers == 32
    cfg, scaling = bench.build_engine_config(bench.parse_args(["--config", "masks", "--model", "tiny"]), 2)
    assert (cfg.tokens_per_step, cfg.mask, scaling, cfg.tp_size, cfg.dcp_size) == (131072, "mixed", "strong", 1, 0)
    # the defaults give a run that finishes in minutes on one GPU
    d = bench.parse_args([])
    assert (d.gpus, d.impl) == (1, "ours") and d.warmup >= 3 and d.steps >= 1


def test_parallel_layout_groups_partition_the_world():
    """TP x CP x DP rank layout: every family of groups partitions the ranks, a dcp group and a tp
    group share exactly one rank, and the optimizer groups are the ranks of equal tp index."""
    from dcp_b200.train import parallel_layout
    for world, tp, dcp in [(8, 2, 2), (8, 1, 4), (8, 4, 0), (16, 2, 4), (2, 2, 0), (8, 1, 0), (6, 3, 1)]:
        lay = parallel_layout(world, tp, dcp)
        n_cp, d = world // tp, (dcp or world // tp)
        assert (lay["n_cp"], lay["dcp"]) == (n_cp, d)
        for name, size in (("dcp_groups", d), ("tp_groups", tp), ("opt_groups", n_cp)):
            flat = sorted(r for g in lay[name] for r in g)
            assert flat == list(range(world)) and all(len(g) == size for g in lay[name]), name
        for dg in lay["dcp_groups"]:
            assert len({r % tp for r in dg}) == 1                     # one tp index per attention group
            assert len({r // tp // d for r in dg}) == 1               # one replica per attention group
            for tg in lay["tp_groups"]:
                assert len(set(dg) & set(tg)) <= 1
        for t, og in enumerate(lay["opt_groups"]):
            assert all(r % tp == t for r in og)
        for tg in lay["tp_groups"]:
            assert tg == list(range(tg[0], tg[0] + tp))               # tensor-parallel ranks are adjacent


def test_bench_clock_log_parsing(tmp_path):
    """The bench line's clock record: median SM clock over the sampled rows of the job's own GPUs,
    maximum clock, and every throttle reason that was active in any row; unparsable rows are skipped."""
    import importlib.util
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_main", os.path.join(root, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    log = tmp_path / "clocks.csv"
    log.write_text("0, 1530, 1965, 950.1, 0x0000000000000004, Not Active, Not Active, Not Active, Active\n"
                   "0, 1695, 1965, 990.0, 0x0000000000000004, Not Active, Not Active, Not Active, Active\n"
                   "0, [N/A], 1965, 10.0, 0x0, Not Active, Not Active, Not Active, Not Active\n"
                   "0, 1920, 1965, 400.0, 0x0, Not Active, Not Active, Active, Not Active\n"
                   "garbage\n")
    rec = bench.parse_clock_log(str(log))
    assert rec == {"sm_mhz": 1695.0, "sm_max_mhz": 1965.0, "reasons": ["sw_power_cap", "sw_thermal_slowdown"], "samples": 3}
    sampler = bench.ClockSampler(str(tmp_path / "x.csv"), ["GPU-abc", "GPU-def"])
    assert sampler.stop()["reasons"] == ["nvidia-smi unavailable"]          # never started: no process to read

"""Benchmark tooling that needs no GPU: preprocessing, log parsing, grid runner watchdog, replay."""
import json
import os
import pickle
import sys

from dcp_b200.bench import parse_logs, preprocessing
from dcp_b200.bench.run_experiments import run_cell


def test_preprocessing_scales_and_packs(tmp_path):
    assert preprocessing.scale_lengths([100, 100000, 10], 2.0, 131072) == [200, 131072, 20]
    b = preprocessing.pack_batches([60000, 50000, 40000, 200000, 10], 131072)
    assert b == [[60000, 50000], [40000], [131072], [10]] and preprocessing.max_dp_degree(b) == 1
    out = tmp_path / "b.json"
    preprocessing.main(["--synthetic", "lognormal8k", "--n", "200", "--out", str(out)])
    d = json.load(open(out))
    assert all(sum(x) <= 131072 for x in d["batches"]) and d["max_dp_degree"] >= 1


def test_log_parsers():
    text = "\n".join(f" iteration {i} | elapsed time per iteration (ms): {100 + i}.0 | Training loss: {5 - 0.1 * i:.3f}"
                     for i in range(6)) + "\nDCP: total time 40.0 ms\nUlysses: total time 60.0 ms\n"
    assert parse_logs.parse_iteration_times(text) == (102 + 103 + 104 + 105) / 4
    assert parse_logs.parse_loss_curve(text)[:2] == [5.0, 4.9]
    assert parse_logs.parse_microbenchmark(text, 4) == {"DCP": 10.0, "Ulysses": 15.0}
    assert parse_logs.losses_overlap([5.0, 4.9], [5.01, 4.88]) and not parse_logs.losses_overlap([5.0], [6.0])


def test_grid_runner_detects_failure_and_stall(tmp_path):
    ok = run_cell([sys.executable, "-c", "print('fine')"], str(tmp_path / "a.log"))
    bad = run_cell([sys.executable, "-c", "raise SystemExit(3)"], str(tmp_path / "b.log"))
    stalled = run_cell([sys.executable, "-c", "import time; print('x', flush=True); time.sleep(60)"],
                       str(tmp_path / "c.log"), no_progress_s=3.0)
    assert (ok, bad, stalled) == ("ok", "failed", "stalled")


def test_grid_runner_two_nodes_lock_step(tmp_path):
    """Two runner processes act as two nodes: node 0 publishes the cell through the key-value server,
    both launch their share under torch.distributed.run (one rank each, gloo all-reduce across the
    nodes), node 0 gathers the statuses and writes the summary."""
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    base = [sys.executable, "-m", "dcp_b200.bench.run_experiments", "--kind", "selftest", "--gpus", "1", "--nnodes", "2",
            "--coordinator", "127.0.0.1:29733", "--base-port", "29735", "--out", str(tmp_path), "--batches", "1"]
    env = dict(os.environ, PYTHONPATH=root)
    procs = [subprocess.Popen(base + ["--node-rank", str(r)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                              text=True) for r in (0, 1)]
    outs = [p.communicate(timeout=300)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    rows = list(__import__("csv").DictReader(open(tmp_path / "summary.csv")))
    assert len(rows) == 1 and rows[0]["status"] == "ok" and float(rows[0]["ms_per_batch_Selftest"]) > 0
    assert (tmp_path / "kind-selftest_gpus-1.node1.log").exists()


def test_grid_runner_abort_reaches_the_other_node(tmp_path):
    """A cell that one node gives up is ended on the other node too: the second node's child would
    sleep for a minute, but its watchdog sees the abort key."""
    import threading
    import time
    from dcp_b200.data.kv_store import KVStore
    from dcp_b200.bench.run_experiments import NodeCoordinator, overall_status
    store = KVStore()
    a, b = NodeCoordinator(store, 0, 2), NodeCoordinator(store, 1, 2)
    result = {}

    def node_b():
        result["b"] = run_cell([sys.executable, "-c", "import time; time.sleep(60)"], str(tmp_path / "b.log"),
                               no_progress_s=120, abort_check=lambda: b.aborted(0))
        b.report(0, result["b"])

    t = threading.Thread(target=node_b)
    t0 = time.time()
    t.start()
    a.report(0, run_cell([sys.executable, "-c", "raise SystemExit(3)"], str(tmp_path / "a.log")))
    t.join(timeout=60)
    assert not t.is_alive() and result["b"] == "aborted" and time.time() - t0 < 45
    assert a.gather(0) == ["failed", "aborted"] and overall_status(a.gather(0)) == "failed"
    assert overall_status(["ok", "ok"]) == "ok" and overall_status(["aborted", "stalled"]) == "stalled"


def test_figures_are_written_as_svg(tmp_path):
    """The four figures (microbenchmark bars, iteration-time bars, loss curves, dry-run lines) from
    the runner's tables: well-formed SVG with one bar / line per data point / series."""
    import xml.etree.ElementTree as ET
    from dcp_b200.bench import plotting
    rows = [{"kind": "attention", "framework": fw, "mask": m, "length_dist": "lognormal8k", "block_size": 2048,
             "status": "ok", "ms_per_batch_Forward": 5.0 + i, "ms_per_batch_Backward": 9.0 + i}
            for i, (fw, m) in enumerate([("dcp", "causal"), ("ring", "causal"), ("ulysses", "causal"), ("dcp", "lambda")])]
    rows.append(dict(rows[0], framework="zigzag", status="failed"))          # failed cells are left out
    rows += [{"kind": "train", "mask": "causal", "length_dist": "mixture", "block_size": bs, "ms_per_iteration": 4000 + bs}
             for bs in (1024, 2048)]
    parse_logs.write_table(rows, str(tmp_path / "summary.csv"))
    ns = {"s": "http://www.w3.org/2000/svg"}
    plotting.main(["microbench", str(tmp_path / "summary.csv"), "--out", str(tmp_path / "mb.svg")])
    root = ET.parse(tmp_path / "mb.svg").getroot()
    assert len(root.findall(".//s:rect[@class='bar']", ns)) == 4
    plotting.main(["e2e", str(tmp_path / "summary.csv"), "--out", str(tmp_path / "e2e.svg")])
    assert len(ET.parse(tmp_path / "e2e.svg").getroot().findall(".//s:rect[@class='bar']", ns)) == 2
    for name, shift in (("a.log", 0.0), ("b.log", 0.01)):
        (tmp_path / name).write_text("".join(f"Training loss: {10 - 0.1 * i + shift}\n" for i in range(20)))
    plotting.main(["loss", str(tmp_path / "a.log"), str(tmp_path / "b.log"), "--out", str(tmp_path / "loss.svg")])
    lines = ET.parse(tmp_path / "loss.svg").getroot().findall(".//s:polyline[@class='line']", ns)
    assert len(lines) == 2 and len(lines[0].get("points").split()) == 20
    json.dump({"cells": [{"mask": "causal", "length_dist": "mixture", "n_stages": 4, "block_size": b,
                          "modelled_pipeline_ms": 10.0 + b / 1024} for b in (1024, 2048, 4096)]},
              open(tmp_path / "dry.json", "w"))
    plotting.main(["dryrun", str(tmp_path / "dry.json"), "--out", str(tmp_path / "dry.svg")])
    assert len(ET.parse(tmp_path / "dry.svg").getroot().findall(".//s:polyline[@class='line']", ns)) == 1
    assert plotting._nice_ticks(0, 17.3)[-1] >= 17.3 and plotting._nice_ticks(3, 3)[0] <= 3


def test_replay_of_saved_plans(tmp_path):
    import torch
    from dcp_b200.bench.replay import replay_plans
    from dcp_b200.core.common import get_default_execution_context
    from dcp_b200.planner.compiler import InstrCompiler
    from dcp_b200.planner.workload import generate_workload, pad_seqlens
    ctx = get_default_execution_context(2, 1)
    raw = [400, 250]
    pad = pad_seqlens(raw, 64)
    wl = generate_workload((sum(pad), 4, 16), (sum(pad), 2, 2, 16), raw, pad, 64, 4, ctx.comp_cost_model)
    res = InstrCompiler(ctx).compile(wl)
    p = tmp_path / "plans.pkl"
    pickle.dump(res, open(p, "wb"))
    rep = replay_plans(str(p))
    assert rep["forward"]["attn_units"] == len(res[0].workloads) == rep["backward"]["attn_units"]


def test_ring_baselines_match_dense_attention():
    """Plain and zigzag ring attention (the NCCL point-to-point baselines), forward and backward,
    as two gloo processes against dense causal attention of the packed batch."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    # 2 ranks: plain and zigzag ring; 4 ranks: also the double ring (two inner rings of two) and the
    # hierarchical all-to-all (2) x ring (2) pattern
    for world, port in ((2, 29631), (4, 29633)):
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
               "127.0.0.1", "--master-port", str(port), os.path.join(root, "tests", "ring_worker.py")]
        res = subprocess.run(cmd, env=dict(os.environ, PYTHONPATH=root, OMP_NUM_THREADS="2"), stdout=subprocess.PIPE,
                             stderr=subprocess.STDOUT, text=True, timeout=600)
        assert res.returncode == 0 and "RING_OK" in res.stdout, res.stdout[-3000:]


def test_dry_run_grid_and_best_config(tmp_path):
    """Planner-only grid search: every cell reports balance, traffic and a modelled time; ``best``
    keeps the fastest cell per workload."""
    from dcp_b200.bench import dry_run
    out = tmp_path / "dry.json"
    res = dry_run.main(["--devices", "4", "--nodes", "2", "--tokens", "8192", "--n-heads", "8", "--n-kv-heads", "2",
                        "--block-sizes", "256", "512", "--batches", "1", "--out", str(out)])
    assert len(res["cells"]) == 2 and len(res["best"]) == 1
    for c in res["cells"]:
        assert c["compute_max_over_mean"] >= 1.0 and c["tokens_max_over_mean"] >= 1.0
        assert c["modelled_pipeline_ms"] >= c["max_compute_ms"] > 0
        assert c["inter_node_MB_per_device"] >= 0 and c["n_work_units"] > 0
    assert res["best"][0]["modelled_pipeline_ms"] == min(c["modelled_pipeline_ms"] for c in res["cells"])
    assert json.load(open(out))["best"] == res["best"]


def test_pipeline_stage_boundary():
    """Pipeline-parallel stage links (NCCL / gloo point-to-point with early-posted receives) in
    one-forward-one-backward order on 2 and 3 stages: gradients and losses equal the unsplit model."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for world, port in ((2, 29641), (3, 29643)):
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
               "127.0.0.1", "--master-port", str(port), os.path.join(root, "tests", "pp_worker.py")]
        res = subprocess.run(cmd, env=dict(os.environ, PYTHONPATH=root, OMP_NUM_THREADS="1"), stdout=subprocess.PIPE,
                             stderr=subprocess.STDOUT, text=True, timeout=300)
        assert res.returncode == 0 and "PP_OK" in res.stdout, res.stdout[-3000:]


def test_attention_benchmark_planning_arguments(tmp_path):
    """The microbenchmark's planner-side arguments: default settings leave the planner's own defaults,
    explicit sequence lengths (command line or the preprocessing json, cycled over batches) replace the
    length distribution, tolerances / head block size reach the plan specification."""
    import argparse
    from dcp_b200.bench import attention as A
    args = A.default_args(tokens=8192, block_size=512)
    spec = A.bench_plan_spec(args, 2)
    assert (spec.head_block_size, spec.mem_imbalance_epsilon, spec.comp_imbalance_epsilon) == (0, None, None)
    assert sum(A.plan_for_batch(args, spec, 0, 1).seqlens) <= 8192
    args.seqlens = "3000,1000,2500"
    plans = [A.plan_for_batch(args, spec, 0, r) for r in range(2)]
    assert plans[0].seqlens == [3000, 1000, 2500] and sum(p.tokens.numel() for p in plans) == 6500
    args.seqlens = None
    json.dump({"batches": [[2000, 500], [4096]], "max_dp_degree": 1}, open(tmp_path / "b.json", "w"))
    args.seqlens_config = str(tmp_path / "b.json")
    assert [A.plan_for_batch(args, spec, b, 0).seqlens for b in range(3)] == [[2000, 500], [4096], [2000, 500]]
    tuned = argparse.Namespace(**{**vars(args), "mem_epsilon": 0.1, "comp_epsilon": 0.05, "head_block_size": 8,
                                  "use_block_size_heuristic": True})
    spec = A.bench_plan_spec(tuned, 4)
    assert (spec.head_block_size, spec.mem_imbalance_epsilon, spec.comp_imbalance_epsilon, spec.use_block_size_heuristic) == \
        (8, 0.1, 0.05, True)

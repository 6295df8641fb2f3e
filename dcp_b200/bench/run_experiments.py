"""Experiment grid runner for one multi-GPU box.

Runs a grid of (benchmark, framework, mask, length distribution, GPU count, block size) as child
processes under ``torch.distributed.run``, with the safeguards of the reference's orchestrators
(benchmark/mlm/run_experiments.py:748-845, benchmark/microbenchmark/run_experiments.py:77-221):
failure keywords in the log mark a run failed, a no-progress watchdog ends a silent run, finished
cells are skipped on restart, and every cell's arguments are stored next to its log.  Child
processes are ended through their own process group, never by name pattern.

    python -m dcp_b200.bench.run_experiments --out results --gpus 8 --kind attention
"""
from __future__ import annotations

import argparse
import itertools
import json
import os
import signal
import subprocess
import sys
import time
from typing import Dict, List

from .parse_logs import parse_iteration_times, parse_microbenchmark, write_table

FAIL_KEYWORDS = ("Traceback (most recent call last)", "CUDA error", "NCCL error", "device-side failure detected",
                 "ChildFailedError")


def run_cell(cmd: List[str], log_path: str, no_progress_s: float = 180.0, timeout_s: float = 3600.0) -> str:
    """Run one cell; returns "ok", "failed", "stalled" or "timeout"."""
    with open(log_path, "w") as log:
        proc = subprocess.Popen(cmd, stdout=log, stderr=subprocess.STDOUT, start_new_session=True)
        start = last_change = time.time()
        last_size = 0
        status = None
        while proc.poll() is None:
            time.sleep(2.0)
            size = os.path.getsize(log_path)
            now = time.time()
            if size != last_size:
                last_size, last_change = size, now
                with open(log_path) as f:
                    f.seek(max(0, size - 20000))
                    tail = f.read()
                if any(k in tail for k in FAIL_KEYWORDS):
                    status = "failed"
            if status is None and now - last_change > no_progress_s:
                status = "stalled"
            if status is None and now - start > timeout_s:
                status = "timeout"
            if status is not None:
                try:
                    os.killpg(proc.pid, signal.SIGTERM)   # the child's own process group only
                except ProcessLookupError:
                    pass
                try:
                    proc.wait(timeout=30)
                except subprocess.TimeoutExpired:
                    os.killpg(proc.pid, signal.SIGKILL)
                return status
    return "ok" if proc.returncode == 0 else "failed"


def grid(args) -> List[Dict]:
    cells = []
    if args.kind == "attention":
        for fw, mask, dist, bs in itertools.product(args.frameworks, args.masks, args.length_dists, args.block_sizes):
            if fw != "dcp" and mask != "causal":
                continue
            cells.append({"kind": "attention", "framework": fw, "mask": mask, "length_dist": dist, "block_size": bs,
                          "gpus": args.gpus})
    else:
        for mask, dist, bs in itertools.product(args.masks, args.length_dists, args.block_sizes):
            cells.append({"kind": "train", "mask": mask, "length_dist": dist, "block_size": bs, "gpus": args.gpus})
    return cells


def command(cell: Dict, port: int, args) -> List[str]:
    launch = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={cell['gpus']}",
              "--master-addr", "127.0.0.1", "--master-port", str(port)]
    if cell["kind"] == "attention":
        return launch + ["-m", "dcp_b200.bench.attention", "--framework", cell["framework"], "--mask", cell["mask"],
                         "--length-dist", cell["length_dist"], "--block-size", str(cell["block_size"]), "--tokens",
                         str(args.tokens), "--batches", str(args.batches)]
    return launch + ["-m", "dcp_b200.train", "--iters", str(args.iters), "--tokens-per-step", str(args.tokens),
                     "--dcp-mask-type", cell["mask"], "--length-dist", cell["length_dist"], "--dcp-block-size",
                     str(cell["block_size"]), "--model", args.model]


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="results")
    ap.add_argument("--kind", default="attention", choices=["attention", "train"])
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--frameworks", nargs="+", default=["dcp", "ulysses", "zigzag", "ring"])
    ap.add_argument("--masks", nargs="+", default=["causal", "lambda", "causal_blockwise", "shared_question"])
    ap.add_argument("--length-dists", nargs="+", default=["lognormal8k"])
    ap.add_argument("--block-sizes", nargs="+", type=int, default=[1024, 2048, 4096])
    ap.add_argument("--tokens", type=int, default=131072)
    ap.add_argument("--batches", type=int, default=5)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--no-progress-s", type=float, default=180.0)
    args = ap.parse_args(argv)
    os.makedirs(args.out, exist_ok=True)
    rows = []
    for i, cell in enumerate(grid(args)):
        name = "_".join(f"{k}-{v}" for k, v in cell.items())
        log_path = os.path.join(args.out, name + ".log")
        done_path = os.path.join(args.out, name + ".json")
        if os.path.exists(done_path):
            rows.append(json.load(open(done_path)))
            continue
        json.dump(cell, open(os.path.join(args.out, name + ".args.json"), "w"))
        status = run_cell(command(cell, 29700 + i % 200, args), log_path, args.no_progress_s)
        text = open(log_path).read()
        res = dict(cell, status=status)
        if cell["kind"] == "attention":
            res.update({f"ms_per_batch_{k}": v for k, v in parse_microbenchmark(text, args.batches).items()})
        else:
            res["ms_per_iteration"] = parse_iteration_times(text)
        json.dump(res, open(done_path, "w"))
        rows.append(res)
        print(res, flush=True)
    write_table(rows, os.path.join(args.out, "summary.csv"))


if __name__ == "__main__":
    main()

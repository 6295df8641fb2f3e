"""Experiment grid runner for one multi-GPU box or several of them.

Runs a grid of (benchmark, framework, mask, length distribution, GPU count, block size) as child
processes under ``torch.distributed.run``, with the safeguards of the reference's orchestrators
(benchmark/mlm/run_experiments.py:748-845, benchmark/microbenchmark/run_experiments.py:77-221):
failure keywords in the log mark a run failed, a no-progress watchdog ends a silent run, finished
cells are skipped on restart, and every cell's arguments are stored next to its log.  Child
processes are ended through their own process group, never by name pattern.

    python -m dcp_b200.bench.run_experiments --out results --gpus 8 --kind attention

Several boxes: start the same command on every node with ``--nnodes N --node-rank r --coordinator
HOST:PORT`` (HOST = node 0).  Node 0 owns the grid and a key-value server (the role of the
reference's Redis store, benchmark/utils.py:17-215); it publishes one cell at a time, every node
launches its ``torch.distributed.run`` share of the cell, reports its status, and a failure,
stall or timeout seen by one node ends the cell's children on all of them before the next cell.
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


def run_cell(cmd: List[str], log_path: str, no_progress_s: float = 180.0, timeout_s: float = 3600.0,
             abort_check=None) -> str:
    """Run one cell; returns "ok", "failed", "stalled", "timeout" or "aborted" (``abort_check()``
    became true: another node gave the cell up)."""
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
            if status is None and abort_check is not None and abort_check():
                status = "aborted"
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
    elif args.kind == "selftest":
        cells.append({"kind": "selftest", "gpus": args.gpus})
    else:
        for mask, dist, bs in itertools.product(args.masks, args.length_dists, args.block_sizes):
            cells.append({"kind": "train", "mask": mask, "length_dist": dist, "block_size": bs, "gpus": args.gpus})
    return cells


def command(cell: Dict, port: int, args) -> List[str]:
    nnodes = getattr(args, "nnodes", 1)
    launch = [sys.executable, "-m", "torch.distributed.run", f"--nnodes={nnodes}", f"--nproc-per-node={cell['gpus']}",
              "--master-addr", getattr(args, "master_addr", None) or "127.0.0.1", "--master-port", str(port)]
    if nnodes > 1:
        launch += [f"--node-rank={args.node_rank}"]
    if cell["kind"] == "selftest":
        return launch + ["-m", "dcp_b200.bench.run_experiments", "--selftest-worker"]
    if cell["kind"] == "attention":
        return launch + ["-m", "dcp_b200.bench.attention", "--framework", cell["framework"], "--mask", cell["mask"],
                         "--length-dist", cell["length_dist"], "--block-size", str(cell["block_size"]), "--tokens",
                         str(args.tokens), "--batches", str(args.batches)] + \
            (["--seqlens-config", args.seqlens_config] if getattr(args, "seqlens_config", None) else [])
    return launch + ["-m", "dcp_b200.train", "--iters", str(args.iters), "--tokens-per-step", str(args.tokens),
                     "--dcp-mask-type", cell["mask"], "--length-dist", cell["length_dist"], "--dcp-block-size",
                     str(cell["block_size"]), "--model", args.model]


class NodeCoordinator:
    """Lock step of the nodes of one grid over the key-value store.  Keys: ``cell/<i>`` (published by
    node 0; None ends the grid), ``status/<i>/<node>``, ``abort/<i>`` (set by the first node that
    gives cell i up; the others poll it from their watchdog loop)."""

    def __init__(self, store, node_rank: int, n_nodes: int, wait_s: float = 7200.0):
        self.store, self.node_rank, self.n_nodes, self.wait_s = store, node_rank, n_nodes, wait_s

    def publish(self, i: int, cell) -> None:
        self.store.set(f"cell/{i}", cell)

    def fetch(self, i: int):
        return self.store.get(f"cell/{i}", self.wait_s)

    def aborted(self, i: int) -> bool:
        return self.store.exists(f"abort/{i}")

    def report(self, i: int, status: str) -> None:
        if status not in ("ok", "aborted"):
            self.store.set(f"abort/{i}", self.node_rank)
        self.store.set(f"status/{i}/{self.node_rank}", status)

    def wait_followers(self, timeout_s: float = 120.0) -> None:
        deadline = time.time() + timeout_s
        while self.store.add("followers_done", 0) < self.n_nodes - 1 and time.time() < deadline:
            time.sleep(0.2)

    def gather(self, i: int) -> List[str]:
        return [self.store.get(f"status/{i}/{n}", self.wait_s) for n in range(self.n_nodes)]


def overall_status(statuses: List[str]) -> str:
    """One status for a cell from its nodes' statuses: ok only if all are; else the first real cause."""
    bad = [s for s in statuses if s not in ("ok", "aborted")]
    return "ok" if all(s == "ok" for s in statuses) else (bad[0] if bad else "aborted")


def selftest_worker() -> None:
    """Child of a ``selftest`` cell: a gloo all-reduce over all ranks of all nodes, reported in the
    microbenchmark log format."""
    import torch
    import torch.distributed as dist
    dist.init_process_group("gloo")
    t0 = time.time()
    x = torch.ones(4) * (dist.get_rank() + 1)
    dist.all_reduce(x)
    w = dist.get_world_size()
    assert x[0].item() == w * (w + 1) / 2
    if dist.get_rank() == 0:
        print(f"Selftest: total time {1e3 * (time.time() - t0):.3f} ms", flush=True)
    dist.barrier()
    dist.destroy_process_group()


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="results")
    ap.add_argument("--kind", default="attention", choices=["attention", "train", "selftest"])
    ap.add_argument("--nnodes", type=int, default=1)
    ap.add_argument("--node-rank", type=int, default=0)
    ap.add_argument("--coordinator", default=None, help="HOST:PORT of node 0's key-value server (several nodes)")
    ap.add_argument("--master-addr", default=None, help="rendezvous address of the children (default: coordinator host)")
    ap.add_argument("--base-port", type=int, default=29700)
    ap.add_argument("--selftest-worker", action="store_true", help=argparse.SUPPRESS)
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--frameworks", nargs="+", default=["dcp", "ulysses", "zigzag", "ring", "double-ring", "a2a+p2p"])
    ap.add_argument("--masks", nargs="+", default=["causal", "lambda", "causal_blockwise", "shared_question"])
    ap.add_argument("--length-dists", nargs="+", default=["lognormal8k"])
    ap.add_argument("--block-sizes", nargs="+", type=int, default=[1024, 2048, 4096])
    ap.add_argument("--tokens", type=int, default=131072)
    ap.add_argument("--batches", type=int, default=5)
    ap.add_argument("--seqlens-config", default=None,
                    help="json of explicit batches for the attention cells (written by dcp_b200.bench.preprocessing)")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--no-progress-s", type=float, default=180.0)
    args = ap.parse_args(argv)
    if args.selftest_worker:
        selftest_worker()
        return
    os.makedirs(args.out, exist_ok=True)
    coord = None
    if args.nnodes > 1:
        from ..data.kv_store import KVServer, KVStore
        assert args.coordinator, "--coordinator HOST:PORT is needed with --nnodes > 1"
        host, port = args.coordinator.rsplit(":", 1)
        server = KVServer(host, int(port), args.nnodes) if args.node_rank == 0 else None   # kept alive by this name
        coord = NodeCoordinator(KVStore(host, int(port), timeout_s=600.0), args.node_rank, args.nnodes)
        args.master_addr = args.master_addr or host
    if coord is not None and args.node_rank > 0:
        follow(coord, args)
        return
    rows = []
    seq = 0
    for i, cell in enumerate(grid(args)):
        name = "_".join(f"{k}-{v}" for k, v in cell.items())
        log_path = os.path.join(args.out, name + ".log")
        done_path = os.path.join(args.out, name + ".json")
        if os.path.exists(done_path):
            rows.append(json.load(open(done_path)))
            continue
        json.dump(cell, open(os.path.join(args.out, name + ".args.json"), "w"))
        port = args.base_port + i % 200
        if coord is None:
            status = run_cell(command(cell, port, args), log_path, args.no_progress_s)
        else:
            coord.publish(seq, {"cell": cell, "port": port, "name": name})
            mine = run_cell(command(cell, port, args), log_path, args.no_progress_s,
                            abort_check=lambda s=seq: coord.aborted(s))
            coord.report(seq, mine)
            status = overall_status(coord.gather(seq))
            seq += 1
        text = open(log_path).read()
        res = dict(cell, status=status)
        if cell["kind"] in ("attention", "selftest"):
            res.update({f"ms_per_batch_{k}": v for k, v in parse_microbenchmark(text, args.batches).items()})
        else:
            res["ms_per_iteration"] = parse_iteration_times(text)
        json.dump(res, open(done_path, "w"))
        rows.append(res)
        print(res, flush=True)
    if coord is not None:
        coord.publish(seq, None)               # end of the grid
        coord.wait_followers()                 # the key-value server lives in this process: leave last
    write_table(rows, os.path.join(args.out, "summary.csv"))


def follow(coord: NodeCoordinator, args) -> None:
    """Nodes other than 0: run this node's share of every published cell until the grid ends."""
    seq = 0
    while True:
        item = coord.fetch(seq)
        if item is None:
            coord.store.add("followers_done", 1)
            return
        log_path = os.path.join(args.out, f"{item['name']}.node{args.node_rank}.log")
        status = run_cell(command(item["cell"], item["port"], args), log_path, args.no_progress_s,
                          abort_check=lambda s=seq: coord.aborted(s))
        coord.report(seq, status)
        seq += 1


if __name__ == "__main__":
    main()

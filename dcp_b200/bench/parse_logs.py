"""Log parsers and result tables (benchmark/plotting/utils.py:10-31,
plot_microbenchmark_results.py:380-399); ``bench/plotting.py`` draws the figures from them.

* training logs: mean "elapsed time per iteration (ms)" skipping the first two log lines, and the
  "Training loss:" curve;
* microbenchmark logs: "<Name>: total time X ms" lines -> average ms per batch per framework.
"""
from __future__ import annotations

import csv
import json
import re
import sys
from typing import Dict, List, Optional

_ITER = re.compile(r"elapsed time per iteration \(ms\):\s*([0-9.]+)")
_LOSS = re.compile(r"Training loss:\s*([0-9.eE+-]+)")
_TOTAL = re.compile(r"^(\w+): total time ([0-9.]+) ms", re.M)


def parse_iteration_times(text: str, skip: int = 2) -> Optional[float]:
    vals = [float(m.group(1)) for m in _ITER.finditer(text)]
    vals = vals[skip:]
    return sum(vals) / len(vals) if vals else None


def parse_loss_curve(text: str) -> List[float]:
    return [float(m.group(1)) for m in _LOSS.finditer(text)]


def parse_microbenchmark(text: str, n_batches: int) -> Dict[str, float]:
    return {m.group(1): float(m.group(2)) / max(n_batches, 1) for m in _TOTAL.finditer(text)}


def losses_overlap(a: List[float], b: List[float], rel_tol: float = 0.02) -> bool:
    """Convergence-equivalence check between two runs' loss curves (the reference compares them by eye)."""
    n = min(len(a), len(b))
    return n > 0 and all(abs(x - y) <= rel_tol * max(abs(x), abs(y), 1e-9) for x, y in zip(a[:n], b[:n]))


def write_table(rows: List[dict], path: str) -> None:
    if path.endswith(".json"):
        json.dump(rows, open(path, "w"), indent=1)
        return
    keys = sorted({k for r in rows for k in r})
    with open(path, "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=keys)
        w.writeheader()
        w.writerows(rows)


if __name__ == "__main__":
    text = open(sys.argv[1]).read()
    print(json.dumps({"ms_per_iteration": parse_iteration_times(text), "losses": parse_loss_curve(text)[:5],
                      "microbenchmark": parse_microbenchmark(text, int(sys.argv[2]) if len(sys.argv) > 2 else 1)}))

"""Dataset preprocessing for benchmarks: sequence-length extraction, length scaling and packing
sequences into token-budget batches (the reference's benchmark/preprocessing/**:
get_longalign_variations.py:16-22 scales every length by 0.5/1/2/4, get_longalign_batches.py:5-41
packs <=131072-token batches into {"batches": [[len, ...], ...], "max_dp_degree": n}).

    python -m dcp_b200.bench.preprocessing --lengths lengths.json --scale 2.0 --budget 131072 --out batches.json
    python -m dcp_b200.bench.preprocessing --synthetic lognormal8k --n 2000 --out batches.json
"""
from __future__ import annotations

import argparse
import json
from typing import List, Sequence

import numpy as np

from ..data import synth


def scale_lengths(lengths: Sequence[int], scale: float, max_len: int = 131072, min_len: int = 16) -> List[int]:
    return [int(min(max(round(n * scale), min_len), max_len)) for n in lengths]


def pack_batches(lengths: Sequence[int], budget: int = 131072, min_fill: float = 0.0) -> List[List[int]]:
    """Greedy in-order packing; a sequence longer than the budget is truncated to it."""
    batches, cur, tok = [], [], 0
    for n in lengths:
        n = min(int(n), budget)
        if cur and tok + n > budget:
            if tok >= min_fill * budget:
                batches.append(cur)
            cur, tok = [], 0
        cur.append(n)
        tok += n
    if cur and tok >= min_fill * budget:
        batches.append(cur)
    return batches


def max_dp_degree(batches: Sequence[Sequence[int]]) -> int:
    """Largest data-parallel degree every batch supports (at least one sequence per replica)."""
    return min((len(b) for b in batches), default=1)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--lengths", help="json list of sequence lengths (e.g. token counts of a dataset)")
    ap.add_argument("--synthetic", choices=["lognormal8k", "lognormal16k", "mixture"])
    ap.add_argument("--n", type=int, default=1000)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--scale", type=float, default=1.0)
    ap.add_argument("--budget", type=int, default=131072)
    ap.add_argument("--out", required=True)
    args = ap.parse_args(argv)
    if args.lengths:
        lengths = json.load(open(args.lengths))
    else:
        dist = {"lognormal8k": synth.LOGNORMAL_8K, "lognormal16k": synth.LOGNORMAL_16K, "mixture": synth.MIXTURE}[
            args.synthetic or "lognormal8k"]
        rng = np.random.default_rng(args.seed)
        lengths = [synth._draw(rng, dist) for _ in range(args.n)]
    lengths = scale_lengths(lengths, args.scale, args.budget)
    batches = pack_batches(lengths, args.budget)
    json.dump({"batches": batches, "max_dp_degree": max_dp_degree(batches)}, open(args.out, "w"))
    print(f"{len(lengths)} sequences -> {len(batches)} batches, max_dp_degree {max_dp_degree(batches)}")


if __name__ == "__main__":
    main()

"""Seeded synthetic workloads: sequence-length distributions and token batches.

The length distributions are the ones the B200 benchmark configurations name (lognormal
heavy-tailed lengths clipped to a range, and a uniform/lognormal mixture), drawn until a token
budget is filled.  Token ids are uniform over the vocabulary; labels are the next token inside
each sequence.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np


@dataclass
class LengthDist:
    kind: str = "lognormal"           # "lognormal" | "mixture" | "fixed"
    median: float = 8192.0
    sigma: float = 1.0
    lo: int = 512
    hi: int = 131072
    # mixture: with probability p_uniform draw U[u_lo, u_hi], else lognormal(median, sigma) clipped to hi
    p_uniform: float = 0.7
    u_lo: int = 1024
    u_hi: int = 8192
    fixed: int = 8192


LOGNORMAL_8K = LengthDist("lognormal", 8192.0, 1.0, 512, 131072)
LOGNORMAL_16K = LengthDist("lognormal", 16384.0, 0.8, 4096, 131072)
MIXTURE = LengthDist("mixture", 65536.0, 0.5, 1024, 131072, 0.7, 1024, 8192)


def _draw(rng: np.random.Generator, dist: LengthDist) -> int:
    if dist.kind == "fixed":
        return int(dist.fixed)
    if dist.kind == "mixture" and rng.random() < dist.p_uniform:
        return int(rng.integers(dist.u_lo, dist.u_hi + 1))
    x = float(np.exp(np.log(dist.median) + dist.sigma * rng.standard_normal()))
    return int(min(max(x, dist.lo), dist.hi))


def sample_seqlens(token_budget: int, dist: LengthDist, seed: int, min_len: int = 16) -> List[int]:
    """Draw lengths until ``token_budget`` tokens are filled; the last draw is truncated to fit."""
    rng = np.random.default_rng(seed)
    out, left = [], int(token_budget)
    while left >= min_len:
        n = min(_draw(rng, dist), left)
        out.append(n)
        left -= n
    if left > 0 and out:
        out[-1] += left
    return out


def assign_mask_kinds(seqlens: Sequence[int], seed: int, kinds=("lambda", "chunked_first_chunk", "shared_question"),
                      params: Optional[Dict[str, dict]] = None) -> List[dict]:
    """Per-sequence structured-mask assignment (seeded), as ``mask_fn_info`` for ``mixed_mask_fn``."""
    default = {"lambda": {"n_starting": 64, "l_pretrain": 4096}, "chunked_first_chunk": {"chunk_size": 4096},
               "shared_question": {"question_tokens": 2048, "n_answers": 4}, "causal": {}}
    params = {**default, **(params or {})}
    rng = np.random.default_rng(seed + 7)
    return [{"kind": (k := kinds[int(rng.integers(len(kinds)))]), "params": params.get(k, {})} for _ in seqlens]


def make_token_batch(seqlens: Sequence[int], vocab: int, seed: int):
    """-> dict of int64 arrays over the packed batch: tokens, labels (-100 at sequence ends), positions."""
    rng = np.random.default_rng(seed + 13)
    total = int(sum(seqlens))
    tokens = rng.integers(0, vocab, size=total, dtype=np.int64)
    labels = np.empty(total, dtype=np.int64)
    positions = np.empty(total, dtype=np.int64)
    off = 0
    for n in seqlens:
        labels[off:off + n - 1] = tokens[off + 1:off + n]
        labels[off + n - 1] = -100
        positions[off:off + n] = np.arange(n)
        off += n
    return {"tokens": tokens, "labels": labels, "positions": positions}

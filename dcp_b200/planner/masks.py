"""Range-mask library: every query token may see up to two half-open key intervals.

A ``mask_fn(raw_seqlens, padded_seqlens, mask_dtype, mask_fn_info, **params)`` returns an int32
tensor over the padded packed batch, ``[sum(padded), 2]`` (one interval: start, end) or
``[sum(padded), 2, 2]`` (interval, bound), in per-sequence key coordinates; padding rows are
``[0, 0)``.  Same contract and the same built-in masks as
dcp/runtime/flash_attention/utils.py:501-683, computed with array arithmetic instead of
per-token loops, plus the parameterisations the B200 benchmark configurations name
(4096-token chunked causal-blockwise, 2048-token shared prefix).
"""
from __future__ import annotations

from typing import Callable, Dict, Optional, Sequence

import numpy as np
import torch


def _alloc(padded_seqlens: Sequence[int], two: bool) -> np.ndarray:
    shape = (int(sum(padded_seqlens)), 2, 2) if two else (int(sum(padded_seqlens)), 2)
    return np.zeros(shape, dtype=np.int64)


def _offsets(padded_seqlens: Sequence[int]) -> np.ndarray:
    return np.concatenate([[0], np.cumsum(np.asarray(padded_seqlens, dtype=np.int64))])


def _finish(a: np.ndarray, mask_dtype) -> torch.Tensor:
    return torch.from_numpy(a).to(mask_dtype if mask_dtype is not None else torch.int32)


def causal_range_mask_fn(raw_seqlens, padded_seqlens, mask_dtype=torch.int32, mask_fn_info=None):
    out, off = _alloc(padded_seqlens, False), _offsets(padded_seqlens)
    for s, n in enumerate(raw_seqlens):
        out[off[s]:off[s] + n, 1] = np.arange(1, n + 1)
    return _finish(out, mask_dtype)


def lambda_mask_fn(raw_seqlens, padded_seqlens, mask_dtype=torch.int32, mask_fn_info=None, n_starting: int = 64,
                   l_pretrain: int = 4096):
    """Attention sink of ``n_starting`` tokens plus a causal sliding window of ``l_pretrain``."""
    out, off = _alloc(padded_seqlens, True), _offsets(padded_seqlens)
    for s, n in enumerate(raw_seqlens):
        i = np.arange(n)
        v = out[off[s]:off[s] + n]
        v[:, 0, 1] = np.minimum(n_starting, i + 1)
        v[:, 1, 0] = np.maximum(0, i - l_pretrain + 1)
        v[:, 1, 1] = i + 1
    return _finish(out, mask_dtype)


def shared_question_mask_fn(raw_seqlens, padded_seqlens, mask_dtype=torch.int32, mask_fn_info=None,
                            question_proportion: float = 0.2, n_answers: int = 4,
                            question_tokens: Optional[int] = None):
    """A causal question prefix followed by ``n_answers`` answers that each see the whole question
    and themselves causally.  ``question_tokens`` fixes the prefix length (capped at the sequence)
    instead of taking a proportion of it."""
    out, off = _alloc(padded_seqlens, True), _offsets(padded_seqlens)
    for s, n in enumerate(raw_seqlens):
        nq = int(n * question_proportion) if question_tokens is None else min(int(question_tokens), n)
        per = max((n - nq) // n_answers, 1)
        i = np.arange(n)
        v = out[off[s]:off[s] + n]
        is_q = i < nq
        ans_idx = np.minimum((i - nq) // per, n_answers - 1)
        ans_start = nq + ans_idx * per
        v[:, 0, 0] = 0
        v[:, 0, 1] = np.where(is_q, i + 1, nq)
        v[:, 1, 0] = np.where(is_q, i + 1, ans_start)
        v[:, 1, 1] = i + 1
    return _finish(out, mask_dtype)


def causal_blockwise_mask_fn(raw_seqlens, padded_seqlens, mask_dtype=torch.int32, mask_fn_info=None,
                             block_size: int = 256, k_local: int = 2):
    """Chunked attention: first chunk causal; middle chunks see the first chunk and a window of
    ``k_local`` previous chunks; the last chunk sees everything before it."""
    out, off = _alloc(padded_seqlens, True), _offsets(padded_seqlens)
    for s, n in enumerate(raw_seqlens):
        i = np.arange(n)
        blk = i // block_size
        n_blocks = -(-n // block_size)
        first, last = blk == 0, (blk == n_blocks - 1) & (blk != 0)
        prev_end_last = (blk - 1) * block_size
        win_start = np.maximum(block_size, i - k_local * block_size)
        v = out[off[s]:off[s] + n]
        v[:, 0, 0] = 0
        v[:, 0, 1] = np.where(first, i + 1, np.where(last, prev_end_last, block_size))
        v[:, 1, 0] = np.where(first, i + 1, np.where(last, prev_end_last, win_start))
        v[:, 1, 1] = i + 1
    return _finish(out, mask_dtype)


def chunked_first_chunk_mask_fn(raw_seqlens, padded_seqlens, mask_dtype=torch.int32, mask_fn_info=None,
                                chunk_size: int = 4096):
    """Each ``chunk_size`` chunk attends causally to itself and fully to the first chunk."""
    out, off = _alloc(padded_seqlens, True), _offsets(padded_seqlens)
    for s, n in enumerate(raw_seqlens):
        i = np.arange(n)
        chunk_start = (i // chunk_size) * chunk_size
        first = chunk_start == 0
        v = out[off[s]:off[s] + n]
        v[:, 0, 0] = 0
        v[:, 0, 1] = np.where(first, i + 1, min(chunk_size, n))
        v[:, 1, 0] = np.where(first, i + 1, chunk_start)
        v[:, 1, 1] = i + 1
    return _finish(out, mask_dtype)


def modality_specific_mask_fn(raw_seqlens, padded_seqlens, mask_dtype=torch.int32, mask_fn_info=None,
                              limit_image_attn_to_self: bool = False):
    """Text tokens are causal; image tokens are bidirectional inside their image (and, unless
    ``limit_image_attn_to_self``, also see everything before it).  ``mask_fn_info[s]`` carries
    ``image_size`` and ``text_lengths`` (an image sits between consecutive text spans)."""
    assert mask_fn_info is not None and len(mask_fn_info) == len(raw_seqlens)
    out, off = _alloc(padded_seqlens, False), _offsets(padded_seqlens)
    for s, n in enumerate(raw_seqlens):
        info = mask_fn_info[s]
        image_size, text_lengths = int(info["image_size"]), list(info["text_lengths"])
        cur = 0
        v = out[off[s]:off[s] + n]
        for idx, t_len in enumerate(text_lengths):
            v[cur:cur + t_len, 0] = 0
            v[cur:cur + t_len, 1] = np.arange(cur + 1, cur + t_len + 1)
            cur += t_len
            if idx < len(text_lengths) - 1:
                v[cur:cur + image_size, 0] = cur if limit_image_attn_to_self else 0
                v[cur:cur + image_size, 1] = cur + image_size
                cur += image_size
    return _finish(out, mask_dtype)


def modality_specific_sparse_mask_fn(raw_seqlens, padded_seqlens, mask_dtype=torch.int32, mask_fn_info=None):
    return modality_specific_mask_fn(raw_seqlens, padded_seqlens, mask_dtype, mask_fn_info, True)


def mixed_mask_fn(raw_seqlens, padded_seqlens, mask_dtype=torch.int32, mask_fn_info=None):
    """Per-sequence mask kind taken from ``mask_fn_info[s]['kind']`` (and optional ``params``)."""
    assert mask_fn_info is not None
    out, off = _alloc(padded_seqlens, True), _offsets(padded_seqlens)
    for s, (n, p) in enumerate(zip(raw_seqlens, padded_seqlens)):
        info = mask_fn_info[s]
        fn = MASK_FNS[info["kind"]]
        m = fn([n], [p], torch.int64, [info], **info.get("params", {})).numpy()
        out[off[s]:off[s] + p] = to_two_range(m)
    return _finish(out, mask_dtype)


MASK_FNS: Dict[str, Callable] = {
    "causal": causal_range_mask_fn,
    "lambda": lambda_mask_fn,
    "shared_question": shared_question_mask_fn,
    "causal_blockwise": causal_blockwise_mask_fn,
    "chunked_first_chunk": chunked_first_chunk_mask_fn,
    "modality_specific": modality_specific_mask_fn,
    "modality_specific_sparse": modality_specific_sparse_mask_fn,
    "mixed": mixed_mask_fn,
}


def get_mask_fn(name: str) -> Callable:
    if name not in MASK_FNS:
        raise KeyError(f"unknown mask type {name!r}; known: {sorted(MASK_FNS)}")
    return MASK_FNS[name]


def to_two_range(mask) -> np.ndarray:
    """[T,2] or [T,2,2] -> int64 [T,2,2]; a single interval gets an empty second one."""
    m = mask.numpy() if isinstance(mask, torch.Tensor) else np.asarray(mask)
    m = m.astype(np.int64)
    if m.ndim == 2:
        out = np.zeros((m.shape[0], 2, 2), dtype=np.int64)
        out[:, 0] = m
        return out
    return m


def to_flat4(mask) -> np.ndarray:
    """-> int32 [T, 4] = (s0, e0, s1, e1) with ends clamped to be >= starts."""
    m = to_two_range(mask).reshape(-1, 4).copy()
    m[:, 1] = np.maximum(m[:, 1], m[:, 0])
    m[:, 3] = np.maximum(m[:, 3], m[:, 2])
    return m.astype(np.int32)


def dense_from_ranges(mask, n_q: int, n_k: int) -> torch.Tensor:
    """Boolean [n_q, n_k] from the first ``n_q`` rows of a range mask (testing helper)."""
    m = torch.from_numpy(to_two_range(mask)[:n_q])
    pos = torch.arange(n_k)[None, :]
    return ((pos >= m[:, 0, 0:1]) & (pos < m[:, 0, 1:2])) | ((pos >= m[:, 1, 0:1]) & (pos < m[:, 1, 1:2]))

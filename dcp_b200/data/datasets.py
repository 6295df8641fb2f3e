"""Datasets and the token-budget batch sampler.

``OrderedBatchSampler`` packs whole sequences into batches of at most ``batch_size_in_tokens``
tokens, dropping batches filled below 75 % (dcp/data/hf_dataset.py:440-484) and, unlike the
reference, can resume from ``consumed_samples``.  ``HuggingFaceDataset`` tokenises a text dataset
when the optional ``datasets`` / tokenizer packages are present; the synthetic datasets need
nothing beyond NumPy.  Samples are dicts with ``tokens, labels, loss_mask, position_ids`` like the
reference's (dcp/data/hf_dataset.py:249-312).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, Iterator, List, Optional

import numpy as np
import torch
from torch.utils.data import Dataset, Sampler

from . import synth


def _sample_from_tokens(tok: np.ndarray) -> Dict[str, torch.Tensor]:
    tok = np.asarray(tok, dtype=np.int64)
    n = len(tok) - 1
    return {"tokens": torch.from_numpy(tok[:-1].copy()), "labels": torch.from_numpy(tok[1:].copy()),
            "loss_mask": torch.ones(n, dtype=torch.float32), "position_ids": torch.arange(n, dtype=torch.int64)}


class SyntheticLengthDataset(Dataset):
    """Random token sequences whose lengths follow a ``synth.LengthDist`` (seeded per index)."""

    def __init__(self, n_samples: int, dist: synth.LengthDist, vocab: int = 32000, seed: int = 0):
        self.n, self.dist, self.vocab, self.seed = n_samples, dist, vocab, seed
        rng = np.random.default_rng(seed)
        self.seqlens = [synth._draw(rng, dist) for _ in range(n_samples)]

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        rng = np.random.default_rng(self.seed * 7919 + i)
        return _sample_from_tokens(rng.integers(0, self.vocab, size=self.seqlens[i] + 1))


class MockGPTLowLevelDataset(Dataset):
    """Fixed-length random documents (the mock dataset of dcp/data/hf_dataset.py:487-520)."""

    def __init__(self, n_samples: int = 1024, seq_len: int = 2048, vocab: int = 32000, seed: int = 0):
        self.n, self.seq_len, self.vocab, self.seed = n_samples, seq_len, vocab, seed
        self.seqlens = [seq_len] * n_samples

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        rng = np.random.default_rng(self.seed + i)
        return _sample_from_tokens(rng.integers(0, self.vocab, size=self.seq_len + 1))


class DummyMultiModelDataset(Dataset):
    """Interleaved text / image token layouts for the modality-specific masks
    (dcp/data/hf_dataset.py:341-437): each sample is text, image, text, ..., text and carries the
    ``image_size`` / ``text_lengths`` the mask function needs."""

    def __init__(self, n_samples: int = 256, image_size: int = 576, max_images: int = 4, mean_text: int = 512,
                 vocab: int = 32000, seed: int = 0):
        self.n, self.image_size, self.vocab, self.seed = n_samples, image_size, vocab, seed
        rng = np.random.default_rng(seed)
        self.layouts = []
        for _ in range(n_samples):
            n_img = int(rng.integers(1, max_images + 1))
            texts = [int(max(8, rng.exponential(mean_text))) for _ in range(n_img + 1)]
            self.layouts.append(texts)
        self.seqlens = [sum(t) + (len(t) - 1) * image_size for t in self.layouts]

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        rng = np.random.default_rng(self.seed * 31 + i)
        s = _sample_from_tokens(rng.integers(0, self.vocab, size=self.seqlens[i] + 1))
        s["mask_fn_info"] = {"image_size": self.image_size, "text_lengths": list(self.layouts[i])}
        return s


@dataclass
class HuggingFaceDatasetConfig:
    dataset_name: str = ""           # a `datasets` name / local path, or "" when `texts` are passed directly
    tokenizer_name: str = ""         # a `transformers` tokenizer name / path, or "bytes" for the built-in byte tokenizer
    split: str = "train"
    text_key: str = "text"
    max_seq_len: int = 131072
    min_seq_len: int = 16
    cache_dir: Optional[str] = None  # tokenised samples are cached here (one .npz per configuration)
    seqlen_scale: float = 1.0        # the benchmark's x0.5 / x2 / x4 length scaling


def byte_tokenizer(text: str) -> List[int]:
    """UTF-8 bytes + 1 with 0 as the begin-of-text id: a dependency-free tokenizer (vocabulary 257)."""
    return [0] + [b + 1 for b in text.encode("utf-8")]


class HuggingFaceDataset(Dataset):
    """Text dataset, tokenised once and cached (dcp/data/hf_dataset.py:24-312).

    Sources: a ``datasets`` dataset (optional package, local copy: there is no network in the build
    image) or an in-memory list of ``texts``; tokenizer: a ``transformers`` tokenizer, a callable
    text -> ids, or the built-in byte tokenizer.  Tokenisation, length scaling and the length
    filter run once; the result is written to ``cache_dir`` as one ``.npz`` keyed by everything
    that determines it and loaded from there afterwards.  Under ``torch.distributed`` the first
    rank of every node (``LOCAL_RANK`` 0; with ``DCP_DATASET_INIT_WITH_GLOBAL_RANK=1`` only global
    rank 0, for a cache directory all nodes share) builds the cache while the other ranks wait at a
    barrier, then they load it (the reference's rank-0-first protocol, hf_dataset.py:118-135,174-247)."""

    def __init__(self, config: HuggingFaceDatasetConfig, texts: Optional[List[str]] = None, tokenizer=None):
        self.config = config
        self.built_from_cache = False
        path = self._cache_path(texts)
        rank0, distributed = True, False
        try:
            import torch.distributed as dist
            distributed = dist.is_available() and dist.is_initialized()
            if distributed:
                by_global = os.environ.get("DCP_DATASET_INIT_WITH_GLOBAL_RANK", "0") not in ("0", "", "false", "False")
                rank0 = dist.get_rank() == 0 if by_global or "LOCAL_RANK" not in os.environ \
                    else int(os.environ["LOCAL_RANK"]) == 0
        except Exception:  # pragma: no cover - torch without distributed support
            pass
        if path is not None and not rank0:
            dist.barrier()                      # rank 0 is tokenising
        if path is not None and os.path.exists(path):
            data = np.load(path)
            flat, cu = data["tokens"], data["offsets"]
            self.ids = [flat[cu[i]:cu[i + 1]] for i in range(len(cu) - 1)]
            self.built_from_cache = True
        else:
            self.ids = self._tokenise(texts, tokenizer)
            if path is not None and rank0:
                os.makedirs(os.path.dirname(path), exist_ok=True)
                cu = np.zeros(len(self.ids) + 1, dtype=np.int64)
                np.cumsum([len(t) for t in self.ids], out=cu[1:])
                tmp = f"{path}.{os.getpid()}.tmp.npz"
                np.savez(tmp, tokens=np.concatenate(self.ids) if self.ids else np.zeros(0, np.int64), offsets=cu)
                os.replace(tmp, path)           # atomic: readers never see a partial file
        if path is not None and rank0 and distributed:
            dist.barrier()                      # the cache is complete: let the other ranks load it
        self.seqlens = [len(t) - 1 for t in self.ids]

    def _cache_path(self, texts) -> Optional[str]:
        c = self.config
        if not c.cache_dir:
            return None
        import hashlib
        key = repr((c.dataset_name, c.tokenizer_name, c.split, c.text_key, c.max_seq_len, c.min_seq_len, c.seqlen_scale,
                    None if texts is None else hashlib.sha1("\x00".join(texts).encode()).hexdigest()))
        return os.path.join(c.cache_dir, "tokenised_" + hashlib.sha1(key.encode()).hexdigest()[:16] + ".npz")

    def _tokenise(self, texts, tokenizer) -> List[np.ndarray]:
        c = self.config
        if tokenizer is None:
            if c.tokenizer_name in ("", "bytes"):
                tokenizer = byte_tokenizer
            else:
                try:
                    from transformers import AutoTokenizer
                except ImportError as e:  # pragma: no cover - optional dependency
                    raise ImportError("a named tokenizer needs the `transformers` package") from e
                tok = AutoTokenizer.from_pretrained(c.tokenizer_name)
                tokenizer = lambda text: tok(text, add_special_tokens=True)["input_ids"]
        if texts is None:
            try:
                import datasets as hf
            except ImportError as e:  # pragma: no cover - optional dependency
                raise ImportError("loading a named dataset needs the `datasets` package") from e
            texts = (row[c.text_key] for row in hf.load_dataset(c.dataset_name, split=c.split, cache_dir=c.cache_dir))
        ids = []
        for text in texts:
            t = list(tokenizer(text))
            if c.seqlen_scale != 1.0:
                reps = int(np.ceil(c.seqlen_scale))
                t = (t * reps)[:max(2, int(len(t) * c.seqlen_scale))]
            t = t[:c.max_seq_len + 1]
            if len(t) - 1 >= c.min_seq_len:
                ids.append(np.asarray(t, dtype=np.int64))
        return ids

    def __len__(self):
        return len(self.ids)

    def __getitem__(self, i):
        return _sample_from_tokens(self.ids[i])


class OrderedBatchSampler(Sampler):
    """Yields lists of sample indices whose lengths sum to at most ``batch_size_in_tokens``."""

    def __init__(self, dataset, batch_size_in_tokens: int, shuffle: bool = True, seed: int = 24,
                 min_fill: float = 0.75, consumed_samples: int = 0):
        self.seqlens = list(dataset.seqlens)
        self.budget = int(batch_size_in_tokens)
        self.shuffle, self.seed, self.min_fill = shuffle, seed, min_fill
        self.consumed_samples = consumed_samples
        self.epoch = 0

    def _order(self) -> List[int]:
        idx = list(range(len(self.seqlens)))
        if self.shuffle:
            rng = np.random.default_rng(self.seed + self.epoch)
            idx = rng.permutation(len(idx)).tolist()
        return idx

    def _batches(self) -> List[List[int]]:
        batches, cur, tok = [], [], 0
        for i in self._order():
            n = min(self.seqlens[i], self.budget)
            if cur and tok + n > self.budget:
                if tok >= self.min_fill * self.budget:
                    batches.append(cur)
                cur, tok = [], 0
            cur.append(i)
            tok += n
        if cur and tok >= self.min_fill * self.budget:
            batches.append(cur)
        return batches

    def __iter__(self) -> Iterator[List[int]]:
        seen = 0
        for b in self._batches():
            if seen >= self.consumed_samples:
                self.consumed_samples += len(b)
                yield b
            seen += len(b)
        self.epoch += 1
        self.consumed_samples = 0

    def __len__(self) -> int:
        return len(self._batches())

    def state_dict(self) -> dict:
        return {"consumed_samples": self.consumed_samples, "epoch": self.epoch, "seed": self.seed}

    def load_state_dict(self, sd: dict) -> None:
        self.consumed_samples, self.epoch, self.seed = sd["consumed_samples"], sd["epoch"], sd["seed"]

"""Datasets and the token-budget batch sampler.

``OrderedBatchSampler`` packs whole sequences into batches of at most ``batch_size_in_tokens``
tokens, dropping batches filled below 75 % (dcp/data/hf_dataset.py:440-484) and, unlike the
reference, can resume from ``consumed_samples``.  ``HuggingFaceDataset`` tokenises a text dataset
when the optional ``datasets`` / tokenizer packages are present; the synthetic datasets need
nothing beyond NumPy.  Samples are dicts with ``tokens, labels, loss_mask, position_ids`` like the
reference's (dcp/data/hf_dataset.py:249-312).
"""
from __future__ import annotations

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
    dataset_name: str = ""
    tokenizer_name: str = ""
    split: str = "train"
    text_key: str = "text"
    max_seq_len: int = 131072
    min_seq_len: int = 16
    cache_dir: Optional[str] = None
    seqlen_scale: float = 1.0        # the benchmark's x0.5 / x2 / x4 length scaling


class HuggingFaceDataset(Dataset):
    """Text dataset tokenised on first use.  Needs the optional ``datasets`` and ``transformers``
    packages and local copies of the data (there is no network in the build image)."""

    def __init__(self, config: HuggingFaceDatasetConfig):
        try:
            import datasets  # noqa: F401
            from transformers import AutoTokenizer
        except ImportError as e:  # pragma: no cover - optional dependency
            raise ImportError("HuggingFaceDataset needs the `datasets` and `transformers` packages") from e
        import datasets as hf
        self.config = config
        tok = AutoTokenizer.from_pretrained(config.tokenizer_name)
        ds = hf.load_dataset(config.dataset_name, split=config.split, cache_dir=config.cache_dir)
        ids = []
        for row in ds:
            t = tok(row[config.text_key], add_special_tokens=True)["input_ids"]
            if config.seqlen_scale != 1.0:
                reps = int(np.ceil(config.seqlen_scale))
                t = (t * reps)[:max(2, int(len(t) * config.seqlen_scale))]
            t = t[:config.max_seq_len + 1]
            if len(t) - 1 >= config.min_seq_len:
                ids.append(np.asarray(t, dtype=np.int64))
        self.ids = ids
        self.seqlens = [len(t) - 1 for t in ids]

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

"""Sample construction over document datasets (reference: mintext/data/dataset.py).

``DocumentDataSource`` takes one split of the documents, shuffles them per epoch, lays them end to end and cuts
consecutive samples of ``seq_len (+1)`` tokens; the (document position, offset) of every cut is the *sample
index*, cached on disk under an md5 of the build parameters.  ``BlendedDataSource`` interleaves several sources
so that the running share of each tracks its weight.  The index builders run in C++ when the native runtime is
available and in NumPy otherwise; both produce identical arrays.
"""

from __future__ import annotations

import hashlib
import json
import logging
from pathlib import Path

import numpy as np

from .indexed_dataset import ArrayRecordDocDataset, MMapIndexedDataset

logger = logging.getLogger(__name__)


def _native():
    from mintext_b200.ops._ext import io_ext

    return io_ext()


def _build_document_index(num_documents: int, num_epochs: int, rng: np.random.RandomState) -> np.ndarray:
    """One independent permutation of the documents per epoch, concatenated (int32)."""
    epochs = []
    for _ in range(num_epochs):
        order = np.arange(num_documents, dtype=np.int32)
        rng.shuffle(order)
        epochs.append(order)
    return np.concatenate(epochs) if epochs else np.zeros(0, dtype=np.int32)


def _build_sample_index_numpy(document_index, doc_lengths, seq_len: int, add_extra_token: bool = True) -> np.ndarray:
    target = seq_len + int(add_extra_token)
    rows = [(0, 0)]
    pos, offset, remaining = 0, 0, target
    n = len(document_index)
    while pos < n:
        dlen = int(doc_lengths[int(document_index[pos])])
        avail = dlen - offset
        if avail <= 0:
            pos, offset = pos + 1, 0
        elif avail >= remaining:
            offset += remaining
            rows.append((pos, offset))
            remaining = target
            if offset >= dlen:
                pos, offset = pos + 1, 0
        else:
            remaining -= avail
            pos, offset = pos + 1, 0
    return np.asarray(rows, dtype=np.int64)


def _build_sample_index(document_index, doc_lengths, seq_len: int, add_extra_token: bool = True) -> np.ndarray:
    """``[num_samples + 1, 2]`` int64 rows of (position in document_index, offset in that document)."""
    nat = _native()
    if nat is not None and len(document_index) > 0:
        import torch

        out = nat.build_sample_index(torch.from_numpy(np.ascontiguousarray(doc_lengths).astype(np.int64)),
                                     torch.from_numpy(np.ascontiguousarray(document_index).astype(np.int64)),
                                     int(seq_len), bool(add_extra_token))
        return out.numpy()
    return _build_sample_index_numpy(document_index, doc_lengths, seq_len, add_extra_token)


class DocumentDataSource:
    """Random-access source of ``{"tokens": int array of seq_len + add_extra_token}`` samples."""

    def __init__(self, data_path: str, data_type: str, seq_len: int, seed: int, num_epochs: int,
                 split: tuple[float, float, float], split_index: int, cache_dir: str | None = None,
                 add_extra_token: bool = True) -> None:
        self._seq_len = seq_len
        self._seed = seed
        self._add_extra_token = add_extra_token
        if data_type == "mmap":
            self._backend = MMapIndexedDataset(data_path)
        elif data_type == "arecord":
            self._backend = ArrayRecordDocDataset(data_path)
        else:
            raise ValueError(f"Unknown data_type: {data_type}")
        all_lengths = self._backend.doc_lengths
        total_docs = len(all_lengths)
        fracs = [s / sum(split) for s in split]
        bounds = [0]
        for f in fracs:
            bounds.append(bounds[-1] + int(round(f * total_docs)))
        bounds[-1] = total_docs
        lo, hi = bounds[split_index], bounds[split_index + 1]
        self._doc_ids = np.arange(lo, hi, dtype=np.int32)
        self._split_doc_lengths = all_lengths[lo:hi]
        self._document_index = np.zeros(0, dtype=np.int32)
        if len(self._doc_ids) == 0:
            self._sample_index = np.zeros((1, 2), dtype=np.int64)
            return
        if cache_dir:
            cache = Path(cache_dir)
        else:
            cache = Path(data_path if Path(data_path).is_dir() else Path(data_path).parent) / "cache"
        self._document_index, self._sample_index = self._load_or_build_indices(
            data_path, seq_len, seed, num_epochs, (lo, hi), cache, add_extra_token)

    def __len__(self) -> int:
        return max(0, len(self._sample_index) - 1)

    def __getitem__(self, idx: int) -> dict[str, np.ndarray]:
        target = self._seq_len + int(self._add_extra_token)
        pos, offset = (int(v) for v in self._sample_index[idx])
        parts, remaining = [], target
        while remaining > 0 and pos < len(self._document_index):
            doc = int(self._document_index[pos])
            avail = int(self._split_doc_lengths[doc]) - offset
            if avail <= 0:
                pos, offset = pos + 1, 0
                continue
            take = min(avail, remaining)
            parts.append(self._backend.get(int(self._doc_ids[doc]), offset=offset, length=take))
            remaining -= take
            if take >= avail:
                pos, offset = pos + 1, 0
            else:
                offset += take
        tokens = np.concatenate(parts) if parts else np.zeros(0, dtype=np.int32)
        if len(tokens) < target:
            tokens = np.pad(tokens, (0, target - len(tokens)), constant_values=0)
        return {"tokens": tokens[:target]}

    def _load_or_build_indices(self, data_path, seq_len, seed, num_epochs, split, cache_dir: Path,
                               add_extra_token: bool = True):
        key = json.dumps({"add_extra_token": add_extra_token, "dataset_path": data_path, "sequence_length": seq_len,
                          "random_seed": seed, "split": f"{split[0]}:{split[1]}", "num_epochs": num_epochs},
                         indent=4, sort_keys=True)
        digest = hashlib.md5(key.encode()).hexdigest()
        cache_dir.mkdir(parents=True, exist_ok=True)
        doc_path = cache_dir / f"{digest}-document_index.npy"
        smp_path = cache_dir / f"{digest}-sample_index.npy"
        if doc_path.exists() and smp_path.exists():
            logger.info("Loading cached indices from %s", cache_dir)
            return np.load(doc_path), np.load(smp_path)
        logger.info("Building indices (seq_len=%d, epochs=%d, docs=%d)...", seq_len, num_epochs, len(self._doc_ids))
        rng = np.random.RandomState(seed)
        document_index = _build_document_index(len(self._doc_ids), num_epochs, rng)
        sample_index = _build_sample_index(document_index, self._split_doc_lengths, seq_len, add_extra_token)
        np.save(doc_path, document_index)
        np.save(smp_path, sample_index)
        logger.info("Built %d samples, cached to %s", len(sample_index) - 1, cache_dir)
        return document_index, sample_index


class BlendedDataSource:
    """Weighted interleave of sources (greedy by deficit; lowest index wins ties)."""

    def __init__(self, sources: list, weights: list[float], size: int) -> None:
        if len(sources) != len(weights):
            raise ValueError("sources and weights must have same length")
        if not sources:
            raise ValueError("Must provide at least one source")
        self._sources = sources
        self._size = size
        lens = [len(s) for s in sources]
        nat = _native()
        if nat is not None:
            import torch

            ds, si = nat.build_blend_index(torch.tensor(weights, dtype=torch.float64),
                                           torch.tensor(lens, dtype=torch.int64), int(size))
            self._dataset_index, self._dataset_sample_index = ds.numpy(), si.numpy()
        else:
            total = float(sum(weights))
            w = [x / total for x in weights]
            self._dataset_index = np.zeros(size, dtype=np.int32)
            self._dataset_sample_index = np.zeros(size, dtype=np.int64)
            counts = [0] * len(sources)
            for i in range(size):
                errs = [w[k] * (i + 1) - counts[k] for k in range(len(sources))]
                best = int(np.argmax(errs))
                self._dataset_index[i] = best
                self._dataset_sample_index[i] = counts[best] % lens[best] if lens[best] else 0
                counts[best] += 1

    def __len__(self) -> int:
        return self._size

    def __getitem__(self, idx: int) -> dict[str, np.ndarray]:
        return self._sources[int(self._dataset_index[idx])][int(self._dataset_sample_index[idx])]

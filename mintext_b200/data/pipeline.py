"""Training / evaluation iterators over tokenised data (reference: mintext/data/pipeline.py, built on Grain).

The loader here is self-contained: a seeded per-epoch permutation of the sample ids, sharded round-robin over
the data-parallel ranks, ``ShiftTokens``, fixed-size batches (remainder dropped) and a pool of prefetch threads
filling a bounded queue (``grain_worker_count`` threads, ``grain_prefetch_buffer_size`` samples).  The iterator
is infinite and *resumable*: ``state_dict()`` / ``load_state_dict()`` carry the number of batches produced, so a
restarted run continues with the very next batch.
"""

from __future__ import annotations

import logging
import queue
import threading
from pathlib import Path
from typing import Iterator

import numpy as np

from .dataset import BlendedDataSource, DocumentDataSource

logger = logging.getLogger(__name__)


def _parse_data_path(data_path: str) -> list[tuple[float, str]]:
    """``"w1 p1 w2 p2 ..."`` -> weighted entries; a single token (or a string that does not start with a number)
    is one path of weight 1."""
    parts = data_path.strip().split()
    if len(parts) == 1:
        return [(1.0, parts[0])]
    entries: list[tuple[float, str]] = []
    i = 0
    while i < len(parts):
        try:
            w = float(parts[i])
        except ValueError:
            if not entries:
                return [(1.0, data_path.strip())]
            raise
        if i + 1 >= len(parts):
            raise ValueError(f"Weight {w} at position {i} has no path")
        entries.append((w, parts[i + 1]))
        i += 2
    return entries


def _detect_data_type(path: str) -> str:
    p = Path(path)
    if Path(f"{path}.idx").exists() and (Path(f"{path}.bin").exists() or Path(f"{path}.bin.00000").exists()):
        return "mmap"
    if p.is_dir():
        if list(p.glob("*.arecord")):
            return "arecord"
    elif p.suffix == ".arecord":
        return "arecord"
    raise ValueError(f"Cannot detect data type for '{path}'. Expected .bin+.idx files or .arecord files/directory.")


def _parse_split(split_str: str) -> tuple[float, float, float]:
    parts = [float(x) for x in split_str.split(",")]
    if len(parts) != 3:
        raise ValueError(f"data_split must have 3 values, got: {split_str}")
    return parts[0], parts[1], parts[2]


class ShiftTokens:
    """``tokens`` -> ``input_tokens`` / ``target_tokens``: with the extra token the two are the length-``seq_len``
    prefixes shifted by one; without it the target is the input rolled left by one."""

    def __init__(self, add_extra_token: bool = True):
        self._add_extra_token = add_extra_token

    def map(self, element: dict[str, np.ndarray]) -> dict[str, np.ndarray]:
        t = element["tokens"]
        if self._add_extra_token:
            return {"input_tokens": t[:-1], "target_tokens": t[1:]}
        return {"input_tokens": t, "target_tokens": np.roll(t, -1)}

    __call__ = map


class BatchIterator:
    """Infinite iterator of ``{"input_tokens", "target_tokens"}`` int32 arrays ``[batch, seq]`` for one rank."""

    def __init__(self, source, batch_size: int, seed: int, shuffle: bool, rank: int = 0, world: int = 1,
                 add_extra_token: bool = True, workers: int = 0, buffer_size: int = 64):
        if len(source) < world * batch_size:
            raise ValueError(f"data source has {len(source)} samples, fewer than one global batch "
                             f"({world} x {batch_size})")
        self.source, self.batch_size, self.seed, self.shuffle = source, batch_size, seed, shuffle
        self.rank, self.world = rank, world
        self.shift = ShiftTokens(add_extra_token)
        self.batches_done = 0
        self.workers = workers
        self.buffer_size = max(buffer_size // max(batch_size, 1), 2)
        self._q: queue.Queue | None = None
        self._threads: list[threading.Thread] = []
        self._stop = threading.Event()
        self._perm_cache: dict[int, np.ndarray] = {}
        self._perm_lock = threading.Lock()

    # position -> sample id ------------------------------------------------------------
    def _epoch_perm(self, epoch: int) -> np.ndarray:
        """Sample order of one epoch.  Prefetch workers straddle an epoch boundary, so the two most recent epochs
        stay cached and the array itself is returned under the lock (never looked up again after an eviction)."""
        with self._perm_lock:
            ids = self._perm_cache.get(epoch)
            if ids is None:
                ids = np.arange(len(self.source))
                if self.shuffle:
                    np.random.RandomState((self.seed + 1000003 * epoch) % (2 ** 31)).shuffle(ids)
                keep = {e: v for e, v in self._perm_cache.items() if abs(e - epoch) <= 1}
                keep[epoch] = ids
                self._perm_cache = keep
            return ids

    def _sample_ids(self, batch_index: int) -> list[int]:
        per_epoch = (len(self.source) // (self.world * self.batch_size)) * self.world * self.batch_size
        out = []
        for j in range(self.batch_size):
            g = (batch_index * self.batch_size + j) * self.world + self.rank
            epoch, within = divmod(g, per_epoch)
            out.append(int(self._epoch_perm(epoch)[within]))
        return out

    def _make_batch(self, batch_index: int) -> dict[str, np.ndarray]:
        rows = [self.shift(self.source[i]) for i in self._sample_ids(batch_index)]
        return {k: np.stack([r[k] for r in rows]).astype(np.int32) for k in rows[0]}

    # prefetch ----------------------------------------------------------------------------
    def _start(self) -> None:
        self._q = queue.Queue(maxsize=self.buffer_size)
        self._stop.clear()
        self._next_to_schedule = self.batches_done
        self._pending: dict[int, dict] = {}
        self._lock = threading.Lock()

        def work():
            while not self._stop.is_set():
                with self._lock:
                    b = self._next_to_schedule
                    self._next_to_schedule += 1
                try:
                    batch = self._make_batch(b)
                except BaseException as exc:  # handed to the consumer: a dead worker must not become a silent hang
                    batch = exc
                while not self._stop.is_set():
                    try:
                        self._q.put((b, batch), timeout=0.1)
                        break
                    except queue.Full:
                        continue

        self._threads = [threading.Thread(target=work, daemon=True) for _ in range(self.workers)]
        for t in self._threads:
            t.start()

    def close(self) -> None:
        self._stop.set()
        for t in self._threads:
            t.join(timeout=1)
        self._threads, self._q = [], None

    def __iter__(self) -> Iterator[dict[str, np.ndarray]]:
        return self

    def __next__(self) -> dict[str, np.ndarray]:
        if self.workers <= 0:
            batch = self._make_batch(self.batches_done)
        else:
            if self._q is None:
                self._start()
            want = self.batches_done
            while want not in self._pending:
                try:
                    b, data = self._q.get(timeout=1.0)
                except queue.Empty:
                    if not any(t.is_alive() for t in self._threads):
                        raise RuntimeError(f"data workers exited before producing batch {want}")
                    continue
                self._pending[b] = data
            batch = self._pending.pop(want)
            if isinstance(batch, BaseException):
                self.close()
                raise RuntimeError(f"data worker failed while building batch {want}") from batch
        self.batches_done += 1
        return batch

    # resume -------------------------------------------------------------------------------
    def state_dict(self) -> dict:
        return {"batches_done": self.batches_done, "seed": self.seed}

    def load_state_dict(self, state: dict) -> None:
        self.close()
        self.batches_done = int(state["batches_done"])


def _create_iterator(config, mesh, split_index: int, shuffle: bool) -> BatchIterator:
    split = _parse_split(config.data_split)
    sources, weights = [], []
    for weight, path in _parse_data_path(config.data_path):
        dtype = _detect_data_type(path) if config.dataset_type == "auto" else config.dataset_type
        sources.append(DocumentDataSource(
            data_path=path, data_type=dtype, seq_len=config.seq_length, seed=config.seed,
            num_epochs=config.num_data_epochs, split=split, split_index=split_index,
            cache_dir=config.data_cache_dir or None, add_extra_token=config.add_extra_token))
        weights.append(weight)
    source = sources[0] if len(sources) == 1 else BlendedDataSource(sources, weights, sum(len(s) for s in sources))
    logger.info("Data source: %d samples, %d source(s), split_index=%d", len(source), len(sources), split_index)
    rank, world = 0, 1
    try:
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized():
            world = dist.get_world_size()
            rank = dist.get_rank()
            if mesh is not None:
                rank, world = mesh.batch_rank(rank)  # tensor-parallel peers read the same rows
    except Exception:
        pass
    batch = config.per_device_batch_size * config.gradient_accumulation_steps
    return BatchIterator(source, batch, config.seed, shuffle, rank, world, config.add_extra_token,
                         workers=config.grain_worker_count, buffer_size=config.grain_prefetch_buffer_size)


def create_train_iterator(config, mesh=None) -> BatchIterator:
    """Shuffled, infinite iterator over split 0."""
    return _create_iterator(config, mesh, split_index=0, shuffle=True)


def create_eval_iterator(config, mesh=None) -> BatchIterator:
    """Unshuffled iterator over split 1."""
    return _create_iterator(config, mesh, split_index=1, shuffle=False)

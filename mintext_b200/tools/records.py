"""Sharded per-document record output shared by the converters: ``shard-XXXXX-of-YYYYY.arecord`` files (size
capped) plus ``doc_lengths.npy``.  Uses Google's ``array_record`` writer when it is installed, else this package's
record container (both are read back by ``ArrayRecordDocDataset``)."""

from __future__ import annotations

from pathlib import Path

import numpy as np

from mintext_b200.data.indexed_dataset import RecordFileWriter


def _open_writer(path: str):
    try:
        from array_record.python.array_record_module import ArrayRecordWriter  # type: ignore

        return ArrayRecordWriter(path, "group_size:1")
    except ImportError:
        return RecordFileWriter(path)


class ShardedRecordWriter:
    def __init__(self, out_dir: str, max_shard_bytes: int, dtype=np.uint16):
        self.out_dir = Path(out_dir)
        self.out_dir.mkdir(parents=True, exist_ok=True)
        self.max_shard_bytes = max_shard_bytes
        self.dtype = np.dtype(dtype)
        self._tmp: list[Path] = []
        self._writer = None
        self._bytes = 0
        self.doc_lengths: list[int] = []

    def _roll(self) -> None:
        if self._writer is not None:
            self._writer.close()
        path = self.out_dir / f"tmp-shard-{len(self._tmp):05d}.arecord"
        self._tmp.append(path)
        self._writer = _open_writer(str(path))
        self._bytes = 0

    def write_document(self, tokens) -> None:
        arr = np.asarray(tokens, dtype=self.dtype)
        if len(arr) == 0:
            return
        data = arr.tobytes()
        if self._writer is None or (self._bytes + len(data) > self.max_shard_bytes and self._bytes > 0):
            self._roll()
        self._writer.write(data)
        self._bytes += len(data)
        self.doc_lengths.append(len(arr))

    def close(self) -> list[Path]:
        if self._writer is not None:
            self._writer.close()
        total = len(self._tmp)
        final = []
        for i, p in enumerate(self._tmp):
            q = self.out_dir / f"shard-{i:05d}-of-{total:05d}.arecord"
            p.rename(q)
            final.append(q)
        np.save(self.out_dir / "doc_lengths.npy", np.asarray(self.doc_lengths, dtype=np.int32))
        return final

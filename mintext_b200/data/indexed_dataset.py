"""Document-level readers for tokenised corpora (reference: mintext/data/indexed_dataset.py).

``MMapIndexedDataset``: Megatron ``.idx`` + ``.bin`` (or multi-part ``.bin.00000`` ...).  The ``.idx`` header is
``MMIDIDX\\0\\0`` | version u64 = 1 | dtype code u8 | sequence count u64 | document count u64, followed by int32
sequence lengths, int64 byte pointers and int64 document boundaries.  Slices are read straight from the mapping
(the reference materialises the whole document first).

``ArrayRecordDocDataset``: one record per document plus a ``doc_lengths.npy`` companion.  Google's
``array_record`` library is used when importable; otherwise the files must be in this package's own record
container (see :class:`RecordFileWriter`), which the conversion tools write when ``array_record`` is absent.
"""

from __future__ import annotations

import itertools
import struct
from pathlib import Path

import numpy as np

_IDX_MAGIC = b"MMIDIDX\x00\x00"
_IDX_HEADER_SIZE = 34
_DTYPE_CODES = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float64, 7: np.float32,
                8: np.uint16}
_CODE_OF_DTYPE = {np.dtype(v): k for k, v in _DTYPE_CODES.items()}


def write_mmap_dataset(path_prefix: str, documents, dtype=np.uint16, parts: int = 1) -> None:
    """Write ``documents`` (iterable of 1-D integer arrays, one sequence per document) as ``.idx`` + ``.bin``
    (``parts > 1`` splits the data file at sequence boundaries into ``.bin.00000`` ...)."""
    docs = [np.asarray(d, dtype=dtype) for d in documents]
    lengths = np.array([len(d) for d in docs], dtype=np.int32)
    itemsize = np.dtype(dtype).itemsize
    pointers = np.zeros(len(docs), dtype=np.int64)
    if len(docs) > 1:
        pointers[1:] = np.cumsum(lengths[:-1].astype(np.int64)) * itemsize
    doc_idx = np.arange(len(docs) + 1, dtype=np.int64)
    with open(f"{path_prefix}.idx", "wb") as f:
        f.write(_IDX_MAGIC)
        f.write(struct.pack("<Q", 1))
        f.write(struct.pack("<B", _CODE_OF_DTYPE[np.dtype(dtype)]))
        f.write(struct.pack("<Q", len(docs)))
        f.write(struct.pack("<Q", len(doc_idx)))
        f.write(lengths.tobytes())
        f.write(pointers.tobytes())
        f.write(doc_idx.tobytes())
    if parts <= 1:
        with open(f"{path_prefix}.bin", "wb") as f:
            for d in docs:
                f.write(d.tobytes())
        return
    per = max((len(docs) + parts - 1) // parts, 1)
    for p in range(parts):
        chunk = docs[p * per:(p + 1) * per]
        if not chunk and p > 0:  # fewer documents than parts: no empty trailing files (they cannot be mapped)
            break
        with open(f"{path_prefix}.bin.{p:05d}", "wb") as f:
            for d in chunk:
                f.write(d.tobytes())


class MMapIndexedDataset:
    def __init__(self, path_prefix: str) -> None:
        idx_path = Path(f"{path_prefix}.idx")
        if not idx_path.exists():
            raise FileNotFoundError(f"Index file not found: {idx_path}")
        with open(idx_path, "rb") as f:
            magic = f.read(9)
            if magic != _IDX_MAGIC:
                raise ValueError(f"Invalid .idx magic: {magic!r}")
            (version,) = struct.unpack("<Q", f.read(8))
            if version != 1:
                raise ValueError(f"Unsupported .idx version: {version}")
            (code,) = struct.unpack("<B", f.read(1))
            if code not in _DTYPE_CODES:
                raise ValueError(f"Unknown dtype code: {code}")
            (seq_count,) = struct.unpack("<Q", f.read(8))
            (doc_count,) = struct.unpack("<Q", f.read(8))
        self._dtype = np.dtype(_DTYPE_CODES[code])
        self._dtype_size = self._dtype.itemsize
        raw = np.memmap(idx_path, mode="r", order="C")
        off = _IDX_HEADER_SIZE
        self._sequence_lengths = np.frombuffer(raw, dtype=np.int32, count=seq_count, offset=off)
        off += 4 * seq_count
        self._sequence_pointers = np.frombuffer(raw, dtype=np.int64, count=seq_count, offset=off)
        off += 8 * seq_count
        self._document_indices = np.frombuffer(raw, dtype=np.int64, count=doc_count, offset=off)
        self._idx_mmap = raw
        single = Path(f"{path_prefix}.bin")
        if single.exists():
            paths = [single]
        else:
            paths = []
            for i in itertools.count():
                p = Path(f"{path_prefix}.bin.{i:05d}")
                if not p.exists():
                    break
                paths.append(p)
            if not paths:
                raise FileNotFoundError(f"Data file not found: {single} (also tried {path_prefix}.bin.00000)")
        self._bin_parts = [np.memmap(p, mode="r", dtype=np.uint8) if p.stat().st_size > 0 else np.zeros(0, dtype=np.uint8)
                           for p in paths]
        self._part_cumulative = np.concatenate([[0], np.cumsum([len(m) for m in self._bin_parts])]).astype(np.int64)
        self._num_docs = len(self._document_indices) - 1
        cs = np.zeros(seq_count + 1, dtype=np.int64)
        np.cumsum(self._sequence_lengths, out=cs[1:])
        self._seq_token_start = cs  # token offset of every sequence within the logical token stream

    def __len__(self) -> int:
        return self._num_docs

    def _check(self, idx: int) -> int:
        if idx < 0:
            idx += self._num_docs
        if idx < 0 or idx >= self._num_docs:
            raise IndexError(f"Document index {idx} out of range [0, {self._num_docs})")
        return idx

    def _read_bytes(self, pointer: int, nbytes: int) -> np.ndarray:
        """Bytes ``[pointer, pointer + nbytes)`` of the logical data stream (may straddle part files)."""
        out = np.empty(nbytes, dtype=np.uint8)
        done = 0
        while done < nbytes:
            part = int(np.searchsorted(self._part_cumulative, pointer + done, side="right")) - 1
            local = pointer + done - int(self._part_cumulative[part])
            take = min(nbytes - done, len(self._bin_parts[part]) - local)
            out[done:done + take] = self._bin_parts[part][local:local + take]
            done += take
        return out

    def _read_sequence(self, seq_idx: int, offset: int = 0, length: int | None = None) -> np.ndarray:
        n = int(self._sequence_lengths[seq_idx])
        length = n - offset if length is None else min(length, n - offset)
        if length <= 0:
            return np.zeros(0, dtype=self._dtype)
        ptr = int(self._sequence_pointers[seq_idx]) + offset * self._dtype_size
        return self._read_bytes(ptr, length * self._dtype_size).view(self._dtype)

    def __getitem__(self, idx: int) -> np.ndarray:
        idx = self._check(idx)
        s0, s1 = int(self._document_indices[idx]), int(self._document_indices[idx + 1])
        if s1 - s0 == 1:
            return self._read_sequence(s0)
        return np.concatenate([self._read_sequence(s) for s in range(s0, s1)])

    def get(self, idx: int, offset: int = 0, length: int | None = None) -> np.ndarray:
        """``document[idx][offset:offset+length]`` without reading the rest of the document."""
        idx = self._check(idx)
        s0, s1 = int(self._document_indices[idx]), int(self._document_indices[idx + 1])
        doc_len = int(self._seq_token_start[s1] - self._seq_token_start[s0])
        end = doc_len if length is None else min(doc_len, offset + length)
        if offset >= end:
            return np.zeros(0, dtype=self._dtype)
        parts = []
        base = int(self._seq_token_start[s0])
        for s in range(s0, s1):
            a = int(self._seq_token_start[s]) - base
            b = int(self._seq_token_start[s + 1]) - base
            lo, hi = max(a, offset), min(b, end)
            if lo < hi:
                parts.append(self._read_sequence(s, lo - a, hi - lo))
        return parts[0] if len(parts) == 1 else np.concatenate(parts)

    @property
    def doc_lengths(self) -> np.ndarray:
        starts = self._document_indices[:-1].astype(np.intp)
        ends = self._document_indices[1:].astype(np.intp)
        return (self._seq_token_start[ends] - self._seq_token_start[starts]).astype(np.int32)


# ---------------------------------------------------------------------------------------------- record files
_REC_MAGIC = b"MTRECORD1"


class RecordFileWriter:
    """This package's record container, used for ``.arecord`` shards when Google's ``array_record`` library is not
    installed: ``MTRECORD1`` | records back to back | int64 offsets table | record count u64 | table position u64."""

    def __init__(self, path: str):
        self._f = open(path, "wb")
        self._f.write(_REC_MAGIC)
        self._offsets = [len(_REC_MAGIC)]

    def write(self, record: bytes) -> None:
        self._f.write(record)
        self._offsets.append(self._offsets[-1] + len(record))

    def close(self) -> None:
        table_pos = self._offsets[-1]
        self._f.write(np.asarray(self._offsets, dtype=np.int64).tobytes())
        self._f.write(struct.pack("<QQ", len(self._offsets) - 1, table_pos))
        self._f.close()


class _RecordFileReader:
    def __init__(self, path: str):
        self._mm = np.memmap(path, mode="r", dtype=np.uint8)
        if bytes(self._mm[: len(_REC_MAGIC)]) != _REC_MAGIC:
            raise ValueError(f"{path} is not a record file of this package (and array_record is not installed)")
        n, table_pos = struct.unpack("<QQ", bytes(self._mm[-16:]))
        self._offsets = np.frombuffer(self._mm, dtype=np.int64, count=n + 1, offset=table_pos)
        self._n = n

    def num_records(self) -> int:
        return self._n

    def read(self, indices):
        return [bytes(self._mm[int(self._offsets[i]):int(self._offsets[i + 1])]) for i in indices]


def _open_record_reader(path: str):
    try:
        from array_record.python.array_record_module import ArrayRecordReader  # type: ignore

        with open(path, "rb") as f:
            if f.read(len(_REC_MAGIC)) != _REC_MAGIC:
                return ArrayRecordReader(path)
    except ImportError:
        pass
    return _RecordFileReader(path)


class ArrayRecordDocDataset:
    def __init__(self, path: str) -> None:
        p = Path(path)
        if p.is_dir():
            files = sorted(p.glob("*.arecord"))
            if not files:
                raise FileNotFoundError(f"No .arecord files found in {p}")
            lengths_path = p / "doc_lengths.npy"
        else:
            files = [p]
            lengths_path = p.parent / "doc_lengths.npy"
        if not lengths_path.exists():
            raise FileNotFoundError(f"Companion doc_lengths.npy not found: {lengths_path}")
        self._doc_lengths_arr = np.load(lengths_path).astype(np.int32)
        self._readers = [_open_record_reader(str(f)) for f in files]
        counts = [r.num_records() for r in self._readers]
        self._shard_offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)
        self._total_docs = int(self._shard_offsets[-1])
        if len(self._doc_lengths_arr) != self._total_docs:
            raise ValueError(f"doc_lengths.npy has {len(self._doc_lengths_arr)} entries "
                             f"but arecord files have {self._total_docs} records")
        first = self._readers[0].read([0])[0] if self._total_docs else b""
        self._token_dtype = np.uint16 if len(first) == int(self._doc_lengths_arr[0]) * 2 and self._total_docs else np.int32

    def __len__(self) -> int:
        return self._total_docs

    def __getitem__(self, idx: int) -> np.ndarray:
        if idx < 0:
            idx += self._total_docs
        if idx < 0 or idx >= self._total_docs:
            raise IndexError(f"Document index {idx} out of range [0, {self._total_docs})")
        shard = int(np.searchsorted(self._shard_offsets, idx, side="right")) - 1
        rec = self._readers[shard].read([idx - int(self._shard_offsets[shard])])[0]
        return np.frombuffer(rec, dtype=self._token_dtype).copy()

    def get(self, idx: int, offset: int = 0, length: int | None = None) -> np.ndarray:
        tokens = self[idx]
        return tokens[offset:] if length is None else tokens[offset:offset + length]

    @property
    def doc_lengths(self) -> np.ndarray:
        return self._doc_lengths_arr

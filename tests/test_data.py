"""Dataset readers, index builders, blending, the loader and its resume behaviour (mirrors tests/test_data.py)."""

import numpy as np
import pytest

from mintext_b200 import MinTextConfig
from mintext_b200.data import (ArrayRecordDocDataset, BlendedDataSource, DocumentDataSource, MMapIndexedDataset,
                               ShiftTokens, create_eval_iterator, create_train_iterator)
from mintext_b200.data.dataset import _build_document_index, _build_sample_index, _build_sample_index_numpy
from mintext_b200.data.indexed_dataset import RecordFileWriter, write_mmap_dataset
from mintext_b200.data.pipeline import _detect_data_type, _parse_data_path, _parse_split


def make_docs(n=20, seed=0, lo=5, hi=40, vocab=1000):
    rng = np.random.RandomState(seed)
    return [rng.randint(1, vocab, size=rng.randint(lo, hi)).astype(np.uint16) for _ in range(n)]


@pytest.fixture
def mmap_path(tmp_path):
    docs = make_docs()
    write_mmap_dataset(str(tmp_path / "corpus"), docs)
    return str(tmp_path / "corpus"), docs


@pytest.fixture
def arecord_dir(tmp_path):
    docs = make_docs(seed=1)
    d = tmp_path / "rec"
    d.mkdir()
    for shard in range(2):
        w = RecordFileWriter(str(d / f"shard-{shard:05d}-of-00002.arecord"))
        for doc in docs[shard * 10:(shard + 1) * 10]:
            w.write(doc.tobytes())
        w.close()
    np.save(d / "doc_lengths.npy", np.array([len(x) for x in docs], dtype=np.int32))
    return str(d), docs


def test_mmap_reader(mmap_path):
    path, docs = mmap_path
    ds = MMapIndexedDataset(path)
    assert len(ds) == 20 and np.array_equal(ds[3], docs[3]) and np.array_equal(ds[-1], docs[-1])
    assert np.array_equal(ds.get(4, offset=2, length=3), docs[4][2:5]) and np.array_equal(ds.get(4, offset=2), docs[4][2:])
    assert np.array_equal(ds.doc_lengths, [len(d) for d in docs])
    with pytest.raises(IndexError):
        ds[20]
    with pytest.raises(FileNotFoundError):
        MMapIndexedDataset(path + "_missing")


def test_mmap_bad_magic(tmp_path):
    (tmp_path / "x.idx").write_bytes(b"BADMAGIC!" + b"\0" * 40)
    (tmp_path / "x.bin").write_bytes(b"")
    with pytest.raises(ValueError, match="magic"):
        MMapIndexedDataset(str(tmp_path / "x"))


def test_multipart_bin_equivalence(tmp_path):
    docs = make_docs(n=13)
    write_mmap_dataset(str(tmp_path / "one"), docs)
    write_mmap_dataset(str(tmp_path / "many"), docs, parts=4)
    a, b = MMapIndexedDataset(str(tmp_path / "one")), MMapIndexedDataset(str(tmp_path / "many"))
    for i in range(13):
        assert np.array_equal(a[i], b[i])
        assert np.array_equal(a.get(i, 1, 4), b.get(i, 1, 4))


def test_arecord_reader(arecord_dir):
    path, docs = arecord_dir
    ds = ArrayRecordDocDataset(path)
    assert len(ds) == 20 and np.array_equal(ds[12], docs[12]) and np.array_equal(ds.get(12, 1, 3), docs[12][1:4])
    assert np.array_equal(ds.doc_lengths, [len(d) for d in docs])


def test_document_and_sample_index_builders():
    di = _build_document_index(5, 2, np.random.RandomState(0))
    assert len(di) == 10 and sorted(di[:5]) == list(range(5)) and sorted(di[5:]) == list(range(5))
    lens = np.array([5, 3, 10, 2], dtype=np.int32)
    order = np.arange(4, dtype=np.int32)
    si = _build_sample_index_numpy(order, lens, seq_len=3, add_extra_token=True)  # 20 tokens / 4 per sample
    assert si.shape == (6, 2) and si[0].tolist() == [0, 0] and si[1].tolist() == [0, 4] and si[2].tolist() == [1, 3]
    assert np.array_equal(si, _build_sample_index(order, lens, 3, True))  # native builder agrees
    si2 = _build_sample_index(order, lens, seq_len=4, add_extra_token=False)
    assert len(si2) - 1 == 5
    rng = np.random.RandomState(3)
    big_lens = rng.randint(1, 50, size=300).astype(np.int32)
    big_order = _build_document_index(300, 3, rng)
    assert np.array_equal(_build_sample_index(big_order, big_lens, 17, True),
                          _build_sample_index_numpy(big_order, big_lens, 17, True))


@pytest.mark.parametrize("kind", ["mmap", "arecord"])
def test_document_data_source_covers_the_corpus(kind, mmap_path, arecord_dir, tmp_path):
    path, docs = mmap_path if kind == "mmap" else arecord_dir
    src = DocumentDataSource(path, kind, seq_len=16, seed=0, num_epochs=1, split=(1, 0, 0), split_index=0,
                             cache_dir=str(tmp_path / "cache"))
    total = sum(len(d) for d in docs)
    assert len(src) == total // 17
    s = src[0]["tokens"]
    assert s.shape == (17,) and s.dtype.kind in "iu"
    order = src._document_index
    stream = np.concatenate([docs[i] for i in order])
    for i in (0, 1, len(src) - 1):
        assert np.array_equal(src[i]["tokens"], stream[i * 17:(i + 1) * 17])
    again = DocumentDataSource(path, kind, 16, 0, 1, (1, 0, 0), 0, cache_dir=str(tmp_path / "cache"))
    assert np.array_equal(again._sample_index, src._sample_index)  # served from the cache files
    assert len(list((tmp_path / "cache").glob("*.npy"))) == 2


def test_splits(mmap_path, tmp_path):
    path, _ = mmap_path
    tr = DocumentDataSource(path, "mmap", 8, 0, 1, (80, 20, 0), 0, cache_dir=str(tmp_path / "c"))
    ev = DocumentDataSource(path, "mmap", 8, 0, 1, (80, 20, 0), 1, cache_dir=str(tmp_path / "c"))
    te = DocumentDataSource(path, "mmap", 8, 0, 1, (80, 20, 0), 2, cache_dir=str(tmp_path / "c"))
    assert len(tr._doc_ids) == 16 and len(ev._doc_ids) == 4 and len(te) == 0


def test_blending_proportions():
    class Fake:
        def __init__(self, tag, n):
            self.tag, self.n = tag, n

        def __len__(self):
            return self.n

        def __getitem__(self, i):
            return {"tokens": np.array([self.tag, i])}

    b = BlendedDataSource([Fake(0, 50), Fake(1, 30)], [0.7, 0.3], size=1000)
    tags = np.array([b[i]["tokens"][0] for i in range(1000)])
    assert abs((tags == 0).mean() - 0.7) < 0.05
    assert b[0]["tokens"].tolist() == [0, 0]
    with pytest.raises(ValueError):
        BlendedDataSource([Fake(0, 1)], [1.0, 2.0], 10)


def test_shift_tokens_both_modes():
    t = np.arange(6)
    a = ShiftTokens(True).map({"tokens": t})
    assert a["input_tokens"].tolist() == [0, 1, 2, 3, 4] and a["target_tokens"].tolist() == [1, 2, 3, 4, 5]
    b = ShiftTokens(False).map({"tokens": t})
    assert b["input_tokens"].tolist() == list(range(6)) and b["target_tokens"].tolist() == [1, 2, 3, 4, 5, 0]


def test_path_type_split_parsing(mmap_path, arecord_dir):
    assert _parse_data_path("/a/b") == [(1.0, "/a/b")]
    assert _parse_data_path("0.3 /a 0.7 /b") == [(0.3, "/a"), (0.7, "/b")]
    assert _parse_data_path("/path with space") == [(1.0, "/path with space")]
    with pytest.raises(ValueError):
        _parse_data_path("0.3 /a 0.7")
    assert _detect_data_type(mmap_path[0]) == "mmap" and _detect_data_type(arecord_dir[0]) == "arecord"
    with pytest.raises(ValueError, match="Cannot detect"):
        _detect_data_type("/nonexistent/path")
    assert _parse_split("99,1,0") == (99.0, 1.0, 0.0)
    with pytest.raises(ValueError):
        _parse_split("1,2")


def _cfg(path, tmp_path, **kw):
    base = dict(dataset_type="auto", data_path=path, seq_length=8, per_device_batch_size=2, data_split="80,20,0",
                data_cache_dir=str(tmp_path / "cache"), grain_worker_count=2, grain_prefetch_buffer_size=8)
    base.update(kw)
    return MinTextConfig(**base)


def test_iterators_shapes_determinism_and_resume(mmap_path, tmp_path):
    path, _ = mmap_path
    it = create_train_iterator(_cfg(path, tmp_path))
    batches = [next(it) for _ in range(6)]
    assert batches[0]["input_tokens"].shape == (2, 8) and batches[0]["input_tokens"].dtype == np.int32
    assert np.array_equal(batches[0]["input_tokens"][:, 1:], batches[0]["target_tokens"][:, :-1])
    it.close()
    it2 = create_train_iterator(_cfg(path, tmp_path, grain_worker_count=0))  # no worker threads: same stream
    for b in batches:
        assert np.array_equal(next(it2)["input_tokens"], b["input_tokens"])
    it3 = create_train_iterator(_cfg(path, tmp_path))
    it3.load_state_dict({"batches_done": 4})  # restart after 4 batches continues with the 5th
    assert np.array_equal(next(it3)["input_tokens"], batches[4]["input_tokens"])
    it3.close()
    ev = create_eval_iterator(_cfg(path, tmp_path, seq_length=4))
    assert next(ev)["input_tokens"].shape == (2, 4)
    ev.close()


def test_rank_sharding_is_disjoint(mmap_path, tmp_path):
    from mintext_b200.data.pipeline import BatchIterator

    path, _ = mmap_path
    src = DocumentDataSource(path, "mmap", 8, 0, 1, (1, 0, 0), 0, cache_dir=str(tmp_path / "c"))
    a = BatchIterator(src, 2, 0, True, rank=0, world=2)
    b = BatchIterator(src, 2, 0, True, rank=1, world=2)
    ia = sum((a._sample_ids(i) for i in range(5)), [])
    ib = sum((b._sample_ids(i) for i in range(5)), [])
    assert not set(ia) & set(ib) and len(set(ia)) == 10


class _ArraySource:
    """Tiny in-memory source: sample ``i`` is ``seq_len + 1`` tokens all equal to ``i``."""

    def __init__(self, n, seq_len=4, fail_at=None):
        self.n, self.seq_len, self.fail_at = n, seq_len, fail_at

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        if self.fail_at is not None and i == self.fail_at:
            raise OSError(f"cannot read sample {i}")
        return {"tokens": np.full(self.seq_len + 1, i, dtype=np.int32)}


def test_prefetch_workers_cross_epoch_boundaries_in_order():
    from mintext_b200.data.pipeline import BatchIterator

    src = _ArraySource(10)
    serial = BatchIterator(src, 2, 7, True, workers=0)
    threaded = BatchIterator(src, 2, 7, True, workers=4, buffer_size=8)
    try:
        for _ in range(40):  # 5 batches per epoch: eight epoch boundaries
            a, b = next(serial), next(threaded)
            assert np.array_equal(a["input_tokens"], b["input_tokens"])
    finally:
        threaded.close()


def test_worker_exception_reaches_the_consumer():
    from mintext_b200.data.pipeline import BatchIterator

    it = BatchIterator(_ArraySource(8, fail_at=5), 2, 0, False, workers=3, buffer_size=8)
    with pytest.raises(RuntimeError, match="data worker failed") as info:
        for _ in range(8):
            next(it)
    assert isinstance(info.value.__cause__, OSError)
    it.close()

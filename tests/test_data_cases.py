"""Single-behaviour tests of the data stack (readers, index builders, sources, parsers), one assertion group per
test, after the cases the reference checks in tests/test_data.py."""

import numpy as np
import pytest

from mintext_b200.data import (ArrayRecordDocDataset, BlendedDataSource, DocumentDataSource, MMapIndexedDataset,
                               ShiftTokens)
from mintext_b200.data.dataset import _build_document_index, _build_sample_index, _build_sample_index_numpy
from mintext_b200.data.indexed_dataset import RecordFileWriter, write_mmap_dataset
from mintext_b200.data.pipeline import _detect_data_type, _parse_data_path, _parse_split
from mintext_b200.utils.filesize import parse_file_size


def _docs(n=12, seed=0, lo=3, hi=30):
    rng = np.random.RandomState(seed)
    return [rng.randint(1, 500, size=rng.randint(lo, hi)).astype(np.uint16) for _ in range(n)]


@pytest.fixture
def mmap(tmp_path):
    docs = _docs()
    write_mmap_dataset(str(tmp_path / "c"), docs)
    return MMapIndexedDataset(str(tmp_path / "c")), docs, str(tmp_path / "c")


@pytest.fixture
def arecord(tmp_path):
    docs = _docs(seed=4)
    d = tmp_path / "rec"
    d.mkdir()
    w = RecordFileWriter(str(d / "shard-00000-of-00001.arecord"))
    for doc in docs:
        w.write(doc.tobytes())
    w.close()
    np.save(d / "doc_lengths.npy", np.array([len(x) for x in docs], dtype=np.int32))
    return ArrayRecordDocDataset(str(d)), docs, str(d)


# ---- mmap reader ------------------------------------------------------------------------------------------------
def test_mmap_len(mmap):
    ds, docs, _ = mmap
    assert len(ds) == len(docs)


def test_mmap_getitem_every_document(mmap):
    ds, docs, _ = mmap
    for i, d in enumerate(docs):
        assert np.array_equal(ds[i], d)


def test_mmap_negative_index(mmap):
    ds, docs, _ = mmap
    assert np.array_equal(ds[-1], docs[-1]) and np.array_equal(ds[-len(docs)], docs[0])


def test_mmap_index_past_the_end(mmap):
    ds, docs, _ = mmap
    with pytest.raises(IndexError):
        ds[len(docs)]
    with pytest.raises(IndexError):
        ds[-len(docs) - 1]


def test_mmap_get_slice(mmap):
    ds, docs, _ = mmap
    assert np.array_equal(ds.get(2, offset=1, length=2), docs[2][1:3])


def test_mmap_get_without_length_runs_to_the_document_end(mmap):
    ds, docs, _ = mmap
    assert np.array_equal(ds.get(5, offset=2), docs[5][2:])


def test_mmap_doc_lengths(mmap):
    ds, docs, _ = mmap
    assert ds.doc_lengths.tolist() == [len(d) for d in docs]


def test_mmap_dtype_is_preserved(tmp_path):
    docs = [np.arange(70000, 70010, dtype=np.int32)]
    write_mmap_dataset(str(tmp_path / "w"), docs, dtype=np.int32)
    got = MMapIndexedDataset(str(tmp_path / "w"))[0]
    assert got.dtype == np.int32 and got.tolist() == docs[0].tolist()


def test_mmap_missing_files(tmp_path):
    with pytest.raises(FileNotFoundError):
        MMapIndexedDataset(str(tmp_path / "nothing"))


def test_mmap_rejects_foreign_index_file(tmp_path):
    (tmp_path / "x.idx").write_bytes(b"NOTANIDX\x00" + b"\0" * 64)
    (tmp_path / "x.bin").write_bytes(b"\0" * 8)
    with pytest.raises(ValueError):
        MMapIndexedDataset(str(tmp_path / "x"))


# ---- multi-part .bin ---------------------------------------------------------------------------------------------
def test_multipart_reads_equal_single_part(tmp_path):
    docs = _docs(n=17, seed=2)
    write_mmap_dataset(str(tmp_path / "a"), docs)
    write_mmap_dataset(str(tmp_path / "b"), docs, parts=3)
    a, b = MMapIndexedDataset(str(tmp_path / "a")), MMapIndexedDataset(str(tmp_path / "b"))
    assert len(a) == len(b)
    for i in range(len(docs)):
        assert np.array_equal(a[i], b[i])


def test_multipart_doc_lengths(tmp_path):
    docs = _docs(n=9, seed=3)
    write_mmap_dataset(str(tmp_path / "b"), docs, parts=4)
    assert MMapIndexedDataset(str(tmp_path / "b")).doc_lengths.tolist() == [len(d) for d in docs]


def test_multipart_slices_that_cross_a_part_boundary(tmp_path):
    docs = [np.arange(100, dtype=np.uint16) + 7 * i for i in range(6)]
    write_mmap_dataset(str(tmp_path / "b"), docs, parts=5)
    ds = MMapIndexedDataset(str(tmp_path / "b"))
    for i in range(6):
        assert np.array_equal(ds.get(i, 13, 70), docs[i][13:83])


def test_multipart_is_detected_as_mmap(tmp_path):
    write_mmap_dataset(str(tmp_path / "b"), _docs(n=5), parts=2)
    assert _detect_data_type(str(tmp_path / "b")) == "mmap"


def test_index_without_any_bin_file(tmp_path):
    write_mmap_dataset(str(tmp_path / "b"), _docs(n=4))
    (tmp_path / "b.bin").unlink()
    with pytest.raises(FileNotFoundError):
        MMapIndexedDataset(str(tmp_path / "b"))


# ---- record-file reader ------------------------------------------------------------------------------------------
def test_arecord_len_and_items(arecord):
    ds, docs, _ = arecord
    assert len(ds) == len(docs)
    assert np.array_equal(ds[0], docs[0]) and np.array_equal(ds[len(docs) - 1], docs[-1])


def test_arecord_negative_index(arecord):
    ds, docs, _ = arecord
    assert np.array_equal(ds[-2], docs[-2])


def test_arecord_get_slice(arecord):
    ds, docs, _ = arecord
    assert np.array_equal(ds.get(3, 1, 2), docs[3][1:3])


def test_arecord_doc_lengths(arecord):
    ds, docs, _ = arecord
    assert ds.doc_lengths.tolist() == [len(d) for d in docs]


def test_arecord_without_doc_lengths_file(tmp_path):
    d = tmp_path / "rec"
    d.mkdir()
    w = RecordFileWriter(str(d / "shard-00000-of-00001.arecord"))
    w.write(np.arange(4, dtype=np.uint16).tobytes())
    w.close()
    with pytest.raises(FileNotFoundError):
        ArrayRecordDocDataset(str(d))


# ---- index builders ----------------------------------------------------------------------------------------------
def test_document_index_one_epoch_is_a_permutation():
    di = _build_document_index(9, 1, np.random.RandomState(0))
    assert sorted(di.tolist()) == list(range(9))


def test_document_index_epochs_are_each_a_permutation():
    di = _build_document_index(6, 3, np.random.RandomState(1))
    assert len(di) == 18
    for e in range(3):
        assert sorted(di[6 * e:6 * e + 6].tolist()) == list(range(6))


def test_document_index_depends_on_the_generator_state():
    a = _build_document_index(50, 1, np.random.RandomState(0))
    b = _build_document_index(50, 1, np.random.RandomState(1))
    assert not np.array_equal(a, b)


@pytest.mark.parametrize("builder", [_build_sample_index, _build_sample_index_numpy])
def test_sample_index_inside_one_document(builder):
    si = builder(np.array([0], dtype=np.int32), np.array([13], dtype=np.int32), 3, True)
    assert si.tolist() == [[0, 0], [0, 4], [0, 8], [0, 12]]  # three samples of 4 tokens, then the end marker


@pytest.mark.parametrize("builder", [_build_sample_index, _build_sample_index_numpy])
def test_sample_index_crosses_documents(builder):
    lens = np.array([3, 3, 3], dtype=np.int32)
    si = builder(np.arange(3, dtype=np.int32), lens, 3, True)  # 9 tokens, 4 per sample
    assert si[:3].tolist() == [[0, 0], [1, 1], [2, 2]]


@pytest.mark.parametrize("builder", [_build_sample_index, _build_sample_index_numpy])
def test_sample_index_exact_fit(builder):
    si = builder(np.array([0, 1], dtype=np.int32), np.array([4, 4], dtype=np.int32), 3, True)
    assert len(si) - 1 == 2


@pytest.mark.parametrize("builder", [_build_sample_index, _build_sample_index_numpy])
def test_sample_index_without_the_extra_token(builder):
    si = builder(np.array([0], dtype=np.int32), np.array([12], dtype=np.int32), 4, False)
    assert len(si) - 1 == 3 and si[1].tolist() == [0, 4]


# ---- sources -----------------------------------------------------------------------------------------------------
def test_source_sample_length_with_extra_token(mmap, tmp_path):
    _, _, path = mmap
    src = DocumentDataSource(path, "mmap", 8, 0, 1, (1, 0, 0), 0, cache_dir=str(tmp_path / "k"))
    assert src[0]["tokens"].shape == (9,)


def test_source_sample_length_without_extra_token(mmap, tmp_path):
    _, _, path = mmap
    src = DocumentDataSource(path, "mmap", 8, 0, 1, (1, 0, 0), 0, cache_dir=str(tmp_path / "k"), add_extra_token=False)
    assert src[0]["tokens"].shape == (8,)


def test_source_on_record_files(arecord, tmp_path):
    _, docs, path = arecord
    src = DocumentDataSource(path, "arecord", 5, 0, 1, (1, 0, 0), 0, cache_dir=str(tmp_path / "k"))
    assert len(src) == sum(len(d) for d in docs) // 6


def test_source_index_cache_is_reused(mmap, tmp_path):
    _, _, path = mmap
    a = DocumentDataSource(path, "mmap", 8, 3, 2, (1, 0, 0), 0, cache_dir=str(tmp_path / "k"))
    files = sorted(p.name for p in (tmp_path / "k").iterdir())
    stamps = [p.stat().st_mtime_ns for p in sorted((tmp_path / "k").iterdir())]
    b = DocumentDataSource(path, "mmap", 8, 3, 2, (1, 0, 0), 0, cache_dir=str(tmp_path / "k"))
    assert sorted(p.name for p in (tmp_path / "k").iterdir()) == files
    assert [p.stat().st_mtime_ns for p in sorted((tmp_path / "k").iterdir())] == stamps
    assert np.array_equal(a._document_index, b._document_index)


def test_source_seed_changes_the_order(mmap, tmp_path):
    _, _, path = mmap
    a = DocumentDataSource(path, "mmap", 8, 0, 1, (1, 0, 0), 0, cache_dir=str(tmp_path / "k"))
    b = DocumentDataSource(path, "mmap", 8, 1, 1, (1, 0, 0), 0, cache_dir=str(tmp_path / "k"))
    assert not np.array_equal(a._document_index, b._document_index)


def test_source_splits_partition_the_documents(mmap, tmp_path):
    _, docs, path = mmap
    parts = [DocumentDataSource(path, "mmap", 4, 0, 1, (50, 25, 25), i, cache_dir=str(tmp_path / "k")) for i in range(3)]
    ids = [set(p._doc_ids.tolist()) for p in parts]
    assert sum(len(s) for s in ids) == len(docs) and not (ids[0] & ids[1]) and not (ids[1] & ids[2])


class _Tagged:
    def __init__(self, tag, n):
        self.tag, self.n = tag, n

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        return {"tokens": np.array([self.tag, i])}


def test_blend_draws_from_every_source():
    b = BlendedDataSource([_Tagged(0, 10), _Tagged(1, 10), _Tagged(2, 10)], [1, 1, 1], size=300)
    tags = {int(b[i]["tokens"][0]) for i in range(300)}
    assert tags == {0, 1, 2}


def test_blend_follows_the_weights():
    b = BlendedDataSource([_Tagged(0, 40), _Tagged(1, 40)], [0.9, 0.1], size=2000)
    frac = np.mean([b[i]["tokens"][0] == 0 for i in range(2000)])
    assert abs(frac - 0.9) < 0.03


def test_blend_wraps_small_sources():
    b = BlendedDataSource([_Tagged(0, 3)], [1.0], size=10)
    assert [int(b[i]["tokens"][1]) for i in range(10)] == [i % 3 for i in range(10)]


def test_blend_length_is_the_requested_size():
    assert len(BlendedDataSource([_Tagged(0, 3), _Tagged(1, 5)], [0.5, 0.5], size=77)) == 77


def test_blend_rejects_mismatched_weights():
    with pytest.raises(ValueError):
        BlendedDataSource([_Tagged(0, 3)], [0.5, 0.5], size=4)


# ---- token shift -------------------------------------------------------------------------------------------------
def test_shift_with_extra_token():
    out = ShiftTokens(True).map({"tokens": np.array([5, 6, 7, 8])})
    assert out["input_tokens"].tolist() == [5, 6, 7] and out["target_tokens"].tolist() == [6, 7, 8]


def test_shift_without_extra_token_rolls_the_targets():
    out = ShiftTokens(False).map({"tokens": np.array([5, 6, 7, 8])})
    assert out["input_tokens"].tolist() == [5, 6, 7, 8] and out["target_tokens"].tolist() == [6, 7, 8, 5]


# ---- parsers -----------------------------------------------------------------------------------------------------
def test_data_path_single():
    assert _parse_data_path("/data/corpus") == [(1.0, "/data/corpus")]


def test_data_path_two_weighted():
    assert _parse_data_path("0.25 /a 0.75 /b") == [(0.25, "/a"), (0.75, "/b")]


def test_data_path_three_weighted():
    assert [w for w, _ in _parse_data_path("1 /a 2 /b 3 /c")] == [1.0, 2.0, 3.0]


def test_data_path_with_spaces_is_one_path():
    assert _parse_data_path("/my data/corpus one") == [(1.0, "/my data/corpus one")]


def test_data_path_dangling_weight():
    with pytest.raises(ValueError):
        _parse_data_path("0.5 /a 0.5")


def test_detect_mmap_prefix(mmap):
    assert _detect_data_type(mmap[2]) == "mmap"


def test_detect_record_directory(arecord):
    assert _detect_data_type(arecord[2]) == "arecord"


def test_detect_single_record_file(arecord):
    import os

    f = [p for p in os.listdir(arecord[2]) if p.endswith(".arecord")][0]
    assert _detect_data_type(os.path.join(arecord[2], f)) == "arecord"


def test_detect_unknown_path(tmp_path):
    with pytest.raises(ValueError):
        _detect_data_type(str(tmp_path / "void"))


def test_split_three_numbers():
    assert _parse_split("90,5,5") == (90.0, 5.0, 5.0)


@pytest.mark.parametrize("bad", ["90,10", "a,b,c", ""])
def test_split_malformed(bad):
    with pytest.raises(ValueError):
        _parse_split(bad)


@pytest.mark.parametrize("text,expected", [("1G", 2 ** 30), ("2GB", 2 * 2 ** 30), ("512M", 512 * 2 ** 20),
                                           ("64MB", 64 * 2 ** 20), ("1T", 2 ** 40), ("4K", 4096), ("123", 123),
                                           ("1g", 2 ** 30), ("  8M ", 8 * 2 ** 20), ("1.5G", int(1.5 * 2 ** 30))])
def test_file_size_forms(text, expected):
    assert parse_file_size(text) == expected


@pytest.mark.parametrize("bad", ["", "abc", "12Q", "G"])
def test_file_size_malformed(bad):
    with pytest.raises(ValueError):
        parse_file_size(bad)

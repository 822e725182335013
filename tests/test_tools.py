"""Data-preparation tools: sample corpus -> record shards / mmap -> readable by the dataset classes; .bin splitting."""

import numpy as np

from mintext_b200.data import ArrayRecordDocDataset, MMapIndexedDataset
from mintext_b200.data.indexed_dataset import write_mmap_dataset
from mintext_b200.tools import generate_sample_jsonl, mmap_to_arecord, split_mmap, text_to_arecord


def _encode(text):
    return [(hash(w) % 5000) + 1 for w in text.split()]


def test_jsonl_to_records_and_mmap(tmp_path):
    src = tmp_path / "s.jsonl"
    generate_sample_jsonl.generate(str(src), 50, 5, 40, 0)
    n = text_to_arecord.convert([str(src)], str(tmp_path / "rec"), tokenizer="", max_bytes=2000, encode_fn=_encode)
    assert n == 50
    ds = ArrayRecordDocDataset(str(tmp_path / "rec"))
    assert len(ds) == 50 and len(list((tmp_path / "rec").glob("shard-*-of-*.arecord"))) > 1
    first = next(text_to_arecord.iter_texts(str(src), "text"))
    assert ds[0].tolist() == _encode(first)
    n2 = text_to_arecord.convert([str(src)], str(tmp_path / "mm"), tokenizer="", fmt="mmap", encode_fn=_encode)
    mm = MMapIndexedDataset(str(tmp_path / "mm"))
    assert n2 == 50 and mm[0].tolist() == _encode(first)
    assert mmap_to_arecord.convert(str(tmp_path / "mm"), str(tmp_path / "rec2"), 1 << 20) == 1
    assert np.array_equal(ArrayRecordDocDataset(str(tmp_path / "rec2"))[7], mm[7])


def test_split_mmap_keeps_documents(tmp_path):
    rng = np.random.RandomState(0)
    docs = [rng.randint(1, 1000, size=rng.randint(50, 200)).astype(np.uint16) for _ in range(40)]
    write_mmap_dataset(str(tmp_path / "c"), docs)
    parts = split_mmap.split(str(tmp_path / "c"), str(tmp_path / "out"), 2000)
    assert parts > 2
    ds = MMapIndexedDataset(str(tmp_path / "out"))
    for i in (0, 13, 39):
        assert np.array_equal(ds[i], docs[i])
    assert split_mmap.split(str(tmp_path / "c"), str(tmp_path / "same"), 10 ** 9) == 1

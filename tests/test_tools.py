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


def test_orbax_tree_mapping_and_native_round_trip(tmp_path, monkeypatch):
    """The Orbax converter without Orbax: path mapping both ways, and a reference-shaped TrainState tree written to
    and read back from this framework's layout; the CPU trainer restores from the converted checkpoint."""
    import numpy as np
    import torch

    from mintext_b200 import MinTextConfig, trainer
    from mintext_b200.checkpoint import create_checkpoint_manager, restore_checkpoint
    from mintext_b200.models import Transformer
    from mintext_b200.tools import convert_orbax as co

    c = MinTextConfig(num_hidden_layers=1, hidden_size=32, num_attention_heads=2, intermediate_size=64, vocab_size=64,
                      seq_length=8, dtype="float32", checkpoint_dir=str(tmp_path / "native"), enable_tensorboard=False)
    model = Transformer(c, rngs=3)
    # a tree shaped like the reference's saved TrainState: NNX-style nesting with {"value": array} leaves, optax
    # chain state with mu / nu subtrees that mirror the parameters
    flat_params = {("params",) + tuple(n.split(".")) + ("value",): p.detach().numpy().copy()
                   for n, p in model.named_parameters()}
    mu = {("opt_state", "1", "0", "mu") + k[1:]: np.full_like(v, 0.5) for k, v in flat_params.items()}
    nu = {("opt_state", "1", "0", "nu") + k[1:]: np.full_like(v, 0.25) for k, v in flat_params.items()}
    tree = co.unflatten_tree({**flat_params, **mu, **nu, ("step",): np.int64(7), ("opt_state", "1", "0", "count"): np.int64(7)})
    native = co.orbax_to_native(tree)
    name = "layers.0.attention.query.kernel"
    assert f"params/{name}" in native and f"opt_state/mu/{name}" in native and f"opt_state/nu/{name}" in native
    assert int(native["step"]) == 7 and int(native["opt_state/count"]) == 7
    back = co.flatten_tree(co.native_to_orbax(native))
    assert ("params", "layers", "0", "attention", "query", "kernel", "value") in back
    assert ("opt_state", "mu", "layers", "0", "attention", "query", "kernel", "value") in back

    monkeypatch.setattr(co, "load_orbax_tree", lambda path: tree)   # stands in for PyTreeCheckpointer().restore
    co.main(["from-orbax", "unused", str(tmp_path / "native")])
    got = co.read_native(str(tmp_path / "native"), 7)
    assert np.array_equal(got[f"params/{name}"], native[f"params/{name}"])
    # the converted checkpoint restores into a fresh trainer state
    fresh = Transformer(c, rngs=99)
    state = trainer.create_train_state(fresh, c)
    state, step = restore_checkpoint(create_checkpoint_manager(c), state)
    assert step == 7 and state.step == 7
    assert torch.equal(dict(fresh.named_parameters())[name], dict(model.named_parameters())[name])
    assert float(state.opt_state.mu[name].mean()) == 0.5 and float(state.opt_state.nu[name].mean()) == 0.25

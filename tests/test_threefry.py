"""Counter-based synthetic token stream: cipher known answers, tensor path vs integer path, row slicing, resume."""

import torch

from mintext_b200 import MinTextConfig
from mintext_b200.utils import threefry as tf


def test_threefry2x32_known_answers():
    # Random123 known-answer vectors for Threefry-2x32-20
    assert tf.threefry2x32(0, 0, 0, 0) == (0x6B200159, 0x99BA4EFE)
    assert tf.threefry2x32(0xFFFFFFFF, 0xFFFFFFFF, 0xFFFFFFFF, 0xFFFFFFFF) == (0x1CB996FC, 0xBB002BE7)
    assert tf.threefry2x32(0x13198A2E, 0x03707344, 0x243F6A88, 0x85A308D3) == (0xC4923A9C, 0x483DF7A0)


def test_tensor_path_equals_integer_path_and_split_is_a_cipher_block():
    k = tf.key(42)
    assert k == (0, 42)
    bits = tf.random_bits(k, 5, 16)
    for j in range(16):
        y0, y1 = tf.threefry2x32(k[0], k[1], 0, 5 + j)
        assert int(bits[j]) == y0 ^ y1
    a, b = tf.split(k)
    assert a == tf.threefry2x32(0, 42, 0, 0) and b == tf.threefry2x32(0, 42, 0, 1) and a != b


def test_randint_range_rows_and_uniformity():
    k = tf.key(7)
    full = tf.randint(k, (8, 64), 1000)
    assert full.dtype == torch.int64 and int(full.min()) >= 0 and int(full.max()) < 1000
    # a rank drawing only its rows gets exactly those rows of the global batch
    assert torch.equal(tf.randint_rows(k, 2, 3, 64, 1000), full[2:5])
    big = tf.randint(tf.key(1), (64, 4096), 16).reshape(-1)
    counts = torch.bincount(big, minlength=16).float()
    assert (counts / counts.mean() - 1).abs().max() < 0.05
    assert not torch.equal(tf.randint(tf.key(8), (8, 64), 1000), full)
    assert int(tf.randint(k, (4, 4), 1).max()) == 0                      # span 1
    assert int(tf.randint(k, (64, 64), 128256).max()) < 128256           # a span that is not a power of two


def test_synthetic_stream_resumes_and_shards():
    from mintext_b200.train import _SyntheticStream

    c = MinTextConfig(vocab_size=500, seq_length=16, seed=3, synthetic_shift_targets=True)
    whole = _SyntheticStream(c, 4, 0, torch.device("cpu"))
    batches = [whole.next() for _ in range(3)]
    assert torch.equal(batches[0]["target_tokens"], batches[0]["input_tokens"].roll(-1, dims=1))
    assert not torch.equal(batches[0]["input_tokens"], batches[1]["input_tokens"])
    resumed = _SyntheticStream(c, 4, 0, torch.device("cpu"))
    resumed.skip(2)
    assert torch.equal(resumed.next()["input_tokens"], batches[2]["input_tokens"])
    # two data-parallel ranks with two rows each see the halves of the four-row global batch
    r0, r1 = (_SyntheticStream(c, 2, r, torch.device("cpu")).next()["input_tokens"] for r in (0, 1))
    assert torch.equal(torch.cat([r0, r1]), batches[0]["input_tokens"])
    legacy = _SyntheticStream(c.model_copy(update={"synthetic_rng": "torch"}), 4, 0, torch.device("cpu")).next()
    assert legacy["input_tokens"].shape == (4, 16)

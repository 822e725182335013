"""Runs under ``MT_DEBUG_BOUNDS=1`` (the range-checked build of the kernels): ragged and odd shapes through the ops
that index memory with values read from memory must leave the bounds report clean; deliberately bad indices must be
reported with their value and limit while the accesses themselves are skipped, so nothing faults and the context
stays usable."""

import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def main() -> None:
    from mintext_b200 import MinTextConfig
    from mintext_b200.models import Transformer
    from mintext_b200.ops import moe as moe_ops
    from mintext_b200.ops._ext import check_bounds, check_status, debug_bounds_enabled, ext
    from mintext_b200.parallel.engine import TrainEngine

    assert debug_bounds_enabled() and ext().debug_bounds_units() >= 4, "not the range-checked build"
    out = {"units": int(ext().debug_bounds_units())}
    dev = "cuda"
    torch.manual_seed(0)

    # 1. clean runs: ragged expert loads (empty experts, one-row experts), odd token counts, a whole training step
    for n_tok, E, K in ((37, 8, 2), (1000, 16, 4), (129, 4, 1)):
        x = torch.randn(n_tok, 256, device=dev, dtype=torch.bfloat16)
        idx = torch.randint(0, E, (n_tok, K), device=dev)
        idx[:, 0] = torch.where(idx[:, 0] == 1, torch.zeros_like(idx[:, 0]), idx[:, 0])  # expert 1 mostly idle
        w = torch.rand(n_tok, K, device=dev)
        gu = (torch.randn(E, 256, 256, device=dev) * 0.05).bfloat16()
        dn = (torch.randn(E, 128, 256, device=dev) * 0.05).bfloat16()
        y = moe_ops.experts_forward(x.requires_grad_(True), idx, w, gu.requires_grad_(True), dn.requires_grad_(True), "silu")
        y.float().sum().backward()
    cfg = MinTextConfig(num_hidden_layers=2, hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                        intermediate_size=512, vocab_size=1000, seq_length=128, num_experts=8, num_experts_per_tok=2,
                        moe_intermediate_size=128, n_group=4, topk_group=2, first_k_dense_replace=1, n_shared_experts=1,
                        enable_tensorboard=False, enable_checkpointing=False, tie_word_embeddings=True)
    eng = TrainEngine(Transformer(cfg, rngs=0), cfg, device=dev)
    tok = torch.randint(0, cfg.vocab_size, (2, cfg.seq_length), device=dev)
    losses = [float(eng.train_step({"input_tokens": tok, "target_tokens": tok.roll(-1, 1)}, num_micro=1)["loss"]) for _ in range(2)]
    eng.check()
    check_bounds()
    out["clean_losses"] = losses

    # 2. bad indices are reported, not dereferenced
    table = torch.randn(100, 64, device=dev, dtype=torch.bfloat16)
    ids = torch.tensor([[3, 99, 100, 7]], device=dev)            # 100 is one past the table
    emb = torch.zeros(4, 64, device=dev, dtype=torch.bfloat16)
    ext().embedding_fwd(table, ids.reshape(-1), emb, 1.0)
    torch.cuda.synchronize()
    try:
        check_bounds()
        out["embedding_report"] = None
    except IndexError as e:
        out["embedding_report"] = str(e)
    assert torch.equal(emb[0], table[3]) and torch.equal(emb[1], table[99]) and torch.equal(emb[3], table[7])
    assert torch.count_nonzero(emb[2]).item() == 0                # the bad row was skipped

    pos = torch.tensor([0, 5, 2, 1], device=dev)                  # 5 is beyond the 3 rows of y
    yrows = torch.ones(3, 64, device=dev, dtype=torch.bfloat16)
    res, _ = ext().moe_combine_rows(yrows, pos, None, 2, 2, True, None)
    torch.cuda.synchronize()
    try:
        check_bounds()
        out["combine_report"] = None
    except IndexError as e:
        out["combine_report"] = str(e)
    assert res[0].float().sum().item() == 64.0 and res[1].float().sum().item() == 128.0   # one slot dropped, two kept
    check_bounds()            # reports were reset: clean again
    check_status()
    # the context is still healthy
    assert torch.allclose((torch.ones(8, device=dev) * 2).sum(), torch.tensor(16.0, device=dev))
    print(json.dumps(out))


if __name__ == "__main__":
    main()

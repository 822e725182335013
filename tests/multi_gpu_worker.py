"""Worker for the multi-GPU tests (launched with torch.distributed.run, one process per GPU).

Trains a small Llama-style model for a few steps three ways from the same initial weights and global batch:
peer-memory optimizer kernels, NCCL composition, and writes the per-step losses of each to a JSON file.
"""

import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def main(out_path: str) -> None:
    rank = int(os.environ["RANK"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from mintext_b200 import MinTextConfig
    from mintext_b200.models import Transformer
    from mintext_b200.parallel.engine import TrainEngine, local_batch_rows

    world = dist.get_world_size()
    results = {}
    g = torch.Generator().manual_seed(7)
    global_tok = torch.randint(0, 1024, (8, 128), generator=g)
    lo, hi = local_batch_rows(8, world, rank)
    tok = global_tok[lo:hi].to(dev)
    for name, fused in (("fused", True), ("nccl", False), ("muon", False), ("muon_peer", True)):
        cfg = MinTextConfig(optimizer="muon" if name.startswith("muon") else "adamw",
                            num_hidden_layers=2, hidden_size=256, num_attention_heads=4, num_key_value_heads=2,
                            head_dim=64, intermediate_size=512, vocab_size=1024, seq_length=128, steps=20,
                            learning_rate=1e-3, enable_tensorboard=False, enable_checkpointing=False,
                            fused_collectives=fused)
        eng = TrainEngine(Transformer(cfg, rngs=0), cfg, device=dev)
        if name.startswith("muon"):  # Muon's own publication: peer loads (fused collectives) or the NCCL all-gather
            assert (eng._muon_comm is not None) == fused, name
        else:
            assert eng.use_fused == fused, (name, eng.use_fused)
        if name.startswith("muon"):  # matrix-aligned shards: no parameter straddles two ranks' optimizer shards
            for sl in eng.big.slots:
                assert sl.offset // eng.shard_size == (sl.offset + sl.numel - 1) // eng.shard_size, sl.name
        losses, norms = [], []
        for _ in range(5):
            out = eng.train_step({"input_tokens": tok, "target_tokens": tok}, num_micro=1)
            losses.append(float(out["loss"]))
            norms.append(float(out["grad_norm"]))
        eng.check()
        # every rank must hold identical parameters after the publication step
        flat = eng.param_flat.float()
        ref = flat.clone()
        dist.broadcast(ref, src=0)
        assert torch.equal(flat, ref), f"{name}: parameters diverged across ranks"
        results[name] = {"losses": losses, "grad_norms": norms}
    if rank == 0:
        Path(out_path).write_text(json.dumps(results))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1])

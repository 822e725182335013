"""Worker for the checkpoint resharding GPU test: trains on all ranks, saves the engine state (flat fp32 master
and moments written as one chunk per rank), trains on, and records the losses after the save."""

import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def ckpt_config(ckpt_dir: str, optimizer: str = "adamw"):
    from mintext_b200 import MinTextConfig

    return MinTextConfig(optimizer=optimizer, num_hidden_layers=2, hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                         intermediate_size=512, vocab_size=1024, seq_length=128, steps=20, learning_rate=1e-3,
                         enable_tensorboard=False, enable_checkpointing=True, checkpoint_dir=ckpt_dir,
                         checkpoint_period=1, async_checkpointing=False)


def global_batch():
    return torch.randint(0, 1024, (8, 128), generator=torch.Generator().manual_seed(7))


def main(ckpt_dir: str, out_path: str, optimizer: str = "adamw") -> None:
    rank = int(os.environ["RANK"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from mintext_b200.checkpoint.manager import create_checkpoint_manager, save_checkpoint, wait_for_checkpoint
    from mintext_b200.models import Transformer
    from mintext_b200.parallel.engine import TrainEngine, local_batch_rows

    world = dist.get_world_size()
    cfg = ckpt_config(ckpt_dir, optimizer)
    eng = TrainEngine(Transformer(cfg, rngs=0), cfg, device=dev)
    lo, hi = local_batch_rows(8, world, rank)
    tok = global_batch()[lo:hi].to(dev)
    batch = {"input_tokens": tok, "target_tokens": tok}
    for _ in range(3):
        eng.train_step(batch, num_micro=1)
    mgr = create_checkpoint_manager(cfg)
    save_checkpoint(mgr, 3, eng, force=True)
    wait_for_checkpoint(mgr)
    after = [float(eng.train_step(batch, num_micro=1)["loss"]) for _ in range(3)]
    eng.check()
    if rank == 0:
        Path(out_path).write_text(json.dumps({"after": after, "world": world}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main(*sys.argv[1:4])

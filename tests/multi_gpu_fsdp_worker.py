"""Worker for the parameter-sharded engine test (torch.distributed.run, one process per GPU).

Trains the same small Llama-style model from the same weights and global batch in the resident mode and in the
parameter-sharded mode (layer weights gathered one layer ahead, layer gradients reduce-scattered per layer), with one
and with two micro-batches per step and with full rematerialisation, and writes losses, gradient norms and the largest
difference between the final fp32 master weights of the two modes.
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
    from mintext_b200.parallel.fsdp import ParamShardedEngine

    world = dist.get_world_size()
    g = torch.Generator().manual_seed(7)
    global_tok = torch.randint(0, 1024, (16, 128), generator=g)
    lo, hi = local_batch_rows(16, world, rank)
    tok = global_tok[lo:hi].to(dev)
    results = {}
    for case, n_micro, remat in (("one_micro", 1, "none"), ("two_micro", 2, "none"), ("remat", 2, "full")):
        runs = {}
        for mode in ("resident", "sharded"):
            cfg = MinTextConfig(num_hidden_layers=5, hidden_size=256, num_attention_heads=4, num_key_value_heads=2,
                                head_dim=64, intermediate_size=512, vocab_size=1024, seq_length=128, steps=20,
                                learning_rate=1e-3, enable_tensorboard=False, enable_checkpointing=False,
                                remat_policy=remat, fsdp_shard_params=(mode == "sharded"))
            torch.cuda.reset_peak_memory_stats(dev)
            cls = ParamShardedEngine if mode == "sharded" else TrainEngine
            eng = cls(Transformer(cfg, rngs=0), cfg, device=dev)
            losses, norms = [], []
            for _ in range(5):
                out = eng.train_step({"input_tokens": tok, "target_tokens": tok.roll(-1, dims=1)}, num_micro=n_micro)
                losses.append(float(out["loss"]))
                norms.append(float(out["grad_norm"]))
            ev = float(eng.eval_step({"input_tokens": tok, "target_tokens": tok.roll(-1, dims=1)})["eval_loss"])
            eng.check()
            runs[mode] = {"losses": losses, "grad_norms": norms, "eval_loss": ev,
                          "master": eng.named_master_parameters()}
            if mode == "sharded":
                assert eng.param_flat is None and eng.grad_flat is None
                # a rank persists 1/world of the layer weights; the staging buffers hold two layers
                layer_elems = sum(s.numel for s in eng.big.slots if s.bucket != eng._res_index)
                assert eng.stage_param.numel() < layer_elems
                eng.close()
            del eng
        diffs = [(runs["resident"]["master"][k].float() - v.float()).abs() for k, v in runs["sharded"]["master"].items()]
        diff = max(float(d.max()) for d in diffs)
        mean = sum(float(d.sum()) for d in diffs) / sum(d.numel() for d in diffs)
        results[case] = {m: {k: v for k, v in r.items() if k != "master"} for m, r in runs.items()}
        results[case]["max_master_diff"] = diff
        results[case]["mean_master_diff"] = mean
    if rank == 0:
        Path(out_path).write_text(json.dumps(results))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1])

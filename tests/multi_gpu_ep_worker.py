"""Worker for the expert-parallel GPU test (one process per GPU): trains a small MoE model with the experts
distributed over all ranks, once with the peer-memory token exchange and once with the collective exchange."""

import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def moe_config(fused: bool, ep: int):
    from mintext_b200 import MinTextConfig

    return MinTextConfig(num_hidden_layers=2, hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                         intermediate_size=512, vocab_size=1024, seq_length=128, steps=20, learning_rate=1e-3,
                         num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128, n_group=4, topk_group=2,
                         first_k_dense_replace=1, n_shared_experts=1, enable_tensorboard=False,
                         enable_checkpointing=False, fused_collectives=fused, ici_expert_parallelism=ep)


def main(out_path: str) -> None:
    rank = int(os.environ["RANK"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from mintext_b200.models import Transformer
    from mintext_b200.parallel.engine import TrainEngine, local_batch_rows
    from mintext_b200.parallel.ep import ExpertParallel, set_current_ep

    world = dist.get_world_size()
    g = torch.Generator().manual_seed(7)
    global_tok = torch.randint(0, 1024, (8, 128), generator=g)
    lo, hi = local_batch_rows(8, world, rank)
    tok = global_tok[lo:hi].to(dev)
    results = {}
    # "peer": dispatch by peer stores, down projection fused with the combine all-to-all (one kernel);
    # "peer_unfused": the same exchange with the combine as a separate pull kernel; "collective": NCCL baseline
    # "peer_tight": receive buffers smaller than the rows routed to a rank - the excess rows are dropped cleanly
    for name, fused, fuse_combine in (("peer", True, "1"), ("peer_unfused", True, "0"), ("collective", False, "1"),
                                      ("peer_tight", True, "1")):
        os.environ["MT_EP_FUSED_COMBINE"] = fuse_combine
        cfg = moe_config(fused, world)
        capacity = 0.62 if name == "peer_tight" else cfg.moe_capacity_factor
        ep = ExpertParallel(dist.group.WORLD, dev, capacity, fused=fused)
        set_current_ep(ep)
        eng = TrainEngine(Transformer(cfg, rngs=0), cfg, device=dev)
        assert len(eng.exp.slots) == 2, [s.name for s in eng.exp.slots]
        losses = []
        for _ in range(5):
            out = eng.train_step({"input_tokens": tok, "target_tokens": tok}, num_micro=1)
            losses.append(float(out["loss"]))
        eng.check()
        ep.check_overflow()
        if fused:  # the fused expert-GEMM + combine kernel ran exactly where it was asked for
            assert (getattr(ep, "fused_combines", 0) > 0) == (fuse_combine == "1"), (name, getattr(ep, "fused_combines", 0))
        dropped = torch.tensor([ep.dropped_rows() if fused else 0], device=dev)
        dist.all_reduce(dropped)
        results[name] = {"losses": losses, "grad_norm": float(out["grad_norm"]), "dropped": int(dropped.item())}
        set_current_ep(None)
    if rank == 0:
        Path(out_path).write_text(json.dumps(results))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1])

"""Worker for the tensor-parallel GPU test (one process per GPU, all ranks in one tensor-parallel group).

Part 1 compares the fused projections (gather folded into the GEMM, GEMM scattering its tiles) with the NCCL
composition on random data, values and gradients.  Part 2 trains a small model with both variants."""

import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


MIXED = {  # families with multi-head-latent attention / Gated Delta Rule layers and mixture-of-experts blocks
    "deepseek": dict(model_type="deepseek_v3", attention_type="mla", q_lora_rank=128, kv_lora_rank=128,
                     qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, num_experts=8, num_experts_per_tok=2,
                     moe_intermediate_size=128, n_group=4, topk_group=2, first_k_dense_replace=1, n_shared_experts=1),
    "qwen3_next": dict(model_type="qwen3_next", use_qk_norm=True, full_attention_interval=2, partial_rotary_factor=0.25,
                       linear_key_head_dim=64, linear_value_head_dim=64, linear_num_key_heads=2,
                       linear_num_value_heads=4, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=128,
                       n_group=1, topk_group=1, first_k_dense_replace=0, router_type="softmax_topk",
                       shared_expert_gate=True, n_shared_experts=1, router_aux_loss_coef=0.01),
    # embedding table and output head sharded over the vocabulary as well (z-loss on, so every softmax reduction counts)
    "vocab_parallel": dict(tp_vocab_parallel=True, z_loss_weight=1e-4),
}


def tp_config(fused: bool, tp: int, kind: str = "dense"):
    from mintext_b200 import MinTextConfig

    extra = MIXED.get(kind, {})
    return MinTextConfig(**extra, num_hidden_layers=2, hidden_size=512, num_attention_heads=8, num_key_value_heads=8, head_dim=64,
                         intermediate_size=1024, vocab_size=1024, seq_length=128, steps=20, learning_rate=1e-3,
                         enable_tensorboard=False, enable_checkpointing=False, fused_collectives=fused,
                         ici_tensor_parallelism=tp)


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))


def op_level(dev, rank, world):
    from mintext_b200.parallel import tp as tpm

    fused = tpm.TensorParallel(dist.group.WORLD, dev, fused=True)
    plain = tpm.TensorParallel(dist.group.WORLD, dev, fused=False)
    g = torch.Generator().manual_seed(100 + rank)
    Tl, K = 512, 256
    errs = {}
    for trial in range(3):  # several calls: exercises the parity double-buffering
        x = (torch.randn(Tl, K, generator=g) * 0.5).to(dev, torch.bfloat16)
        gw = torch.Generator().manual_seed(5 + trial)
        ws = [(torch.randn(K, n, generator=gw) / 16).to(dev, torch.bfloat16) for n in (384, 128)]
        wo = (torch.randn(384, K, generator=gw) / 16).to(dev, torch.bfloat16)
        outs = {}
        for name, ctx in (("fused", fused), ("plain", plain)):
            xx = x.clone().requires_grad_(True)
            wl = [w.clone().requires_grad_(True) for w in ws]
            wol = wo.clone().requires_grad_(True)
            xg, (a, b) = tpm.column_linear(xx, wl, ctx, torch.bfloat16)
            y = tpm.row_linear(torch.tanh(a.float()).to(torch.bfloat16), wol, ctx, torch.bfloat16)
            loss = (y.float() ** 2).sum() + (b.float() ** 2).sum() * 0.1
            loss.backward()
            outs[name] = [xg.detach(), a.detach(), b.detach(), y.detach(), xx.grad, wl[0].grad, wl[1].grad, wol.grad]
        for i, key in enumerate(("gathered", "col0", "col1", "row", "dx", "dw0", "dw1", "dwo")):
            errs[key] = max(errs.get(key, 0.0), _rel(outs["fused"][i], outs["plain"][i]))
    # fully sharded weight: gather inside the GEMM vs an explicit all-gather + matmul
    from mintext_b200.ops import tp_gemm

    gw = torch.Generator().manual_seed(11)
    K, N, T = 256 * world, 384, 640
    w = (torch.randn(K, N, generator=gw) / 16).to(torch.bfloat16)
    sw = tp_gemm.ShardedWeight(w, dist.group.WORLD, dev)
    for trial in range(2):
        x = (torch.randn(T, K, generator=g) * 0.5).to(dev, torch.bfloat16).requires_grad_(True)
        y = tp_gemm.fsdp_linear(x, sw)
        (y.float() ** 2).sum().backward()
        xr = x.detach().clone().requires_grad_(True)
        wr = w.to(dev).float().requires_grad_(True)
        yr = xr.float() @ wr
        (yr ** 2).sum().backward()
        dwr = wr.grad.clone()
        dist.all_reduce(dwr)
        rows = K // world
        errs["fsdp_y"] = max(errs.get("fsdp_y", 0.0), _rel(y, yr))
        errs["fsdp_dx"] = max(errs.get("fsdp_dx", 0.0), _rel(x.grad, xr.grad))
        errs["fsdp_dw"] = max(errs.get("fsdp_dw", 0.0), _rel(sw.shard.grad, dwr[rank * rows:(rank + 1) * rows]))
        sw.shard.grad = None
    return errs


def main(out_path: str, kind: str = "dense") -> None:
    rank = int(os.environ["RANK"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from mintext_b200.models import Transformer
    from mintext_b200.ops._ext import check_status
    from mintext_b200.parallel.engine import TrainEngine
    from mintext_b200.parallel.tp import TensorParallel, set_current_tp

    world = dist.get_world_size()
    results = {}
    if kind == "dense":
        results["ops"] = op_level(dev, rank, world)
        check_status(dev)
        assert results["ops"]["gathered"] == 0.0 and all(v < 2e-2 for v in results["ops"].values()), results["ops"]
    g = torch.Generator().manual_seed(7)
    tok = torch.randint(0, 1024, (8, 128), generator=g).to(dev)  # one tensor-parallel group: all ranks share the batch
    for name, fused in (("fused", True), ("nccl", False)) if kind == "dense" else (("fused", True),):
        cfg = tp_config(fused, world, kind)
        set_current_tp(TensorParallel(dist.group.WORLD, dev, fused=fused))
        eng = TrainEngine(Transformer(cfg, rngs=0), cfg, device=dev)
        losses = []
        for _ in range(5):
            out = eng.train_step({"input_tokens": tok, "target_tokens": tok}, num_micro=1)
            losses.append(float(out["loss"]))
        eng.check()
        results[name] = {"losses": losses, "grad_norm": float(out["grad_norm"])}
        set_current_tp(None)
    if rank == 0:
        Path(out_path).write_text(json.dumps(results))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main(*sys.argv[1:3])

"""Library-composed comparator for the headline benchmark: the same Llama-shaped model and training step written
with stock PyTorch pieces only - cuBLAS matmuls (``torch.nn.functional.linear``), the fused scaled-dot-product
attention that ships with torch (flash / cuDNN backend), ``torch.optim.AdamW(fused=True)`` and, on several GPUs,
torch's own FSDP (``fully_shard``, NCCL all-gather / reduce-scatter) or DDP.  None of this repository's kernels,
modules or engine is imported here.

It is NOT the reference (which is a JAX program and cannot run on this image); it stands in for "a framework
that composes vendor libraries" on the same box, same shapes, same batch, same optimizer, same precision policy
(bf16 compute, fp32 master weights and optimizer state), so that ``bench.py --impl library`` gives the headline
number something measured on identical hardware to stand against.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        return F.rms_norm(x.float(), (x.shape[-1],), self.weight.float(), self.eps).to(x.dtype)


def _rope_tables(seq: int, dim: int, theta: float, device):
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, device=device, dtype=torch.float32) / dim))
    ang = torch.outer(torch.arange(seq, device=device, dtype=torch.float32), inv)
    return ang.cos(), ang.sin()


def _apply_rope(x, cos, sin):  # x [B, H, S, dh], rotate-half convention
    x1, x2 = x.float().chunk(2, dim=-1)
    c, s = cos[None, None], sin[None, None]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


class Block(nn.Module):
    def __init__(self, d, heads, kv_heads, dh, ffn, eps):
        super().__init__()
        self.heads, self.kv_heads, self.dh = heads, kv_heads, dh
        self.norm1, self.norm2 = RMSNorm(d, eps), RMSNorm(d, eps)
        self.q = nn.Linear(d, heads * dh, bias=False)
        self.k = nn.Linear(d, kv_heads * dh, bias=False)
        self.v = nn.Linear(d, kv_heads * dh, bias=False)
        self.o = nn.Linear(heads * dh, d, bias=False)
        self.gate = nn.Linear(d, ffn, bias=False)
        self.up = nn.Linear(d, ffn, bias=False)
        self.down = nn.Linear(ffn, d, bias=False)

    def forward(self, x, cos, sin):
        B, S, _ = x.shape
        h = self.norm1(x)
        q = self.q(h).view(B, S, self.heads, self.dh).transpose(1, 2)
        k = self.k(h).view(B, S, self.kv_heads, self.dh).transpose(1, 2)
        v = self.v(h).view(B, S, self.kv_heads, self.dh).transpose(1, 2)
        q, k = _apply_rope(q, cos, sin), _apply_rope(k, cos, sin)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=self.heads != self.kv_heads)
        x = x + self.o(a.transpose(1, 2).reshape(B, S, self.heads * self.dh))
        h = self.norm2(x)
        return x + self.down(F.silu(self.gate(h)) * self.up(h))


class Llama(nn.Module):
    def __init__(self, vocab, d, layers, heads, kv_heads, dh, ffn, eps=1e-5, theta=500000.0, tied=True):
        super().__init__()
        self.embed = nn.Embedding(vocab, d)
        self.blocks = nn.ModuleList([Block(d, heads, kv_heads, dh, ffn, eps) for _ in range(layers)])
        self.norm = RMSNorm(d, eps)
        self.head = None if tied else nn.Linear(d, vocab, bias=False)
        self.dh, self.theta = dh, theta
        for p in self.parameters():
            if p.dim() >= 2:
                nn.init.normal_(p, std=0.02)

    def forward(self, tokens, targets):
        cos, sin = _rope_tables(tokens.shape[1], self.dh, self.theta, tokens.device)
        x = self.embed(tokens)
        for blk in self.blocks:
            x = blk(x, cos, sin)
        x = self.norm(x)
        w = self.embed.weight if self.head is None else self.head.weight
        logits = F.linear(x, w.to(x.dtype) if w.dtype != x.dtype else w)
        return F.cross_entropy(logits.float().view(-1, logits.shape[-1]), targets.reshape(-1))


LLAMA_1B = dict(vocab=128256, d=2048, layers=16, heads=32, kv_heads=8, dh=64, ffn=8192, eps=1e-5, theta=500000.0,
                tied=True)


class LibraryTrainer:
    """``step(tokens [rows, S]) -> loss``: micro-batches of ``micro_batch`` rows with gradient accumulation, global
    norm clip at 1.0, fused AdamW with a cosine schedule - the optimizer settings of the headline run."""

    def __init__(self, shape: dict, device, world: int, micro_batch: int, lr: float = 3e-4, total_steps: int = 10):
        torch.manual_seed(0)
        self.world, self.micro_batch = world, micro_batch
        self.parallel = "single"
        model = Llama(**shape).to(device)
        if world > 1:
            try:
                from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

                mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
                for blk in model.blocks:
                    fully_shard(blk, mp_policy=mp)
                fully_shard(model, mp_policy=mp)
                self.parallel = f"torch fully_shard (FSDP2) over {world}"
            except Exception:
                from torch.nn.parallel import DistributedDataParallel as DDP

                model = DDP(model, device_ids=[device.index])
                self.parallel = f"torch DDP over {world}"
        self.model = model
        self.autocast = self.parallel.startswith("single") or "DDP" in self.parallel  # FSDP2 casts by policy
        self.opt = torch.optim.AdamW(model.parameters(), lr=lr, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1,
                                     fused=device.type == "cuda")
        warm = max(int(0.1 * total_steps), 1)
        self.sched = torch.optim.lr_scheduler.LambdaLR(self.opt, lambda s: min(1.0, (s + 1) / warm) * (
            0.1 + 0.9 * 0.5 * (1 + math.cos(math.pi * min(s, total_steps) / max(total_steps, 1)))))

    def _sync_gradients(self, on: bool) -> None:
        if hasattr(self.model, "set_requires_gradient_sync"):      # FSDP2
            self.model.set_requires_gradient_sync(on)
        elif hasattr(self.model, "require_backward_grad_sync"):    # DDP
            self.model.require_backward_grad_sync = on

    # the engine interface bench.py drives
    def train_step(self, batch: dict, num_micro: int | None = None) -> dict:
        return {"loss": self.step(batch["input_tokens"])}

    def check(self) -> None:
        pass

    def step(self, tokens: torch.Tensor) -> torch.Tensor:
        rows = tokens.shape[0]
        n = max(rows // self.micro_batch, 1)
        total = torch.zeros((), device=tokens.device)
        self.opt.zero_grad(set_to_none=True)
        for i in range(n):
            tok = tokens[i * self.micro_batch:(i + 1) * self.micro_batch]
            self._sync_gradients(i == n - 1)  # communicate gradients on the last micro-batch only
            with torch.autocast("cuda" if tok.is_cuda else "cpu", dtype=torch.bfloat16, enabled=self.autocast):
                loss = self.model(tok, tok.roll(-1, dims=1))
            (loss / n).backward()
            total += loss.detach()
        torch.nn.utils.clip_grad_norm_(self.model.parameters(), 1.0)
        self.opt.step()
        self.sched.step()
        return total / n

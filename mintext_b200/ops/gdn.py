"""CUDA front-end of the chunked Gated Delta Rule (falls back to the oracle until the kernels are loaded)."""

from __future__ import annotations

import torch

from . import functional as F
from ._ext import ext


def cuda_path(q: torch.Tensor) -> bool:
    return q.is_cuda and F._backend() != "oracle" and hasattr(ext(), "gdn_chunk_fwd")


def chunk_gated_delta_rule_cuda(q, k, v, beta, g, chunk_size=64):  # pragma: no cover - needs a GPU
    raise NotImplementedError

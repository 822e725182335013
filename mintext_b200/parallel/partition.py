"""Model construction under a mesh (reference: mintext/distributed/partition.py)."""

from __future__ import annotations


def create_sharded_model(config, mesh=None, model_cls=None):
    """Build the model from ``config.seed``.  Parameters are created on the host in ``weight_dtype``; the
    training engine places them (flat bf16 compute copy per rank, fp32 master and optimizer state sharded)."""
    if model_cls is None:
        from mintext_b200.models import Transformer as model_cls
    return model_cls(config, rngs=int(config.seed), mesh=mesh)

"""Model construction under a mesh (reference: mintext/distributed/partition.py)."""

from __future__ import annotations


def create_sharded_model(config, mesh=None, model_cls=None, init_device=None):
    """Build the model from ``config.seed`` in ``weight_dtype``; the training engine places the parameters (flat
    bf16 compute copy per rank, fp32 master and optimizer state sharded).  Parameters are drawn on the host unless
    ``init_device`` names a GPU, in which case the large tensors are sampled there (see
    :class:`mintext_b200.modules.linear.init_on_device`)."""
    if model_cls is None:
        from mintext_b200.models import Transformer as model_cls
    from mintext_b200.modules.linear import init_on_device

    with init_on_device(init_device):
        return model_cls(config, rngs=int(config.seed), mesh=mesh)

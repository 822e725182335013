"""The reference keeps its decoder in ``mintext/models/base.py``; here it lives in :mod:`.transformer`.  This module
serves imports of the old location with the same objects."""

from .transformer import (  # noqa: F401
    REMAT_POLICIES,
    DecoderLayer,
    Transformer,
    _all_layers_scannable,
    apply_layer_with_remat,
    make_causal_mask,
)

_apply_layer_with_remat = apply_layer_with_remat

__all__ = ["Transformer", "DecoderLayer", "make_causal_mask", "apply_layer_with_remat", "REMAT_POLICIES"]

"""Compatibility shim for the reference's TPU flag presets (mintext/utils/xla_flags.py).

There is no XLA in this framework, so nothing here changes how kernels run; the functions exist so that configs
and launch scripts written for the reference (``tpu_type``, ``xla_flags``, ``MINTEXT_TPU_TYPE``) keep working.
``get_flags_for_device`` returns an empty preset for every device type, ``set_xla_flags`` records the user's
extra flags in ``LIBTPU_INIT_ARGS`` unchanged and returns them.
"""

from __future__ import annotations

import os

KNOWN_TPU_TYPES = ("v4", "v5e", "v5p", "v6e", "v6p")


def detect_tpu_type() -> str | None:
    """TPU generation from ``MINTEXT_TPU_TYPE`` / ``TPU_ACCELERATOR_TYPE`` if any, else None (always None on a
    GPU machine)."""
    for var in ("MINTEXT_TPU_TYPE", "TPU_ACCELERATOR_TYPE"):
        v = os.environ.get(var, "").lower()
        for t in KNOWN_TPU_TYPES:
            if v.startswith(t):
                return t
    return None


def get_flags_for_device(tpu_type: str = "auto", num_slices: int = 1) -> str:
    return ""


def set_xla_flags(tpu_type: str = "auto", num_slices: int = 1, extra_flags: str = "") -> str:
    flags = (get_flags_for_device(tpu_type, num_slices) + " " + (extra_flags or "")).strip()
    if flags:
        os.environ["LIBTPU_INIT_ARGS"] = flags
    return flags

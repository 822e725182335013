"""Loader for the compiled extension.

The CUDA path is mandatory on a GPU machine: if a CUDA device is present and the extension cannot be loaded,
:func:`ext` raises instead of silently falling back to PyTorch ops.
"""

from __future__ import annotations

import importlib.util
import os
import threading
from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parents[1]
_lock = threading.Lock()
_mods: dict[str, object] = {}
_status: dict[int, torch.Tensor] = {}

STATUS_MESSAGES = {
    0: "ok",
    1: "timeout waiting for a TMA stage (full barrier)",
    2: "timeout waiting for a free stage (empty barrier)",
    3: "timeout waiting for an accumulator (tmem full)",
    4: "timeout waiting for the epilogue (tmem empty)",
    5: "timeout waiting for a global-memory flag",
    6: "bad kernel arguments",
}


def _load(name: str):
    with _lock:
        if name in _mods:
            return _mods[name]
        path = _PKG / f"{name}.so"
        if not path.exists():
            from . import build

            if name == "_mt_C_dbg":
                build.build_cuda(debug_bounds=True)
            else:
                (build.build_cuda if name == "_mt_C" else build.build_io)()
        spec = importlib.util.spec_from_file_location(name, path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        if name in ("_mt_C", "_mt_C_dbg"):
            from . import launch_counter

            launch_counter.install(mod)
        _mods[name] = mod
        return mod


def debug_bounds_enabled() -> bool:
    """True when ``MT_DEBUG_BOUNDS=1`` selects the range-checked build of the kernels."""
    return os.environ.get("MT_DEBUG_BOUNDS", "0") == "1"


def ext():
    """The CUDA extension module (built on first use when the shared object is missing).  With
    ``MT_DEBUG_BOUNDS=1`` this is the build whose kernels range-check every index they read from memory."""
    return _load("_mt_C_dbg" if debug_bounds_enabled() else "_mt_C")


def check_bounds(reset: bool = True) -> None:
    """Debug-bounds build: raise if any kernel met an out-of-range index (the access itself was skipped); a no-op
    report in the ordinary build.  Synchronises."""
    torch.cuda.synchronize()
    rep = ext().debug_bounds_report()
    if rep:
        if reset:
            ext().debug_bounds_reset()
        msgs = [f"{Path(f).name}:{line}: index {idx} outside [0, {lim})" for f, line, idx, lim in rep]
        raise IndexError("out-of-range index in a kernel: " + "; ".join(msgs))


def io_ext():
    """The host-only C++ runtime module, or None when it has not been built and cannot be."""
    try:
        return _load("_mt_io")
    except Exception:  # pragma: no cover - the pure-Python paths take over
        return None


def cuda_available() -> bool:
    return torch.cuda.is_available()


def status_word(device: torch.device | int | None = None) -> torch.Tensor:
    """Per-device int32 word that kernels with bounded waits write an error code to."""
    idx = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    if idx not in _status:
        _status[idx] = torch.zeros(4, dtype=torch.int32, device=f"cuda:{idx}")
    return _status[idx]


def check_status(device=None) -> None:
    """Synchronously read the status word; raise if any kernel recorded a bounded-wait expiry."""
    code = int(status_word(device)[0].item())
    if code != 0:
        status_word(device).zero_()
        raise RuntimeError(f"mintext_b200 kernel error {code}: {STATUS_MESSAGES.get(code, 'unknown')}")

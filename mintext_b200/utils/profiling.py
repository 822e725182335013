"""Step-window profiler (reference: mintext/utils/profiling.py, which wraps jax.profiler).

Traces steps ``[skip_first_n_profiler_steps, skip_first_n_profiler_steps + profiler_steps)`` with
``torch.profiler`` (CPU + CUDA activities) and writes a Chrome trace under ``<base>/<run>/profiles``.
"""

from __future__ import annotations

import logging
from pathlib import Path

logger = logging.getLogger(__name__)

_NVTX = False


class nvtx_range:
    """NVTX range around a model region (per decoder layer, loss, optimizer step), emitted only while the profiler
    window is open on a CUDA device so that the steady-state loop pays nothing."""

    def __init__(self, name: str):
        self.name = name
        self.on = False

    def __enter__(self):
        if _NVTX:
            import torch

            torch.cuda.nvtx.range_push(self.name)
            self.on = True
        return self

    def __exit__(self, *exc):
        if self.on:
            import torch

            torch.cuda.nvtx.range_pop()
        return False


class Profiler:
    def __init__(self, config):
        self.enabled = bool(config.enable_profiler)
        self.start_step = int(config.skip_first_n_profiler_steps)
        self.end_step = self.start_step + int(config.profiler_steps)
        self.output_dir = str(Path(config.base_output_directory) / config.run_name / "profiles")
        self.active = False
        self._prof = None

    def maybe_activate(self, step: int) -> None:
        if self.enabled and not self.active and step == self.start_step:
            self._start()

    def maybe_deactivate(self, step: int) -> None:
        if self.active and step + 1 >= self.end_step:
            self.stop()

    def _start(self) -> None:
        import torch

        Path(self.output_dir).mkdir(parents=True, exist_ok=True)
        acts = [torch.profiler.ProfilerActivity.CPU]
        if torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        self._prof = torch.profiler.profile(activities=acts)
        self._prof.__enter__()
        self.active = True
        global _NVTX
        _NVTX = torch.cuda.is_available()
        logger.info("Profiler started, writing to %s", self.output_dir)

    def stop(self) -> None:
        if not self.active:
            return
        self._prof.__exit__(None, None, None)
        try:
            self._prof.export_chrome_trace(str(Path(self.output_dir) / "trace.json"))
        except Exception as e:  # pragma: no cover
            logger.warning("could not export trace: %s", e)
        self._prof = None
        self.active = False
        global _NVTX
        _NVTX = False
        logger.info("Profiler stopped")


def kernel_share_table(step_fn, header: str = "", top: int = 40) -> str:
    """Run ``step_fn()`` once under ``torch.profiler`` and return a text table of the device kernels by total time
    (calls, milliseconds, share of the summed kernel time).  Times taken under the profiler are for shares only."""
    import time
    from collections import defaultdict

    import torch
    from torch.profiler import ProfilerActivity, profile

    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
        t0 = time.time()
        step_fn()
        host_ms = (time.time() - t0) * 1e3
        torch.cuda.synchronize()
        wall_ms = (time.time() - t0) * 1e3
    agg = defaultdict(lambda: [0, 0.0])
    for ev in prof.events():
        if ev.device_type == torch.autograd.DeviceType.CUDA:
            a = agg[ev.name]
            a[0] += 1
            a[1] += ev.device_time
    total = sum(v[1] for v in agg.values()) or 1.0
    lines = [header] if header else []
    lines.append(f"under profiler: wall {wall_ms:.1f} ms, host issue time {host_ms:.1f} ms, sum of kernel time "
                 f"{total / 1e3:.1f} ms, launches {sum(v[0] for v in agg.values())}")
    lines.append(f"{'kernel':90s} {'calls':>6s} {'ms':>9s} {'share':>7s}")
    for name, (n, us) in sorted(agg.items(), key=lambda kv: -kv[1][1])[:top]:
        lines.append(f"{name[:90]:90s} {n:6d} {us / 1e3:9.2f} {us / total * 100:6.1f}%")
    return "\n".join(lines)

"""Console / TensorBoard / JSONL metric logging (reference: mintext/utils/logging.py).

Console line and TensorBoard tags are the reference's; the line additionally carries ``MFU=..%`` (the
reference's own benchmark runner greps for it) and, when given, the device-timed step.  Only rank 0 writes.
"""

from __future__ import annotations

import json
import logging
import os
from pathlib import Path
from typing import Any

from .pytree import calculate_tflops_per_device, calculate_tokens_per_device, count_params

logger = logging.getLogger("mintext_b200")

NOMINAL_BF16_TFLOPS = 2250.0  # B200 dense bf16


def peak_tflops() -> float:
    """Denominator for MFU: nominal B200 dense bf16 unless ``MINTEXT_PEAK_TFLOPS`` overrides it."""
    return float(os.environ.get("MINTEXT_PEAK_TFLOPS", NOMINAL_BF16_TFLOPS))


def _rank() -> int:
    return int(os.environ.get("RANK", "0"))


class MetricLogger:
    def __init__(self, config, params: Any = None):
        self.tflops_per_device = calculate_tflops_per_device(config)
        self.tokens_per_device = calculate_tokens_per_device(config)
        self.writer = None
        self.jsonl = None
        self.is_main = _rank() == 0
        if self.is_main and config.enable_tensorboard:
            try:
                from torch.utils.tensorboard import SummaryWriter

                Path(config.tensorboard_dir).mkdir(parents=True, exist_ok=True)
                self.writer = SummaryWriter(config.tensorboard_dir)
                logger.info("TensorBoard logging to %s", config.tensorboard_dir)
            except Exception as e:  # tensorboard not installed
                logger.warning("TensorBoard disabled: %s", e)
        if self.is_main and config.log_dir:
            try:
                Path(config.log_dir).mkdir(parents=True, exist_ok=True)
                self.jsonl = open(Path(config.log_dir) / "metrics.jsonl", "a")
            except OSError:
                self.jsonl = None
        if params is not None and self.is_main:
            n = count_params(params)
            logger.info("Model parameters: %s (%.2fM)", f"{n:,}", n / 1e6)
            logger.info("Estimated TFLOP/device/step: %.2f", self.tflops_per_device)
            logger.info("Tokens/device/step: %d", self.tokens_per_device)
            if self.writer is not None:
                self.writer.add_text("config/model_params", f"{n:,}")
                self.writer.add_text("config/model_name", config.model_name)

    def log_step(self, step: int, metrics: dict[str, Any], step_time: float) -> None:
        if not self.is_main:
            return
        loss = float(metrics["loss"])
        lr = float(metrics["learning_rate"])
        gn = float(metrics["grad_norm"])
        tflops = self.tflops_per_device / step_time if step_time > 0 else 0.0
        tps = self.tokens_per_device / step_time if step_time > 0 else 0.0
        mfu = 100.0 * tflops / peak_tflops()
        logger.info(
            "step=%d loss=%.4f lr=%.2e grad_norm=%.4f step_time=%.3fs TFLOP/s/device=%.1f tokens/s/device=%.0f MFU=%.1f%%",
            step, loss, lr, gn, step_time, tflops, tps, mfu)
        if self.writer is not None:
            w = self.writer
            w.add_scalar("learning/loss", loss, step)
            w.add_scalar("learning/learning_rate", lr, step)
            w.add_scalar("learning/grad_norm", gn, step)
            if metrics.get("param_norm") is not None:
                w.add_scalar("learning/param_norm", float(metrics["param_norm"]), step)
            w.add_scalar("perf/step_time_seconds", step_time, step)
            w.add_scalar("perf/tflops_per_sec_per_device", tflops, step)
            w.add_scalar("perf/tokens_per_sec_per_device", tps, step)
        if self.jsonl is not None:
            rec = {"step": step, "loss": loss, "lr": lr, "grad_norm": gn, "step_time": step_time,
                   "tflops_per_device": tflops, "tokens_per_sec_per_device": tps, "mfu_pct": mfu}
            if metrics.get("device_step_ms") is not None:
                rec["device_step_ms"] = float(metrics["device_step_ms"])
            self.jsonl.write(json.dumps(rec) + "\n")
            self.jsonl.flush()

    def close(self) -> None:
        if self.writer is not None:
            self.writer.close()
            self.writer = None
        if self.jsonl is not None:
            self.jsonl.close()
            self.jsonl = None

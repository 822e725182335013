"""Checkpoint manager (reference: mintext/checkpoint/manager.py, which wraps Orbax).

Layout on disk: ``<checkpoint_dir>/<step>/default/`` holds one raw little-endian file per leaf of the state
tree (``step``, ``params/<dotted name>``, ``opt_state/...``), named by the leaf path with ``/`` -> ``__``, plus
``_METADATA`` (JSON: path -> dtype, shape, file; a flat buffer saved by several ranks lists ``chunks`` with their
element ranges, a tensor- or expert-parallel parameter lists ``shards`` with the dimension it is split along, the
shard's index and the shard count, so that a restore under another parallel degree reassembles it along that
dimension) and, once everything is on disk,
``<step>/_CHECKPOINT_METADATA`` as the commit marker; a step without the marker is ignored (a crash mid-save
never yields a loadable half checkpoint).  Saves snapshot device tensors into pinned host memory and hand the
buffers to background writer threads (C++ when the native runtime is built), so training continues while files
are written.  Retention keeps the newest ``max_to_keep`` committed steps.

State objects: anything exposing ``checkpoint_tree() -> {path: tensor | int | float | dict}`` and
``load_checkpoint_tree(read)``; :class:`mintext_b200.trainer.TrainState` and the GPU ``TrainEngine`` both do.
"""

from __future__ import annotations

import json
import logging
import os
import shutil
import threading
from pathlib import Path

import numpy as np
import torch

logger = logging.getLogger(__name__)

_COMMIT = "_CHECKPOINT_METADATA"
_NP_OF = {torch.float32: np.float32, torch.float64: np.float64, torch.float16: np.float16, torch.int64: np.int64,
          torch.int32: np.int32, torch.int16: np.int16, torch.uint8: np.uint8, torch.bool: np.bool_,
          torch.bfloat16: np.uint16}


class CheckpointCorrupt(RuntimeError):
    """A committed checkpoint whose files do not match its metadata."""


def _rank() -> int:
    import torch.distributed as dist

    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def _world() -> int:
    import torch.distributed as dist

    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def _barrier() -> None:
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized():
        dist.barrier()


class _PyWriter:
    """Thread-based fallback of the native asynchronous writer."""

    def __init__(self, threads: int = 4):
        self._jobs: list[threading.Thread] = []
        self._errors: list[Exception] = []

    def submit(self, path: str, host: torch.Tensor) -> None:
        def run():
            try:
                tmp = path + ".tmp"
                arr = host.view(torch.uint8).numpy() if host.dtype == torch.bfloat16 else host.numpy()
                with open(tmp, "wb") as f:
                    f.write(arr.tobytes())
                    f.flush()
                    os.fsync(f.fileno())
                os.replace(tmp, path)
            except Exception as e:  # surfaced by wait()
                self._errors.append(e)

        t = threading.Thread(target=run, daemon=True)
        t.start()
        self._jobs.append(t)

    def wait(self) -> None:
        for t in self._jobs:
            t.join()
        self._jobs = []
        if self._errors:
            e = self._errors[0]
            self._errors = []
            raise e

    def pending(self) -> int:
        return sum(t.is_alive() for t in self._jobs)


def _make_writer():
    from mintext_b200.ops._ext import io_ext

    nat = io_ext()
    return nat.AsyncFileWriter(4) if nat is not None else _PyWriter()


class CheckpointManager:
    def __init__(self, directory: str, save_interval_steps: int = 1, max_to_keep: int | None = None,
                 enable_async: bool = True, read_only: bool = False):
        self.directory = Path(directory)
        self.save_interval_steps = max(int(save_interval_steps), 1)
        self.max_to_keep = max_to_keep
        self.enable_async = enable_async
        self.read_only = read_only
        self._writer = None
        self._inflight: list[tuple[int, Path]] = []
        self._pending_meta: dict | None = None
        if not read_only and _rank() == 0:
            self.directory.mkdir(parents=True, exist_ok=True)

    # ---------------------------------------------------------------- queries
    def all_steps(self) -> list[int]:
        if not self.directory.exists():
            return []
        steps = []
        for p in self.directory.iterdir():
            if p.is_dir() and p.name.isdigit() and (p / _COMMIT).exists():
                steps.append(int(p.name))
        return sorted(steps)

    def latest_step(self) -> int | None:
        steps = self.all_steps()
        return steps[-1] if steps else None

    def should_save(self, step: int) -> bool:
        return step % self.save_interval_steps == 0

    # ---------------------------------------------------------------- save
    def save(self, step: int, state, force: bool = False) -> bool:
        if self.read_only:
            raise RuntimeError("checkpoint manager is read-only")
        if not force and not self.should_save(step):
            return False
        if step in self.all_steps():
            return False
        self.wait_until_finished()  # one save in flight at a time
        tree = state.checkpoint_tree()
        step_dir = self.directory / str(step)
        leaf_dir = step_dir / "default"
        if _rank() == 0:
            leaf_dir.mkdir(parents=True, exist_ok=True)
        _barrier()
        if self._writer is None:
            self._writer = _make_writer()
        meta: dict[str, dict] = {}
        flat_items = []
        for path, value in tree.items():  # a list holds several chunks of the same entry written by this rank
            for v in (value if isinstance(value, list) else [value]):
                flat_items.append((path, v))
        for path, value in flat_items:
            entry = value if isinstance(value, dict) else {"tensor": value}
            writer_rank = entry.get("writer_rank", 0)
            t = entry.get("tensor")
            if not isinstance(t, torch.Tensor):
                meta[path] = {"scalar": t}
                continue
            fname = path.replace("/", "__") + entry.get("suffix", "") + ".bin"
            info = {"dtype": str(t.dtype).replace("torch.", ""), "shape": list(t.shape), "file": fname}
            if "flat_range" in entry:
                info["flat_range"] = list(entry["flat_range"])
                info["flat_total"] = int(entry["flat_total"])
            if "flat_range" in entry:
                meta.setdefault(path, {"chunks": []})["chunks"].append(info)
            elif "shard" in entry:
                info["shard"] = [int(v) for v in entry["shard"]]
                meta.setdefault(path, {"shards": []})["shards"].append(info)
            else:
                meta[path] = info
            if writer_rank is not None and writer_rank != _rank():
                continue
            host = torch.empty(t.shape, dtype=t.dtype, device="cpu",
                               pin_memory=t.is_cuda and torch.cuda.is_available())
            host.copy_(t.detach(), non_blocking=False)
            buf = host.view(torch.uint8) if host.dtype == torch.bfloat16 else host
            self._writer.submit(str(leaf_dir / fname), buf.contiguous())
        if _world() > 1:
            import torch.distributed as dist

            gathered = [None] * _world()
            dist.all_gather_object(gathered, meta)
            merged: dict[str, dict] = {}
            for m in gathered:
                for k, v in m.items():
                    if "chunks" in v or "shards" in v:
                        kind = "chunks" if "chunks" in v else "shards"
                        merged.setdefault(k, {kind: []})[kind].extend(
                            c for c in v[kind] if c not in merged[k][kind])
                    else:
                        merged[k] = v
            meta = merged
        self._inflight.append((step, step_dir))
        self._pending_meta = meta
        if not self.enable_async:
            self.wait_until_finished()
        return True

    def wait_until_finished(self) -> None:
        """Block until the save in flight is on disk and committed.  A write error on any rank fails the save on
        every rank: nothing is committed, the step's directory is removed, and all ranks raise together (a rank
        that raised alone would leave its peers waiting in the barrier)."""
        error: Exception | None = None
        if self._writer is not None:
            try:
                self._writer.wait()
            except Exception as e:
                error = e
        if not self._inflight:
            if error is not None:
                raise error
            return
        ok = error is None
        if _world() > 1:
            import torch.distributed as dist

            flags = [None] * _world()
            dist.all_gather_object(flags, ok)
            ok = all(flags)
        inflight, self._inflight, meta, self._pending_meta = self._inflight, [], self._pending_meta, None
        if not ok:
            if _rank() == 0:
                for _, step_dir in inflight:
                    shutil.rmtree(step_dir, ignore_errors=True)
            _barrier()
            steps = [s for s, _ in inflight]
            if error is not None:
                raise RuntimeError(f"checkpoint write failed for step(s) {steps}; nothing was committed") from error
            raise RuntimeError(f"checkpoint write failed on another rank for step(s) {steps}; nothing was committed")
        for step, step_dir in inflight:
            if _rank() == 0:
                with open(step_dir / "default" / "_METADATA", "w") as f:
                    json.dump(meta, f)
                with open(step_dir / _COMMIT, "w") as f:
                    json.dump({"step": step, "world_size": _world()}, f)
        _barrier()
        self._apply_retention()

    def _apply_retention(self) -> None:
        if self.max_to_keep is None or _rank() != 0:
            return
        steps = self.all_steps()
        for s in steps[: max(0, len(steps) - self.max_to_keep)]:
            shutil.rmtree(self.directory / str(s), ignore_errors=True)

    # ---------------------------------------------------------------- restore
    def verify(self, step: int) -> None:
        """Raise :class:`CheckpointCorrupt` unless every file the step's metadata names exists with exactly the size
        its shape and dtype imply (a truncated or partly copied checkpoint must not be loaded)."""
        leaf_dir = self.directory / str(step) / "default"
        try:
            with open(leaf_dir / "_METADATA") as f:
                meta = json.load(f)
        except (OSError, ValueError) as e:
            raise CheckpointCorrupt(f"step {step}: unreadable metadata ({e})") from e
        for path, info in meta.items():
            for leaf in info.get("chunks", info.get("shards", [info] if "file" in info else [])):
                want = int(np.prod(leaf["shape"], dtype=np.int64)) * np.dtype(_NP_OF[getattr(torch, leaf["dtype"])]).itemsize
                f = leaf_dir / leaf["file"]
                have = f.stat().st_size if f.exists() else -1
                if have != want:
                    raise CheckpointCorrupt(f"step {step}: '{path}' file {leaf['file']} has {have} bytes, expected {want}")

    def restore(self, step: int, state) -> None:
        leaf_dir = self.directory / str(step) / "default"
        if not (self.directory / str(step) / _COMMIT).exists():
            raise FileNotFoundError(f"No committed checkpoint for step {step} in {self.directory}")
        self.verify(step)
        with open(leaf_dir / "_METADATA") as f:
            meta = json.load(f)

        def read_file(info) -> torch.Tensor:
            dt = getattr(torch, info["dtype"])
            raw = np.fromfile(leaf_dir / info["file"], dtype=_NP_OF[dt])
            t = torch.from_numpy(raw)
            if dt == torch.bfloat16:
                t = t.view(torch.bfloat16)
            return t.reshape(info["shape"])

        def read(path: str, flat_range: tuple[int, int] | None = None, shard: tuple[int, int, int] | None = None):
            """``flat_range``: element range of a flat buffer saved in per-rank chunks.  ``shard = (dim, index,
            count)``: the caller holds slice ``index`` of ``count`` along ``dim``; the saved entry may be whole or
            split into any number of shards along the same dimension."""
            if path not in meta:
                raise KeyError(f"checkpoint has no entry '{path}'")
            info = meta[path]
            if "scalar" in info:
                return info["scalar"]
            if "shards" in info:
                parts = sorted(info["shards"], key=lambda c: c["shard"][1])
                dim, _, count = parts[0]["shard"]
                if len(parts) != count or any(c["shard"][0] != dim or c["shard"][2] != count for c in parts):
                    raise CheckpointCorrupt(f"step {step}: '{path}' has {len(parts)} of {count} shards")
                if shard is not None and shard[0] != dim:
                    raise ValueError(f"'{path}' was saved split along dim {dim}, requested along dim {shard[0]}")
                if shard is not None and shard[2] == count:
                    return read_file(parts[shard[1]])
                full = torch.cat([read_file(c) for c in parts], dim=dim)
            elif "chunks" not in info:
                full = read_file(info)
            else:
                # flat buffer saved as per-rank chunks: assemble the requested range from the chunks that overlap it
                lo, hi = flat_range if flat_range is not None else (0, info["chunks"][0]["flat_total"])
                first = info["chunks"][0]
                out = torch.zeros(hi - lo, dtype=getattr(torch, first["dtype"]))
                for c in info["chunks"]:
                    a, b = c["flat_range"]
                    s, e = max(a, lo), min(b, hi)
                    if s < e:
                        out[s - lo:e - lo] = read_file(c)[s - a:e - a]
                return out
            if shard is None:
                return full
            dim, idx, cnt = shard
            if full.shape[dim] % cnt != 0:
                raise ValueError(f"'{path}' dim {dim} ({full.shape[dim]}) does not split into {cnt} shards")
            per = full.shape[dim] // cnt
            return full.narrow(dim, idx * per, per).contiguous()

        read.paths = list(meta.keys())  # type: ignore[attr-defined]
        state.load_checkpoint_tree(read)


# ------------------------------------------------------------------------------------ functional API
def create_checkpoint_manager(config) -> CheckpointManager:
    return CheckpointManager(config.checkpoint_dir, save_interval_steps=config.checkpoint_period,
                             max_to_keep=config.max_checkpoints, enable_async=config.async_checkpointing)


def save_checkpoint(manager: CheckpointManager, step: int, state, force: bool = False) -> bool:
    """Save when ``step`` is a multiple of the interval (or ``force``); returns whether a save was started."""
    saved = manager.save(step, state, force=force)
    if saved:
        logger.info("Saved checkpoint at step %d", step)
    return saved


def restore_checkpoint(manager: CheckpointManager, state, step: int | None = None):
    """Restore ``step`` (default: latest) into ``state``; returns ``(state, step)``."""
    if step is None:
        step = manager.latest_step()
    if step is None:
        raise FileNotFoundError(f"No checkpoint found in {manager.directory}")
    manager.restore(step, state)
    logger.info("Restored checkpoint from step %d", step)
    return state, step


def maybe_restore_checkpoint(manager: CheckpointManager | None, state, config, model=None):
    """Resume priority: (1) latest step in the run's own ``checkpoint_dir``; (2) ``load_checkpoint`` (whole state,
    or parameters only with ``load_params_only`` -> step 0); (3) ``load_hf_checkpoint`` (parameters, step 0);
    (4) start from scratch.  Returns ``(state, start_step)``."""
    if manager is not None and manager.latest_step() is not None:
        # newest first; a step whose files are damaged is skipped in favour of the one before it
        for step in reversed(manager.all_steps()):
            try:
                manager.verify(step)
            except CheckpointCorrupt as e:
                logger.warning("Skipping damaged checkpoint: %s", e)
                continue
            state, step = restore_checkpoint(manager, state, step)
            logger.info("Resuming from step %d", step)
            return state, step
        raise CheckpointCorrupt(f"every checkpoint in {manager.directory} is damaged")
    if config.load_checkpoint:
        src = CheckpointManager(config.load_checkpoint, read_only=True)
        step = src.latest_step()
        if step is None:
            raise FileNotFoundError(f"No checkpoint found in {config.load_checkpoint}")
        if config.load_params_only:
            state.params_only_restore = True
            try:
                src.restore(step, state)
            finally:
                state.params_only_restore = False
            state.reset_step()
            logger.info("Loaded parameters only from %s (step %d); optimizer and step reset", config.load_checkpoint, step)
            return state, 0
        src.restore(step, state)
        return state, step
    if config.load_hf_checkpoint:
        if model is None:
            raise ValueError("load_hf_checkpoint requires the model")
        from .conversion import load_hf_checkpoint

        load_hf_checkpoint(config.load_hf_checkpoint, config, model)
        state.refresh_from_model()
        state.reset_step()
        logger.info("Loaded HF checkpoint from %s", config.load_hf_checkpoint)
        return state, 0
    return state, 0


def wait_for_checkpoint(manager: CheckpointManager | None) -> None:
    if manager is not None:
        manager.wait_until_finished()

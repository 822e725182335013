"""Command-line entry point and the training loop (reference: mintext/train.py).

    python -m mintext_b200.train --config configs/base.yml --config configs/models/<model>.yml key=value ...
    python -m mintext_b200.train --help-config

``--config`` may be repeated; files are merged left to right (each still follows its ``base_config`` chain),
then ``key=value`` overrides, then ``MINTEXT_<KEY>`` environment variables with the documented priority.
On a machine with CUDA the loop runs through :class:`mintext_b200.parallel.engine.TrainEngine` (this
repository's kernels, sharded fused optimizer, device-timed steps); without a GPU it runs the same model through
the plain-PyTorch path.
"""

from __future__ import annotations

import argparse
import logging
import os
import sys
import time

import torch

from mintext_b200.config import MinTextConfig, load_config, parse_cli_overrides, print_help_config

logger = logging.getLogger("mintext_b200.train")


def _make_synthetic_batch(config, generator: torch.Generator, batch_rows: int, device) -> dict[str, torch.Tensor]:
    """Uniform random token ids.  Targets equal the inputs unless ``synthetic_shift_targets`` is set (then the
    target is the next token), matching the reference's synthetic task by default."""
    tok = torch.randint(0, config.vocab_size, (batch_rows, config.seq_length), generator=generator, dtype=torch.int64)
    tgt = tok.roll(-1, dims=1) if config.synthetic_shift_targets else tok
    if device.type == "cuda":
        tok, tgt = tok.pin_memory().to(device, non_blocking=True), tgt.pin_memory().to(device, non_blocking=True)
    return {"input_tokens": tok, "target_tokens": tgt}


class _SyntheticStream:
    """Source of the synthetic batches of one data-parallel rank (``synthetic_rng``).  With the counter-based
    generator the key is split once per step and the rank draws rows ``[dp_rank * rows, (dp_rank + 1) * rows)`` of
    the step's global batch directly on its device; ``skip`` advances past the steps a resumed run has consumed."""

    def __init__(self, config, rows: int, dp_rank: int, device):
        from mintext_b200.utils import threefry

        self.config, self.rows, self.dp_rank, self.device = config, rows, dp_rank, device
        self.counter_based = str(config.synthetic_rng) == "threefry"
        self.key = threefry.key(config.seed)
        self.gen = torch.Generator(device="cpu").manual_seed(config.seed * 1000003 + dp_rank)

    def skip(self, steps: int) -> None:
        from mintext_b200.utils import threefry

        for _ in range(steps):
            if self.counter_based:
                self.key = threefry.split(self.key)[0]
            else:
                _make_synthetic_batch(self.config, self.gen, self.rows, torch.device("cpu"))

    def next(self) -> dict[str, torch.Tensor]:
        if not self.counter_based:
            return _make_synthetic_batch(self.config, self.gen, self.rows, self.device)
        from mintext_b200.utils import threefry

        self.key, batch_key = threefry.split(self.key)
        cfg = self.config
        tok = threefry.randint_rows(batch_key, self.dp_rank * self.rows, self.rows, cfg.seq_length, cfg.vocab_size,
                                    self.device)
        tgt = tok.roll(-1, dims=1) if cfg.synthetic_shift_targets else tok
        return {"input_tokens": tok, "target_tokens": tgt}


def _apply_moe_tiling(config, result, model=None) -> MinTextConfig:
    """Copy autotuned grouped-GEMM tilings into the config and, when the model is already built, into its expert
    modules, which hand them to the grouped kernels (single-CTA or CTA-pair tiles per projection)."""
    if model is not None:
        from mintext_b200.modules.moe import MoEExperts

        for m in model.modules():
            if isinstance(m, MoEExperts):
                m.gate_up_tiling, m.down_tiling = tuple(result.gate_up_tiling), tuple(result.down_tiling)
    return config.model_copy(update={"moe_gate_up_tiling": list(result.gate_up_tiling),
                                     "moe_down_tiling": list(result.down_tiling)})


def _device_init_wanted(config) -> bool:
    mode = str(config.init_weights_on_device).lower()
    if mode in ("true", "1", "yes"):
        return True
    if mode in ("false", "0", "no"):
        return False
    from mintext_b200.utils.pytree import estimate_param_count

    return estimate_param_count(config) > 2e9


def setup_training(config: MinTextConfig):
    """Everything between a config and the first step: join the process group, build the mesh, install the
    expert- / tensor-parallel contexts the modules consult while they are constructed, build the model and hand it
    to the engine (GPU) or the plain-PyTorch train state (CPU).  Returns ``(mesh, model, state, device, use_gpu)``;
    ``bench.py`` calls this too, so a benchmarked model is set up exactly as a trained one."""
    from mintext_b200.parallel import create_sharded_model, initialize_distributed, setup_mesh

    initialize_distributed(config.jax_distributed_init_timeout)
    mesh = setup_mesh(config)
    use_gpu = torch.cuda.is_available() and config.kernel_backend != "oracle"
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if use_gpu else torch.device("cpu")
    if use_gpu:
        torch.cuda.set_device(device)
    rank = 0
    if mesh.size > 1:
        import torch.distributed as dist

        rank = dist.get_rank()
    # peer-memory kernels only among ranks of one NVSwitch domain; a group that spans nodes composes NCCL collectives
    fused_ok = lambda ranks: bool(config.fused_collectives) and mesh.within_one_slice(ranks)  # noqa: E731
    if config.ici_expert_parallelism > 1 and config.num_experts > 0:
        from mintext_b200.parallel.ep import ExpertParallel, set_current_ep

        set_current_ep(ExpertParallel(mesh.group(("expert",)), device, config.moe_capacity_factor,
                                      fused=fused_ok(mesh.expert_group_ranks(rank))))
    # Replica groups for the parameters a rank holds a slice of: tensor slices are replicated on the ranks of the same
    # tensor coordinate, expert slices on the ranks at the same expert position (across the tensor axis too, since the
    # routed experts treat a tensor-parallel group as data parallelism).
    local_reduce_group = expert_reduce_group = None
    tp_on = mesh.shape["tensor"] > 1
    ep_on = config.ici_expert_parallelism > 1 and config.num_experts > 0
    dp = mesh.shape["data"] * mesh.shape["fsdp"]
    if tp_on:
        from mintext_b200.parallel.tp import TensorParallel, set_current_tp

        set_current_tp(TensorParallel(mesh.group(("tensor",)), device, fused=fused_ok(mesh.ranks_along("tensor", rank))))
        if dp > 1:
            local_reduce_group = mesh.group(("data", "fsdp"))
    if ep_on:
        replicas = dp // config.ici_expert_parallelism * mesh.shape["tensor"]
        if replicas > 1:
            group = _expert_replica_group(mesh, config.ici_expert_parallelism)
            if tp_on:
                expert_reduce_group = group
            else:
                local_reduce_group = group
    init_device = device if (use_gpu and _device_init_wanted(config)) else None
    model = create_sharded_model(config, mesh, init_device=init_device)
    if use_gpu:
        from mintext_b200.utils.pytree import wants_sharded_params

        engine_config = config
        if mesh.num_slices > 1 and config.fused_collectives:
            # the optimizer's reduce-scatter / all-gather span every rank, hence every node: NCCL composition
            logger.info("mesh spans %d NVSwitch domains: the sharded optimizer step uses NCCL collectives", mesh.num_slices)
            engine_config = config.model_copy(update={"fused_collectives": False})
        if wants_sharded_params(engine_config, mesh.size):
            from mintext_b200.parallel.fsdp import ParamShardedEngine as Engine
        else:
            from mintext_b200.parallel.engine import TrainEngine as Engine
        state = Engine(model, engine_config, device=device, local_reduce_group=local_reduce_group,
                       expert_reduce_group=expert_reduce_group)
    else:
        from mintext_b200 import trainer

        # several CPU processes: gradients are averaged as the GPU engine would (replicas, slices and their groups)
        groups = None
        if mesh.size > 1:
            groups = trainer.ReduceGroups(slice_group=local_reduce_group, expert_group=expert_reduce_group)
        state = trainer.create_train_state(model, config, groups)
    return mesh, model, state, device, use_gpu


def _expert_replica_ranks(mesh, ep: int, rank: int) -> tuple[int, ...]:
    """Ranks that hold the same experts as ``rank``: the rank at the same position of every expert-parallel block of
    the batch-sharding ranks, in every tensor column."""
    dp = mesh.ranks_along(("data", "fsdp"), rank)
    pos = dp.index(rank) % ep
    members = []
    for column_peer in mesh.ranks_along("tensor", rank):
        members.extend(mesh.ranks_along(("data", "fsdp"), column_peer)[pos::ep])
    return tuple(sorted(members))


def _expert_replica_group(mesh, ep: int):
    """Process group of :func:`_expert_replica_ranks` for the calling rank (every rank creates every group)."""
    import torch.distributed as dist

    rank = dist.get_rank()
    mine = None
    seen = set()
    for r in range(mesh.size):
        members = _expert_replica_ranks(mesh, ep, r)
        if members in seen:
            continue
        seen.add(members)
        g = dist.new_group(list(members))
        if rank in members:
            mine = g
    return mine


def train(config: MinTextConfig) -> dict:
    """Run ``config.steps`` optimizer steps.  Returns the metrics of the last step (floats)."""
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(name)s %(message)s")
    from mintext_b200.checkpoint import (create_checkpoint_manager, maybe_restore_checkpoint, save_checkpoint,
                                         wait_for_checkpoint)
    from mintext_b200.utils import MetricLogger, Profiler

    mesh, model, state, device, use_gpu = setup_training(config)
    metric_logger = MetricLogger(config, params=model)
    profiler = Profiler(config)

    manager = create_checkpoint_manager(config) if config.enable_checkpointing else None
    state, start_step = maybe_restore_checkpoint(manager, state, config, model=model)

    if config.moe_autotune and config.num_experts > 0 and use_gpu:
        from mintext_b200.kernels.autotuner import MoETuningConfig, autotune_moe

        tokens = config.per_device_batch_size * config.seq_length * config.num_experts_per_tok
        res = autotune_moe(MoETuningConfig(config.num_experts, config.hidden_size, config.moe_intermediate_size,
                                           tokens, config.dtype), cache_dir=config.moe_autotune_cache_dir or None)
        config = _apply_moe_tiling(config, res, model)

    world = mesh.size
    tp = mesh.shape["tensor"]
    dp_world = world // tp
    rows = config.per_device_batch_size * config.gradient_accumulation_steps
    train_iter = eval_iter = None
    if config.dataset_type != "synthetic":
        from mintext_b200.data import create_eval_iterator, create_train_iterator

        train_iter = create_train_iterator(config, mesh)
        if start_step > 0:
            train_iter.load_state_dict({"batches_done": start_step})
        if config.eval_period > 0:
            eval_iter = create_eval_iterator(config, mesh)
    rank = int(os.environ.get("RANK", "0"))
    synthetic = _SyntheticStream(config, rows, mesh.batch_rank(rank)[0] if world > 1 else 0, device)
    if train_iter is None:
        synthetic.skip(start_step)  # resume: past the batches already consumed

    heartbeat = None
    if config.heartbeat_interval > 0 and world > 1:
        import torch.distributed as dist

        from mintext_b200.parallel.health import Heartbeat

        heartbeat = Heartbeat(dist.distributed_c10d._get_default_store(), rank, world, config.heartbeat_interval,
                              config.heartbeat_timeout)
        heartbeat.wait_all_alive(config.jax_distributed_init_timeout)
    last = {}
    ev0 = ev1 = None
    if use_gpu:
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for step in range(start_step, config.steps):
        profiler.maybe_activate(step)
        if heartbeat is not None:
            heartbeat.check()  # a dead peer becomes an exception here, not a hang in the step's first collective
        t0 = time.time()
        if train_iter is not None:
            nb = next(train_iter)
            batch = {k: torch.from_numpy(v).long().to(device, non_blocking=True) for k, v in nb.items()}
        else:
            batch = synthetic.next()
        if use_gpu:
            ev0.record()
            metrics = state.train_step(batch)
            ev1.record()
            loss_value = float(metrics["loss"])  # device -> host sync, as the reference blocks on the loss
            metrics["device_step_ms"] = ev0.elapsed_time(ev1)
            state.check()
        else:
            from mintext_b200 import trainer

            state, metrics = trainer.train_step(state, batch, model, config)
            loss_value = float(metrics["loss"])
        step_time = time.time() - t0
        if config.num_experts > 0 and metrics.get("moe_expert_counts") is not None:
            if use_gpu:
                state.update_expert_biases(metrics["moe_expert_counts"])
            else:
                from mintext_b200 import trainer

                state = trainer.update_expert_biases(state, metrics["moe_expert_counts"], config)
        if step % config.log_period == 0 or step == config.steps - 1:
            metric_logger.log_step(step, metrics, step_time)
        if eval_iter is not None and config.eval_period > 0 and (step + 1) % config.eval_period == 0:
            losses = []
            for _ in range(config.eval_steps):
                eb = {k: torch.from_numpy(v).long().to(device) for k, v in next(eval_iter).items()}
                if use_gpu:
                    losses.append(float(state.eval_step(eb)["eval_loss"]))
                else:
                    from mintext_b200 import trainer

                    losses.append(float(trainer.eval_step(state, eb, model, config)["eval_loss"]))
            logger.info("step=%d eval_loss=%.4f", step, sum(losses) / len(losses))
        if manager is not None:
            save_checkpoint(manager, step + 1, state)
        profiler.maybe_deactivate(step)
        last = {"loss": loss_value, "step": step, "step_time": step_time,
                "grad_norm": float(metrics["grad_norm"]), "learning_rate": float(metrics["learning_rate"])}
    if manager is not None:
        if config.steps not in manager.all_steps() and config.steps > start_step:
            save_checkpoint(manager, config.steps, state, force=True)
        wait_for_checkpoint(manager)
    if heartbeat is not None:
        # ranks that finish early must not take the store down under a peer that is still checking it
        import torch.distributed as dist

        dist.barrier()
        heartbeat.close()
    if use_gpu:
        free_b, total_b = torch.cuda.mem_get_info(device)  # includes symmetric-memory and communicator buffers
        last["peak_memory_gb"] = round(max(torch.cuda.max_memory_reserved(device), total_b - free_b) / 2 ** 30, 2)
        logger.info("peak device memory on rank %d: %.2f GB", rank, last["peak_memory_gb"])
    profiler.stop()
    metric_logger.close()
    if train_iter is not None:
        train_iter.close()
    return last


def main(argv: list[str] | None = None) -> None:
    ap = argparse.ArgumentParser(description="mintext_b200 training")
    ap.add_argument("--config", action="append", default=None, help="YAML config file (repeatable)")
    ap.add_argument("--help-config", action="store_true", help="print every config field and exit")
    args, rest = ap.parse_known_args(argv)
    if args.help_config:
        print_help_config()
        return
    if not args.config:
        ap.error("--config is required")
    overrides = parse_cli_overrides(rest)
    config = load_config(args.config, overrides or None)
    train(config)


if __name__ == "__main__":
    main()

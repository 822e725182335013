"""Mesh construction, logical sharding rules, distributed bootstrap (mocked env and real gloo ranks)."""

import os
from unittest import mock

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mintext_b200 import MinTextConfig
from mintext_b200.parallel import (add_data_axis_to_sharding, create_mesh, create_named_sharding, create_sharded_model,
                                   get_input_data_sharding, get_logical_axis_rules, get_model_param_shardings,
                                   logical_to_pspec, setup_mesh)
from mintext_b200.parallel.mesh import _resolve_auto_parallelism, get_global_mesh
from mintext_b200.parallel.sharding import NamedSharding


def test_auto_axis_resolution_and_errors():
    assert _resolve_auto_parallelism({"data": 1, "fsdp": -1, "tensor": 2}, 8) == {"data": 1, "fsdp": 4, "tensor": 2}
    assert _resolve_auto_parallelism({"data": 2, "fsdp": 2, "tensor": 2}, 8)["fsdp"] == 2
    with pytest.raises(ValueError, match="At most one"):
        _resolve_auto_parallelism({"data": -1, "fsdp": -1, "tensor": 1}, 8)
    with pytest.raises(ValueError, match="not divisible"):
        _resolve_auto_parallelism({"data": 3, "fsdp": -1, "tensor": 1}, 8)
    with pytest.raises(ValueError, match="product"):
        _resolve_auto_parallelism({"data": 2, "fsdp": 2, "tensor": 1}, 8)


def test_mesh_shapes_and_groups():
    c = MinTextConfig(ici_data_parallelism=2, ici_fsdp_parallelism=2, ici_tensor_parallelism=2, ici_expert_parallelism=2)
    m = create_mesh(c, devices=list(range(8)))
    assert m.shape == {"data": 2, "fsdp": 2, "tensor": 2, "expert": 2} and m.size == 8
    assert m.coords(5) == {"data": 1, "fsdp": 0, "tensor": 1}
    assert m.ranks_along("tensor", 5) == [4, 5]
    assert m.ranks_along(("data", "fsdp"), 5) == [1, 3, 5, 7]
    assert m.expert_group_ranks(5) == [5, 7]
    with pytest.raises(ValueError, match="ici_expert_parallelism"):
        create_mesh(MinTextConfig(ici_expert_parallelism=3), devices=list(range(8)))
    one = setup_mesh(MinTextConfig())
    assert one.size == 1 and get_global_mesh() is one
    with pytest.raises(ValueError, match="multi-slice"):
        create_mesh(MinTextConfig(num_slices=2), devices=[0])       # one device does not split into two slices


def test_logical_rules_and_specs():
    c = MinTextConfig()
    rules = get_logical_axis_rules(c)
    assert ("embed", "fsdp") in rules
    mesh = create_mesh(MinTextConfig(ici_fsdp_parallelism=4, ici_tensor_parallelism=2), devices=list(range(8)))
    assert logical_to_pspec(("embed", "mlp"), rules, mesh) == ("fsdp", "tensor")
    assert logical_to_pspec(("batch", "length"), rules, mesh) == (None, None)  # data axis has size 1 -> dropped
    assert logical_to_pspec(("unknown",), rules, mesh) == (None,)
    sh = create_named_sharding(mesh, ("embed", "mlp"), rules)
    assert sh.shard_shape((128, 64)) == (32, 32)
    t = torch.arange(128 * 64).view(128, 64)
    assert torch.equal(sh.shard(t, 3), t[32:64, 32:64])  # rank 3 = (fsdp 1, tensor 1)
    with pytest.raises(ValueError):
        sh.shard_shape((130, 64))
    assert get_input_data_sharding(c, mesh).spec == (None, None)


def test_zero1_data_axis_helper():
    mesh = create_mesh(MinTextConfig(ici_data_parallelism=2, ici_fsdp_parallelism=2), devices=list(range(4)))
    assert add_data_axis_to_sharding(NamedSharding(mesh, ("fsdp", None))).spec == ("fsdp", "data")
    assert add_data_axis_to_sharding(NamedSharding(mesh, ("fsdp", "tensor"))).spec == (("data", "fsdp"), "tensor")
    assert add_data_axis_to_sharding(NamedSharding(mesh, ("data", None))).spec == ("data", None)
    one = create_mesh(MinTextConfig(), devices=[0])
    assert add_data_axis_to_sharding(NamedSharding(one, (None,))).spec == (None,)


def test_sharded_model_creation_and_param_shardings():
    c = MinTextConfig(dtype="float32")
    mesh = setup_mesh(c)
    model = create_sharded_model(c, mesh)
    tok = torch.randint(0, c.vocab_size, (1, 8))
    assert model(tok)[0].shape == (1, 8, c.vocab_size)
    sh = get_model_param_shardings(model, c, mesh)
    assert set(sh) == {n for n, _ in model.named_parameters()} and all(isinstance(v, NamedSharding) for v in sh.values())
    big = create_mesh(MinTextConfig(ici_fsdp_parallelism=2, ici_tensor_parallelism=2), devices=list(range(4)))
    assert get_model_param_shardings(model, c, big)["layers.0.mlp.gate.kernel"].spec == ("fsdp", "tensor")


def test_scan_eligibility():
    from mintext_b200.models import _all_layers_scannable

    assert _all_layers_scannable(MinTextConfig())
    assert not _all_layers_scannable(MinTextConfig(scan_layers=False))
    assert not _all_layers_scannable(MinTextConfig(num_experts=4))
    assert not _all_layers_scannable(MinTextConfig(model_type="gemma3", num_hidden_layers=6))


def test_initialize_distributed_env_aliases():
    from mintext_b200.parallel import mesh as mesh_mod

    env = {"JAX_COORDINATOR_IP": "10.0.0.1", "JAX_COORDINATOR_PORT": "1234", "NNODES": "2", "NODE_RANK": "1",
           "GPUS_PER_NODE": "1"}
    with mock.patch.dict(os.environ, env, clear=False), \
            mock.patch.object(dist, "is_initialized", return_value=False), \
            mock.patch.object(dist, "init_process_group") as init, \
            mock.patch.object(dist, "get_rank", return_value=1), mock.patch.object(dist, "get_world_size", return_value=2):
        os.environ.pop("MASTER_ADDR", None)
        os.environ.pop("WORLD_SIZE", None)
        os.environ.pop("RANK", None)
        assert mesh_mod.initialize_distributed(timeout=5)
        assert os.environ["MASTER_ADDR"] == "10.0.0.1" and os.environ["MASTER_PORT"] == "1234"
        assert os.environ["WORLD_SIZE"] == "2" and os.environ["RANK"] == "1"
        assert init.call_args[0][0] in ("gloo", "nccl")
        for k in ("MASTER_ADDR", "MASTER_PORT", "WORLD_SIZE", "RANK"):
            os.environ.pop(k, None)
    with mock.patch.dict(os.environ, {}, clear=False), mock.patch.object(dist, "is_initialized", return_value=False):
        os.environ.pop("WORLD_SIZE", None)
        os.environ.pop("NNODES", None)
        assert not mesh_mod.initialize_distributed()


# ------------------------------------------------------------------ real gloo ranks
def _worker(rank, world, port, fn, ret):
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "RANK": str(rank), "WORLD_SIZE": str(world)})
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ret[rank] = fn(rank, world)
    finally:
        dist.destroy_process_group()


def _usable_port(port: int) -> int:
    """``port`` if it can be bound right now, else a free one (a rerun shortly after another may find the
    rendezvous port of the previous run still in TIME_WAIT)."""
    import socket

    for candidate in (port, 0):
        with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
            try:
                s.bind(("127.0.0.1", candidate))
                return s.getsockname()[1]
            except OSError:
                continue
    return port


def run_ranks(fn, world, port):
    port = _usable_port(port)
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, fn, ret), nprocs=world, join=True)
    return dict(ret)


def _mesh_groups(rank, world):
    c = MinTextConfig(ici_data_parallelism=1, ici_fsdp_parallelism=2, ici_tensor_parallelism=2)
    m = create_mesh(c)
    g = m.group("tensor")
    t = torch.tensor([float(rank)])
    dist.all_reduce(t, group=g)
    g2 = m.group(("data", "fsdp"))
    u = torch.tensor([float(rank)])
    dist.all_reduce(u, group=g2)
    return (t.item(), u.item())


def test_mesh_process_groups_on_gloo():
    out = run_ranks(_mesh_groups, 4, 29611)
    assert out == {0: (1.0, 2.0), 1: (1.0, 4.0), 2: (5.0, 2.0), 3: (5.0, 4.0)}


# ------------------------------------------------------------------ gradient bucket layout of the engine
def test_bucket_plan_gives_every_rank_an_aligned_slice_of_every_bucket():
    from mintext_b200.parallel.engine import bucket_of, plan_buckets

    assert bucket_of("layers.3.mlp.gate.kernel") == 4 and bucket_of("token_embedder") == 0
    assert bucket_of("output_proj.kernel") == 0 and bucket_of("layers.x.y") == 0
    sizes = [(0, 70000), (1, 5000), (1, 130), (2, 4097), (2, 64), (0, 9000)]   # model order, buckets interleaved
    for world in (1, 2, 4, 8):
        offsets, buckets, total = plan_buckets(sizes, world)
        assert [b for b, _, _ in buckets] == [0, 1, 2]
        spans = {b: (off, off + length) for b, off, length in buckets}
        assert sum(length for _, _, length in buckets) == total
        seen = []
        for (b, n), off in zip(sizes, offsets):
            lo, hi = spans[b]
            assert lo <= off and off + n <= hi and off % 64 == 0      # inside its bucket, TMA-aligned
            seen.append((off, off + n))
        seen.sort()
        assert all(a[1] <= b[0] for a, b in zip(seen, seen[1:]))       # parameters do not overlap
        for _, off, length in buckets:
            assert length % (world * 1024) == 0 and off % 1024 == 0    # every rank's slice is vector-aligned


def test_engine_segments_cover_the_flat_buffer_once():
    """The shard arrays of all ranks, laid back into the flat order, tile it exactly (pure index arithmetic)."""
    from mintext_b200.parallel.engine import plan_buckets

    world = 4
    _, buckets, total = plan_buckets([(0, 3000), (1, 9000), (2, 100), (3, 4096)], world)
    covered = [0] * (total // 1024)
    per_rank = total // world
    for rank in range(world):
        local = 0
        for _, boff, blen in buckets:
            sl = blen // world
            for k in range((boff + rank * sl) // 1024, (boff + (rank + 1) * sl) // 1024):
                covered[k] += 1
            local += sl
        assert local == per_rank
    assert set(covered) == {1}


# ------------------------------------------------------------------ process groups of the shipped benchmark configs
def _benchmark_groups(rank, world):
    """What ``setup_training`` builds between the mesh and the engine for every shipped benchmark config, on 8 ranks:
    tensor group, expert group and the replica groups of rank-local slices; one all-reduce per group proves it works."""
    from pathlib import Path

    from mintext_b200.config import load_config
    from mintext_b200.train import _expert_replica_group

    out = {}
    root = Path(__file__).resolve().parents[1] / "configs" / "benchmarks"
    for f in sorted(root.glob("*.yml")):
        c = load_config(f)
        m = create_mesh(c)
        sizes = {}
        dp = m.shape["data"] * m.shape["fsdp"]
        groups = {}
        if c.ici_tensor_parallelism > 1:
            groups["tensor"] = m.group(("tensor",))
            if dp > 1:
                groups["tensor_replicas"] = m.group(("data", "fsdp"))
        if c.ici_expert_parallelism > 1 and c.num_experts > 0:
            groups["expert"] = m.group(("expert",))
            if dp // c.ici_expert_parallelism * m.shape["tensor"] > 1:
                groups["expert_replicas"] = _expert_replica_group(m, c.ici_expert_parallelism)
        for name, g in groups.items():
            t = torch.ones(1)
            dist.all_reduce(t, group=g)
            sizes[name] = int(t.item())
        out[f.name] = (dict(m.shape), sizes)
    return out


def test_benchmark_configs_build_their_process_groups_on_eight_ranks():
    res = run_ranks(_benchmark_groups, 8, 29651)
    for r in range(8):
        assert res[r] == res[0]  # every rank sees groups of the same sizes
    got = res[0]
    assert got["llama-3-8b-b200.yml"] == ({"data": 1, "fsdp": 4, "tensor": 2, "expert": 1},
                                          {"tensor": 2, "tensor_replicas": 4})
    assert got["qwen3-30b-a3b-b200.yml"] == ({"data": 1, "fsdp": 8, "tensor": 1, "expert": 8}, {"expert": 8})
    assert got["deepseek-v3-4l-b200.yml"] == ({"data": 1, "fsdp": 8, "tensor": 1, "expert": 8}, {"expert": 8})
    assert got["llama-3.2-1b-b200.yml"] == ({"data": 1, "fsdp": 8, "tensor": 1, "expert": 1}, {})

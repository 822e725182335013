"""Single-behaviour tests of the mesh, the logical sharding rules and the scan eligibility (after the cases of the
reference's tests/test_sharding.py), plus the expert axis and the rank arithmetic this build adds."""

import os
from unittest import mock

import pytest
import torch
import torch.distributed as dist

from mintext_b200 import MinTextConfig
from mintext_b200.parallel import (add_data_axis_to_sharding, create_mesh, create_named_sharding, create_sharded_model,
                                   get_input_data_sharding, get_logical_axis_rules, get_model_param_shardings,
                                   logical_to_pspec, setup_mesh)
from mintext_b200.parallel.mesh import _resolve_auto_parallelism, get_global_mesh
from mintext_b200.parallel.sharding import NamedSharding


# ---- auto axis ---------------------------------------------------------------------------------------------------
def test_auto_all_explicit_passes_through():
    assert _resolve_auto_parallelism({"data": 2, "fsdp": 2, "tensor": 2}, 8) == {"data": 2, "fsdp": 2, "tensor": 2}


def test_auto_fsdp():
    assert _resolve_auto_parallelism({"data": 1, "fsdp": -1, "tensor": 1}, 8)["fsdp"] == 8


def test_auto_data():
    assert _resolve_auto_parallelism({"data": -1, "fsdp": 2, "tensor": 2}, 8)["data"] == 2


def test_auto_tensor():
    assert _resolve_auto_parallelism({"data": 2, "fsdp": 1, "tensor": -1}, 8)["tensor"] == 4


def test_auto_product_mismatch():
    with pytest.raises(ValueError, match="product"):
        _resolve_auto_parallelism({"data": 2, "fsdp": 2, "tensor": 1}, 8)


def test_auto_two_unknowns():
    with pytest.raises(ValueError, match="At most one"):
        _resolve_auto_parallelism({"data": -1, "fsdp": -1, "tensor": 1}, 8)


def test_auto_not_divisible():
    with pytest.raises(ValueError, match="not divisible"):
        _resolve_auto_parallelism({"data": 3, "fsdp": -1, "tensor": 1}, 8)


def test_auto_rejects_zero_and_other_negatives():
    with pytest.raises(ValueError):
        _resolve_auto_parallelism({"data": 0, "fsdp": -1, "tensor": 1}, 8)
    with pytest.raises(ValueError):
        _resolve_auto_parallelism({"data": -2, "fsdp": 4, "tensor": 1}, 8)


# ---- mesh --------------------------------------------------------------------------------------------------------
def test_mesh_on_one_device():
    m = create_mesh(MinTextConfig(), devices=[0])
    assert m.size == 1 and m.shape == {"data": 1, "fsdp": 1, "tensor": 1, "expert": 1}


def test_mesh_auto_fsdp_takes_all_devices():
    assert create_mesh(MinTextConfig(), devices=list(range(4))).shape["fsdp"] == 4


def test_mesh_tensor_is_the_fastest_axis():
    m = create_mesh(MinTextConfig(ici_fsdp_parallelism=2, ici_tensor_parallelism=2), devices=list(range(4)))
    assert m.ranks_along("tensor", 0) == [0, 1] and m.ranks_along("fsdp", 0) == [0, 2]


def test_mesh_coords_round_trip():
    m = create_mesh(MinTextConfig(ici_data_parallelism=2, ici_fsdp_parallelism=2, ici_tensor_parallelism=2),
                    devices=list(range(8)))
    for r in range(8):
        c = m.coords(r)
        assert r == (c["data"] * 2 + c["fsdp"]) * 2 + c["tensor"]


def test_mesh_ranks_along_contains_the_rank_itself():
    m = create_mesh(MinTextConfig(ici_data_parallelism=2, ici_fsdp_parallelism=2, ici_tensor_parallelism=2),
                    devices=list(range(8)))
    for r in range(8):
        for axes in ("data", "fsdp", "tensor", ("data", "fsdp")):
            assert r in m.ranks_along(axes, r)


def test_mesh_data_parallel_groups_partition_the_job():
    m = create_mesh(MinTextConfig(ici_fsdp_parallelism=4, ici_tensor_parallelism=2), devices=list(range(8)))
    groups = {tuple(m.ranks_along(("data", "fsdp"), r)) for r in range(8)}
    assert sorted(sum(map(list, groups), [])) == list(range(8)) and len(groups) == 2


def test_expert_axis_is_carved_out_of_data_and_fsdp():
    m = create_mesh(MinTextConfig(ici_expert_parallelism=4), devices=list(range(8)))
    assert m.shape["expert"] == 4 and m.shape["fsdp"] == 8
    assert len(m.expert_group_ranks(0)) == 4


def test_expert_groups_partition_the_data_parallel_ranks():
    m = create_mesh(MinTextConfig(ici_expert_parallelism=2), devices=list(range(8)))
    groups = {tuple(m.expert_group_ranks(r)) for r in range(8)}
    assert sorted(sum(map(list, groups), [])) == list(range(8)) and all(len(g) == 2 for g in groups)


def test_expert_axis_must_divide_the_data_parallel_ranks():
    with pytest.raises(ValueError, match="ici_expert_parallelism"):
        create_mesh(MinTextConfig(ici_expert_parallelism=3), devices=list(range(8)))


def test_expert_axis_with_tensor_parallelism_counts_only_data_ranks():
    with pytest.raises(ValueError, match="ici_expert_parallelism"):
        create_mesh(MinTextConfig(ici_tensor_parallelism=2, ici_expert_parallelism=8), devices=list(range(8)))


def test_multi_slice_mesh_puts_the_slice_index_on_the_slow_part_of_every_axis():
    """Two nodes of 8 (ranks numbered node by node): data across the nodes, fsdp x tensor inside each."""
    m = create_mesh(MinTextConfig(num_slices=2, dcn_data_parallelism=2, ici_fsdp_parallelism=4, ici_tensor_parallelism=2),
                    devices=list(range(16)))
    assert dict(m.shape) == {"data": 2, "fsdp": 4, "tensor": 2, "expert": 1}
    assert m.num_slices == 2 and m.dcn_shape == (2, 1, 1)
    assert m.ranks_along("tensor", 9) == [8, 9] and m.within_one_slice(m.ranks_along("tensor", 9))
    assert m.ranks_along("fsdp", 9) == [9, 11, 13, 15] and m.within_one_slice(m.ranks_along("fsdp", 9))
    assert m.ranks_along("data", 9) == [1, 9] and not m.within_one_slice(m.ranks_along("data", 9))
    assert [m.slice_of(r) for r in (0, 7, 8, 15)] == [0, 0, 1, 1]


def test_multi_slice_axis_split_over_nodes_and_gpus():
    """fsdp 2 (nodes) x 4 (GPUs): the node index is the slow part of the axis; tensor pairs stay inside a node."""
    m = create_mesh(MinTextConfig(num_slices=2, dcn_fsdp_parallelism=-1, ici_fsdp_parallelism=-1, ici_tensor_parallelism=2),
                    devices=list(range(16)))
    assert dict(m.shape) == {"data": 1, "fsdp": 8, "tensor": 2, "expert": 1} and m.dcn_shape == (1, 2, 1)
    assert m.ranks_along("fsdp", 0) == [0, 2, 4, 6, 8, 10, 12, 14]
    assert all(m.within_one_slice(m.ranks_along("tensor", r)) for r in range(16))
    # expert-parallel blocks of 4 are consecutive batch-sharding ranks: inside one node
    e = create_mesh(MinTextConfig(num_slices=2, dcn_fsdp_parallelism=2, ici_fsdp_parallelism=8, ici_expert_parallelism=4),
                    devices=list(range(16)))
    assert e.expert_group_ranks(9) == [8, 9, 10, 11] and e.within_one_slice(e.expert_group_ranks(9))


def test_slices_follow_from_the_dcn_settings_and_are_validated():
    m = create_mesh(MinTextConfig(dcn_data_parallelism=2), devices=[0, 1])        # num_slices left at 1
    assert m.num_slices == 2 and dict(m.shape)["data"] == 2
    with pytest.raises(ValueError, match="multi-slice"):
        create_mesh(MinTextConfig(num_slices=2), devices=[0])                       # 1 device, 2 slices
    with pytest.raises(ValueError, match="DCN"):
        create_mesh(MinTextConfig(num_slices=4, dcn_data_parallelism=2), devices=list(range(8)))   # product != slices
    with pytest.raises(ValueError, match="num_slices"):
        create_mesh(MinTextConfig(dcn_data_parallelism=-1), devices=list(range(8)))
    flat = create_mesh(MinTextConfig(ici_fsdp_parallelism=-1), devices=list(range(16)))  # all DCN settings 1: one slice
    assert flat.num_slices == 1 and dict(flat.shape)["fsdp"] == 16


def test_setup_mesh_sets_the_global_mesh():
    m = setup_mesh(MinTextConfig())
    assert get_global_mesh() is m


# ---- rules and specs ---------------------------------------------------------------------------------------------
def test_default_rules_cover_the_reference_axes():
    rules = dict(get_logical_axis_rules(MinTextConfig()))
    for axis, target in (("batch", "data"), ("embed", "fsdp"), ("mlp", "tensor"), ("heads", "tensor"), ("vocab", "tensor")):
        assert rules[axis] == target, axis


def test_rules_come_from_the_config():
    c = MinTextConfig(logical_axis_rules=[["embed", "tensor"], ["mlp", None]])
    assert get_logical_axis_rules(c) == [("embed", "tensor"), ("mlp", None)]


@pytest.fixture
def mesh42():
    return create_mesh(MinTextConfig(ici_fsdp_parallelism=4, ici_tensor_parallelism=2), devices=list(range(8)))


def test_spec_of_a_weight(mesh42):
    assert logical_to_pspec(("embed", "mlp"), get_logical_axis_rules(MinTextConfig()), mesh42) == ("fsdp", "tensor")


def test_spec_with_unsharded_axes(mesh42):
    assert logical_to_pspec((None, None), get_logical_axis_rules(MinTextConfig()), mesh42) == (None, None)


def test_spec_of_a_norm_scale(mesh42):
    assert logical_to_pspec(("norm",), get_logical_axis_rules(MinTextConfig()), mesh42) == (None,)


def test_spec_drops_axes_of_size_one(mesh42):
    assert logical_to_pspec(("batch",), get_logical_axis_rules(MinTextConfig()), mesh42) == (None,)


def test_spec_of_an_unknown_logical_axis(mesh42):
    assert logical_to_pspec(("no_such_axis",), get_logical_axis_rules(MinTextConfig()), mesh42) == (None,)


def test_named_sharding_shard_shape(mesh42):
    sh = create_named_sharding(mesh42, ("embed", "mlp"), get_logical_axis_rules(MinTextConfig()))
    assert isinstance(sh, NamedSharding) and sh.shard_shape((64, 32)) == (16, 16)


def test_named_sharding_rejects_indivisible_shapes(mesh42):
    sh = create_named_sharding(mesh42, ("embed", "mlp"), get_logical_axis_rules(MinTextConfig()))
    with pytest.raises(ValueError):
        sh.shard_shape((66, 32))


def test_named_sharding_slices_tile_the_tensor(mesh42):
    sh = create_named_sharding(mesh42, ("embed", "mlp"), get_logical_axis_rules(MinTextConfig()))
    t = torch.arange(16 * 8).view(16, 8)
    seen = torch.zeros_like(t)
    for r in range(8):
        sl = sh.local_slices(t.shape, r)
        seen[sl] += 1
        assert torch.equal(sh.shard(t, r), t[sl])
    assert bool((seen == 1).all())


def test_input_sharding_follows_the_batch_rule():
    c = MinTextConfig(ici_data_parallelism=2, ici_fsdp_parallelism=2)
    m = create_mesh(c, devices=list(range(4)))
    assert get_input_data_sharding(c, m).spec[0] == "data"


def test_zero1_adds_data_to_an_unsharded_dimension():
    m = create_mesh(MinTextConfig(ici_data_parallelism=2, ici_fsdp_parallelism=2), devices=list(range(4)))
    assert add_data_axis_to_sharding(NamedSharding(m, ("fsdp", None))).spec == ("fsdp", "data")


def test_zero1_leaves_data_sharded_specs_alone():
    m = create_mesh(MinTextConfig(ici_data_parallelism=2, ici_fsdp_parallelism=2), devices=list(range(4)))
    assert add_data_axis_to_sharding(NamedSharding(m, ("data", None))).spec == ("data", None)


def test_zero1_compounds_when_every_dimension_is_sharded():
    m = create_mesh(MinTextConfig(ici_data_parallelism=2, ici_fsdp_parallelism=2), devices=list(range(4)))
    assert add_data_axis_to_sharding(NamedSharding(m, ("fsdp", "tensor"))).spec == (("data", "fsdp"), "tensor")


def test_zero1_on_a_scalar_spec():
    m = create_mesh(MinTextConfig(ici_data_parallelism=2, ici_fsdp_parallelism=2), devices=list(range(4)))
    assert add_data_axis_to_sharding(NamedSharding(m, ())).spec == ()


def test_zero1_without_a_data_axis_is_the_identity():
    m = create_mesh(MinTextConfig(), devices=[0])
    assert add_data_axis_to_sharding(NamedSharding(m, (None, "fsdp"))).spec == (None, "fsdp")


# ---- model creation ----------------------------------------------------------------------------------------------
def test_create_sharded_model_runs():
    c = MinTextConfig(dtype="float32")
    model = create_sharded_model(c, setup_mesh(c))
    out, _ = model(torch.randint(0, c.vocab_size, (2, 6)))
    assert out.shape == (2, 6, c.vocab_size) and bool(torch.isfinite(out).all())


def test_param_shardings_cover_every_parameter():
    c = MinTextConfig(dtype="float32")
    mesh = setup_mesh(c)
    model = create_sharded_model(c, mesh)
    sh = get_model_param_shardings(model, c, mesh)
    assert set(sh) == {n for n, _ in model.named_parameters()}


def test_param_shardings_follow_the_rules():
    c = MinTextConfig(dtype="float32")
    model = create_sharded_model(c, setup_mesh(c))
    big = create_mesh(MinTextConfig(ici_fsdp_parallelism=2, ici_tensor_parallelism=2), devices=list(range(4)))
    sh = get_model_param_shardings(model, c, big)
    assert sh["layers.0.mlp.down.kernel"].spec == ("tensor", "fsdp")
    assert sh["final_norm.scale"].spec == (None,)


# ---- distributed bootstrap ---------------------------------------------------------------------------------------
def test_initialize_distributed_without_a_launcher():
    from mintext_b200.parallel.mesh import initialize_distributed

    clean = {k: v for k, v in os.environ.items()
             if k not in ("WORLD_SIZE", "RANK", "NNODES", "NODE_RANK", "JAX_COORDINATOR_IP", "MASTER_ADDR")}
    with mock.patch.dict(os.environ, clean, clear=True), mock.patch.object(dist, "is_initialized", return_value=False), \
            mock.patch.object(dist, "init_process_group") as init:
        assert initialize_distributed() is False
        init.assert_not_called()


def test_initialize_distributed_when_already_joined():
    from mintext_b200.parallel.mesh import initialize_distributed

    with mock.patch.object(dist, "is_initialized", return_value=True), \
            mock.patch.object(dist, "get_world_size", return_value=4), \
            mock.patch.object(dist, "init_process_group") as init:
        assert initialize_distributed() is True
        init.assert_not_called()


def test_initialize_distributed_world_of_one_is_not_joined():
    from mintext_b200.parallel.mesh import initialize_distributed

    with mock.patch.dict(os.environ, {"WORLD_SIZE": "1", "RANK": "0"}), \
            mock.patch.object(dist, "is_initialized", return_value=False), \
            mock.patch.object(dist, "init_process_group") as init:
        assert initialize_distributed() is False
        init.assert_not_called()


# ---- layer scan key ----------------------------------------------------------------------------------------------
def test_scan_homogeneous_layers():
    from mintext_b200.models import _all_layers_scannable

    assert _all_layers_scannable(MinTextConfig(num_hidden_layers=4))


def test_scan_disabled_by_the_config():
    from mintext_b200.models import _all_layers_scannable

    assert not _all_layers_scannable(MinTextConfig(scan_layers=False))


def test_scan_mixture_of_experts_layers():
    from mintext_b200.models import _all_layers_scannable

    assert not _all_layers_scannable(MinTextConfig(num_experts=4))


def test_scan_mixed_layer_types():
    from mintext_b200.models import _all_layers_scannable

    assert not _all_layers_scannable(MinTextConfig(model_type="gemma3", num_hidden_layers=6))


def test_scanned_and_looped_forward_agree():
    tok = torch.randint(0, 256, (2, 8))
    outs = []
    for scan in (True, False):
        c = MinTextConfig(dtype="float32", scan_layers=scan, num_hidden_layers=3, vocab_size=256)
        from mintext_b200.models import Transformer

        outs.append(Transformer(c, rngs=0)(tok)[0])
    assert outs[0].shape == (2, 8, 256) and torch.allclose(outs[0], outs[1], atol=1e-6)


# ---- NVLink multicast probe --------------------------------------------------------------------------------------
def test_multicast_probe_reads_the_handle_and_never_raises():
    from mintext_b200.parallel.symm import multicast_available

    class Plain:
        multicast_ptr = 0

    class Bound:
        multicast_ptr = 0x7F0000000000

    class Broken:
        @property
        def multicast_ptr(self):
            raise RuntimeError("driver says no")

    assert not multicast_available(Plain()) and multicast_available(Bound())
    assert not multicast_available(object()) and not multicast_available(Broken())


# ---- replica groups of expert slices -----------------------------------------------------------------------------
def test_expert_replicas_without_tensor_parallelism():
    from mintext_b200.train import _expert_replica_ranks

    m = create_mesh(MinTextConfig(ici_expert_parallelism=2), devices=list(range(8)))
    # expert-parallel blocks (0,1) (2,3) (4,5) (6,7): position 0 of each block holds the same experts
    assert _expert_replica_ranks(m, 2, 0) == (0, 2, 4, 6) and _expert_replica_ranks(m, 2, 5) == (1, 3, 5, 7)


def test_expert_replicas_span_the_tensor_axis():
    from mintext_b200.train import _expert_replica_ranks

    m = create_mesh(MinTextConfig(ici_fsdp_parallelism=4, ici_tensor_parallelism=2, ici_expert_parallelism=2),
                    devices=list(range(8)))
    # tensor column 0 = ranks 0,2,4,6 with expert blocks (0,2) (4,6); column 1 = ranks 1,3,5,7 likewise
    assert m.expert_group_ranks(0) == [0, 2] and m.expert_group_ranks(5) == [5, 7]
    assert _expert_replica_ranks(m, 2, 0) == (0, 1, 4, 5)      # position 0 of every block, both columns
    assert _expert_replica_ranks(m, 2, 6) == (2, 3, 6, 7)
    groups = {_expert_replica_ranks(m, 2, r) for r in range(8)}
    assert sorted(sum(map(list, groups), [])) == list(range(8))


def test_expert_replicas_when_every_data_rank_is_its_own_expert_position():
    from mintext_b200.train import _expert_replica_ranks

    m = create_mesh(MinTextConfig(ici_fsdp_parallelism=2, ici_tensor_parallelism=2, ici_expert_parallelism=2),
                    devices=list(range(4)))
    assert _expert_replica_ranks(m, 2, 0) == (0, 1) and _expert_replica_ranks(m, 2, 3) == (2, 3)


def test_engine_lays_tensor_slices_before_expert_slices_when_both_have_replica_groups():
    """With tensor and expert parallelism combined the rank-local flat buffers hold the tensor slices first and the
    expert slices behind them, so that each range is reduced over its own replica group (storage layout only: runs on
    the CPU with stand-in groups)."""
    from mintext_b200.models import Transformer
    from mintext_b200.parallel.engine import TrainEngine

    c = MinTextConfig(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, vocab_size=128,
                      intermediate_size=128, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, n_group=2,
                      topk_group=1, first_k_dense_replace=1, n_shared_experts=1)
    model = Transformer(c, rngs=0)
    for n, p in model.named_parameters():
        if ".experts." in n:
            p.expert_parallel = True
        elif ".attention." in n and p.dim() >= 2:
            p.tensor_parallel = True
    with mock.patch.object(dist, "get_world_size", side_effect=lambda g=None: {"tp_replicas": 2, "ep_replicas": 4}[g]):
        eng = TrainEngine(model, c, device="cpu", local_reduce_group="tp_replicas", expert_reduce_group="ep_replicas")
    kinds = [bool(getattr(s.param, "expert_parallel", False)) for s in eng.exp.slots]
    assert kinds == sorted(kinds) and any(kinds) and not all(kinds)
    first_expert = next(s for s in eng.exp.slots if getattr(s.param, "expert_parallel", False))
    assert eng._exp_split == first_expert.offset
    ranges = eng._exp_ranges()
    assert [(lo, hi) for lo, hi, _, _ in ranges] == [(0, eng._exp_split), (eng._exp_split, eng.exp.total)]
    assert [(g, n) for _, _, g, n in ranges] == [("tp_replicas", 2), ("ep_replicas", 4)]
    # offsets are back to back and every parameter views its own range of the flat buffers
    for s in eng.exp.slots:
        assert s.param.data_ptr() == eng.exp_param[s.offset:].data_ptr()
    plain = TrainEngine(Transformer(c, rngs=0), c, device="cpu")
    assert plain._exp_split is None and plain._exp_ranges() == [(0, plain.exp.total, None, 1)]


# ---- resident or parameter-sharded engine ------------------------------------------------------------------------
def _llama8b(**kw):
    base = dict(num_hidden_layers=32, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                intermediate_size=14336, vocab_size=128256)
    base.update(kw)
    return MinTextConfig(**base)


def test_resident_bytes_count_six_per_parameter():
    from mintext_b200.utils.pytree import estimate_param_count, resident_param_bytes_per_rank

    c = _llama8b()
    assert resident_param_bytes_per_rank(c) == pytest.approx(6 * estimate_param_count(c))
    halved = resident_param_bytes_per_rank(_llama8b(ici_tensor_parallelism=2, ici_fsdp_parallelism=1))
    assert halved == pytest.approx(3 * estimate_param_count(c))


def test_resident_bytes_divide_the_experts_by_the_expert_axis():
    from mintext_b200.utils.pytree import resident_param_bytes_per_rank

    moe = dict(num_experts=64, num_experts_per_tok=4, moe_intermediate_size=1024, first_k_dense_replace=0)
    one = resident_param_bytes_per_rank(_llama8b(**moe))
    eight = resident_param_bytes_per_rank(_llama8b(**moe, ici_expert_parallelism=8))
    experts = 6.0 * 3 * 4096 * 1024 * 64 * 32
    assert one - eight == pytest.approx(experts * 7 / 8)


def test_explicit_flag_decides():
    from mintext_b200.utils.pytree import wants_sharded_params

    assert wants_sharded_params(_llama8b(fsdp_shard_params=True), 8)
    assert not wants_sharded_params(_llama8b(fsdp_shard_params=False), 8)
    assert _llama8b(fsdp_shard_params="true").fsdp_shard_params is True
    assert _llama8b(fsdp_shard_params="No").fsdp_shard_params is False


def test_auto_shards_when_the_resident_copy_exceeds_the_budget():
    from mintext_b200.utils.pytree import wants_sharded_params

    big = _llama8b(fsdp_shard_params="auto", fsdp_resident_budget_gb=40.0)     # 8 B parameters x 6 bytes = 45 GB
    roomy = _llama8b(fsdp_shard_params="auto", fsdp_resident_budget_gb=60.0)
    assert wants_sharded_params(big, 8) and not wants_sharded_params(roomy, 8)


def test_auto_stays_resident_where_the_sharded_mode_does_not_apply():
    from mintext_b200.utils.pytree import wants_sharded_params

    tight = dict(fsdp_shard_params="auto", fsdp_resident_budget_gb=1.0)
    assert not wants_sharded_params(_llama8b(**tight), 1)                                   # nothing to shard over
    assert not wants_sharded_params(_llama8b(**tight, optimizer="muon"), 8)
    assert not wants_sharded_params(_llama8b(**tight, fused_collectives=False), 8)
    assert not wants_sharded_params(_llama8b(**tight, ici_tensor_parallelism=2, ici_fsdp_parallelism=4), 8)
    assert wants_sharded_params(_llama8b(**tight), 8)


def test_unknown_mode_is_rejected():
    with pytest.raises(ValueError, match="true, false or auto"):
        _llama8b(fsdp_shard_params="sometimes")


def test_auto_from_the_environment(tmp_path, monkeypatch):
    import yaml

    from mintext_b200.config import load_config

    p = tmp_path / "c.yml"
    p.write_text(yaml.safe_dump({"steps": 1}))
    monkeypatch.setenv("MINTEXT_FSDP_SHARD_PARAMS", "auto")
    assert load_config(p).fsdp_shard_params == "auto"
    monkeypatch.setenv("MINTEXT_FSDP_SHARD_PARAMS", "true")
    assert load_config(p).fsdp_shard_params is True

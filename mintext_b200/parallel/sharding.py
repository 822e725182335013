"""Logical-axis sharding rules (reference: mintext/distributed/sharding.py).

Parameters carry logical axis names (``("embed", "mlp")`` ...).  The rules map each logical axis to a mesh axis
(first match wins); a mesh axis of size 1 is dropped from the result.  A *partition spec* is a tuple with one
entry per tensor dimension: a mesh-axis name, a tuple of names, or None.  :class:`NamedSharding` pairs a spec
with a mesh and can compute the local shard of a tensor for a rank.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .mesh import Mesh

PartitionSpec = tuple


def get_logical_axis_rules(config) -> list[tuple[str, str | None]]:
    return [tuple(r) for r in config.logical_axis_rules]


def logical_to_pspec(logical_names, rules, mesh: Mesh | None = None) -> PartitionSpec:
    out = []
    for name in logical_names:
        target = None
        for logical, physical in rules:
            if logical == name:
                target = physical
                break
        if target is not None and mesh is not None and mesh.shape.get(target, 1) == 1:
            target = None
        out.append(target)
    return tuple(out)


@dataclass(frozen=True)
class NamedSharding:
    mesh: Mesh
    spec: PartitionSpec

    def _axis_sizes(self, entry) -> int:
        if entry is None:
            return 1
        names = entry if isinstance(entry, tuple) else (entry,)
        n = 1
        for a in names:
            n *= self.mesh.shape[a]
        return n

    def shard_shape(self, shape) -> tuple[int, ...]:
        out = []
        for dim, entry in zip(shape, tuple(self.spec) + (None,) * (len(shape) - len(self.spec))):
            n = self._axis_sizes(entry)
            if dim % n != 0:
                raise ValueError(f"dimension {dim} is not divisible by {n} ({entry})")
            out.append(dim // n)
        return tuple(out)

    def local_slices(self, shape, rank: int) -> tuple[slice, ...]:
        coords = self.mesh.coords(rank)
        sl = []
        for dim, entry in zip(shape, tuple(self.spec) + (None,) * (len(shape) - len(self.spec))):
            if entry is None:
                sl.append(slice(0, dim))
                continue
            names = entry if isinstance(entry, tuple) else (entry,)
            idx, n = 0, 1
            for a in names:
                idx = idx * self.mesh.shape[a] + coords[a]
                n *= self.mesh.shape[a]
            per = dim // n
            sl.append(slice(idx * per, (idx + 1) * per))
        return tuple(sl)

    def shard(self, tensor: torch.Tensor, rank: int) -> torch.Tensor:
        return tensor[self.local_slices(tensor.shape, rank)]


def create_named_sharding(mesh: Mesh, logical_names, rules) -> NamedSharding:
    return NamedSharding(mesh, logical_to_pspec(logical_names, rules, mesh))


def add_data_axis_to_sharding(sharding: NamedSharding, mesh: Mesh | None = None) -> NamedSharding:
    """ZeRO-1 helper: additionally shard over ``data``: the first unsharded dimension gets it, otherwise the
    first dimension becomes a compound ``("data", existing)`` axis.  No change when ``data`` has size 1 or is
    already used."""
    mesh = mesh or sharding.mesh
    spec = list(sharding.spec)
    if mesh.shape.get("data", 1) == 1:
        return sharding
    for entry in spec:
        names = entry if isinstance(entry, tuple) else (entry,)
        if "data" in names:
            return sharding
    for i, entry in enumerate(spec):
        if entry is None:
            spec[i] = "data"
            return NamedSharding(mesh, tuple(spec))
    if spec:
        first = spec[0] if isinstance(spec[0], tuple) else (spec[0],)
        spec[0] = ("data",) + tuple(first)
    return NamedSharding(mesh, tuple(spec))


def get_input_data_sharding(config, mesh: Mesh) -> NamedSharding:
    """Token batches ``[B, S]``: logical axes ``("batch", "length")``.  Note that the engine additionally
    splits the batch over ``fsdp`` (true FSDP); this function states the rule table's answer."""
    return create_named_sharding(mesh, ("batch", "length"), get_logical_axis_rules(config))


def get_model_param_shardings(model: torch.nn.Module, mesh, rules=None, *, config=None) -> dict[str, NamedSharding]:
    """``{parameter name: NamedSharding}`` from every parameter's logical axes
    (mintext/distributed/sharding.py:130-165: ``(model, mesh, rules=None)``, default rules when none are given).
    ``(model, config, mesh)`` is accepted as well: the rules then come from the config."""
    if not isinstance(mesh, Mesh) and isinstance(rules, Mesh):   # (model, config, mesh)
        config, mesh, rules = mesh, rules, None
    if rules is None:
        from mintext_b200.config import DEFAULT_LOGICAL_AXIS_RULES

        rules = get_logical_axis_rules(config) if config is not None else list(DEFAULT_LOGICAL_AXIS_RULES)
    out = {}
    for name, p in model.named_parameters():
        axes = getattr(p, "logical_axes", (None,) * p.dim())
        out[name] = create_named_sharding(mesh, axes, rules)
    return out

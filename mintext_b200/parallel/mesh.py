"""Process-group bootstrap and the device mesh (reference: mintext/distributed/mesh.py).

One process drives one GPU.  The mesh has the reference's three axes plus ``expert``:
``("data", "fsdp", "tensor", "expert")``.  ``data`` and ``fsdp`` both shard the batch (and together shard the
optimizer state); ``tensor`` splits heads / MLP width / vocabulary inside a layer; ``expert`` distributes MoE
experts and is carved out of the data-parallel ranks (a rank's expert-parallel peers are data-parallel peers
for the dense parts of the model).

Several NVSwitch domains (nodes) form a hybrid mesh as the reference's multi-slice meshes do
(mintext/distributed/mesh.py:133-199): a slice is a node, ``dcn_*_parallelism`` says how the nodes are laid out on
the axes and ``ici_*_parallelism`` how the GPUs of one node are; along every axis the node index is the slow one,
so the peers a rank has along the fast part of an axis sit on its own NVSwitch.
"""

from __future__ import annotations

import datetime
import logging
import os
from dataclasses import dataclass, field

import numpy as np

logger = logging.getLogger(__name__)

AXES = ("data", "fsdp", "tensor")


def _resolve_auto_parallelism(values: dict[str, int], num_devices: int, kind: str = "ICI") -> dict[str, int]:
    """Replace the single ``-1`` entry by whatever makes the product equal ``num_devices``; validate."""
    auto = [k for k, v in values.items() if v == -1]
    if len(auto) > 1:
        raise ValueError(f"At most one {kind} parallelism axis can be -1 (auto), got {auto}")
    out = dict(values)
    if auto:
        known = 1
        for k, v in values.items():
            if v != -1:
                if v < 1:
                    raise ValueError(f"{kind} parallelism for '{k}' must be >= 1 or -1, got {v}")
                known *= v
        if num_devices % known != 0:
            raise ValueError(
                f"Cannot auto-resolve {kind} axis '{auto[0]}': {num_devices} devices not divisible by {known}")
        out[auto[0]] = num_devices // known
    prod = 1
    for v in out.values():
        if v < 1:
            raise ValueError(f"{kind} parallelism values must be >= 1, got {out}")
        prod *= v
    if prod != num_devices:
        raise ValueError(f"{kind} parallelism product {prod} != number of devices {num_devices} ({out})")
    return out


@dataclass
class Mesh:
    """Ranks arranged on named axes.  ``devices[i_data, i_fsdp, i_tensor]`` is a global rank."""

    devices: np.ndarray
    axis_names: tuple[str, ...] = AXES
    expert: int = 1
    num_slices: int = 1                                   # NVSwitch domains (nodes) the mesh spans
    dcn_shape: tuple[int, ...] = (1, 1, 1)                # nodes along each axis (the slow part of the axis)
    _groups: dict = field(default_factory=dict, repr=False)

    @property
    def shape(self) -> dict[str, int]:
        d = dict(zip(self.axis_names, self.devices.shape))
        d["expert"] = self.expert
        return d

    @property
    def size(self) -> int:
        return int(self.devices.size)

    def coords(self, rank: int) -> dict[str, int]:
        idx = np.argwhere(self.devices == rank)
        if idx.size == 0:
            raise ValueError(f"rank {rank} is not on the mesh")
        return dict(zip(self.axis_names, (int(i) for i in idx[0])))

    def ranks_along(self, axes: tuple[str, ...] | str, rank: int) -> list[int]:
        """Ranks that differ from ``rank`` only in the given axes (the communicator of those axes)."""
        axes = (axes,) if isinstance(axes, str) else tuple(axes)
        c = self.coords(rank)
        index = tuple(slice(None) if n in axes else c[n] for n in self.axis_names)
        return [int(r) for r in np.asarray(self.devices[index]).reshape(-1)]

    def batch_rank(self, rank: int) -> tuple[int, int]:
        """``(index, count)`` of ``rank`` among the batch-sharding positions (``data x fsdp``): which rows of the
        global batch it reads.  The ranks of a tensor-parallel group share an index."""
        c = self.coords(rank)
        shape = dict(zip(self.axis_names, self.devices.shape))
        return c["data"] * shape["fsdp"] + c["fsdp"], shape["data"] * shape["fsdp"]

    def slice_of(self, rank: int) -> int:
        """NVSwitch domain of ``rank`` (ranks are numbered slice by slice)."""
        return int(rank) // (self.size // self.num_slices)

    def within_one_slice(self, ranks) -> bool:
        """Whether ``ranks`` share an NVSwitch domain, i.e. may use the peer-memory kernels among themselves."""
        return len({self.slice_of(r) for r in ranks}) <= 1

    def expert_group_ranks(self, rank: int) -> list[int]:
        """Expert-parallel peers: consecutive blocks of ``expert`` ranks inside the batch-sharding ranks."""
        dp = self.ranks_along(("data", "fsdp"), rank)
        pos = dp.index(rank)
        start = pos - pos % self.expert
        return dp[start:start + self.expert]

    def group(self, axes: tuple[str, ...] | str, rank: int | None = None):
        """torch.distributed process group spanning ``axes`` for the calling rank (created on first use; every
        rank must call this with the same axes in the same order)."""
        import torch.distributed as dist

        axes = (axes,) if isinstance(axes, str) else tuple(axes)
        rank = dist.get_rank() if rank is None else rank
        key = axes
        if key not in self._groups:
            mine = None
            seen = set()
            for r in range(self.size):
                members = tuple(self.expert_group_ranks(r) if axes == ("expert",) else self.ranks_along(axes, r))
                if members in seen:
                    continue
                seen.add(members)
                g = dist.new_group(list(members))
                if rank in members:
                    mine = g
            self._groups[key] = mine
        return self._groups[key]


_GLOBAL_MESH: Mesh | None = None


def get_global_mesh() -> Mesh | None:
    return _GLOBAL_MESH


def create_mesh(config, devices=None) -> Mesh:
    """Build the ``data x fsdp x tensor`` grid over ``devices`` (a list of ranks; default: all ranks of the job,
    or a single device when torch.distributed is not initialised)."""
    if devices is None:
        try:
            import torch.distributed as dist

            n = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
        except Exception:
            n = 1
        devices = list(range(n))
    n = len(devices)
    dcn_cfg = {"data": int(config.dcn_data_parallelism), "fsdp": int(config.dcn_fsdp_parallelism),
               "tensor": int(config.dcn_tensor_parallelism)}
    slices = _num_slices(config, dcn_cfg, n)
    if slices > 1:
        if n % slices != 0:
            raise ValueError(f"multi-slice mesh: {n} devices do not split into {slices} slices")
        dcn = _resolve_auto_parallelism(dcn_cfg, slices, "DCN")
    else:
        dcn = {"data": 1, "fsdp": 1, "tensor": 1}
    ici = _resolve_auto_parallelism(
        {"data": config.ici_data_parallelism, "fsdp": config.ici_fsdp_parallelism,
         "tensor": config.ici_tensor_parallelism}, n // slices)
    sizes = {k: dcn[k] * ici[k] for k in AXES}
    ep = int(getattr(config, "ici_expert_parallelism", 1))
    dp = sizes["data"] * sizes["fsdp"]
    if ep < 1 or dp % ep != 0:
        raise ValueError(f"ici_expert_parallelism ({ep}) must divide data x fsdp ({dp})")
    # ranks are numbered slice by slice; on every axis the slice index is the slow part and the index inside the
    # slice the fast part
    grid = np.asarray(devices).reshape(*(dcn[k] for k in AXES), *(ici[k] for k in AXES))
    grid = grid.transpose(0, 3, 1, 4, 2, 5).reshape(sizes["data"], sizes["fsdp"], sizes["tensor"])
    return Mesh(devices=grid, expert=ep, num_slices=slices, dcn_shape=tuple(dcn[k] for k in AXES))


def _num_slices(config, dcn_cfg: dict[str, int], num_devices: int) -> int:
    """Slices (NVSwitch domains) of the job: ``num_slices`` when set above 1, else the product of the
    ``dcn_*_parallelism`` values when that is above 1.  The reference reads the slice of every device from the
    runtime (mintext/distributed/mesh.py:76-81); here the configuration says it, and a job whose DCN settings are all 1
    is laid out as one slice however many nodes it runs on."""
    if int(config.num_slices) > 1:
        return int(config.num_slices)
    known = 1
    for v in dcn_cfg.values():
        if v != -1:
            known *= v
    if -1 in dcn_cfg.values():
        raise ValueError("a DCN parallelism axis of -1 (auto) needs num_slices > 1 to resolve against")
    return known if known > 1 else 1


def setup_mesh(config) -> Mesh:
    """Create the mesh and make it the process-wide default."""
    global _GLOBAL_MESH
    _GLOBAL_MESH = create_mesh(config)
    logger.info("Mesh: %s", _GLOBAL_MESH.shape)
    return _GLOBAL_MESH


def initialize_distributed(timeout: int = 300) -> bool:
    """Join the job's process group if the launcher's environment describes one.

    Accepts torchrun variables (``RANK``, ``WORLD_SIZE``, ``LOCAL_RANK``, ``MASTER_ADDR``, ``MASTER_PORT``) and,
    as aliases, the reference launcher's ``JAX_COORDINATOR_IP`` / ``JAX_COORDINATOR_PORT`` / ``NNODES`` /
    ``NODE_RANK``.  Returns True when a multi-process group was initialised.  NCCL on GPUs, gloo on CPU-only hosts.
    """
    import torch
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size() > 1
    env = os.environ
    if "MASTER_ADDR" not in env and "JAX_COORDINATOR_IP" in env:
        env["MASTER_ADDR"] = env["JAX_COORDINATOR_IP"]
        env.setdefault("MASTER_PORT", env.get("JAX_COORDINATOR_PORT", "29500"))
    if "WORLD_SIZE" not in env and "NNODES" in env:
        per_node = int(env.get("GPUS_PER_NODE", "1"))
        env["WORLD_SIZE"] = str(int(env["NNODES"]) * per_node)
        env.setdefault("RANK", str(int(env.get("NODE_RANK", "0")) * per_node + int(env.get("LOCAL_RANK", "0"))))
    world = int(env.get("WORLD_SIZE", "1"))
    if world <= 1:
        return False
    env.setdefault("MASTER_ADDR", "127.0.0.1")
    env.setdefault("MASTER_PORT", "29500")
    use_cuda = torch.cuda.is_available()
    kwargs = {}
    if use_cuda:
        local = int(env.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        kwargs["device_id"] = torch.device("cuda", local)
    dist.init_process_group("nccl" if use_cuda else "gloo", timeout=datetime.timedelta(seconds=timeout), **kwargs)
    logger.info("Joined process group: rank %d of %d", dist.get_rank(), dist.get_world_size())
    return True

"""Distributed runtime: mesh, sharding rules, the training engine and the peer-memory communication kernels."""

from .mesh import Mesh, create_mesh, initialize_distributed, setup_mesh
from .partition import create_sharded_model
from .sharding import (NamedSharding, add_data_axis_to_sharding, create_named_sharding, get_input_data_sharding,
                       get_logical_axis_rules, get_model_param_shardings, logical_to_pspec)

__all__ = ["Mesh", "create_mesh", "setup_mesh", "initialize_distributed", "create_sharded_model", "NamedSharding",
           "get_logical_axis_rules", "logical_to_pspec", "create_named_sharding", "add_data_axis_to_sharding",
           "get_input_data_sharding", "get_model_param_shardings"]

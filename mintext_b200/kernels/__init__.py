"""MoE kernel API with the reference's names: route, unroute, grouped_matmul, grouped_matmul_vjp, tgmm."""

from .grouped_matmul import grouped_matmul, grouped_matmul_vjp, tgmm
from .moe_dispatch import route, unroute

__all__ = ["route", "unroute", "grouped_matmul", "grouped_matmul_vjp", "tgmm"]

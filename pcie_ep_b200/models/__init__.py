"""Model-level building blocks on top of the EP buffer: the expert-parallel MoE layer."""

from .moe_layer import MoELayer, dense_moe_reference

__all__ = ["MoELayer", "dense_moe_reference"]

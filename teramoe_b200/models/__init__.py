"""Model-level modules built on the expert-parallel layer."""
from .moe_layer import MoEBlock, TeraMoELayer, TopKRouter

__all__ = ["TeraMoELayer", "TopKRouter", "MoEBlock"]

"""Models built on the communication buffers: the expert-parallel MoE layer."""
from .moe_layer import MoEConfig, MoELayer

__all__ = ['MoEConfig', 'MoELayer']

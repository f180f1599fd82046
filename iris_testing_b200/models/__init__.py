"""Model-level modules: the expert-parallel MoE block."""
from .moe_layer import MoELayer, default_cap_rows, heap_bytes_needed

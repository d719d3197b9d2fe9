from . import fmha
from .fmha import AttentionBias, memory_efficient_attention

__all__ = ["fmha", "AttentionBias", "memory_efficient_attention"]

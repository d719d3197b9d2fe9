from . import attn_bias, flash
from .attn_bias import AttentionBias


def memory_efficient_attention(*args, **kwargs):
    raise NotImplementedError("xformers is not installed; use attn_impl='sdpa'")

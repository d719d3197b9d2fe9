"""h_t = gates_t * h_{t-1} + tokens_t along the last dim, as a log-depth parallel scan of PyTorch ops (twelve
elementwise passes for 4096 steps): the restated baseline for the reference's warp / Triton scan kernels."""
import torch


def _scan_last_dim(a, b):
    a, b = a.float(), b.float().clone()
    a = a.clone()
    L = a.shape[-1]
    d = 1
    while d < L:
        b[..., d:] = a[..., d:] * b[..., :-d] + b[..., d:]
        a[..., d:] = a[..., d:] * a[..., :-d]
        d *= 2
    return b


def scan(gates, tokens, reverse=False):
    if reverse:
        return _scan_last_dim(gates.flip(-1), tokens.flip(-1)).flip(-1).to(tokens.dtype)
    return _scan_last_dim(gates, tokens).to(tokens.dtype)

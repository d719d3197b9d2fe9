"""Call-compatible restatement of accelerated_scan.warp (forward and backward of the linear recurrence)."""
import torch

from .ref import _scan_last_dim


def warpscan_forward(gates, tokens, output, reverse=False):
    if reverse:
        output.copy_(_scan_last_dim(gates.flip(-1), tokens.flip(-1)).flip(-1))
    else:
        output.copy_(_scan_last_dim(gates, tokens))


def warpscan_backward(gates, states, dout, d_gates, d_tokens):
    """lambda_t = dout_t + gates_{t+1} * lambda_{t+1}; d_tokens = lambda; d_gates_t = lambda_t * states_{t-1}."""
    g_next = torch.cat([gates[..., 1:], torch.zeros_like(gates[..., :1])], dim=-1)
    lam = _scan_last_dim(g_next.flip(-1), dout.flip(-1)).flip(-1)
    d_tokens.copy_(lam)
    prev = torch.cat([torch.zeros_like(states[..., :1]), states[..., :-1]], dim=-1)
    d_gates.copy_(lam * prev.float())

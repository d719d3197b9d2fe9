"""PyTorch restatement of causal_conv1d.causal_conv1d_varlen.causal_conv1d_varlen_states."""
import torch


def causal_conv1d_varlen_states(x, cu_seqlens, state_len):
    """x [total_tokens, dim] packed documents -> [n_docs, dim, state_len]: the last `state_len` inputs of each
    document, zero-padded on the left."""
    ends = cu_seqlens[1:].long()
    starts = cu_seqlens[:-1].long()
    idx = ends.view(-1, 1) - state_len + torch.arange(state_len, device=x.device).view(1, -1)
    valid = idx >= starts.view(-1, 1)
    g = x[idx.clamp(min=0)]
    g = torch.where(valid.unsqueeze(-1), g, torch.zeros_like(g))
    return g.permute(0, 2, 1).contiguous()

"""PyTorch restatement of the `causal_conv1d_cuda` extension for the reference arm of the benchmark.

The reference's recurrent models call a CUDA extension that cannot be built offline. These functions keep its
call signatures (as used by apps/mamba/component/causal_conv1d_compilable.py of the reference) and compute the
same results with ordinary PyTorch ops, so that the reference's own model code can be timed as a baseline:
depthwise causal convolution along the last dim of x [batch, channels, length] with weight [channels, width],
optional bias, optional SiLU, and `seq_idx` [batch, length] document ids that the window must not cross.
"""
import torch
import torch.nn.functional as F


def _conv_math(x, weight, bias, seq_idx, activation):
    B, C, L = x.shape
    W = weight.shape[1]
    xf = x.float()
    if seq_idx is None:
        out = F.conv1d(F.pad(xf, (W - 1, 0)), weight.float().unsqueeze(1), None if bias is None else bias.float(), groups=C)
    else:
        out = torch.zeros_like(xf)
        for j in range(W):
            shift = W - 1 - j
            xs = F.pad(xf, (shift, 0))[..., :L]
            ids = F.pad(seq_idx, (shift, 0), value=-1)[..., :L]
            same = (ids == seq_idx).unsqueeze(1)
            out = out + weight[:, j].float().view(1, C, 1) * torch.where(same, xs, torch.zeros_like(xs))
        if bias is not None:
            out = out + bias.float().view(1, C, 1)
    if activation:
        out = F.silu(out)
    return out


def _conv(x, weight, bias, seq_idx, activation):
    out = _conv_math(x, weight, bias, seq_idx, activation)
    # same memory layout as the input (the extension writes channel-last outputs for channel-last inputs, and the
    # reference's traced graph relies on it)
    res = torch.empty_like(x)
    res.copy_(out)
    return res


def causal_conv1d_fwd(x, weight, bias, seq_idx, initial_states, final_states_out, activation):
    assert initial_states is None and final_states_out is None
    return _conv(x, weight, bias, seq_idx, activation)


def causal_conv1d_bwd(x, weight, bias, dout, seq_idx, initial_states, dfinal_states, dx, return_dinitial_states,
                      activation):
    """Gradients written out by hand: the body of a custom op runs below autograd, so nothing can be recorded here."""
    B, C, L = x.shape
    W = weight.shape[1]
    xf, wf, g = x.float(), weight.float(), dout.float()
    if activation:
        pre = _conv_math(x, weight, bias, seq_idx, False)
        sig = torch.sigmoid(pre)
        g = g * sig * (1 + pre * (1 - sig))
    dxf = torch.zeros_like(xf)
    dw = torch.zeros_like(wf)
    for j in range(W):
        shift = W - 1 - j  # out[t] takes w[:, j] * x[t - shift]
        xs = F.pad(xf, (shift, 0))[..., :L]
        if seq_idx is not None:
            ids = F.pad(seq_idx, (shift, 0), value=-1)[..., :L]
            same = (ids == seq_idx).unsqueeze(1)
            xs = torch.where(same, xs, torch.zeros_like(xs))
            gm = torch.where(same, g, torch.zeros_like(g))
        else:
            gm = g
        dw[:, j] = (gm * xs).sum(dim=(0, 2))
        # x[t] receives w[:, j] * g[t + shift]
        dxf = dxf + wf[:, j].view(1, C, 1) * F.pad(gm, (0, shift))[..., shift:]
    dbias = g.sum(dim=(0, 2)).to(bias.dtype) if bias is not None else torch.empty((0,), device=x.device)
    dx_out = torch.empty_like(x)
    dx_out.copy_(dxf)
    return dx_out, dw.to(weight.dtype), dbias, None


def causal_conv1d_update(x, conv_state, weight, bias, activation, cache_seqlens):
    """x [batch, channels, 1]; conv_state [batch, channels, state_len] shifted in place."""
    assert cache_seqlens is None
    W = weight.shape[1]
    conv_state.copy_(torch.roll(conv_state, shifts=-1, dims=-1))
    conv_state[:, :, -1] = x[:, :, 0]
    out = (conv_state[:, :, -W:].float() * weight.float().unsqueeze(0)).sum(-1)
    if bias is not None:
        out = out + bias.float()
    if activation:
        out = F.silu(out)
    return out.to(x.dtype).unsqueeze(-1)

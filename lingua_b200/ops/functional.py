"""Raw (non-autograd) ops: each has a native sm_100a kernel and a PyTorch reference.

The reference implementations restate the math of lingua/transformer.py in fp32
(cross_entropy :51-56, apply_rotary_emb :126-139, RMSNorm :283-289, FeedForward :467-472)
and serve both as the CPU path and as the oracle of the kernel tests. CUDA tensors always
take the native kernel; there is no PyTorch fallback on a GPU.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from . import _lib

ACT_SILU, ACT_RELU2 = 0, 1


def _L():
    return _lib.load()


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


# ----------------------------------------------------------------------------- RMSNorm
def rmsnorm_fwd_ref(x, w, eps, res=None):
    h = x.float() if res is None else (x.float() + res.float()).to(x.dtype).float()
    rstd = torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps)
    y = (h * rstd * w.float()).to(x.dtype)
    return y, (h.to(x.dtype) if res is not None else None), rstd.squeeze(-1)


def rmsnorm_fwd(x: torch.Tensor, w: torch.Tensor, eps: float, res: Optional[torch.Tensor] = None):
    """y = rmsnorm(x + res) * w. Returns (y, h, rstd) with h = x + res (None when res is None)."""
    if not x.is_cuda:
        return rmsnorm_fwd_ref(x, w, eps, res)
    D = x.shape[-1]
    x2 = x.reshape(-1, D)
    assert x2.is_contiguous() and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    M = x2.shape[0]
    y = torch.empty_like(x2)
    h = torch.empty_like(x2) if res is not None else None
    rstd = torch.empty(M, dtype=torch.float32, device=x.device)
    if res is not None:
        assert res.is_contiguous() and res.numel() == x.numel()
    rc = _L().lb_rmsnorm_fwd(x2.data_ptr(), _ptr(res), w.data_ptr(), y.data_ptr(), _ptr(h), rstd.data_ptr(),
                             M, D, eps, _lib.stream_ptr())
    _lib.check(rc, "lb_rmsnorm_fwd")
    return y.view(x.shape), (h.view(x.shape) if h is not None else None), rstd


def rmsnorm_bwd_ref(dy, h, w, rstd, dres=None):
    hf, dyf = h.float(), dy.float()
    xhat = hf * rstd.unsqueeze(-1)
    g = dyf * w.float()
    dx = rstd.unsqueeze(-1) * (g - xhat * (g * xhat).mean(-1, keepdim=True))
    if dres is not None:
        dx = dx + dres.float()
    dw = (dyf * xhat).reshape(-1, h.shape[-1]).sum(0)
    return dx.to(h.dtype), dw


def rmsnorm_bwd(dy, h, w, rstd, dres=None, dw_out: Optional[torch.Tensor] = None):
    """Returns (dh, dw). dw is accumulated into ``dw_out`` (fp32) when given."""
    if not dy.is_cuda:
        dx, dw = rmsnorm_bwd_ref(dy, h, w, rstd.view(h.shape[:-1]), dres)
        if dw_out is not None:
            dw_out.add_(dw.to(dw_out.dtype))
            dw = dw_out
        return dx, dw
    D = h.shape[-1]
    M = h.numel() // D
    assert dy.is_contiguous() and h.is_contiguous()
    dx = torch.empty_like(h)
    if dw_out is None:
        dw_out = torch.zeros(D, dtype=torch.float32, device=h.device)
    assert dw_out.dtype == torch.float32
    rc = _L().lb_rmsnorm_bwd(dy.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr(), _ptr(dres), dx.data_ptr(),
                             dw_out.data_ptr(), M, D, _lib.stream_ptr())
    _lib.check(rc, "lb_rmsnorm_bwd")
    return dx, dw_out


# ----------------------------------------------------------------------------- RoPE
def rope_table(head_dim: int, end: int, theta: float, device=None) -> torch.Tensor:
    """[end, head_dim/2, 2] fp32 table of (cos, sin) of pos * theta^(-2i/head_dim)
    (the angles of lingua/transformer.py:72-94)."""
    freqs = 1.0 / (theta ** (torch.arange(0, head_dim, 2)[: head_dim // 2].float() / head_dim))
    t = torch.arange(end)
    ang = torch.outer(t, freqs).float()
    return torch.stack((ang.cos(), ang.sin()), dim=-1).to(device)


def rope_ref(x, cs, pos=None, backward=False):
    """x: [B, S, H, Dh]; interleaved pairs rotated by the table row of each position."""
    B, S, H, Dh = x.shape
    tab = cs[:S] if pos is None else cs[pos.view(B, S).long()]
    cos, sin = tab[..., 0], tab[..., 1]
    if backward:
        sin = -sin
    if pos is None:
        cos, sin = cos.view(1, S, 1, Dh // 2), sin.view(1, S, 1, Dh // 2)
    else:
        cos, sin = cos.view(B, S, 1, Dh // 2), sin.view(B, S, 1, Dh // 2)
    xf = x.float().reshape(B, S, H, Dh // 2, 2)
    a, b = xf[..., 0], xf[..., 1]
    out = torch.stack((a * cos - b * sin, a * sin + b * cos), dim=-1)
    return out.reshape(B, S, H, Dh).to(x.dtype)


def rope_(qkv: torch.Tensor, cs: torch.Tensor, n_rot_heads: int, head_dim: int, seq_len: int,
          pos: Optional[torch.Tensor] = None, backward: bool = False) -> torch.Tensor:
    """In-place rotation of the first ``n_rot_heads`` heads of every row of ``qkv`` [tokens, heads*head_dim]."""
    n_tok = qkv.shape[0]
    if not qkv.is_cuda:
        B = n_tok // seq_len
        part = qkv[:, : n_rot_heads * head_dim].reshape(B, seq_len, n_rot_heads, head_dim)
        qkv[:, : n_rot_heads * head_dim] = rope_ref(part, cs, pos, backward).reshape(n_tok, -1)
        return qkv
    assert qkv.stride(-1) == 1 and qkv.dtype == torch.bfloat16 and cs.dtype == torch.float32
    if pos is not None:
        assert pos.dtype == torch.int32 and pos.numel() == n_tok
    rc = _L().lb_rope(qkv.data_ptr(), cs.data_ptr(), _ptr(pos), n_tok, seq_len, qkv.stride(0), n_rot_heads,
                      head_dim, int(backward), _lib.stream_ptr())
    _lib.check(rc, "lb_rope")
    return qkv


# ----------------------------------------------------------------------------- activations
def _act_ref(g, mode):
    return torch.nn.functional.silu(g) if mode == ACT_SILU else torch.relu(g).pow(2)


def glu_fwd(gu: torch.Tensor, mode: int = ACT_SILU) -> torch.Tensor:
    """gu: [M, 2H] = [gate | up] -> act(gate) * up, [M, H]."""
    M, H2 = gu.shape
    H = H2 // 2
    if not gu.is_cuda:
        g, u = gu[:, :H].float(), gu[:, H:].float()
        return (_act_ref(g, mode) * u).to(gu.dtype)
    assert gu.is_contiguous()
    out = torch.empty(M, H, dtype=gu.dtype, device=gu.device)
    _lib.check(_L().lb_glu_fwd(gu.data_ptr(), out.data_ptr(), M, H, mode, _lib.stream_ptr()), "lb_glu_fwd")
    return out


def glu_bwd(gu: torch.Tensor, dout: torch.Tensor, mode: int = ACT_SILU, inplace: bool = False) -> torch.Tensor:
    M, H2 = gu.shape
    H = H2 // 2
    if not gu.is_cuda:
        g = gu[:, :H].float().detach().requires_grad_(True)
        u = gu[:, H:].float().detach().requires_grad_(True)
        with torch.enable_grad():
            o = _act_ref(g, mode) * u
        dg, du = torch.autograd.grad(o, (g, u), dout.float())
        return torch.cat((dg, du), dim=1).to(gu.dtype)
    assert gu.is_contiguous() and dout.is_contiguous()
    dgu = gu if inplace else torch.empty_like(gu)
    _lib.check(_L().lb_glu_bwd(gu.data_ptr(), dout.data_ptr(), dgu.data_ptr(), M, H, mode, _lib.stream_ptr()),
               "lb_glu_bwd")
    return dgu


def act_fwd(x: torch.Tensor, mode: int) -> torch.Tensor:
    if not x.is_cuda:
        return _act_ref(x.float(), mode).to(x.dtype)
    assert x.is_contiguous()
    y = torch.empty_like(x)
    _lib.check(_L().lb_act_fwd(x.data_ptr(), y.data_ptr(), x.numel(), mode, _lib.stream_ptr()), "lb_act_fwd")
    return y


def act_bwd(x: torch.Tensor, dy: torch.Tensor, mode: int) -> torch.Tensor:
    if not x.is_cuda:
        xf = x.float().detach().requires_grad_(True)
        with torch.enable_grad():
            y = _act_ref(xf, mode)
        return torch.autograd.grad(y, xf, dy.float())[0].to(x.dtype)
    dx = torch.empty_like(x)
    _lib.check(_L().lb_act_bwd(x.data_ptr(), dy.data_ptr(), dx.data_ptr(), x.numel(), mode, _lib.stream_ptr()),
               "lb_act_bwd")
    return dx


def add(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    if not a.is_cuda:
        return (a.float() + b.float()).to(a.dtype)
    assert a.is_contiguous() and b.is_contiguous() and a.numel() == b.numel()
    out = torch.empty_like(a)
    _lib.check(_L().lb_add(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), _lib.stream_ptr()), "lb_add")
    return out


# ----------------------------------------------------------------------------- embedding
def embed_fwd(tokens: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    if not table.is_cuda:
        return table[tokens.reshape(-1)].view(*tokens.shape, table.shape[1])
    tok = tokens.reshape(-1).contiguous()
    assert tok.dtype == torch.int64
    V, D = table.shape
    out = torch.empty(tok.numel(), D, dtype=table.dtype, device=table.device)
    _lib.check(_L().lb_embed_fwd(tok.data_ptr(), table.data_ptr(), out.data_ptr(), tok.numel(), D, V,
                                 _lib.stream_ptr()), "lb_embed_fwd")
    return out.view(*tokens.shape, D)


def embed_bwd(tokens: torch.Tensor, dy: torch.Tensor, dtable: torch.Tensor) -> torch.Tensor:
    """dtable[tokens] += dy; dtable is an fp32 accumulation buffer [V, D]."""
    V, D = dtable.shape
    tok = tokens.reshape(-1).contiguous()
    if not dtable.is_cuda:
        dtable.index_add_(0, tok, dy.reshape(-1, D).to(dtable.dtype))
        return dtable
    assert dtable.dtype == torch.float32 and dy.is_contiguous()
    _lib.check(_L().lb_embed_bwd(tok.data_ptr(), dy.data_ptr(), dtable.data_ptr(), tok.numel(), D, V,
                                 _lib.stream_ptr()), "lb_embed_bwd")
    return dtable


# ----------------------------------------------------------------------------- cross-entropy
def ce_fwd(logits: torch.Tensor, target: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-row (loss, lse) of fp32 logits [rows, V]; rows with target < 0 get loss 0."""
    if not logits.is_cuda:
        lf = logits.float()
        lse = torch.logsumexp(lf, dim=-1)
        valid = target >= 0
        tgt = lf.gather(1, target.clamp(min=0).unsqueeze(1)).squeeze(1)
        return torch.where(valid, lse - tgt, torch.zeros_like(lse)), lse
    rows, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and target.dtype == torch.int64
    loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
    lse = torch.empty_like(loss)
    _lib.check(_L().lb_ce_fwd(logits.data_ptr(), target.data_ptr(), loss.data_ptr(), lse.data_ptr(), rows, V,
                              logits.stride(0), _lib.stream_ptr()), "lb_ce_fwd")
    return loss, lse


def ce_bwd(logits, target, lse, scale: float, gscale: Optional[torch.Tensor] = None, out_dtype=torch.bfloat16,
           out: Optional[torch.Tensor] = None):
    """dlogits = (softmax - onehot) * scale * gscale[0]; rows with target < 0 get zeros.

    ``out``: optional [rows, V] bf16 destination (unit stride along V, row pitch a multiple of 8)."""
    if not logits.is_cuda:
        p = torch.exp(logits.float() - lse.unsqueeze(1))
        valid = (target >= 0).unsqueeze(1)
        p.scatter_add_(1, target.clamp(min=0).unsqueeze(1), -torch.ones_like(p[:, :1]))
        g = scale * (gscale.float().reshape(()) if gscale is not None else 1.0)
        res = (p * valid * g).to(out_dtype)
        if out is not None:
            out.copy_(res)
            return out
        return res
    rows, V = logits.shape
    if out is not None:
        assert out.shape == (rows, V) and out.dtype == torch.bfloat16 and out.stride(1) == 1 and out.stride(0) % 8 == 0
        d = out
    else:
        d = torch.empty(rows, (V + 7) // 8 * 8, dtype=torch.bfloat16, device=logits.device)[:, :V]
    _lib.check(_L().lb_ce_bwd(logits.data_ptr(), target.data_ptr(), lse.data_ptr(), _ptr(gscale), scale,
                              d.data_ptr(), rows, V, logits.stride(0), d.stride(0), _lib.stream_ptr()), "lb_ce_bwd")
    return d


# ----------------------------------------------------------------------------- optimiser
def sumsq(g: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[0] += sum(g^2) for a flat fp32 tensor."""
    if not g.is_cuda:
        out += g.float().pow(2).sum()
        return out
    assert g.dtype == torch.float32 and g.is_contiguous() and out.dtype == torch.float32
    _lib.check(_L().lb_sumsq(g.data_ptr(), g.numel(), out.data_ptr(), _lib.stream_ptr()), "lb_sumsq")
    return out


def adamw_step(p, m, v, g, p16, *, step: int, lr: float, beta1: float, beta2: float, eps: float, wd: float,
               sumsq_t: Optional[torch.Tensor] = None, max_norm: float = 0.0, grad_mul: float = 1.0) -> None:
    """One AdamW update of flat fp32 (p, m, v) from flat fp32 g (torch.optim.AdamW arithmetic,
    lingua/optim.py:151-158), with clipping by the global norm sqrt(sumsq_t[0]) * grad_mul folded in
    and the bf16 copy ``p16`` refreshed."""
    if not p.is_cuda:
        clip = grad_mul
        if sumsq_t is not None and max_norm > 0:
            nrm = float(sumsq_t.sqrt()) * grad_mul
            clip *= min(1.0, max_norm / (nrm + 1e-6))
        gg = g.float() * clip
        p.mul_(1 - lr * wd)
        m.mul_(beta1).add_(gg, alpha=1 - beta1)
        v.mul_(beta2).addcmul_(gg, gg, value=1 - beta2)
        bc1 = 1 - beta1 ** step
        bc2 = 1 - beta2 ** step
        denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
        p.addcdiv_(m, denom, value=-lr / bc1)
        if p16 is not None:
            p16.copy_(p)
        return
    rc = _L().lb_adamw(p.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(), _ptr(p16), p.numel(),
                       _ptr(sumsq_t), max_norm, grad_mul, lr, beta1, beta2, eps, wd, step, _lib.stream_ptr())
    _lib.check(rc, "lb_adamw")


def cast_f32_bf16(src: torch.Tensor, dst: torch.Tensor) -> None:
    if not src.is_cuda:
        dst.copy_(src)
        return
    _lib.check(_L().lb_cast_f32_bf16(src.data_ptr(), dst.data_ptr(), src.numel(), _lib.stream_ptr()), "lb_cast")

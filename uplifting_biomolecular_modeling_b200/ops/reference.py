"""Plain PyTorch statements of every fused op.

These are the framework's ``off`` path and the oracle of every kernel test: each function is the
textbook form of the op (LayerNorm, Linear, softmax written out), runs on CPU or GPU in whatever
dtype its inputs have, and allocates the intermediates a fused kernel avoids.  Parameter naming
follows the upstream modules the kits patch (Boltz-2 layers:
boltz2/stock/src/boltz/model/layers/triangular_mult.py:49-54, transition.py, attentionv2.py,
triangular_attention/attention.py:44-50, outer_product_mean.py).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F


def layer_norm(x, weight=None, bias=None, eps: float = 1e-5):
    return F.layer_norm(x, (x.shape[-1],), weight, bias, eps)


def transition(x, norm_w, norm_b, fc1, fc2, fc3, residual: bool = False, eps: float = 1e-5):
    """SwiGLU transition: fc3(silu(fc1 n) * fc2 n), n = LN(x).  fc1/fc2: [hidden, c], fc3: [c, hidden]."""
    n = layer_norm(x, norm_w, norm_b, eps)
    y = F.linear(F.silu(F.linear(n, fc1)) * F.linear(n, fc2), fc3)
    return x + y if residual else y


def triangle_multiplication(z, mask, norm_in_w, norm_in_b, p_in, g_in, norm_out_w, norm_out_b, p_out, g_out,
                            outgoing: bool = True, residual: bool = False, eps: float = 1e-5):
    """z: [..., N, N, c]; mask: [..., N, N] or None; p_in/g_in: [2c_h, c]; p_out/g_out: [c, c_h]."""
    x = layer_norm(z, norm_in_w, norm_in_b, eps)
    x_in = x
    x = F.linear(x, p_in) * torch.sigmoid(F.linear(x, g_in))
    if mask is not None:
        x = x * mask.unsqueeze(-1).to(x.dtype)
    a, b = torch.chunk(x.float(), 2, dim=-1)
    if outgoing:
        x = torch.einsum("...ikd,...jkd->...ijd", a, b)
    else:
        x = torch.einsum("...kid,...kjd->...ijd", a, b)
    x = x.to(z.dtype)
    x = F.linear(layer_norm(x, norm_out_w, norm_out_b, eps), p_out) * torch.sigmoid(F.linear(x_in, g_out))
    return z + x if residual else x


def attention_with_bias(q, k, v, bias=None, key_mask=None, scale: Optional[float] = None):
    """softmax(scale * q k^T + bias) v.  q: [..., H, Q, D]; k, v: [..., H, K, D]; bias broadcastable to
    [..., H, Q, K]; key_mask: [..., K] (1 = keep)."""
    d = q.shape[-1]
    scale = (1.0 / math.sqrt(d)) if scale is None else scale
    s = torch.einsum("...qd,...kd->...qk", q.float(), k.float()) * scale
    if bias is not None:
        s = s + bias.float()
    if key_mask is not None:
        s = s.masked_fill(~key_mask.bool()[..., None, None, :], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("...qk,...kd->...qd", p, v.float()).to(q.dtype)


def triangle_attention(z, mask, ln_w, ln_b, w_bias, w_q, w_k, w_v, w_g, b_g, w_o, b_o, heads: int,
                       starting: bool = True, residual: bool = False, eps: float = 1e-5, inf: float = 1e9):
    """Triangle attention around the starting (rows) or ending (columns) node.

    z: [N, N, c]; mask: [N, N] or None.  w_bias: [H, c]; w_q/k/v/g: [H*D, c]; w_o: [c, H*D].
    The ending-node form is the starting-node form on the transposed pair tensor.
    """
    x = z if starting else z.transpose(-2, -3)
    m = None if mask is None else (mask if starting else mask.transpose(-1, -2))
    n = layer_norm(x, ln_w, ln_b, eps)
    N = n.shape[-2]
    tri_bias = F.linear(n, w_bias).permute(2, 0, 1)                      # [H, j, k]
    q = F.linear(n, w_q).view(*n.shape[:-1], heads, -1).transpose(-2, -3)  # [i, H, j, D]
    k = F.linear(n, w_k).view(*n.shape[:-1], heads, -1).transpose(-2, -3)
    v = F.linear(n, w_v).view(*n.shape[:-1], heads, -1).transpose(-2, -3)
    g = torch.sigmoid(F.linear(n, w_g, b_g))
    bias = tri_bias.unsqueeze(0).float()
    if m is not None:
        bias = bias + (inf * (m.float() - 1.0))[:, None, None, :]
    o = attention_with_bias(q, k, v, bias)                               # [i, H, j, D]
    o = o.transpose(-2, -3).reshape(*n.shape[:-1], -1)
    o = F.linear(o * g, w_o, b_o)
    if not starting:
        o = o.transpose(-2, -3)
    return z + o if residual else o


def attention_pair_bias(s, z, mask, norm_s_w, norm_s_b, w_q, b_q, w_k, w_v, w_g, norm_z_w, norm_z_b, w_z, w_o,
                        heads: int, residual: bool = False, k_in=None, eps: float = 1e-5, inf: float = 1e6,
                        pre_normed: bool = False):
    """Single-representation attention with pair bias (AttentionPairBias).  s: [B, N, c_s]; z: [B, N, N, c_z]."""
    x = s if pre_normed else layer_norm(s, norm_s_w, norm_s_b, eps)
    kin = x if k_in is None else k_in
    B, N, _ = x.shape
    q = F.linear(x, w_q, b_q).view(B, N, heads, -1).transpose(1, 2)
    k = F.linear(kin, w_k).view(B, kin.shape[1], heads, -1).transpose(1, 2)
    v = F.linear(kin, w_v).view(B, kin.shape[1], heads, -1).transpose(1, 2)
    g = torch.sigmoid(F.linear(x, w_g))
    bias = F.linear(layer_norm(z, norm_z_w, norm_z_b, eps), w_z).permute(0, 3, 1, 2).float()
    if mask is not None:
        bias = bias + ((1.0 - mask.float()) * -inf)[:, None, None, :]
    o = attention_with_bias(q, k, v, bias)
    o = o.transpose(1, 2).reshape(B, N, -1)
    o = F.linear(g * o, w_o)
    return s + o if residual else o


def outer_product_mean(m, mask, norm_w, norm_b, w_a, w_b, w_o, b_o, eps: float = 1e-5):
    """m: [B, S, N, c_m]; mask: [B, S, N]; w_a/w_b: [c_h, c_m]; w_o: [c_z, c_h*c_h]."""
    n = layer_norm(m, norm_w, norm_b, eps)
    mk = mask.unsqueeze(-1).to(n.dtype)
    a = F.linear(n, w_a) * mk
    b = F.linear(n, w_b) * mk
    num = torch.einsum("bsic,bsjd->bijcd", a.float(), b.float())
    cnt = torch.einsum("bsi,bsj->bij", mask.float(), mask.float()).clamp(min=1.0)
    z = (num / cnt[..., None, None]).reshape(*num.shape[:3], -1).to(m.dtype)
    return F.linear(z, w_o, b_o)


def pair_weighted_averaging(m, z, mask, norm_m_w, norm_m_b, norm_z_w, norm_z_b, w_m, w_g, w_z, w_o, heads: int,
                            eps: float = 1e-5, inf: float = 1e6):
    """m: [B, S, N, c_m]; z: [B, N, N, c_z]; mask: [B, N, N]; weights softmax_j(w_z LN(z)) shared over S."""
    mn = layer_norm(m, norm_m_w, norm_m_b, eps)
    zn = layer_norm(z, norm_z_w, norm_z_b, eps)
    B, S, N, _ = mn.shape
    v = F.linear(mn, w_m).view(B, S, N, heads, -1).permute(0, 3, 1, 2, 4)   # [B, H, S, N, c]
    b = F.linear(zn, w_z).permute(0, 3, 1, 2).float()                       # [B, H, N, N]
    b = b + ((1.0 - mask.float()) * -inf)[:, None]
    w = torch.softmax(b, dim=-1)
    g = torch.sigmoid(F.linear(mn, w_g))
    o = torch.einsum("bhij,bhsjd->bhsid", w, v.float()).to(m.dtype)
    o = o.permute(0, 2, 3, 1, 4).reshape(B, S, N, -1)
    return F.linear(g * o, w_o)


def adaln(a, s, s_norm_w, w_scale, b_scale, w_shift, eps: float = 1e-5):
    """Adaptive LayerNorm: sigmoid(Linear(LN(s))) * LN_noaffine(a) + LinearNoBias(LN(s))."""
    an = F.layer_norm(a, (a.shape[-1],), None, None, eps)
    sn = F.layer_norm(s, (s.shape[-1],), s_norm_w, None, eps)
    return torch.sigmoid(F.linear(sn, w_scale, b_scale)) * an + F.linear(sn, w_shift)


def window_attention(q, k, v, bias, wq: int = 32, wk: int = 128):
    """Atom attention in windows: query window w (wq atoms) sees the wk keys centred on it.

    q: [B, H, A, D] with A a multiple of wq; k, v: [B, H, A, D]; bias: [B, H, A/wq, wq, wk] or None.
    Keys outside [0, A) are masked.
    """
    B, H, A, D = q.shape
    nw = A // wq
    pad = (wk - wq) // 2
    kp = F.pad(k, (0, 0, pad, pad))
    vp = F.pad(v, (0, 0, pad, pad))
    idx = (torch.arange(nw, device=q.device) * wq)[:, None] + torch.arange(wk, device=q.device)[None, :]
    kw = kp[:, :, idx]                                   # [B, H, nw, wk, D]
    vw = vp[:, :, idx]
    valid = ((idx - pad) >= 0) & ((idx - pad) < A)       # [nw, wk]
    qw = q.view(B, H, nw, wq, D)
    s = torch.einsum("bhwqd,bhwkd->bhwqk", qw.float(), kw.float()) / math.sqrt(D)
    if bias is not None:
        s = s + bias.float()
    s = s.masked_fill(~valid[None, None, :, None, :], float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = torch.einsum("bhwqk,bhwkd->bhwqd", p, vw.float())
    return o.reshape(B, H, A, D).to(q.dtype)


# ------------------------------------------------------------------------------------------
# Plain statements of the row / sequence kernels in ops.seq (fp32 arithmetic on the given values).
def rmsnorm_rows(x, scale, eps: float = 1e-6):
    x32 = x.float()
    return x32 * torch.rsqrt(x32.pow(2).mean(-1, keepdim=True) + eps) * scale.float()


def causal_fir(x, h, tail=None):
    """x: [B, L, C]; h: [C, K] (h[:, 0] multiplies the current sample); tail: [B, K-1, C] or None."""
    B, L, C = x.shape
    K = h.shape[1]
    pad = x.new_zeros((B, K - 1, C)) if tail is None else tail.to(x.dtype)
    xp = torch.cat([pad, x], 1).float()
    y = torch.zeros((B, L, C), dtype=torch.float32, device=x.device)
    for k in range(K):
        y = y + h[:, k].float() * xp[:, K - 1 - k:K - 1 - k + L]
    return y


def fir_gate3(z, h, tail=None):
    zf = causal_fir(z, h, tail)
    x1, x2, v = zf.chunk(3, -1)
    return x1 * v, x2


def fir_inner_gate(u, h, D, x2, tail=None):
    y = causal_fir(u, h, tail) + u.float() * D.float()
    return y if x2 is None else x2.float() * y


def fftconv_epilogue(y, u, D, x2):
    L = u.shape[1]
    out = y[..., :L].transpose(1, 2).float() + u.float() * D.float()
    return out if x2 is None else x2.float() * out


def pole_step(state, lam, res, u, D, x2):
    s = state * lam.float().unsqueeze(0) + u.float().unsqueeze(-1)
    y = (s * res.float().unsqueeze(0)).sum(-1) + u.float() * D.float()
    return (y if x2 is None else x2.float() * y), s


def gelu_new(x):
    x = x.float()
    return 0.5 * x * (1.0 + torch.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))


def rotary_split_qkv(qkv, pos, heads: int, rot: int, base: float = 10000.0):
    T = qkv.shape[0]
    Dh = qkv.shape[1] // (3 * heads)
    q, k, v = qkv.float().view(T, 3, heads, Dh).unbind(1)
    inv = base ** (-torch.arange(0, rot, 2, device=qkv.device, dtype=torch.float32) / rot)
    ang = pos.float()[:, None] * inv[None, :]
    sn, cs = torch.sin(ang)[:, None, :], torch.cos(ang)[:, None, :]

    def rotate(t):
        t = t.clone()
        a, b = t[..., 0:rot:2], t[..., 1:rot:2]
        t[..., 0:rot:2], t[..., 1:rot:2] = a * cs - b * sn, b * cs + a * sn
        return t
    return rotate(q), rotate(k), v


def pool2(x, mode: str = "max", w=None):
    B, L, C = x.shape
    xp = x.float().view(B, L // 2, 2, C)
    if mode == "max":
        return xp.max(2).values
    if mode == "mean":
        return xp.mean(2)
    return (xp * torch.softmax(w.float().view(B, L // 2, 2, C), 2)).sum(2)


def residual_ln(x, res, gamma, beta, eps: float = 1e-5):
    s = (x.float() + res.float()).to(x.dtype).float()
    return torch.nn.functional.layer_norm(s, (s.shape[-1],), gamma.float(), None if beta is None else beta.float(), eps)


def column_attention(q, k, v, index, bias=None, scale=None):
    """q: [T, H, D]; k, v: [R, T, H, D]; index: [C] clade -> row; bias: [H, C] or None."""
    D = q.shape[-1]
    sc = float(D) ** -0.5 if scale is None else float(scale)
    kc, vc = k.float()[index.long()], v.float()[index.long()]          # [C, T, H, D]
    s = torch.einsum("thd,cthd->thc", q.float(), kc) * sc
    if bias is not None:
        s = s + bias.float().unsqueeze(0)
    return torch.einsum("thc,cthd->thd", torch.softmax(s, -1), vc)


def relative_shift(pos):
    """pos: [..., L, >= 2L - 1] -> [..., L, L] with out[i, j] = pos[i, j - i + L - 1]."""
    L = pos.shape[-2]
    j = torch.arange(L, device=pos.device)
    gather = (j[None, :] - j[:, None] + L - 1).expand(pos.shape[:-2] + (L, L))
    return torch.gather(pos, -1, gather)


def relshift_softmax(content, pos):
    return torch.softmax(content.float() + relative_shift(pos.float()), -1)

"""CPU stand-ins for ``basedxl_b200.ops`` built from the oracle, for testing the
HOST logic (wrappers, comm manager, UNet wrapper, pipeline) on gloo ranks
without a GPU.  Installed by monkeypatching the attributes of the ``ops`` module
inside a test process; nothing in the package refers to this file.

Same calling conventions as the real wrappers: NHWC-contiguous strips,
``[rows, cols]`` matrices, fp32 moments ``[2, B, G]``.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from oracle import patched_ops as po

MODE_LOCAL, MODE_SYNC, MODE_STALE = 0, 1, 2


def _nchw(x):
    return x.permute(0, 3, 1, 2)


def _nhwc(x):
    return x.permute(0, 2, 3, 1).contiguous()


def gemm(a, b, bias=None, residual=None, out=None, b_is_kn=False, out_f32=False):
    y = a @ (b if b_is_kn else b.t())
    if bias is not None:
        y = y + bias
    if residual is not None:
        y = y + residual
    if out is not None:
        out.copy_(y)
        return out
    return y


def gemm_dual(a, w, n1, bias=None, out1=None, out2=None):
    y = a @ w.t()
    if bias is not None:
        y = y + bias
    y1, y2 = y[:, :n1].contiguous(), y[:, n1:].contiguous()
    if out1 is not None:
        out1.copy_(y1)
        y1 = out1
    if out2 is not None:
        out2.copy_(y2)
        y2 = out2
    return y1, y2


def gemm_geglu(a, w_interleaved, bias_interleaved=None, out=None):
    h = a @ w_interleaved.t()
    if bias_interleaved is not None:
        h = h + bias_interleaved
    m, n = h.shape
    h = h.view(m, n // 32, 2, 16)
    y = (h[:, :, 0] * F.gelu(h[:, :, 1])).reshape(m, n // 2)
    if out is not None:
        out.copy_(y)
        return out
    return y


def conv_weight_pack(w):
    co, ci = w.shape[:2]
    return w.permute(0, 2, 3, 1).reshape(co, 9 * ci).contiguous()


def conv3x3(x, w_packed, bias=None, stride=1, top=None, bot=None, bias_rows=None, residual=None, out=None):
    b, h, wd, ci = x.shape
    co = w_packed.shape[0]
    w = w_packed.view(co, 3, 3, ci).permute(0, 3, 1, 2)
    zeros = x.new_zeros(b, 1, wd, ci)
    padded = torch.cat([zeros if top is None else top, x, zeros if bot is None else bot], dim=1)
    y = F.conv2d(_nchw(padded), w, bias, stride=stride, padding=(0, 1))
    if bias_rows is not None:
        y = y + bias_rows[:, :, None, None]
    y = _nhwc(y)
    if residual is not None:
        y = y + residual
    if out is not None:
        out.copy_(y)
        return out
    return y


def halo_pack(x, pad=1, out=None):
    y = torch.stack([x[:, :pad], x[:, -pad:]], dim=0).contiguous()
    if out is not None:
        out.copy_(y.view(out.shape))
        return out
    return y


def groupnorm_stats(x, groups, out=None):
    m = po.groupnorm_moments(_nchw(x).contiguous(), groups).reshape(2, x.shape[0], groups).float()
    if out is not None:
        out.copy_(m)
        return out
    return m


def groupnorm_apply(x, groups, eps, gamma, beta, fresh, peers=None, own=0, mode=MODE_LOCAL, silu=False, out=None):
    b = x.shape[0]
    shape = (2, b, groups, 1, 1, 1)
    xs = _nchw(x).contiguous()
    if mode == MODE_LOCAL:
        y = po.groupnorm_pp(xs, groups, eps, gamma, beta, None, own, "local")
    else:
        pm = [(fresh if (mode == MODE_SYNC and j == own) else p)[: 2 * b * groups].reshape(shape).to(x.dtype) for j, p in enumerate(peers)]
        y = po.groupnorm_pp(xs, groups, eps, gamma, beta, pm, own, "sync" if mode == MODE_SYNC else "stale")
    if silu:
        y = F.silu(y)
    y = _nhwc(y)
    if out is not None:
        out.copy_(y)
        return out
    return y


def groupnorm_fused(x, groups, eps, gamma, beta, peers=None, own=0, mode=MODE_LOCAL, silu=False, fresh_out=None, halo_out=None, out=None):
    fresh = groupnorm_stats(x, groups)
    y = groupnorm_apply(x, groups, eps, gamma, beta, fresh, peers, own, mode, silu=silu, out=out)
    if fresh_out is not None:
        fresh_out.copy_(fresh.view(fresh_out.shape))  # after the stale values have been used
    if halo_out is not None:
        halo_out.copy_(torch.stack([y[:, :1], y[:, -1:]], dim=0).reshape(halo_out.shape))
    return y


def attention(q, kv_slots, heads, scale=None, out=None):
    y = po._sdpa_heads(q, torch.cat(list(kv_slots), dim=1), heads)
    if out is not None:
        out.copy_(y)
        return out
    return y


def upsample2x(x):
    return _nhwc(F.interpolate(_nchw(x), scale_factor=2.0, mode="nearest"))


def layernorm(x, gamma, beta, eps):
    return F.layer_norm(x, (x.shape[-1],), gamma, beta, eps)


def geglu(h):
    a, g = h.chunk(2, dim=-1)
    return a * F.gelu(g)


def install():
    """Replace the kernel wrappers of ``basedxl_b200.ops`` by the functions above."""
    from basedxl_b200 import ops

    for name in ("gemm", "gemm_dual", "gemm_geglu", "conv_weight_pack", "conv3x3", "halo_pack", "groupnorm_stats", "groupnorm_apply", "groupnorm_fused", "attention",
                 "upsample2x", "layernorm", "geglu"):
        setattr(ops, name, globals()[name])

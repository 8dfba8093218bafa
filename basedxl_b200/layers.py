"""Leaf layers of the host UNet graph, backed by the library's kernels.

Each class subclasses the ``torch.nn`` module it stands for, so parameter
names, ``state_dict`` layout and ``isinstance`` checks (the patch-parallel swap
in ``basedxl_b200.unet`` keys on ``nn.Conv2d`` / ``nn.GroupNorm`` / ``Attention``)
are the stock ones; only ``forward`` differs: it launches sm_100a kernels and
has no other path.

Image tensors are ``[B, C, H, W]``-shaped with channels-last strides.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import ops
from .modules.attn import _finish, _folded, _lin, fuse_kv, qkv_project
from .modules.base_module import as_nchw, as_nhwc
from .modules.conv2d import check_conv, packed_weight


class Conv2d(nn.Conv2d):
    supports_fused_epilogue = True

    def forward(self, x, *args, bias_rows=None, residual=None, **kwargs):
        if tuple(self.kernel_size) == (1, 1):
            # 1x1 convolution = a matmul over NHWC pixels
            xh = as_nhwc(x)
            b, h, w, c = xh.shape
            r2 = None if residual is None else as_nhwc(residual).reshape(-1, self.out_channels)
            y = ops.gemm(xh.reshape(-1, c), self.weight.view(self.out_channels, c), bias=self.bias, residual=r2)
            return as_nchw(y.view(b, h, w, self.out_channels))
        check_conv(self)
        fused = {}
        if bias_rows is not None:
            fused["bias_rows"] = bias_rows
        if residual is not None:
            fused["residual"] = as_nhwc(residual)
        y = ops.conv3x3(as_nhwc(x), packed_weight(self), self.bias, stride=self.stride[0], **fused)
        return as_nchw(y)


class GroupNorm(nn.GroupNorm):
    supports_fused_epilogue = True
    fuse_silu = False  # set per instance by the host graph where a SiLU follows

    def forward(self, x, silu=None):
        if silu is None:
            silu = self.fuse_silu
        y = ops.groupnorm_fused(as_nhwc(x), self.num_groups, self.eps, self.weight if self.affine else None,
                                self.bias if self.affine else None, silu=silu)
        return as_nchw(y)


class Linear(nn.Linear):
    supports_fused_epilogue = True

    def forward(self, x, residual=None, ln=None, want_stats: bool = False):
        """``ln = (LayerNorm module, RowStats of x)``: x is un-normalised and the LayerNorm is folded into
        this projection; ``want_stats``: also return the row statistics of the result."""
        return _lin(self, x, residual=residual, ln=ln, want_stats=want_stats)


class LayerNorm(nn.LayerNorm):
    def forward(self, x):
        return ops.layernorm(x if x.is_contiguous() else x.contiguous(), self.weight, self.bias, self.eps)


class Attention(nn.Module):
    """Multi-head attention block with the attribute surface the patch-parallel
    wrappers read: ``to_q, to_k, to_v, to_out[0], to_out[1], heads,
    residual_connection, rescale_output_factor``.  Head dimension 64."""

    supports_fused_epilogue = True
    # forward() accepts ln=(LayerNorm module, RowStats of the un-normalised input) and want_stats
    supports_layernorm_fold = True

    def __init__(self, query_dim: int, heads: int, cross_attention_dim: int | None = None, linear_cls=Linear):
        super().__init__()
        ctx = cross_attention_dim or query_dim
        self.heads = heads
        self.is_cross = cross_attention_dim is not None
        self.to_q = linear_cls(query_dim, query_dim, bias=False)
        self.to_k = linear_cls(ctx, query_dim, bias=False)
        self.to_v = linear_cls(ctx, query_dim, bias=False)
        self.to_out = nn.ModuleList([linear_cls(query_dim, query_dim, bias=True), nn.Dropout(0.0)])
        self.residual_connection = False
        self.rescale_output_factor = 1.0
        self._kv = None
        self._ctx_kv = None   # cross-attention: K/V of the conditioning, reused across steps
        self._ctx_key = None
        self._ctx_ref = None

    def _fused_kv(self) -> nn.Linear:
        key = (self.to_k.weight.data_ptr(), self.to_k.weight._version, self.to_v.weight._version)
        if self._kv is None or self._kv[0] != key:
            self._kv = (key, fuse_kv(self.to_k, self.to_v))
        return self._kv[1]

    def _project_kv(self, ctx: torch.Tensor, out=None) -> torch.Tensor:
        """K|V of ``ctx`` as one ``[B, L, 2C]`` tensor.  With stock Linear projections this is one
        GEMM on the stacked weight; with swapped-in replacements the two projections are called
        as they are and their results laid side by side."""
        if isinstance(self.to_k, nn.Linear):
            return _lin(self._fused_kv(), ctx, out=out)
        kv = torch.cat([_lin(self.to_k, ctx), _lin(self.to_v, ctx)], dim=-1)
        if out is not None:
            out.copy_(kv.reshape(out.shape))
            return out.view(*ctx.shape[:-1], kv.shape[-1])
        return kv

    def context_kv(self, ctx: torch.Tensor, force: bool = False) -> torch.Tensor:
        """K/V projection of the conditioning, computed when the conditioning tensor changes
        (new storage or a new version) and otherwise reused: it is the same for all denoising
        steps of an image (what the reference's patched cross-attention does with its
        ``kv_cache``, basedxl/modules/attn.py:74-78).  Refreshed IN PLACE so that a captured
        step graph keeps reading valid storage."""
        key = (ctx.data_ptr(), ctx._version, tuple(ctx.shape))
        b, l, _ = ctx.shape
        if self._ctx_kv is None or self._ctx_kv.shape[:2] != (b, l):
            self._ctx_kv = self._project_kv(ctx)
        elif force or key != self._ctx_key:
            self._project_kv(ctx, out=self._ctx_kv.view(b * l, -1))
        self._ctx_key = key
        self._ctx_ref = ctx  # keeps the storage alive, so its address cannot be reused by another tensor
        return self._ctx_kv

    def forward(self, hidden_states, encoder_hidden_states=None, scale: float = 1.0, *args, residual=None, ln=None,
                want_stats: bool = False, **kwargs):
        if encoder_hidden_states is None:
            if type(self.to_q) is Linear and self.to_q.out_features % 32 == 0:
                q, kv = qkv_project(self, self.to_q, self._fused_kv(), hidden_states, ln=ln)
            else:
                assert ln is None
                q, kv = _lin(self.to_q, hidden_states), self._project_kv(hidden_states)
        else:
            q = _lin(self.to_q, hidden_states, ln=ln)
            kv = self.context_kv(encoder_hidden_states)
        o = ops.attention(q, [kv], self.heads)
        return _finish(self, o, hidden_states, residual, want_stats=want_stats)


def silu(x):
    return torch.nn.functional.silu(x)


def geglu(h):
    return ops.geglu(h if h.is_contiguous() else h.contiguous())


def linear_geglu(layer: nn.Linear, x, ln=None):
    """GEGLU projection with the gate applied in the GEMM epilogue.  The interleaved copy of
    the weight is cached on the layer (inference: parameters are frozen).  ``ln = (LayerNorm
    module, RowStats of x)`` folds that LayerNorm into the projection."""
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    if ln is not None:
        fold = _folded(layer, "_bxl_geglu_ln", ln[0], layer.weight, layer.bias, interleave=True)
        y = ops.gemm_fused(x2, None, geglu=True, ln=(ln[1], fold))
        return y.view(*lead, fold.weight.shape[0] // 2)
    w = layer.weight
    cache = getattr(layer, "_bxl_geglu", None)
    if cache is None or cache[0] != (w.data_ptr(), w._version):
        layer._bxl_geglu = ((w.data_ptr(), w._version), ops.geglu_interleave(w.detach(), None if layer.bias is None else layer.bias.detach()))
    wi, bi = layer._bxl_geglu[1]
    y = ops.gemm_geglu(x2, wi, bi)
    return y.view(*lead, wi.shape[0] // 2)


def upsample2x(x):
    return as_nchw(ops.upsample2x(as_nhwc(x)))


class KernelLayers:
    """Layer factory handed to the host graph: everything runs on the library."""

    Conv2d, GroupNorm, Linear, LayerNorm, Attention = Conv2d, GroupNorm, Linear, LayerNorm, Attention
    silu = staticmethod(silu)
    geglu = staticmethod(geglu)
    linear_geglu = staticmethod(linear_geglu)
    upsample2x = staticmethod(upsample2x)
    memory_format = torch.channels_last
    batched_time_projection = True   # all residual blocks' time-embedding projections in one GEMM
    fold_layernorm = True            # LayerNorm -> Linear pairs run as one GEMM on the un-normalised input
    linear = staticmethod(lambda x, w, b=None: ops.linear(x, w, b))

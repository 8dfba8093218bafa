"""Patch-parallel attention wrappers (reference: basedxl/modules/attn.py).

``BasedXLSelfAttentionPP``: local queries against the full key/value sequence,
which lives as one ``[B, L_local, 2C]`` slot per strip inside the comm
manager's staging buffers.  The fused ``to_kv`` projection writes this strip's
fresh K/V straight into its own slot, and the attention kernel reads all slots
in place (no concatenation).

``BasedXLCrossAttentionPP``: K/V of the text context are computed once per
image (``counter == 0``) and cached.

The wrapped module must expose what the reference reads off diffusers'
``Attention``: ``to_q, to_k, to_v, to_out[0], to_out[1], heads,
residual_connection, rescale_output_factor`` (attn.py:16-17,69,82,94-101).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops
from ..utils import BasedXLConfig
from .base_module import BaseModule


def fuse_kv(to_k: nn.Linear, to_v: nn.Linear) -> nn.Linear:
    """One Linear with weight [W_k; W_v] (basedxl/modules/attn.py:16-39)."""
    assert isinstance(to_k, nn.Linear) and isinstance(to_v, nn.Linear)
    assert (to_k.bias is None) == (to_v.bias is None)
    assert to_k.weight.shape == to_v.weight.shape
    in_size, out_size = to_k.in_features, to_k.out_features
    to_kv = nn.Linear(in_size, out_size * 2, bias=to_k.bias is not None, device=to_k.weight.device, dtype=to_k.weight.dtype)
    to_kv.weight.data[:out_size].copy_(to_k.weight.data)
    to_kv.weight.data[out_size:].copy_(to_v.weight.data)
    if to_k.bias is not None:
        to_kv.bias.data[:out_size].copy_(to_k.bias.data)
        to_kv.bias.data[out_size:].copy_(to_v.bias.data)
    return to_kv


def fuse_qkv(to_q: nn.Linear, to_kv: nn.Linear):
    """Stacked weight [W_q; W_k; W_v] (and bias) for the single-launch q | k|v projection."""
    w = torch.cat([to_q.weight.detach(), to_kv.weight.detach()], dim=0).contiguous()
    if (to_q.bias is None) != (to_kv.bias is None):
        zq = to_q.bias if to_q.bias is not None else torch.zeros_like(to_q.weight[:, 0])
        zk = to_kv.bias if to_kv.bias is not None else torch.zeros_like(to_kv.weight[:, 0])
        b = torch.cat([zq.detach(), zk.detach()])
    else:
        b = None if to_q.bias is None else torch.cat([to_q.bias.detach(), to_kv.bias.detach()])
    return w, b


def _folded(owner, slot: str, norm: nn.Module, weight: torch.Tensor, bias, interleave: bool = False):
    """``ops.FoldedLayerNorm`` of (norm, weight, bias), cached on ``owner`` (inference: parameters
    are frozen).  ``interleave`` applies the GEGLU row order first."""
    gamma, beta = getattr(norm, "weight", None), getattr(norm, "bias", None)
    key = (weight.data_ptr(), weight._version, None if bias is None else bias._version,
           None if gamma is None else (gamma.data_ptr(), gamma._version), None if beta is None else beta._version)
    cache = getattr(owner, slot, None)
    if cache is None or cache[0] != key:
        w, b = weight.detach(), None if bias is None else bias.detach()
        if interleave:
            w, b = ops.geglu_interleave(w, b)
        cache = (key, ops.FoldedLayerNorm(w, b, gamma, beta, norm.eps))
        setattr(owner, slot, cache)
    return cache[1]


def can_fold_layernorm(norm: nn.Module, *linears) -> bool:
    """A LayerNorm can be folded into the projections that consume it when those are stock
    ``nn.Linear`` layers on a CUDA device in fp16 (swapped-in replacements keep their own path)."""
    return (isinstance(norm, nn.LayerNorm) and len(norm.normalized_shape) == 1
            and all(isinstance(l, nn.Linear) and l.weight.is_cuda and l.weight.dtype == torch.float16 for l in linears))


def qkv_project(owner, to_q: nn.Linear, to_kv: nn.Linear, x: torch.Tensor, kv_out=None, ln=None):
    """q and k|v of self-attention from one GEMM launch; ``kv_out`` (``[rows, 2C]`` view, any row
    stride) receives k|v, e.g. this strip's staging slot.  The stacked weight is cached on
    ``owner`` (inference: parameters are frozen).  ``ln = (norm, RowStats of x)``: ``x`` is the
    UN-normalised input and the LayerNorm is folded into the projection."""
    key = (to_q.weight.data_ptr(), to_q.weight._version, to_kv.weight.data_ptr(), to_kv.weight._version)
    cache = getattr(owner, "_bxl_qkv", None)
    if cache is None or cache[0] != key:
        owner._bxl_qkv = (key, fuse_qkv(to_q, to_kv))
    w, b = owner._bxl_qkv[1]
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    c = to_q.out_features
    if ln is not None:
        norm, stats = ln
        fold = _folded(owner, "_bxl_qkv_ln", norm, w, b)
        q, kv = ops.gemm_fused(x2, None, n_split=c, out2=kv_out, ln=(stats, fold))
    else:
        q, kv = ops.gemm_dual(x2, w, c, bias=b, out2=kv_out)
    return q.view(*lead, c), kv.view(*lead, 2 * c) if kv_out is None else None


def _lin(layer: nn.Module, x: torch.Tensor, residual=None, out=None, ln=None, want_stats: bool = False):
    """``layer(x)`` (+ residual) on the library's GEMM.  ``ln = (norm, RowStats of x)`` folds that
    LayerNorm into the projection (``x`` un-normalised); ``want_stats`` also returns the RowStats
    of the result.  Both need a stock ``nn.Linear``."""
    if not isinstance(layer, nn.Linear):
        assert ln is None and not want_stats
        # a swapped-in replacement (e.g. BasedXLLowPLinear, which keeps its weight as [K, N])
        y = layer(x, residual=residual) if getattr(layer, "supports_fused_epilogue", False) else layer(x)
        if residual is not None and not getattr(layer, "supports_fused_epilogue", False):
            y = y + residual
        if out is not None:
            out.copy_(y.reshape(out.shape))
            return out.view(*x.shape[:-1], out.shape[-1])
        return y
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    r2 = None if residual is None else residual.reshape(-1, layer.out_features)
    if ln is not None or want_stats:
        if x2.stride(1) != 1:
            x2 = x2.contiguous()
        fold = None if ln is None else (ln[1], _folded(layer, "_bxl_ln", ln[0], layer.weight, layer.bias))
        res = ops.gemm_fused(x2, layer.weight, bias=layer.bias, residual=r2, out=out, ln=fold, want_stats=want_stats)
        if want_stats:
            return res[0].view(*lead, layer.out_features), res[1]
        return res.view(*lead, layer.out_features)
    y = ops.gemm(x2, layer.weight, bias=layer.bias, residual=r2, out=out)
    return y.view(*lead, layer.out_features)


def _finish(attn, o: torch.Tensor, hidden_in: torch.Tensor, residual, want_stats: bool = False):
    """to_out projection, then the module's own residual / rescale options
    (basedxl/modules/attn.py:158-166), then the transformer block's outer residual.  The outer
    residual rides in the projection's epilogue only when the module's options leave the
    projection's result untouched; otherwise it is added after them, as the block would.
    ``want_stats`` (plain case only): also return the row statistics of the result."""
    plain = not attn.residual_connection and attn.rescale_output_factor == 1.0
    if want_stats:
        assert plain
        return _lin(attn.to_out[0], o, residual=residual, want_stats=True)
    y = _lin(attn.to_out[0], o, residual=residual if plain else None)
    # to_out[1] is a Dropout; inference only
    if attn.residual_connection:
        y = y + hidden_in
    if attn.rescale_output_factor != 1.0:
        y = y / attn.rescale_output_factor
    if residual is not None and not plain:
        y = y + residual
    return y


def attention_supports_folding(attn_like) -> bool:
    """Whether an attention module (or its patch-parallel wrapper) can take an un-normalised input
    plus its row statistics and can emit the row statistics of its output."""
    m = getattr(attn_like, "module", attn_like)
    return (getattr(attn_like, "supports_layernorm_fold", False) and not m.residual_connection
            and m.rescale_output_factor == 1.0 and isinstance(m.to_q, nn.Linear) and isinstance(m.to_out[0], nn.Linear)
            and m.to_q.weight.is_cuda and m.to_q.weight.dtype == torch.float16 and m.to_q.out_features % 32 == 0)


class BasedXLAttentionPP(BaseModule):
    # forward() accepts ln=(LayerNorm module, RowStats of the un-normalised input) and want_stats
    supports_layernorm_fold = True

    def __init__(self, module: nn.Module, basedxl_config: BasedXLConfig):
        super().__init__(module, basedxl_config)
        self.to_kv = fuse_kv(module.to_k, module.to_v)


class BasedXLCrossAttentionPP(BasedXLAttentionPP):
    def __init__(self, module: nn.Module, basedxl_config: BasedXLConfig):
        super().__init__(module, basedxl_config)
        self.kv_cache = None
        # set by the UNet wrapper in CUDA-graph mode: the cached K/V is then refreshed from outside
        # (``refresh_context_kv``) whenever the conditioning changes, not by the first step of an image
        self.kv_managed = False

    def refresh_context_kv(self, encoder_hidden_states: torch.Tensor):
        """(Re)compute the cached K/V of the conditioning, in place where the cache exists."""
        b, l, _ = encoder_hidden_states.shape
        if self.kv_cache is None or self.kv_cache.shape[:2] != (b, l):
            self.kv_cache = _lin(self.to_kv, encoder_hidden_states)
        else:
            _lin(self.to_kv, encoder_hidden_states, out=self.kv_cache.view(b * l, -1))

    def forward(self, hidden_states, encoder_hidden_states=None, scale: float = 1.0, *args, residual=None, ln=None,
                want_stats: bool = False, **kwargs):
        torch.cuda.nvtx.range_push("cross_attn::forward")
        assert encoder_hidden_states is not None
        attn = self.module
        q = _lin(attn.to_q, hidden_states, ln=ln)
        b, l, _ = encoder_hidden_states.shape
        if self.kv_cache is None or self.kv_cache.shape[:2] != (b, l) or (self.counter == 0 and not self.kv_managed):
            # K/V of the conditioning: once per image (basedxl/modules/attn.py:74-78); refreshed in
            # place, since a captured step graph keeps reading this storage
            self.refresh_context_kv(encoder_hidden_states)
        o = ops.attention(q, [self.kv_cache], attn.heads)
        y = _finish(attn, o, hidden_states, residual, want_stats=want_stats)
        self.counter += 1
        torch.cuda.nvtx.range_pop()
        return y


class BasedXLSelfAttentionPP(BasedXLAttentionPP):
    def __init__(self, module: nn.Module, basedxl_config: BasedXLConfig):
        super().__init__(module, basedxl_config)

    def _forward(self, hidden_states: torch.Tensor, scale: float = 1.0, residual=None, ln=None, want_stats: bool = False):
        attn = self.module
        cfg = self.basedxl_config
        assert self.comm_manager is not None
        n, idx = cfg.n_device_per_batch, cfg.split_idx()
        b, l, c = hidden_states.shape
        fusable = isinstance(attn.to_q, nn.Linear) and c % 32 == 0
        if n > 1 and self.buffer_list is not None:
            # fresh K/V is produced directly in the own staging slot (no concatenation, no staging
            # copy).  Synchronous step: it then goes to every peer and theirs arrive here before the
            # attention runs (attn.py:134-136); displaced step: the peers' slots are one step stale
            # and the fresh slot is queued for the asynchronous gather (attn.py:138-141).
            own = self.buffer_list[idx]
            if fusable:
                q, _ = qkv_project(self, attn.to_q, self.to_kv, hidden_states, kv_out=own.view(b * l, -1), ln=ln)
            else:
                assert ln is None
                q = _lin(attn.to_q, hidden_states)
                _lin(self.to_kv, hidden_states, out=own.view(b * l, -1))
            slots = list(self.buffer_list)
            if self.counter <= cfg.warmup_steps:
                self.comm_manager.sync_exchange(self.idx)
                own = None
        else:
            own = None
            if fusable:
                q, kv = qkv_project(self, attn.to_q, self.to_kv, hidden_states, ln=ln)
            else:
                assert ln is None
                q, kv = _lin(attn.to_q, hidden_states), _lin(self.to_kv, hidden_states)
            # one strip, or no staging buffers yet: own K/V stands in for every strip (attn.py:132-133)
            slots = [kv] * n
        o = ops.attention(q, slots, attn.heads)
        if own is not None:
            # queued only now: a gather that this call triggers is ordered after the attention
            # kernel, which still reads the peers' stale slots in place
            self.comm_manager.enqueue(self.idx, own)
        return _finish(attn, o, hidden_states, residual, want_stats=want_stats)

    def forward(self, hidden_states, encoder_hidden_states=None, scale: float = 1.0, *args, residual=None, ln=None,
                want_stats: bool = False, **kwargs):
        torch.cuda.nvtx.range_push("self_attn::forward")
        cfg = self.basedxl_config
        self._wait_pending()
        b, l, c = hidden_states.shape
        if cfg.n_device_per_batch > 1 and self.buffer_list is None and self.comm_manager is not None:
            if self.comm_manager.buffer_list is None:
                self.idx = self.comm_manager.register_tensor(
                    shape=(b, l, self.to_kv.out_features), torch_dtype=hidden_states.dtype, layer_type="attn"
                )
            else:
                self.buffer_list = self.comm_manager.get_buffer_list(self.idx)
        output = self._forward(hidden_states, scale=scale, residual=residual, ln=ln, want_stats=want_stats)
        self.counter += 1
        torch.cuda.nvtx.range_pop()
        return output

"""Stock ``torch.nn`` leaf layers for the host UNet graph, on the CPU.
Test infrastructure (see ``oracle/__init__.py``).

Handing this factory to ``basedxl_b200.sdxl_unet.UNet2DConditionModel`` gives
the same wiring and the same parameter names as the product graph, evaluated by
PyTorch's own CPU operators; state dicts are interchangeable.  None of these
layers advertises fused epilogues, so the graph performs bias-row adds, residual
adds and SiLU itself, in plain PyTorch.  The reference's patch-parallel wrappers
can be put around these layers unmodified (they are ``nn.Conv2d`` /
``nn.GroupNorm`` / attention modules with the attribute surface the reference
reads, basedxl/modules/attn.py:16-17,69,82,94-101).
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import patched_ops as po


class Attention(nn.Module):
    def __init__(self, query_dim: int, heads: int, cross_attention_dim: int | None = None):
        super().__init__()
        ctx = cross_attention_dim or query_dim
        self.heads = heads
        self.to_q = nn.Linear(query_dim, query_dim, bias=False)
        self.to_k = nn.Linear(ctx, query_dim, bias=False)
        self.to_v = nn.Linear(ctx, query_dim, bias=False)
        self.to_out = nn.ModuleList([nn.Linear(query_dim, query_dim, bias=True), nn.Dropout(0.0)])
        self.residual_connection = False
        self.rescale_output_factor = 1.0

    def forward(self, hidden_states, encoder_hidden_states=None, scale: float = 1.0, **kwargs):
        ctx = hidden_states if encoder_hidden_states is None else encoder_hidden_states
        wkv = torch.cat([self.to_k.weight, self.to_v.weight], dim=0)
        return po.cross_attention(
            hidden_states, ctx, self.to_q.weight, wkv, self.to_out[0].weight, self.to_out[0].bias, self.heads,
            self.residual_connection, self.rescale_output_factor,
        )


def geglu(h):
    a, g = h.chunk(2, dim=-1)
    return a * F.gelu(g)


class TorchLayers:
    Conv2d, GroupNorm, Linear, LayerNorm, Attention = nn.Conv2d, nn.GroupNorm, nn.Linear, nn.LayerNorm, Attention
    silu = staticmethod(F.silu)
    geglu = staticmethod(geglu)
    upsample2x = staticmethod(lambda x: F.interpolate(x, scale_factor=2.0, mode="nearest"))
    memory_format = None

"""Host graph: an SDXL-shaped conditional UNet.

The reference wraps the UNet of the third-party ``diffusers`` package
(basedxl/model.py:17-22, basedxl/unet.py:66-79); that package is not a
dependency here.  This module defines the same architecture from its published
hyper-parameters (three resolution levels of 320/640/1280 channels, two
residual blocks per level, 0/2/10 transformer layers per attention site, 5/10/20
heads of 64, cross-attention on 2048-wide text states, "text_time" additional
conditioning of 2816 inputs, 32-group norms) with the usual module names
(``conv_in``, ``down_blocks.N.resnets.M.conv1``, ``...attentions.M.transformer_blocks.K.attn1``,
``conv_norm_out``, ``conv_out`` ...), which is what the patch-parallel swap keys on.

The graph is written against a *layer factory* (``basedxl_b200.layers.KernelLayers``
by default) so that the same wiring can be instantiated over other leaf
implementations, e.g. stock ``torch.nn`` modules on the CPU for checking.
Fusable epilogues (per-image bias rows from the time embedding, residual adds,
SiLU after a norm) are passed to a leaf only if it advertises
``supports_fused_epilogue``; otherwise the graph performs them itself.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn as nn


@dataclass
class UNetConfig:
    in_channels: int = 4
    out_channels: int = 4
    block_out_channels: tuple = (320, 640, 1280)
    layers_per_block: int = 2
    transformer_layers_per_block: tuple = (0, 2, 10)  # 0 = plain residual stage
    num_attention_heads: tuple = (5, 10, 20)
    cross_attention_dim: int = 2048
    addition_time_embed_dim: int = 256
    projection_class_embeddings_input_dim: int = 2816
    norm_num_groups: int = 32
    norm_eps: float = 1e-5
    sample_size: int = 128

    def get(self, key, default=None):
        return getattr(self, key, default)


def sdxl_config() -> UNetConfig:
    return UNetConfig()


def tiny_config() -> UNetConfig:
    """A two-level miniature with the same structure, for tests."""
    return UNetConfig(
        block_out_channels=(64, 128),
        transformer_layers_per_block=(0, 1),
        num_attention_heads=(1, 2),
        cross_attention_dim=64,
        addition_time_embed_dim=32,
        projection_class_embeddings_input_dim=6 * 32 + 64,
        sample_size=32,
    )


def _fused(layer) -> bool:
    return bool(getattr(layer, "supports_fused_epilogue", False))


def sinusoidal_embedding(t: torch.Tensor, dim: int) -> torch.Tensor:
    """[N] -> [N, dim]: cos half first, then sin half; frequencies 10000^(-i/half)."""
    half = dim // 2
    freqs = torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    args = t.float()[:, None] * freqs[None, :]
    return torch.cat([torch.cos(args), torch.sin(args)], dim=-1)


class TimestepEmbedding(nn.Module):
    def __init__(self, L, in_dim: int, dim: int):
        super().__init__()
        self.L = L
        self.linear_1 = L.Linear(in_dim, dim)
        self.linear_2 = L.Linear(dim, dim)

    def forward(self, x):
        return self.linear_2(self.L.silu(self.linear_1(x)))


class ResnetBlock2D(nn.Module):
    def __init__(self, L, cin: int, cout: int, temb_dim: int, groups: int, eps: float):
        super().__init__()
        self.L = L
        self.norm1 = L.GroupNorm(groups, cin, eps=eps)
        self.conv1 = L.Conv2d(cin, cout, 3, padding=1)
        self.time_emb_proj = L.Linear(temb_dim, cout)
        self.norm2 = L.GroupNorm(groups, cout, eps=eps)
        self.conv2 = L.Conv2d(cout, cout, 3, padding=1)
        self.conv_shortcut = L.Conv2d(cin, cout, 1) if cin != cout else None
        self.t_pre = None   # this step's time-embedding projection, when the UNet computed all of them at once
        for n in (self.norm1, self.norm2):
            if _fused(n):
                n.fuse_silu = True

    def _norm_act(self, norm, x, conv=None):
        """norm + SiLU.  Returns (h, halo_packed): where the norm can write boundary rows and the
        convolution that consumes ``h`` offers its staging range, the rows ``conv`` publishes to the
        neighbouring strips are written by the norm's kernel."""
        # the swap may have wrapped the norm: the wrapper reads fuse_silu off the wrapped module
        inner = getattr(norm, "module", norm)
        if _fused(norm) and getattr(inner, "fuse_silu", False):
            staging = getattr(conv, "halo_staging", None)
            halo = staging() if staging is not None and getattr(norm, "supports_halo_out", False) else None
            if halo is not None:
                return norm(x, halo_out=halo), True
            return norm(x), False
        return self.L.silu(norm(x)), False

    def forward(self, x, temb_act):
        """``temb_act`` = SiLU(time embedding) [B, temb_dim]."""
        h, packed1 = self._norm_act(self.norm1, x, self.conv1)
        t, self.t_pre = self.t_pre, None
        if t is None:
            t = self.time_emb_proj(temb_act)  # [B, cout]
        if _fused(self.conv1):
            h = self.conv1(h, bias_rows=t, halo_packed=True) if packed1 else self.conv1(h, bias_rows=t)
        else:
            h = self.conv1(h) + t[:, :, None, None]
        h, packed2 = self._norm_act(self.norm2, h, self.conv2)
        sc = x if self.conv_shortcut is None else self.conv_shortcut(x)
        if _fused(self.conv2):
            return self.conv2(h, residual=sc, halo_packed=True) if packed2 else self.conv2(h, residual=sc)
        return self.conv2(h) + sc


class FeedForward(nn.Module):
    def __init__(self, L, dim: int):
        super().__init__()
        self.L = L
        self.proj = L.Linear(dim, dim * 8)   # GEGLU: value and gate halves, 4*dim each
        self.out = L.Linear(dim * 4, dim)

    def forward(self, x, residual, ln=None, want_stats: bool = False):
        """``ln = (LayerNorm module, row statistics of x)``: ``x`` is un-normalised and the LayerNorm is
        folded into the projection; ``want_stats``: also return the row statistics of the result."""
        fused_proj = getattr(self.L, "linear_geglu", None)
        if ln is not None:
            h = fused_proj(self.proj, x, ln=ln)
        else:
            h = fused_proj(self.proj, x) if fused_proj is not None and type(self.proj) is self.L.Linear else self.L.geglu(self.proj(x))
        if want_stats:
            return self.out(h, residual=residual, want_stats=True)
        if _fused(self.out):
            return self.out(h, residual=residual)
        return self.out(h) + residual


class BasicTransformerBlock(nn.Module):
    def __init__(self, L, dim: int, heads: int, cross_dim: int):
        super().__init__()
        self.L = L
        self.norm1 = L.LayerNorm(dim)
        self.attn1 = L.Attention(dim, heads)
        self.norm2 = L.LayerNorm(dim)
        self.attn2 = L.Attention(dim, heads, cross_attention_dim=cross_dim)
        self.norm3 = L.LayerNorm(dim)
        self.ff = FeedForward(L, dim)

    @staticmethod
    def _attn(attn, x, ctx, residual):
        if _fused(attn):
            return attn(x, encoder_hidden_states=ctx, residual=residual)
        return attn(x, encoder_hidden_states=ctx) + residual

    def folds_layernorm(self) -> bool:
        """Whether the three LayerNorms of this block can run inside the projections that consume
        them (the layer factory offers it and no projection has been swapped for another type)."""
        L = self.L
        if not getattr(L, "fold_layernorm", False):
            return False
        from .modules.attn import attention_supports_folding, can_fold_layernorm

        a1, a2 = getattr(self.attn1, "module", self.attn1), getattr(self.attn2, "module", self.attn2)
        return (attention_supports_folding(self.attn1) and attention_supports_folding(self.attn2)
                and can_fold_layernorm(self.norm1, a1.to_q, a1.to_k, a1.to_v) and can_fold_layernorm(self.norm2, a2.to_q)
                and can_fold_layernorm(self.norm3, self.ff.proj) and type(self.ff.proj) is L.Linear and type(self.ff.out) is L.Linear)

    def forward(self, h, ctx, stats=None, want_stats: bool = False):
        """``stats``: row statistics of ``h`` left by the GEMM that produced it.  When given, no
        LayerNorm kernel runs: every projection takes the un-normalised rows plus their statistics,
        and every GEMM that closes a residual branch emits the statistics for the next one."""
        if stats is None:
            h = self._attn(self.attn1, self.norm1(h), None, h)
            h = self._attn(self.attn2, self.norm2(h), ctx, h)
            return self.ff(self.norm3(h), residual=h)
        h, stats = self.attn1(h, encoder_hidden_states=None, residual=h, ln=(self.norm1, stats), want_stats=True)
        h, stats = self.attn2(h, encoder_hidden_states=ctx, residual=h, ln=(self.norm2, stats), want_stats=True)
        return self.ff(h, residual=h, ln=(self.norm3, stats), want_stats=want_stats)


class Transformer2DModel(nn.Module):
    def __init__(self, L, dim: int, heads: int, depth: int, cross_dim: int, groups: int):
        super().__init__()
        self.norm = L.GroupNorm(groups, dim, eps=1e-6)
        self.proj_in = L.Linear(dim, dim)
        self.transformer_blocks = nn.ModuleList([BasicTransformerBlock(L, dim, heads, cross_dim) for _ in range(depth)])
        self.proj_out = L.Linear(dim, dim)

    def forward(self, x, ctx):
        b, c, hh, ww = x.shape
        # channels-last image <-> token matrix is a view
        tokens = lambda t: t.permute(0, 2, 3, 1).reshape(b, hh * ww, c)
        res = tokens(x)
        blocks = list(self.transformer_blocks)
        if blocks and type(self.proj_in) is getattr(blocks[0].L, "Linear", None) and all(blk.folds_layernorm() for blk in blocks):
            # LayerNorms folded into the projections: proj_in emits the first row statistics
            h, stats = self.proj_in(tokens(self.norm(x)), want_stats=True)
            for i, blk in enumerate(blocks):
                last = i == len(blocks) - 1
                out = blk(h, ctx, stats=stats, want_stats=not last)
                h, stats = (out, None) if last else out
        else:
            h = self.proj_in(tokens(self.norm(x)))
            for blk in blocks:
                h = blk(h, ctx)
        if _fused(self.proj_out):
            h = self.proj_out(h, residual=res)
        else:
            h = self.proj_out(h) + res
        return h.view(b, hh, ww, c).permute(0, 3, 1, 2)


class Downsample2D(nn.Module):
    def __init__(self, L, ch: int):
        super().__init__()
        self.conv = L.Conv2d(ch, ch, 3, stride=2, padding=1)

    def forward(self, x):
        return self.conv(x)


class Upsample2D(nn.Module):
    def __init__(self, L, ch: int):
        super().__init__()
        self.L = L
        self.conv = L.Conv2d(ch, ch, 3, padding=1)

    def forward(self, x):
        return self.conv(self.L.upsample2x(x))


class DownBlock(nn.Module):
    def __init__(self, L, cfg: UNetConfig, cin, cout, temb_dim, depth, heads, add_downsample):
        super().__init__()
        g, e = cfg.norm_num_groups, cfg.norm_eps
        self.resnets = nn.ModuleList(
            [ResnetBlock2D(L, cin if i == 0 else cout, cout, temb_dim, g, e) for i in range(cfg.layers_per_block)]
        )
        self.attentions = (
            nn.ModuleList([Transformer2DModel(L, cout, heads, depth, cfg.cross_attention_dim, g) for _ in range(cfg.layers_per_block)])
            if depth > 0
            else None
        )
        self.downsamplers = nn.ModuleList([Downsample2D(L, cout)]) if add_downsample else None

    def forward(self, h, temb_act, ctx):
        outs = []
        for i, res in enumerate(self.resnets):
            h = res(h, temb_act)
            if self.attentions is not None:
                h = self.attentions[i](h, ctx)
            outs.append(h)
        if self.downsamplers is not None:
            h = self.downsamplers[0](h)
            outs.append(h)
        return h, outs


class MidBlock(nn.Module):
    def __init__(self, L, cfg: UNetConfig, ch, temb_dim, depth, heads):
        super().__init__()
        g, e = cfg.norm_num_groups, cfg.norm_eps
        self.resnets = nn.ModuleList([ResnetBlock2D(L, ch, ch, temb_dim, g, e) for _ in range(2)])
        self.attentions = nn.ModuleList([Transformer2DModel(L, ch, heads, depth, cfg.cross_attention_dim, g)])

    def forward(self, h, temb_act, ctx):
        h = self.resnets[0](h, temb_act)
        h = self.attentions[0](h, ctx)
        return self.resnets[1](h, temb_act)


class UpBlock(nn.Module):
    def __init__(self, L, cfg: UNetConfig, skip_channels, cprev, cout, temb_dim, depth, heads, add_upsample):
        super().__init__()
        g, e = cfg.norm_num_groups, cfg.norm_eps
        n = cfg.layers_per_block + 1
        self.resnets = nn.ModuleList(
            [ResnetBlock2D(L, (cprev if i == 0 else cout) + skip_channels[i], cout, temb_dim, g, e) for i in range(n)]
        )
        self.attentions = (
            nn.ModuleList([Transformer2DModel(L, cout, heads, depth, cfg.cross_attention_dim, g) for _ in range(n)])
            if depth > 0
            else None
        )
        self.upsamplers = nn.ModuleList([Upsample2D(L, cout)]) if add_upsample else None

    def forward(self, h, skips, temb_act, ctx):
        for i, res in enumerate(self.resnets):
            h = torch.cat([h, skips.pop()], dim=1)
            h = res(h, temb_act)
            if self.attentions is not None:
                h = self.attentions[i](h, ctx)
        if self.upsamplers is not None:
            h = self.upsamplers[0](h)
        return h


class UNet2DConditionModel(nn.Module):
    """``forward(sample, timestep, encoder_hidden_states, added_cond_kwargs, return_dict=False) -> (eps,)``."""

    def __init__(self, config: UNetConfig | None = None, layers=None):
        super().__init__()
        if layers is None:
            from .layers import KernelLayers as layers
        L = self.L = layers
        cfg = self.config = config or sdxl_config()
        ch = cfg.block_out_channels
        temb_dim = ch[0] * 4
        self.conv_in = L.Conv2d(cfg.in_channels, ch[0], 3, padding=1)
        self.time_embedding = TimestepEmbedding(L, ch[0], temb_dim)
        self.add_embedding = TimestepEmbedding(L, cfg.projection_class_embeddings_input_dim, temb_dim)
        levels = len(ch)
        self.down_blocks = nn.ModuleList()
        skip_ch = [ch[0]]
        cin = ch[0]
        for i in range(levels):
            last = i == levels - 1
            self.down_blocks.append(
                DownBlock(L, cfg, cin, ch[i], temb_dim, cfg.transformer_layers_per_block[i], cfg.num_attention_heads[i], not last)
            )
            skip_ch += [ch[i]] * cfg.layers_per_block + ([] if last else [ch[i]])
            cin = ch[i]
        self.mid_block = MidBlock(L, cfg, ch[-1], temb_dim, cfg.transformer_layers_per_block[-1], cfg.num_attention_heads[-1])
        self.up_blocks = nn.ModuleList()
        cprev = ch[-1]
        for j in range(levels):
            i = levels - 1 - j
            n = cfg.layers_per_block + 1
            skips = [skip_ch.pop() for _ in range(n)]
            self.up_blocks.append(
                UpBlock(L, cfg, skips, cprev, ch[i], temb_dim, cfg.transformer_layers_per_block[i], cfg.num_attention_heads[i], j < levels - 1)
            )
            cprev = ch[i]
        self.conv_norm_out = L.GroupNorm(cfg.norm_num_groups, ch[0], eps=cfg.norm_eps)
        if _fused(self.conv_norm_out):
            self.conv_norm_out.fuse_silu = True
        self.conv_out = L.Conv2d(ch[0], cfg.out_channels, 3, padding=1)

    @property
    def dtype(self):
        return next(self.parameters()).dtype

    def _project_time_embedding(self, temb_act):
        """The time-embedding projections of all residual blocks depend only on the step's
        embedding: one GEMM over the concatenated weights replaces 22 launches with two rows
        each.  Every block receives its column slice (rows a full projection apart)."""
        L = self.L
        if not getattr(L, "batched_time_projection", False):
            return
        blocks = [m for m in self.modules() if isinstance(m, ResnetBlock2D)]
        if not blocks or any(type(r.time_emb_proj) is not L.Linear for r in blocks):
            return  # a wrapper replaced some projection: leave them to the blocks
        key = tuple((r.time_emb_proj.weight.data_ptr(), r.time_emb_proj.weight._version, r.time_emb_proj.bias._version) for r in blocks)
        cache = getattr(self, "_time_proj_cache", None)
        if cache is None or cache[0] != key:
            w = torch.cat([r.time_emb_proj.weight.detach() for r in blocks]).contiguous()
            bias = torch.cat([r.time_emb_proj.bias.detach() for r in blocks]).contiguous()
            cache = (key, w, bias)
            self._time_proj_cache = cache
        t_all = L.linear(temb_act, cache[1], cache[2])
        off = 0
        for r in blocks:
            n = r.time_emb_proj.out_features
            r.t_pre = t_all[:, off : off + n]
            off += n

    def embed(self, timestep, batch: int, added_cond_kwargs, device):
        cfg = self.config
        if not torch.is_tensor(timestep):
            timestep = torch.tensor([timestep], dtype=torch.float32, device=device)
        t = timestep.reshape(-1).to(device).expand(batch) if timestep.numel() == 1 else timestep.to(device)
        t_emb = sinusoidal_embedding(t, cfg.block_out_channels[0]).to(self.dtype)
        emb = self.time_embedding(t_emb)
        text_embeds = added_cond_kwargs["text_embeds"]
        time_ids = added_cond_kwargs["time_ids"]
        ids = sinusoidal_embedding(time_ids.reshape(-1), cfg.addition_time_embed_dim).reshape(batch, -1)
        add = torch.cat([text_embeds.to(self.dtype), ids.to(self.dtype)], dim=-1)
        emb = emb + self.add_embedding(add)
        return self.L.silu(emb)

    def forward(self, sample, timestep, encoder_hidden_states, added_cond_kwargs=None, return_dict: bool = False, **kwargs):
        L = self.L
        b = sample.shape[0]
        temb_act = self.embed(timestep, b, added_cond_kwargs or {}, sample.device)
        self._project_time_embedding(temb_act)
        ctx = encoder_hidden_states.to(self.dtype)
        h = sample.to(self.dtype)
        if L.memory_format is not None:
            h = h.contiguous(memory_format=L.memory_format)
        h = self.conv_in(h)
        skips = [h]
        for blk in self.down_blocks:
            h, outs = blk(h, temb_act, ctx)
            skips += outs
        h = self.mid_block(h, temb_act, ctx)
        for blk in self.up_blocks:
            h = blk(h, skips, temb_act, ctx)
        inner = getattr(self.conv_norm_out, "module", self.conv_norm_out)
        if _fused(self.conv_norm_out) and getattr(inner, "fuse_silu", False):
            h = self.conv_norm_out(h)
        else:
            h = L.silu(self.conv_norm_out(h))
        h = self.conv_out(h)
        return (h,)

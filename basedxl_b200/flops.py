"""Algorithmic work of one UNet forward, from the graph's hyper-parameters.

Counts multiply-accumulates of every matmul-shaped operator (linears, 3x3 and
1x1 convolutions, attention score and value products) for a latent of
``h x w`` and one batch item; FLOPs = 2 x MACs.  Used for roofline figures.
"""
from __future__ import annotations

from .sdxl_unet import UNetConfig


def unet_macs(cfg: UNetConfig, h: int, w: int, ctx_len: int = 77) -> dict:
    ch = cfg.block_out_channels
    temb = ch[0] * 4
    macs = {"linear": 0, "conv3x3": 0, "conv1x1": 0, "self_attn": 0, "cross_attn": 0}

    def resnet(cin, cout, hh, ww):
        macs["conv3x3"] += hh * ww * 9 * (cin * cout + cout * cout)
        macs["linear"] += temb * cout
        if cin != cout:
            macs["conv1x1"] += hh * ww * cin * cout

    def transformer(dim, depth, hh, ww):
        L = hh * ww
        macs["linear"] += 2 * L * dim * dim  # proj_in, proj_out
        for _ in range(depth):
            macs["linear"] += L * dim * dim * 4            # attn1: q, k, v, out
            macs["self_attn"] += 2 * L * L * dim           # QK^T and PV over all heads
            macs["linear"] += 2 * L * dim * dim            # attn2: q, out
            macs["linear"] += 2 * ctx_len * cfg.cross_attention_dim * dim  # attn2: k, v of the text
            macs["cross_attn"] += 2 * L * ctx_len * dim
            macs["linear"] += L * dim * dim * 8 + L * dim * 4 * dim  # GEGLU proj + out

    macs["conv3x3"] += h * w * 9 * cfg.in_channels * ch[0]
    macs["linear"] += ch[0] * temb + temb * temb + cfg.projection_class_embeddings_input_dim * temb + temb * temb
    hh, ww = h, w
    skip = [ch[0]]
    cin = ch[0]
    levels = len(ch)
    for i in range(levels):
        for _ in range(cfg.layers_per_block):
            resnet(cin, ch[i], hh, ww)
            cin = ch[i]
            if cfg.transformer_layers_per_block[i]:
                transformer(ch[i], cfg.transformer_layers_per_block[i], hh, ww)
            skip.append(ch[i])
        if i < levels - 1:
            hh, ww = hh // 2, ww // 2
            macs["conv3x3"] += hh * ww * 9 * ch[i] * ch[i]
            skip.append(ch[i])
    resnet(ch[-1], ch[-1], hh, ww)
    transformer(ch[-1], cfg.transformer_layers_per_block[-1], hh, ww)
    resnet(ch[-1], ch[-1], hh, ww)
    cprev = ch[-1]
    for j in range(levels):
        i = levels - 1 - j
        for k in range(cfg.layers_per_block + 1):
            resnet((cprev if k == 0 else ch[i]) + skip.pop(), ch[i], hh, ww)
            if cfg.transformer_layers_per_block[i]:
                transformer(ch[i], cfg.transformer_layers_per_block[i], hh, ww)
        cprev = ch[i]
        if j < levels - 1:
            hh, ww = hh * 2, ww * 2
            macs["conv3x3"] += hh * ww * 9 * ch[i] * ch[i]
    macs["conv3x3"] += hh * ww * 9 * ch[0] * cfg.out_channels
    macs["total"] = sum(macs.values())
    return macs


def unet_flops(cfg: UNetConfig, h: int, w: int, batch: int = 1, ctx_len: int = 77) -> float:
    return 2.0 * batch * unet_macs(cfg, h, w, ctx_len)["total"]

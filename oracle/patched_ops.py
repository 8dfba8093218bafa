"""CPU restatement of the reference's patch-parallel operators.

Test infrastructure (see ``oracle/__init__.py``).  Each function restates one
reference operator as a pure function of explicit inputs: the fresh local
strip, the per-peer exchange buffers (stale or freshly gathered), and the
strip index.  Communication is *not* modelled here; callers hand in whatever
the exchange would have delivered.  All citations are paths inside the
reference project.

Tensors are ordinary NCHW / [B, L, C] host tensors.  Arithmetic is done in the
dtype of the inputs (callers use fp32 for the parity bar).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------
# Conv2d on an H-strip with neighbour halo rows
# --------------------------------------------------------------------------
def conv2d_boundary(x: torch.Tensor, pad: int) -> torch.Tensor:
    """Rows a strip publishes to its neighbours: ``[2, B, C, pad, W]`` with
    index 0 = its top rows and index 1 = its bottom rows
    (basedxl/modules/conv2d.py:92)."""
    return torch.stack([x[:, :, :pad, :], x[:, :, -pad:, :]], dim=0)


def conv2d_pp(
    x: torch.Tensor,
    weight: torch.Tensor,
    bias: torch.Tensor | None,
    stride: int,
    pad: int,
    peer_boundaries: list[torch.Tensor] | None,
    split_idx: int,
    n_split: int,
) -> torch.Tensor:
    """Patched convolution of one strip (basedxl/modules/conv2d.py:74-104).

    ``peer_boundaries[j]`` is strip j's published boundary (layout of
    :func:`conv2d_boundary`).  The strip above contributes its bottom rows,
    the strip below its top rows; the image top/bottom are zero rows.  Height
    is then convolved without padding, width with ``pad``.
    With ``peer_boundaries is None`` (no exchange buffers yet, or a single
    strip) the wrapped convolution runs unchanged (conv2d.py:15-18,53-54,70-71).
    """
    if peer_boundaries is None or n_split == 1:
        return F.conv2d(x, weight, bias, stride=stride, padding=pad)
    b, c, h, w = x.shape
    zeros = x.new_zeros(b, c, pad, w)
    top = zeros if split_idx == 0 else peer_boundaries[split_idx - 1][1]
    bot = zeros if split_idx == n_split - 1 else peer_boundaries[split_idx + 1][0]
    padded = torch.cat([top, x, bot], dim=2)
    return F.conv2d(padded, weight, bias, stride=stride, padding=(0, pad))


def conv2d_first_layer(
    x_full: torch.Tensor,
    weight: torch.Tensor,
    bias: torch.Tensor | None,
    stride: int,
    pad: int,
    split_idx: int,
    n_split: int,
) -> torch.Tensor:
    """First convolution of the network: receives the full-height input and
    produces only this strip's output rows (basedxl/modules/conv2d.py:20-41)."""
    b, c, h, w = x_full.shape
    assert h % n_split == 0
    out_h = h // stride // n_split
    h_begin = out_h * split_idx * stride - pad
    h_end = out_h * (split_idx + 1) * stride + pad
    pad_top = pad_bot = 0
    if h_begin < 0:
        h_begin, pad_top = 0, pad
    if h_end > h:
        h_end, pad_bot = h, pad
    sliced = x_full[:, :, h_begin:h_end, :]
    padded = F.pad(sliced, [pad, pad, pad_top, pad_bot])
    return F.conv2d(padded, weight, bias, stride=stride, padding=0)


# --------------------------------------------------------------------------
# GroupNorm with cross-strip moments
# --------------------------------------------------------------------------
def groupnorm_moments(x: torch.Tensor, num_groups: int) -> torch.Tensor:
    """Per-group first and second raw moments of the local strip,
    ``[2, B, G, 1, 1, 1]`` (basedxl/modules/groupnorm.py:38-42)."""
    n, c, h, w = x.shape
    xg = x.view(n, num_groups, c // num_groups, h, w)
    m1 = xg.mean(dim=[2, 3, 4], keepdim=True)
    m2 = (xg**2).mean(dim=[2, 3, 4], keepdim=True)
    return torch.stack([m1, m2], dim=0)


def groupnorm_pp(
    x: torch.Tensor,
    num_groups: int,
    eps: float,
    gamma: torch.Tensor | None,
    beta: torch.Tensor | None,
    peer_moments: list[torch.Tensor] | None,
    split_idx: int,
    mode: str,
) -> torch.Tensor:
    """Patched GroupNorm (basedxl/modules/groupnorm.py:38-69).

    mode ``"local"``: strip statistics only (:44-45).
    mode ``"sync"``:  ``peer_moments`` hold every strip's *fresh* moments; the
                      full moments are their average (:46-48).
    mode ``"stale"``: ``peer_moments`` hold last step's moments; full =
                      average(stale) + (fresh_own - stale_own) (:49-52).
    Variance = m2 - m1**2; where negative, the strip's own variance is used
    (:56-60); then scaled by N/(N-1) with N the *local* element count per
    group (:62-63).  Output = (x - m1_full) / sqrt(var + eps) * gamma + beta.
    """
    n, c, h, w = x.shape
    gs = c // num_groups
    slice_m = groupnorm_moments(x, num_groups)
    if mode == "local" or peer_moments is None:
        full = slice_m
    elif mode == "sync":
        full = sum(peer_moments) / len(peer_moments)
    elif mode == "stale":
        full = sum(peer_moments) / len(peer_moments) + (slice_m - peer_moments[split_idx])
    else:
        raise ValueError(mode)
    m1, m2 = full[0], full[1]
    var = m2 - m1**2
    svar = slice_m[1] - slice_m[0] ** 2
    var = torch.where(var < 0, svar, var)
    num = gs * h * w
    var = var * (num / (num - 1))
    std = (var + eps).sqrt()
    y = (x.view(n, num_groups, gs, h, w) - m1) / std
    y = y.view(n, c, h, w)
    if gamma is not None:
        y = y * gamma.view(1, -1, 1, 1) + beta.view(1, -1, 1, 1)
    return y


# --------------------------------------------------------------------------
# Attention
# --------------------------------------------------------------------------
def _sdpa_heads(q: torch.Tensor, kv: torch.Tensor, heads: int) -> torch.Tensor:
    """softmax(Q K^T / sqrt(d)) V over ``heads`` heads; ``kv`` carries K in its
    first half of the channel axis and V in the second
    (basedxl/modules/attn.py:143-156)."""
    b = q.shape[0]
    k, v = torch.split(kv, kv.shape[-1] // 2, dim=-1)
    d = k.shape[-1] // heads
    qh = q.view(b, -1, heads, d).transpose(1, 2)
    kh = k.view(b, -1, heads, d).transpose(1, 2)
    vh = v.view(b, -1, heads, d).transpose(1, 2)
    o = F.scaled_dot_product_attention(qh, kh, vh, dropout_p=0.0, is_causal=False)
    return o.transpose(1, 2).reshape(b, -1, heads * d)


def assemble_kv(
    kv_fresh: torch.Tensor, peer_kv: list[torch.Tensor] | None, split_idx: int, n_split: int, mode: str
) -> torch.Tensor:
    """Full-sequence K/V seen by one strip (basedxl/modules/attn.py:129-141).

    ``"local"``: no buffers yet, own K/V repeated n times (:132-133);
    ``"sync"``: concatenation of the gathered fresh slots (:134-136);
    ``"stale"``: stale slots with the own slot replaced by fresh K/V (:138-140).
    """
    if n_split == 1:
        return kv_fresh
    if mode == "local" or peer_kv is None:
        return torch.cat([kv_fresh] * n_split, dim=1)
    if mode == "sync":
        return torch.cat(list(peer_kv), dim=1)
    if mode == "stale":
        slots = list(peer_kv)
        slots[split_idx] = kv_fresh
        return torch.cat(slots, dim=1)
    raise ValueError(mode)


def self_attention_pp(
    x: torch.Tensor,
    wq: torch.Tensor,
    wkv: torch.Tensor,
    wo: torch.Tensor,
    bo: torch.Tensor | None,
    heads: int,
    peer_kv: list[torch.Tensor] | None,
    split_idx: int,
    n_split: int,
    mode: str,
    residual_connection: bool = False,
    rescale_output_factor: float = 1.0,
    bq: torch.Tensor | None = None,
    bkv: torch.Tensor | None = None,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Patched self-attention (basedxl/modules/attn.py:112-168).  Returns the
    block output and the fresh K/V the strip publishes.  ``wkv`` is the fused
    ``[2C, C]`` weight [W_k; W_v] (attn.py:23-39)."""
    q = F.linear(x, wq, bq)
    kv = F.linear(x, wkv, bkv)
    full_kv = assemble_kv(kv, peer_kv, split_idx, n_split, mode)
    o = _sdpa_heads(q, full_kv, heads)
    o = F.linear(o, wo, bo)
    if residual_connection:
        o = o + x
    o = o / rescale_output_factor
    return o, kv


def cross_attention(
    x: torch.Tensor,
    context: torch.Tensor,
    wq: torch.Tensor,
    wkv: torch.Tensor,
    wo: torch.Tensor,
    bo: torch.Tensor | None,
    heads: int,
    residual_connection: bool = False,
    rescale_output_factor: float = 1.0,
) -> torch.Tensor:
    """Patched cross-attention (basedxl/modules/attn.py:57-101): K/V of the
    text context come from the fused weight; the cache only avoids
    recomputation and does not change the result."""
    q = F.linear(x, wq)
    kv = F.linear(context, wkv)
    o = _sdpa_heads(q, kv, heads)
    o = F.linear(o, wo, bo)
    if residual_connection:
        o = o + x
    return o / rescale_output_factor


# --------------------------------------------------------------------------
# Output assembly of the UNet wrapper
# --------------------------------------------------------------------------
def assemble_output(strips: list[torch.Tensor], n_split: int, use_cfg: bool) -> torch.Tensor:
    """What every rank holds after the final world gather
    (basedxl/unet.py:166-175 with CFG, :185-195 without): strips are ordered by
    global rank; with CFG the first ``n_split`` ranks form batch row 0 and the
    rest batch row 1, each concatenated along H."""
    if use_cfg:
        return torch.cat(
            [torch.cat(strips[:n_split], dim=2), torch.cat(strips[n_split:], dim=2)], dim=0
        )
    return torch.cat(strips, dim=2)


def rel_l2(y: torch.Tensor, ref: torch.Tensor) -> float:
    """Relative L2 error in fp64: ||y - ref|| / ||ref||."""
    y64, r64 = y.double().flatten(), ref.double().flatten()
    return float((y64 - r64).norm() / r64.norm().clamp_min(1e-30))

"""Halo-aware 3x3 convolution kernels through the C ABI against the CPU oracle
and the fixtures produced by the reference module."""
import os

import numpy as np
import pytest
import torch

from oracle import patched_ops as po
from tests._util import assert_close, cuda_or_skip, h16, nchw, nhwc

pytestmark = pytest.mark.gpu
T = torch.from_numpy


def _ops():
    from basedxl_b200 import _lib, ops

    return _lib, ops


def _halo_rows(ops, dev, boundaries, idx, n):
    """Device halo rows for strip idx from the peers' NCHW boundary tensors
    [2, B, C, 1, W]: the strip above gives its bottom row, the one below its top row."""
    top = bot = None
    if idx > 0:
        top = nhwc(boundaries[idx - 1][1]).half().to(dev)
    if idx < n - 1:
        bot = nhwc(boundaries[idx + 1][0]).half().to(dev)
    return top, bot


def _conv(ops, dev, x, w, b, stride, top, bot, **kw):
    wp = ops.conv_weight_pack(w.half().to(dev))
    y = ops.conv3x3(nhwc(x).half().to(dev), wp, None if b is None else b.half().to(dev), stride=stride, top=top, bot=bot, **kw)
    return nchw(y)


@pytest.mark.parametrize("Cin,Cout,H,W,stride", [(64, 64, 8, 16, 1), (128, 320, 16, 32, 1), (64, 128, 16, 16, 2), (320, 640, 12, 24, 1)])
@pytest.mark.parametrize("n", [1, 2, 4])
def test_conv_vs_oracle(Cin, Cout, H, W, stride, n):
    dev = cuda_or_skip()
    _lib, ops = _ops()
    if (H // n) % stride or H % n:
        pytest.skip("strip height not divisible")
    gen = torch.Generator().manual_seed(Cin + Cout + H + n)
    x = h16(torch.randn(2, Cin, H, W, generator=gen))
    xp = h16(x + 0.01 * torch.randn(2, Cin, H, W, generator=gen))
    w = h16(torch.randn(Cout, Cin, 3, 3, generator=gen) / (9 * Cin) ** 0.5)
    b = h16(torch.randn(Cout, generator=gen))
    xs, xps = torch.chunk(x, n, 2), torch.chunk(xp, n, 2)
    stale = [po.conv2d_boundary(t, 1) for t in xps]
    for i in range(n):
        ref = po.conv2d_pp(xs[i], w, b, stride, 1, stale if n > 1 else None, i, n)
        top, bot = _halo_rows(ops, dev, stale, i, n) if n > 1 else (None, None)
        y = _conv(ops, dev, xs[i], w, b, stride, top, bot)
        _lib.device_status()
        assert_close(y, ref, what=f"conv {Cin}->{Cout} {H}x{W} s{stride} strip {i}/{n}")


def test_conv_benchmark_shape():
    """2 x 640 x 64 x 64, 640 -> 640, halo 1, split 2/4/8 ways (stale halo)."""
    dev = cuda_or_skip()
    _lib, ops = _ops()
    gen = torch.Generator().manual_seed(0)
    x = h16(torch.randn(2, 640, 64, 64, generator=gen))
    xp = h16(x + 0.01 * torch.randn(2, 640, 64, 64, generator=gen))
    w = h16(torch.randn(640, 640, 3, 3, generator=gen) / (9 * 640) ** 0.5)
    b = h16(torch.randn(640, generator=gen))
    full = torch.nn.functional.conv2d(x, w, b, padding=1)
    y = _conv(ops, dev, x, w, b, 1, None, None)
    _lib.device_status()
    assert_close(y, full, what="conv full")
    for n in (2, 4, 8):
        xs, xps = torch.chunk(x, n, 2), torch.chunk(xp, n, 2)
        stale = [po.conv2d_boundary(t, 1) for t in xps]
        for i in sorted({0, n // 2, n - 1}):  # top-edge, interior and bottom-edge strips
            ref = po.conv2d_pp(xs[i], w, b, 1, 1, stale, i, n)
            top, bot = _halo_rows(ops, dev, stale, i, n)
            y = _conv(ops, dev, xs[i], w, b, 1, top, bot)
            _lib.device_status()
            assert_close(y, ref, what=f"conv strip {i} of n={n}")


def test_conv_fused_epilogue():
    dev = cuda_or_skip()
    _lib, ops = _ops()
    gen = torch.Generator().manual_seed(4)
    x = h16(torch.randn(2, 128, 16, 16, generator=gen))
    w = h16(torch.randn(192, 128, 3, 3, generator=gen) / 34)
    b = h16(torch.randn(192, generator=gen))
    temb = h16(torch.randn(2, 192, generator=gen))
    res = h16(torch.randn(2, 192, 16, 16, generator=gen))
    ref = torch.nn.functional.conv2d(x, w, b, padding=1) + temb[:, :, None, None] + res
    y = _conv(ops, dev, x, w, b, 1, None, None, bias_rows=temb.half().to(dev), residual=nhwc(res).half().to(dev))
    _lib.device_status()
    assert_close(y, ref, what="conv + per-image bias + residual")
    # the per-image bias as a column slice of a wider matrix (all blocks' projections in one GEMM)
    wide = torch.zeros(2, 512, dtype=torch.float16, device=dev)
    wide[:, 128:320] = temb.half().to(dev)
    y2 = _conv(ops, dev, x, w, b, 1, None, None, bias_rows=wide[:, 128:320], residual=nhwc(res).half().to(dev))
    _lib.device_status()
    assert torch.equal(y2, y)


@pytest.mark.parametrize("tag", ["s1", "s2"])
@pytest.mark.parametrize("n", [2, 4])
def test_conv_golden_thin_channels(golden_dir, tag, n):
    """The fixtures use 32 input channels, which the tensor-core path does not take
    (C_in % 64); they pin the halo geometry of the oracle the other tests use, and
    are run here zero-padded to 64 channels."""
    dev = cuda_or_skip()
    _lib, ops = _ops()
    g = np.load(os.path.join(golden_dir, "conv2d_pp.npz"))
    x, xp, w, b = T(g[f"{tag}_x"]), T(g[f"{tag}_x_prev"]), T(g[f"{tag}_w"]), T(g[f"{tag}_b"])
    stride = int(g[f"{tag}_stride"])
    pad_c = lambda t, d: torch.nn.functional.pad(t, [0, 0] * (t.dim() - 1 - d) + [0, 64 - t.shape[d]])
    xz, xpz, wz = pad_c(x, 1), pad_c(xp, 1), pad_c(w, 1)
    xs, xps = torch.chunk(xz, n, 2), torch.chunk(xpz, n, 2)
    stale = [po.conv2d_boundary(t, 1) for t in xps]
    fresh = [po.conv2d_boundary(t, 1) for t in xs]
    for i in range(n):
        top, bot = _halo_rows(ops, dev, stale, i, n)
        y = _conv(ops, dev, xs[i], wz, b, stride, top, bot)
        assert_close(y, T(g[f"{tag}_n{n}_i{i}_stale_y"]), what="golden stale")
        top, bot = _halo_rows(ops, dev, fresh, i, n)
        y = _conv(ops, dev, xs[i], wz, b, stride, top, bot)
        assert_close(y, T(g[f"{tag}_n{n}_i{i}_sync_y"]), what="golden sync")
    _lib.device_status()


@pytest.mark.parametrize("n", [1, 2, 4])
def test_direct_convs_at_network_ends(n):
    """conv_in (4 -> 320, full-height input sliced per strip) and conv_out (320 -> 4)."""
    dev = cuda_or_skip()
    _lib, ops = _ops()
    gen = torch.Generator().manual_seed(9)
    H = W = 32
    x = h16(torch.randn(2, 4, H, W, generator=gen))
    w = h16(torch.randn(320, 4, 3, 3, generator=gen) / 6)
    b = h16(torch.randn(320, generator=gen))
    xd = nhwc(x).half().to(dev)
    wp = ops.conv_weight_pack(w.half().to(dev))
    hl = H // n
    for i in range(n):
        ref = po.conv2d_first_layer(x, w, b, 1, 1, i, n)
        body = xd[:, i * hl : (i + 1) * hl]
        top = xd[:, i * hl - 1 : i * hl] if i > 0 else None
        bot = xd[:, (i + 1) * hl : (i + 1) * hl + 1] if i < n - 1 else None
        y = ops.conv3x3(body, wp, b.half().to(dev), top=top, bot=bot)
        _lib.device_status()
        assert_close(nchw(y), ref, what=f"conv_in strip {i}/{n}")
    x = h16(torch.randn(2, 320, H, W, generator=gen))
    xp = h16(x + 0.01 * torch.randn(2, 320, H, W, generator=gen))
    w = h16(torch.randn(4, 320, 3, 3, generator=gen) / 54)
    b = h16(torch.randn(4, generator=gen))
    xs, xps = torch.chunk(x, n, 2), torch.chunk(xp, n, 2)
    stale = [po.conv2d_boundary(t, 1) for t in xps]
    for i in range(n):
        ref = po.conv2d_pp(xs[i], w, b, 1, 1, stale if n > 1 else None, i, n)
        top, bot = _halo_rows(ops, dev, stale, i, n) if n > 1 else (None, None)
        y = _conv(ops, dev, xs[i], w, b, 1, top, bot)
        _lib.device_status()
        assert_close(y, ref, what=f"conv_out strip {i}/{n}")


@pytest.mark.parametrize("W", [30, 36, 5])
def test_conv_in_ragged_width(W):
    """conv_in on widths that are not a multiple of the four pixels a thread computes."""
    dev = cuda_or_skip()
    _lib, ops = _ops()
    gen = torch.Generator().manual_seed(W)
    x = h16(torch.randn(2, 4, 12, W, generator=gen))
    w = h16(torch.randn(320, 4, 3, 3, generator=gen) / 6)
    b = h16(torch.randn(320, generator=gen))
    ref = torch.nn.functional.conv2d(x, w, b, padding=1)
    y = _conv(ops, dev, x, w, b, 1, None, None)
    _lib.device_status()
    assert_close(y, ref, what=f"conv_in W={W}")


def test_thin_conv_out_off_the_tensor_path():
    """A 4-channel output convolution whose C_in is not a multiple of 64 stays on the direct kernel."""
    dev = cuda_or_skip()
    _lib, ops = _ops()
    gen = torch.Generator().manual_seed(3)
    x = h16(torch.randn(2, 72, 16, 24, generator=gen))
    w = h16(torch.randn(4, 72, 3, 3, generator=gen) / 25)
    b = h16(torch.randn(4, generator=gen))
    ref = torch.nn.functional.conv2d(x, w, b, padding=1)
    y = _conv(ops, dev, x, w, b, 1, None, None)
    _lib.device_status()
    assert_close(y, ref, what="conv 72 -> 4")


def test_halo_pack_is_bit_exact():
    dev = cuda_or_skip()
    _lib, ops = _ops()
    x = torch.randn(2, 320, 16, 64).half()
    packed = ops.halo_pack(nhwc(x).to(dev))
    ref = po.conv2d_boundary(x, 1)  # [2, B, C, 1, W]
    assert torch.equal(packed.cpu().permute(0, 1, 4, 2, 3), ref)
    _lib.device_status()


@pytest.mark.parametrize("bn,split,pair", [(64, 1, 0), (160, 1, 0), (256, 1, 0), (128, 2, 0), (128, 4, 0), (256, 4, 0),
                                           (128, 1, 1), (160, 1, 1), (256, 1, 1)])
def test_conv_forced_tile_width_and_k_split(bn, split, pair):
    """Every tile width, K split and the CTA-pair form (two CTAs, one MMA stream) on a conv with
    stale halo rows; the pair's second tile partly lies past the last image."""
    dev = cuda_or_skip()
    _lib, ops = _ops()
    gen = torch.Generator().manual_seed(bn + split)
    x = h16(torch.randn(2, 128, 16, 32, generator=gen))
    xp = h16(x + 0.01 * torch.randn(2, 128, 16, 32, generator=gen))
    w = h16(torch.randn(320, 128, 3, 3, generator=gen) / 34)
    b = h16(torch.randn(320, generator=gen))
    xs, xps = torch.chunk(x, 2, 2), torch.chunk(xp, 2, 2)
    stale = [po.conv2d_boundary(t, 1) for t in xps]
    l = _lib.lib()
    _lib.check(l.bxl_debug_force_tiles(bn, split, pair), l, kernels=0)
    try:
        for i in range(2):
            ref = po.conv2d_pp(xs[i], w, b, 1, 1, stale, i, 2)
            top, bot = _halo_rows(ops, dev, stale, i, 2)
            y = _conv(ops, dev, xs[i], w, b, 1, top, bot)
            _lib.device_status()
            assert_close(y, ref, what=f"conv bn={bn} split={split} pair={pair} strip {i}")
    finally:
        _lib.check(l.bxl_debug_force_tiles(0, 0, -1), l, kernels=0)


@pytest.mark.parametrize("order", [0, 1])
@pytest.mark.parametrize("bn,split,pair", [(64, 1, 0), (128, 2, 0), (128, 1, 1)])
def test_conv_tile_order(order, bn, split, pair):
    """Both orders in which output tiles are handed to the CTAs (pixels first / output channels
    first, the latter chosen by the library for inputs that do not stay in L2) give the same
    result, with several column tiles per pixel tile, a K split and a CTA pair."""
    dev = cuda_or_skip()
    _lib, ops = _ops()
    gen = torch.Generator().manual_seed(7 + bn)
    x = h16(torch.randn(3, 64, 24, 40, generator=gen))
    w = h16(torch.randn(320, 64, 3, 3, generator=gen) / 24)
    b = h16(torch.randn(320, generator=gen))
    ref = po.conv2d_pp(x, w, b, 1, 1, None, 0, 1)
    l = _lib.lib()
    _lib.check(l.bxl_debug_force_tiles(bn, split, pair), l, kernels=0)
    _lib.check(l.bxl_debug_force_tile_order(order), l, kernels=0)
    try:
        y = _conv(ops, dev, x, w, b, 1, None, None)
        _lib.device_status()
        assert_close(y, ref, what=f"conv order={order} bn={bn} split={split} pair={pair}")
    finally:
        _lib.check(l.bxl_debug_force_tiles(0, 0, -1), l, kernels=0)
        _lib.check(l.bxl_debug_force_tile_order(-1), l, kernels=0)


def test_conv_input_larger_than_l2():
    """63 MB of input (more than stays in L2 beside the output): the library hands out the tiles
    output channels first; result against the oracle."""
    dev = cuda_or_skip()
    _lib, ops = _ops()
    gen = torch.Generator().manual_seed(11)
    x = h16(torch.randn(2, 320, 192, 256, generator=gen))
    w = h16(torch.randn(320, 320, 3, 3, generator=gen) / 54)
    b = h16(torch.randn(320, generator=gen))
    ref = po.conv2d_pp(x, w, b, 1, 1, None, 0, 1)
    y = _conv(ops, dev, x, w, b, 1, None, None)
    _lib.device_status()
    assert_close(y, ref, what="conv 320->320 192x256, tiles handed out channels first")


@pytest.mark.parametrize("n", [1, 2, 4, 8])
def test_auto_tiling_on_every_per_rank_conv_shape(n):
    """The 3x3 convolutions of the UNet on the strips a rank sees when the image is split
    n ways (batch 1), with the tiling the library chooses by itself, against cuDNN fp32."""
    dev = cuda_or_skip()
    _lib, ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(n)
    sites = [(320, 320, 128, 1), (320, 320, 128, 2), (640, 640, 64, 1), (640, 640, 64, 2), (1280, 1280, 32, 1), (2560, 1280, 32, 1),
             (1920, 1280, 32, 1), (1280, 1280, 64, 1), (1920, 640, 64, 1), (960, 640, 64, 1), (640, 640, 128, 1), (960, 320, 128, 1),
             (640, 320, 128, 1), (320, 640, 64, 1), (640, 1280, 32, 1)]
    for (ci, co, hw, stride) in sites:
        hl = hw // n
        if hl < stride or hl % stride:
            continue
        x = torch.randn(1, hl, hw, ci, device=dev, generator=g).half()
        top = torch.randn(1, 1, hw, ci, device=dev, generator=g).half()
        bot = torch.randn(1, 1, hw, ci, device=dev, generator=g).half()
        w = (torch.randn(co, ci, 3, 3, device=dev, generator=g) / (9 * ci) ** 0.5).half()
        b = torch.randn(co, device=dev, generator=g).half()
        y = ops.conv3x3(x, ops.conv_weight_pack(w), b, stride=stride, top=top, bot=bot)
        padded = torch.cat([top, x, bot], dim=1).permute(0, 3, 1, 2).float()
        ref = torch.nn.functional.conv2d(padded, w.float(), b.float(), stride=stride, padding=(0, 1)).permute(0, 2, 3, 1)
        err = float((y.float() - ref).norm() / ref.norm())
        assert torch.isfinite(y).all() and err < 2e-3, f"n={n} {ci}->{co} @{hw} s{stride}: rel-L2 {err:.3e}"
    _lib.device_status()

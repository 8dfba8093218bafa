"""GroupNorm(+SiLU) kernels through the C ABI against the CPU oracle and the
fixtures produced by the reference module."""
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


def _run(ops, dev, x, groups, eps, gamma, beta, peers, own, mode, silu=False):
    xd = nhwc(x).half().to(dev)
    fresh = ops.groupnorm_stats(xd, groups)
    peers_d = None
    if peers is not None:
        peers_d = [p.reshape(2, x.shape[0], groups).float().contiguous().to(dev) for p in peers]
    y = ops.groupnorm_apply(
        xd, groups, eps, gamma.half().to(dev), beta.half().to(dev), fresh, peers_d, own,
        {"local": ops.MODE_LOCAL, "sync": ops.MODE_SYNC, "stale": ops.MODE_STALE}[mode], silu=silu,
    )
    return nchw(y), fresh


@pytest.mark.parametrize("n", [2, 4])
def test_groupnorm_golden(golden_dir, n):
    dev = cuda_or_skip()
    _lib, ops = _ops()
    g = np.load(os.path.join(golden_dir, "groupnorm_pp.npz"))
    x, xp, gamma, beta = T(g["x"]), T(g["x_prev"]), T(g["gamma"]), T(g["beta"])
    eps, groups = float(g["eps"]), int(g["groups"])
    xs, xps = torch.chunk(x, n, 2), torch.chunk(xp, n, 2)
    fresh = [po.groupnorm_moments(h16(t), groups) for t in xs]
    stale = [po.groupnorm_moments(h16(t), groups) for t in xps]
    for i in range(n):
        y, m = _run(ops, dev, xs[i], groups, eps, gamma, beta, None, i, "local")
        assert_close(y, T(g[f"n{n}_i{i}_local_y"]), what="gn local")
        assert_close(m.cpu().reshape(-1), T(g[f"n{n}_i{i}_published"]).reshape(-1), tol=1e-3, what="gn moments")
        y, _ = _run(ops, dev, xs[i], groups, eps, gamma, beta, stale, i, "stale")
        assert_close(y, T(g[f"n{n}_i{i}_stale_y"]), what="gn stale")
        y, _ = _run(ops, dev, xs[i], groups, eps, gamma, beta, fresh, i, "sync")
        assert_close(y, T(g[f"n{n}_i{i}_sync_y"]), what="gn sync")
    _lib.device_status()


@pytest.mark.parametrize("C,H,W", [(1280, 32, 32), (320, 128, 128), (960, 64, 64), (2560, 32, 32), (1920, 8, 32)])
@pytest.mark.parametrize("n", [1, 2, 4, 8])
def test_groupnorm_config_shapes(C, H, W, n):
    """32 groups on SDXL shapes (2 x 1280 x 32 x 32 is the benchmark configuration),
    split n ways along H, stale = current + N(0, 0.01)."""
    if H % n:
        pytest.skip("height not divisible")
    dev = cuda_or_skip()
    _lib, ops = _ops()
    gen = torch.Generator().manual_seed(C + H + n)
    x = torch.randn(2, C, H, W, generator=gen) * 2 + 0.5
    xp = x + 0.01 * torch.randn(2, C, H, W, generator=gen)
    gamma, beta = torch.randn(C, generator=gen), torch.randn(C, generator=gen)
    xs, xps = torch.chunk(h16(x), n, 2), torch.chunk(h16(xp), n, 2)
    stale = [po.groupnorm_moments(t, 32) for t in xps]
    mode = "stale" if n > 1 else "local"
    for i in sorted({0, n // 2, n - 1}):  # first, middle and last strip
        ref = po.groupnorm_pp(xs[i], 32, 1e-5, h16(gamma), h16(beta), stale if n > 1 else None, i, mode)
        y, _ = _run(ops, dev, xs[i], 32, 1e-5, gamma, beta, stale if n > 1 else None, i, mode)
        assert_close(y, ref, what=f"gn {C}x{H}x{W} n={n} strip {i}")
        y, _ = _run(ops, dev, xs[i], 32, 1e-5, gamma, beta, stale if n > 1 else None, i, mode, silu=True)
        assert_close(y, torch.nn.functional.silu(ref), what="gn+silu")
    _lib.device_status()


def test_negative_variance_falls_back_to_strip_variance():
    """Stale moments that make m2 - m1^2 negative (basedxl/modules/groupnorm.py:56-60)."""
    dev = cuda_or_skip()
    _lib, ops = _ops()
    gen = torch.Generator().manual_seed(3)
    x = h16(torch.randn(1, 64, 4, 8, generator=gen))
    fresh = po.groupnorm_moments(x, 32)
    bogus = fresh.clone()
    bogus[0] += 10.0  # huge stale mean on the peer, tiny second moment
    peers = [fresh.clone(), bogus]
    ref = po.groupnorm_pp(x, 32, 1e-5, torch.ones(64), torch.zeros(64), peers, 0, "stale")
    y, _ = _run(ops, dev, x, 32, 1e-5, torch.ones(64), torch.zeros(64), peers, 0, "stale")
    assert_close(y, ref, what="gn negative variance")
    _lib.device_status()


def test_stats_twice_in_a_row_reuses_scratch():
    dev = cuda_or_skip()
    _lib, ops = _ops()
    x = torch.randn(2, 16, 16, 320, device=dev).half()
    m1 = ops.groupnorm_stats(x, 32).clone()
    m2 = ops.groupnorm_stats(x, 32)
    ref = po.groupnorm_moments(x.float().cpu().permute(0, 3, 1, 2), 32).reshape(2, 2, 32)
    assert_close(m1, ref, tol=1e-3)
    assert_close(m2, ref, tol=1e-3)
    _lib.device_status()


# ---------------------------------------------------------------------------------------------
# one-launch form (cluster per image x channel block): same arithmetic, local and stale modes
# ---------------------------------------------------------------------------------------------
def _run_fused(ops, dev, x, groups, eps, gamma, beta, peers, own, mode, silu=False, halo=False, alias_own=False):
    xd = nhwc(x).half().to(dev)
    B, H, W, C = xd.shape
    peers_d = None
    if peers is not None:
        peers_d = [p.reshape(2, B, groups).float().contiguous().to(dev) for p in peers]
    fresh = peers_d[own] if alias_own else torch.full((2, B, groups), float("nan"), device=dev)
    halo_out = torch.zeros(2, B, 1, W, C, device=dev, dtype=torch.float16) if halo else None
    y = ops.groupnorm_fused(xd, groups, eps, gamma.half().to(dev), beta.half().to(dev), peers_d, own,
                            {"local": ops.MODE_LOCAL, "stale": ops.MODE_STALE}[mode], silu=silu, fresh_out=fresh, halo_out=halo_out)
    return nchw(y), fresh, halo_out


@pytest.mark.parametrize("n", [2, 4])
def test_groupnorm_fused_golden(golden_dir, n):
    dev = cuda_or_skip()
    _lib, ops = _ops()
    g = np.load(os.path.join(golden_dir, "groupnorm_pp.npz"))
    x, xp, gamma, beta = T(g["x"]), T(g["x_prev"]), T(g["gamma"]), T(g["beta"])
    eps, groups = float(g["eps"]), int(g["groups"])
    xs, xps = torch.chunk(x, n, 2), torch.chunk(xp, n, 2)
    stale = [po.groupnorm_moments(h16(t), groups) for t in xps]
    for i in range(n):
        y, m, _ = _run_fused(ops, dev, xs[i], groups, eps, gamma, beta, None, i, "local")
        assert_close(y, T(g[f"n{n}_i{i}_local_y"]), what="fused gn local")
        assert_close(m.cpu().reshape(-1), T(g[f"n{n}_i{i}_published"]).reshape(-1), tol=1e-3, what="fused gn moments")
        # the fresh moments go straight into the strip's own (stale) entry: read before written
        y, m, _ = _run_fused(ops, dev, xs[i], groups, eps, gamma, beta, stale, i, "stale", alias_own=True)
        assert_close(y, T(g[f"n{n}_i{i}_stale_y"]), what="fused gn stale")
        assert_close(m.cpu().reshape(-1), T(g[f"n{n}_i{i}_published"]).reshape(-1), tol=1e-3, what="fused gn published")
    _lib.device_status()


@pytest.mark.parametrize("C,H,W", [(1280, 32, 32), (320, 128, 128), (960, 128, 128), (640, 64, 64), (2560, 32, 32), (1920, 8, 32), (64, 6, 8), (32, 4, 8)])
@pytest.mark.parametrize("n", [1, 4])
def test_groupnorm_fused_config_shapes(C, H, W, n):
    """The one-launch form on the UNet's shapes (slab kept in shared memory, or re-read where it
    does not fit: 960 channels at 128 x 128), against the oracle and the two-launch form."""
    if H % n:
        pytest.skip("height not divisible")
    dev = cuda_or_skip()
    _lib, ops = _ops()
    gen = torch.Generator().manual_seed(C + H + n)
    x = torch.randn(2, C, H, W, generator=gen) * 2 + 0.5
    xp = x + 0.01 * torch.randn(2, C, H, W, generator=gen)
    gamma, beta = torch.randn(C, generator=gen), torch.randn(C, generator=gen)
    xs, xps = torch.chunk(h16(x), n, 2), torch.chunk(h16(xp), n, 2)
    stale = [po.groupnorm_moments(t, 32) for t in xps]
    mode = "stale" if n > 1 else "local"
    for i in sorted({0, n - 1}):
        ref = po.groupnorm_pp(xs[i], 32, 1e-5, h16(gamma), h16(beta), stale if n > 1 else None, i, mode)
        y, m, halo = _run_fused(ops, dev, xs[i], 32, 1e-5, gamma, beta, stale if n > 1 else None, i, mode, halo=True)
        assert_close(y, ref, what=f"fused gn {C}x{H}x{W} n={n} strip {i}")
        assert_close(m.cpu().reshape(-1), po.groupnorm_moments(xs[i], 32).reshape(-1), tol=1e-3, what="fused gn moments")
        # boundary rows of the result, bit-identical to the rows of y
        yh = nhwc(y)
        assert torch.equal(halo[0, :, 0], yh[:, 0]) and torch.equal(halo[1, :, 0], yh[:, -1])
        y2, _ = _run(ops, dev, xs[i], 32, 1e-5, gamma, beta, stale if n > 1 else None, i, mode, silu=True)
        y3, _, _ = _run_fused(ops, dev, xs[i], 32, 1e-5, gamma, beta, stale if n > 1 else None, i, mode, silu=True)
        assert_close(y3, torch.nn.functional.silu(ref), what="fused gn+silu")
        assert_close(y3, y2.float().cpu(), tol=5e-4, what="fused vs two-launch")
    _lib.device_status()


def test_groupnorm_fused_negative_variance_fallback():
    dev = cuda_or_skip()
    _lib, ops = _ops()
    gen = torch.Generator().manual_seed(3)
    x = h16(torch.randn(1, 64, 4, 8, generator=gen))
    fresh = po.groupnorm_moments(x, 32)
    bogus = fresh.clone()
    bogus[0] += 10.0
    peers = [fresh.clone(), bogus]
    ref = po.groupnorm_pp(x, 32, 1e-5, torch.ones(64), torch.zeros(64), peers, 0, "stale")
    y, _, _ = _run_fused(ops, dev, x, 32, 1e-5, torch.ones(64), torch.zeros(64), peers, 0, "stale")
    assert_close(y, ref, what="fused gn negative variance")
    _lib.device_status()

"""Host-graph helper kernels against PyTorch fp32 on the CPU."""
import pytest
import torch
import torch.nn.functional as F

from tests._util import assert_close, cuda_or_skip, h16

pytestmark = pytest.mark.gpu


def _ops():
    from basedxl_b200 import _lib, ops

    return _lib, ops


def test_upsample2x():
    dev = cuda_or_skip()
    _lib, ops = _ops()
    x = torch.randn(2, 8, 12, 64).half()
    y = ops.upsample2x(x.to(dev)).cpu()
    ref = F.interpolate(x.permute(0, 3, 1, 2).float(), scale_factor=2.0, mode="nearest").permute(0, 2, 3, 1).half()
    assert torch.equal(y, ref)
    _lib.device_status()


@pytest.mark.parametrize("C", [640, 1280, 320])
def test_layernorm(C):
    dev = cuda_or_skip()
    _lib, ops = _ops()
    x = h16(torch.randn(3, 100, C) * 2 + 1)
    g, b = h16(torch.randn(C)), h16(torch.randn(C))
    y = ops.layernorm(x.half().to(dev), g.half().to(dev), b.half().to(dev), 1e-5)
    assert_close(y, F.layer_norm(x, (C,), g, b, 1e-5), what="layernorm")
    _lib.device_status()


def test_geglu():
    dev = cuda_or_skip()
    _lib, ops = _ops()
    h = h16(torch.randn(2, 77, 2 * 2560))
    y = ops.geglu(h.half().to(dev))
    a, g = h.chunk(2, dim=-1)
    assert_close(y, a * F.gelu(g), what="geglu")
    _lib.device_status()


def test_cfg_euler_step():
    dev = cuda_or_skip()
    _lib, ops = _ops()
    g = torch.Generator().manual_seed(0)
    eps = torch.randn(2, 4, 32, 32, generator=g).half()
    lat = torch.randn(1, 4, 32, 32, generator=g) * 10
    guidance, s0, s1 = 5.0, 3.2, 2.9
    e = eps[0:1].float() + guidance * (eps[1:2].float() - eps[0:1].float())
    ref_lat = lat + e * (s1 - s0)
    ref_in = (ref_lat / (s1 * s1 + 1) ** 0.5).half()
    lat_d = lat.to(dev).clone()
    nxt = torch.empty(2, 4, 32, 32, device=dev, dtype=torch.float16)
    ops.cfg_euler_step(eps.to(dev), lat_d, nxt, guidance, s0, s1)
    _lib.device_status()
    assert torch.allclose(lat_d.cpu(), ref_lat, rtol=1e-6, atol=1e-5)
    assert torch.equal(nxt[0].cpu(), nxt[1].cpu())
    assert (nxt[0:1].float().cpu() - ref_in.float()).abs().max() <= 2e-2

"""Single UNet forward through the library (one GPU) against the same graph
evaluated by stock PyTorch fp32 operators on the CPU."""
import pytest
import torch

from oracle.patched_ops import rel_l2
from oracle.torch_layers import TorchLayers
from tests._util import cuda_or_skip

pytestmark = pytest.mark.gpu


def _pair(cfg, dev, seed=0):
    from basedxl_b200.sdxl_unet import UNet2DConditionModel

    torch.manual_seed(seed)
    ref = UNet2DConditionModel(cfg, layers=TorchLayers).eval()
    # the oracle sees exactly the fp16-rounded weights the device uses
    ref = ref.half().float()
    gpu = UNet2DConditionModel(cfg).eval()
    gpu.load_state_dict(ref.state_dict())
    gpu = gpu.half().to(dev)
    return ref, gpu


def _inputs(cfg, hw, seed=1, ctx_len=77):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(2, 4, hw, hw, generator=g).half().float()
    ehs = torch.randn(2, ctx_len, cfg.cross_attention_dim, generator=g).half().float()
    pooled = cfg.projection_class_embeddings_input_dim - 6 * cfg.addition_time_embed_dim
    added = {
        "text_embeds": torch.randn(2, pooled, generator=g).half().float(),
        "time_ids": torch.tensor([[1024.0, 1024, 0, 0, 1024, 1024]] * 2),
    }
    return x, ehs, added


def _compare(cfg, hw, tol, what):
    dev = cuda_or_skip()
    from basedxl_b200 import _lib

    ref, gpu = _pair(cfg, dev)
    x, ehs, added = _inputs(cfg, hw)
    with torch.no_grad():
        y_ref = ref(x, torch.tensor(999.0), ehs, added_cond_kwargs=added)[0]
        y = gpu(x.to(dev), torch.tensor(999.0, device=dev), ehs.half().to(dev),
                added_cond_kwargs={k: v.to(dev) for k, v in added.items()})[0]
    _lib.device_status()
    err = rel_l2(y.float().cpu(), y_ref)
    print(f"{what}: rel-L2 {err:.3e}")
    assert y.shape == y_ref.shape
    assert err <= tol, f"{what}: rel-L2 {err:.3e} > {tol}"


def test_tiny_unet_forward_matches_oracle():
    from basedxl_b200.sdxl_unet import tiny_config

    _compare(tiny_config(), 32, 2e-3, "tiny UNet forward")


def test_sdxl_unet_forward_matches_oracle_at_reduced_resolution():
    """The full SDXL-shaped graph (2.57 B parameters, all 155 patched-layer sites
    plus conv_in) on a 256 x 256 image (32 x 32 latent) so that the fp32 CPU
    evaluation finishes in seconds."""
    from basedxl_b200.sdxl_unet import sdxl_config

    _compare(sdxl_config(), 32, 2e-3, "SDXL UNet forward, 32x32 latent")


def test_sdxl_unet_forward_matches_oracle_at_full_resolution():
    """The first benchmark configuration at its real size: CFG batch of 2, 128 x 128 latent,
    timestep 999 (one fp32 CPU forward of 13.5 TFLOP: seconds on a multi-core host)."""
    from basedxl_b200.sdxl_unet import sdxl_config

    _compare(sdxl_config(), 128, 2e-3, "SDXL UNet forward, 128x128 latent")


def test_tiny_unet_with_lowp_linear_swap_matches_oracle():
    """``fp16_acc_matmul=True``: every Linear replaced by BasedXLLowPLinear (weights kept as
    [K, N]), as the reference's patch_linear_layers does (basedxl/unet.py:81-87)."""
    dev = cuda_or_skip()
    from basedxl_b200 import _lib
    from basedxl_b200.modules.lowp_linear import BasedXLLowPLinear
    from basedxl_b200.sdxl_unet import tiny_config
    from basedxl_b200.unet import BasedXLUnet
    from basedxl_b200.utils import BasedXLConfig

    cfg = tiny_config()
    ref, gpu = _pair(cfg, dev)
    wrapped = BasedXLUnet(gpu, BasedXLConfig(fp16_acc_matmul=True))
    assert any(isinstance(m, BasedXLLowPLinear) for m in gpu.modules())
    x, ehs, added = _inputs(cfg, 32)
    with torch.no_grad():
        y_ref = ref(x, torch.tensor(999.0), ehs, added_cond_kwargs=added)[0]
        y = wrapped(x.to(dev), torch.tensor(999.0, device=dev), ehs.half().to(dev),
                    added_cond_kwargs={k: v.to(dev) for k, v in added.items()})[0]
    _lib.device_status()
    err = rel_l2(y.float().cpu(), y_ref)
    assert err <= 2e-3, err

"""Host-side structure of the UNet graph and the swap logic (no GPU)."""
import torch
import torch.nn as nn

from basedxl_b200.sdxl_unet import UNet2DConditionModel, sdxl_config, tiny_config
from oracle.torch_layers import TorchLayers


def test_sdxl_inventory_matches_the_reference_workload():
    with torch.device("meta"):
        m = UNet2DConditionModel(sdxl_config())
    assert sum(p.numel() for p in m.parameters()) == 2_567_463_684  # SDXL base UNet parameter count
    convs = [v for _, v in m.named_modules() if isinstance(v, nn.Conv2d) and tuple(v.kernel_size) == (3, 3)]
    gns = [v for _, v in m.named_modules() if isinstance(v, nn.GroupNorm)]
    attn1 = [k for k, _ in m.named_modules() if k.endswith("attn1")]
    attn2 = [k for k, _ in m.named_modules() if k.endswith("attn2")]
    # 39 exchanged convolutions + conv_in, 46 group norms, 70 + 70 attention layers
    assert (len(convs), len(gns), len(attn1), len(attn2)) == (40, 46, 70, 70)
    shapes = sorted({(c.in_channels, c.out_channels, c.stride[0]) for c in convs})
    assert (4, 320, 1) in shapes and (320, 4, 1) in shapes and (2560, 1280, 1) in shapes and (640, 640, 2) in shapes


def test_tiny_graph_runs_on_cpu_with_stock_layers():
    torch.manual_seed(0)
    cfg = tiny_config()
    m = UNet2DConditionModel(cfg, layers=TorchLayers).eval()
    x = torch.randn(2, 4, 16, 16)
    ehs = torch.randn(2, 7, cfg.cross_attention_dim)
    added = {"text_embeds": torch.randn(2, 64), "time_ids": torch.tensor([[128.0, 128, 0, 0, 128, 128]] * 2)}
    with torch.no_grad():
        y = m(x, torch.tensor(999.0), ehs, added_cond_kwargs=added)[0]
    assert y.shape == x.shape and torch.isfinite(y).all()


def test_state_dicts_interchange_between_factories():
    from basedxl_b200.layers import KernelLayers

    a = UNet2DConditionModel(tiny_config(), layers=TorchLayers)
    b = UNet2DConditionModel(tiny_config(), layers=KernelLayers)
    missing, unexpected = b.load_state_dict(a.state_dict(), strict=True)
    assert not missing and not unexpected


def test_batched_time_projection_equals_per_block_projection():
    """One GEMM over the concatenated time-embedding projections of all residual blocks, each
    block reading its column slice, gives the per-block result."""

    class Batched(TorchLayers):
        batched_time_projection = True
        linear = staticmethod(lambda x, w, b=None: torch.nn.functional.linear(x, w, b))

    torch.manual_seed(0)
    cfg = tiny_config()
    a = UNet2DConditionModel(cfg, layers=TorchLayers).eval()
    b = UNet2DConditionModel(cfg, layers=Batched).eval()
    b.load_state_dict(a.state_dict())
    x = torch.randn(2, 4, 16, 16)
    ehs = torch.randn(2, 7, cfg.cross_attention_dim)
    added = {"text_embeds": torch.randn(2, 64), "time_ids": torch.tensor([[128.0, 128, 0, 0, 128, 128]] * 2)}
    with torch.no_grad():
        ya = a(x, torch.tensor(500.0), ehs, added_cond_kwargs=added)[0]
        yb = b(x, torch.tensor(500.0), ehs, added_cond_kwargs=added)[0]
        assert getattr(b, "_time_proj_cache", None) is not None  # the batched path ran
        # a weight update invalidates the cached concatenation
        first = next(m for m in b.modules() if hasattr(m, "time_emb_proj"))
        first.time_emb_proj.bias.add_(1.0)
        next(m for m in a.modules() if hasattr(m, "time_emb_proj")).time_emb_proj.bias.add_(1.0)
        ya2 = a(x, torch.tensor(500.0), ehs, added_cond_kwargs=added)[0]
        yb2 = b(x, torch.tensor(500.0), ehs, added_cond_kwargs=added)[0]
    assert torch.allclose(ya, yb, rtol=1e-5, atol=1e-5)
    assert torch.allclose(ya2, yb2, rtol=1e-5, atol=1e-5) and not torch.allclose(ya, ya2)

"""The single-GPU path the benchmark times: CUDA-graph replay of the UNet step
(``GraphedStep``), cached cross-attention K/V refreshed on new conditioning, the
fused guidance + Euler kernel inside ``BasedXLPipeline.denoise``, and
``BasedXLUnet.forward`` with static weights - against the same loop launched
eagerly and against the CPU oracle loop (stock PyTorch fp32 operators over the
same graph, the scheduler's own un-fused update)."""
import pytest
import torch

from oracle.patched_ops import rel_l2
from oracle.torch_layers import TorchLayers
from tests._util import cuda_or_skip

pytestmark = pytest.mark.gpu
STEPS, TOTAL_STEPS, GUIDANCE = 8, 50, 5.0


def _models(ucfg, dev):
    from basedxl_b200.sdxl_unet import UNet2DConditionModel

    torch.manual_seed(0)
    ref = UNet2DConditionModel(ucfg, layers=TorchLayers).eval().half().float()
    gpu = UNet2DConditionModel(ucfg).eval()
    gpu.load_state_dict(ref.state_dict())
    return ref, gpu.half().to(dev)


def _conditioning(ucfg, hw, seed, ctx_len=77):
    g = torch.Generator().manual_seed(seed)
    pooled = ucfg.projection_class_embeddings_input_dim - 6 * ucfg.addition_time_embed_dim
    r16 = lambda *s: torch.randn(*s, generator=g).half().float()
    return {
        "latents": torch.randn(1, 4, hw, hw, generator=g),
        "prompt_embeds": r16(1, ctx_len, ucfg.cross_attention_dim),
        "negative_prompt_embeds": r16(1, ctx_len, ucfg.cross_attention_dim),
        "pooled_prompt_embeds": r16(1, pooled),
        "negative_pooled_prompt_embeds": r16(1, pooled),
    }


def _oracle_loop(ref, cond, size):
    """The reference loop on the CPU: CFG batch of 2 (row 0 unconditional), guidance, Euler step."""
    from basedxl_b200.scheduler import EulerDiscreteScheduler

    sch = EulerDiscreteScheduler()
    sch.set_timesteps(TOTAL_STEPS)
    lat = cond["latents"].clone().float() * sch.init_noise_sigma
    ehs = torch.cat([cond["negative_prompt_embeds"], cond["prompt_embeds"]])
    added = {"text_embeds": torch.cat([cond["negative_pooled_prompt_embeds"], cond["pooled_prompt_embeds"]]),
             "time_ids": torch.tensor([[float(size), float(size), 0, 0, float(size), float(size)]] * 2)}
    outs = []
    with torch.no_grad():
        for i in range(STEPS):
            # the device loop feeds the UNet an fp16 input
            x = sch.scale_model_input(lat, i).half().float()
            eps = ref(torch.cat([x, x]), sch.timesteps[i], ehs, added_cond_kwargs=added)[0].float()
            outs.append(eps.clone())
            lat = sch.step(eps[0:1] + GUIDANCE * (eps[1:2] - eps[0:1]), i, lat)
    return outs, lat


def _device_image(pipe, cond):
    outs = []
    orig = pipe.unet.forward

    def spy(*a, **k):
        o = orig(*a, **k)
        outs.append(o[0].float().cpu().clone())
        return o

    pipe.unet.forward = spy
    try:
        res = pipe(cond["prompt_embeds"], cond["pooled_prompt_embeds"], cond["negative_prompt_embeds"],
                   cond["negative_pooled_prompt_embeds"], num_inference_steps=TOTAL_STEPS, guidance_scale=GUIDANCE,
                   latents=cond["latents"], last_step=STEPS)
    finally:
        pipe.unet.forward = orig
    return outs, res.latents.float().cpu()


@pytest.mark.parametrize("which", ["tiny", "sdxl"])
def test_graph_replay_loop_matches_eager_and_oracle(which):
    dev = cuda_or_skip()
    from basedxl_b200 import _lib
    from basedxl_b200.model import BasedXLPipeline
    from basedxl_b200.sdxl_unet import sdxl_config, tiny_config
    from basedxl_b200.unet import BasedXLUnet
    from basedxl_b200.utils import BasedXLConfig

    ucfg = tiny_config() if which == "tiny" else sdxl_config()
    hw = 32
    ref, gpu = _models(ucfg, dev)
    cfg = BasedXLConfig(height=hw * 8, width=hw * 8)
    pipe = BasedXLPipeline(BasedXLUnet(gpu, cfg), cfg)
    # two images with DIFFERENT conditioning, one after the other: the second one must not see
    # anything the first one cached (cross-attention K/V, the graph's static conditioning)
    conds = [_conditioning(ucfg, hw, seed=11), _conditioning(ucfg, hw, seed=12)]
    eager = [_device_image(pipe, c) for c in conds]
    pipe.unet.enable_cuda_graph()
    graphed = [_device_image(pipe, c) for c in conds]
    assert pipe.unet._graphed is not None and pipe.unet._graphed.replays >= 2 * STEPS - 1
    # a third image repeating the first conditioning: replay after a change and back
    again = _device_image(pipe, conds[0])
    torch.cuda.synchronize()
    _lib.device_status()
    pipe.unet.release_graph()
    for img in range(2):
        for i in range(STEPS):
            assert torch.equal(graphed[img][0][i], eager[img][0][i]), f"image {img} step {i}: replay differs from eager launches"
        assert torch.equal(graphed[img][1], eager[img][1])
    assert torch.equal(again[1], eager[0][1])
    # the two conditionings really lead to different images
    assert rel_l2(eager[1][1], eager[0][1]) > 1e-2
    for img in range(2):
        outs_ref, lat_ref = _oracle_loop(ref, conds[img], hw * 8)
        per_step = [rel_l2(graphed[img][0][i], outs_ref[i]) for i in range(STEPS)]
        final = rel_l2(graphed[img][1], lat_ref)
        print(f"{which} image {img}: per-step rel-L2 {[f'{e:.2e}' for e in per_step]}, final latents {final:.2e}")
        assert max(per_step) <= 2e-3, per_step
        assert final <= 2e-3, final


def test_first_call_after_loading_weights_packs_before_the_convolution_reads():
    """A convolution reached for the first time inside ``BasedXLUnet.forward`` (static-weights mode:
    the kernel fetches weight tiles before waiting for its predecessor) packs its weight right
    before the launch; the convolution must still read the finished copy.  SDXL's widest case,
    2560 -> 1280 channels, loaded after the wrapper was built so that the packing is lazy."""
    dev = cuda_or_skip()
    from basedxl_b200 import _lib, layers
    from basedxl_b200.unet import BasedXLUnet
    from basedxl_b200.utils import BasedXLConfig

    class OneConv(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.conv = layers.Conv2d(2560, 1280, 3, padding=1)

        def forward(self, sample, timestep, encoder_hidden_states, added_cond_kwargs=None, return_dict=False):
            return (self.conv(sample),)

    torch.manual_seed(3)
    model = OneConv().half().to(dev).eval()
    unet = BasedXLUnet(model, BasedXLConfig(height=256, width=256))
    g = torch.Generator().manual_seed(5)
    w = (torch.randn(1280, 2560, 3, 3, generator=g) / (9 * 2560) ** 0.5).half()
    b = torch.randn(1280, generator=g).half()
    model.load_state_dict({"conv.weight": w, "conv.bias": b})
    x = torch.randn(2, 2560, 32, 32, generator=g).half()
    ref = torch.nn.functional.conv2d(x.float(), w.float(), b.float(), padding=1)
    xd = x.to(dev).contiguous(memory_format=torch.channels_last)
    with torch.no_grad():
        y_first = unet(xd, torch.tensor(999.0, device=dev), None)[0].float().cpu()
        y_second = unet(xd, torch.tensor(999.0, device=dev), None)[0].float().cpu()
    _lib.device_status()
    assert rel_l2(y_first, ref) <= 2e-3, rel_l2(y_first, ref)
    assert torch.equal(y_first, y_second)

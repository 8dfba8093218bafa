"""Pipeline wrapper (reference: basedxl/model.py:10-45).

The reference wraps diffusers' ``StableDiffusionXLPipeline`` (text encoders,
scheduler loop, VAE).  Only the UNet loop is on the accelerated path, so this
wrapper drives exactly that: text conditioning comes in as tensors
(``prompt_embeds`` / ``pooled_prompt_embeds``), the loop is a headless Euler
sampler, and the result is the final latent.  ``from_pretrained`` needs the
third-party package and downloaded weights and says so; ``from_config`` builds
the SDXL-shaped UNet with seeded random weights.
"""
from __future__ import annotations

import torch

from .scheduler import EulerDiscreteScheduler
from .sdxl_unet import UNet2DConditionModel, UNetConfig, sdxl_config
from .unet import BasedXLUnet
from .utils import BasedXLConfig


class PipelineOutput:
    def __init__(self, latents):
        self.latents = latents
        self.images = [latents]  # headless: the "image" is the latent


class BasedXLPipeline:
    def __init__(self, unet: BasedXLUnet, basedxl_config: BasedXLConfig, scheduler=None):
        self.unet = unet
        self.basedxl_config = basedxl_config
        self.scheduler = scheduler or EulerDiscreteScheduler()
        self._progress = basedxl_config.rank == 0

    @staticmethod
    def from_pretrained(basedxl_config: BasedXLConfig, **kwargs):
        raise RuntimeError(
            "from_pretrained needs the `diffusers` package and downloaded SDXL weights, neither of which is a "
            "dependency of this library; build the UNet with BasedXLPipeline.from_config(cfg) and load a state "
            "dict with the usual SDXL parameter names into pipeline.unet.model"
        )

    @staticmethod
    def from_config(basedxl_config: BasedXLConfig, unet_config: UNetConfig | None = None, seed: int = 0, scheduler=None):
        """SDXL-shaped UNet with random weights drawn on the host with ``seed``
        (the device generator gives every rank the same values) and cast to
        the config's dtype."""
        torch.manual_seed(seed)
        with torch.device(basedxl_config.device):
            model = UNet2DConditionModel(unet_config or sdxl_config())
        model = model.to(dtype=basedxl_config.dtype).eval()
        return BasedXLPipeline(BasedXLUnet(model, basedxl_config), basedxl_config, scheduler)

    def set_progress_bar_config(self, disable: bool = False, **kwargs):
        self._progress = not disable

    def prepare_inputs(self, prompt_embeds, pooled_prompt_embeds, negative_prompt_embeds=None,
                       negative_pooled_prompt_embeds=None, latents=None, generator=None):
        """Host or device tensors in, device-resident loop inputs out:
        ``(latents fp32 [1,4,h,w], encoder_hidden_states [2,L,D], added_cond_kwargs)``.
        CFG batch of 2: row 0 unconditional, row 1 conditional."""
        cfg = self.basedxl_config
        dev, dt = cfg.device, cfg.dtype
        h, w = cfg.height // 8, cfg.width // 8
        if latents is None:
            latents = torch.randn((1, 4, h, w), generator=generator, device=generator.device if generator else "cpu")
        latents = latents.to(device=dev, dtype=torch.float32, non_blocking=True)
        if negative_prompt_embeds is None:
            negative_prompt_embeds = torch.zeros_like(prompt_embeds)
        if negative_pooled_prompt_embeds is None:
            negative_pooled_prompt_embeds = torch.zeros_like(pooled_prompt_embeds)
        to = lambda t: t.to(device=dev, dtype=dt, non_blocking=True)
        ehs = torch.cat([to(negative_prompt_embeds), to(prompt_embeds)])
        text = torch.cat([to(negative_pooled_prompt_embeds), to(pooled_prompt_embeds)])
        ids = torch.tensor([[cfg.height, cfg.width, 0, 0, cfg.height, cfg.width]] * 2, dtype=torch.float32, device=dev)
        return latents, ehs, {"text_embeds": text, "time_ids": ids}

    @torch.no_grad()
    def denoise(self, latents, ehs, added, num_inference_steps: int = 50, guidance_scale: float = 5.0,
                first_step: int = 0, last_step: int | None = None, scale_initial: bool = True):
        """Steps ``first_step .. last_step-1`` of a ``num_inference_steps``-step Euler
        schedule on device-resident inputs; returns the latents after the last step."""
        dt = self.basedxl_config.dtype
        sch = self.scheduler
        sch.set_timesteps(num_inference_steps, device=latents.device)
        if first_step == 0 and scale_initial:
            latents = latents * sch.init_noise_sigma
        last_step = num_inference_steps if last_step is None else last_step
        fused = latents.is_cuda and dt == torch.float16 and latents.shape[0] == 1
        if fused:
            from . import ops

            # channels-last throughout: the UNet produces its output in that order (and every strip's
            # rows are then one contiguous range), so the fused update reads it as it is
            cl = torch.channels_last
            latents = latents.contiguous(memory_format=cl).clone()  # updated in place by the fused step
            x2 = torch.empty((2, *latents.shape[1:]), device=latents.device, dtype=dt, memory_format=cl)
            x = sch.scale_model_input(latents, first_step).to(dt)
            x2[0:1], x2[1:2] = x, x
        for i in range(first_step, last_step):
            if fused:
                eps = self.unet(x2, sch.timesteps[i], ehs, added_cond_kwargs=added)[0]
                # guidance + Euler update + scaling of the next input: one kernel
                ops.cfg_euler_step(eps.contiguous(memory_format=cl), latents, x2, guidance_scale, sch.sigmas[i], sch.sigmas[i + 1])
            else:
                x = sch.scale_model_input(latents, i).to(dt)
                eps = self.unet(torch.cat([x, x]), sch.timesteps[i], ehs, added_cond_kwargs=added)[0].float()
                eps = eps[0:1] + guidance_scale * (eps[1:2] - eps[0:1])
                latents = sch.step(eps, i, latents)
        return latents

    @torch.no_grad()
    def __call__(
        self,
        prompt_embeds: torch.Tensor,
        pooled_prompt_embeds: torch.Tensor,
        negative_prompt_embeds: torch.Tensor | None = None,
        negative_pooled_prompt_embeds: torch.Tensor | None = None,
        num_inference_steps: int = 50,
        guidance_scale: float = 5.0,
        latents: torch.Tensor | None = None,
        generator: torch.Generator | None = None,
        last_step: int | None = None,
        **kwargs,
    ):
        """One image.  ``last_step`` (not in the reference) stops after that many steps of the
        ``num_inference_steps``-step schedule and returns the latents reached."""
        cfg = self.basedxl_config
        assert "width" not in kwargs or cfg.width == kwargs["width"]
        assert "height" not in kwargs or cfg.height == kwargs["height"]
        self.unet.reset()  # re-enter the synchronous warm-up phase (basedxl/model.py:44)
        lat, ehs, added = self.prepare_inputs(
            prompt_embeds, pooled_prompt_embeds, negative_prompt_embeds, negative_pooled_prompt_embeds, latents, generator
        )
        lat = self.denoise(lat, ehs, added, num_inference_steps, guidance_scale, last_step=last_step)
        return PipelineOutput(lat)

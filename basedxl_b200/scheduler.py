"""Euler discrete sampler for the denoising loop (epsilon prediction,
scaled-linear betas 0.00085..0.012 over 1000 training steps, "leading" timestep
spacing with offset 1: the SDXL base settings).  The reference takes its
scheduler from the third-party ``diffusers`` package (sample.py:47-50); this is
an independent implementation of the published Euler method (Karras et al.
2022, Alg. 1 without churn) sufficient to drive the UNet loop headlessly.
"""
from __future__ import annotations

import numpy as np
import torch


class EulerDiscreteScheduler:
    def __init__(self, num_train_timesteps=1000, beta_start=0.00085, beta_end=0.012, steps_offset=1):
        betas = np.linspace(beta_start**0.5, beta_end**0.5, num_train_timesteps, dtype=np.float64) ** 2
        alphas_cumprod = np.cumprod(1.0 - betas)
        self.train_sigmas = ((1 - alphas_cumprod) / alphas_cumprod) ** 0.5
        self.num_train_timesteps = num_train_timesteps
        self.steps_offset = steps_offset
        self.timesteps = None
        self.sigmas = None

    def set_timesteps(self, num_inference_steps: int, device="cpu"):
        ratio = self.num_train_timesteps // num_inference_steps
        ts = (np.arange(0, num_inference_steps) * ratio).round()[::-1].astype(np.float64) + self.steps_offset
        sig = np.interp(ts, np.arange(self.num_train_timesteps), self.train_sigmas)
        self.timesteps = torch.tensor(ts, dtype=torch.float32, device=device)
        self.sigmas = [float(s) for s in sig] + [0.0]
        self.init_noise_sigma = float((sig.max() ** 2 + 1) ** 0.5)

    def scale_model_input(self, sample: torch.Tensor, i: int) -> torch.Tensor:
        return sample / ((self.sigmas[i] ** 2 + 1) ** 0.5)

    def step(self, eps: torch.Tensor, i: int, sample: torch.Tensor) -> torch.Tensor:
        # x_{i+1} = x_i + eps * (sigma_{i+1} - sigma_i), evaluated in fp32
        return (sample.float() + eps.float() * (self.sigmas[i + 1] - self.sigmas[i])).to(sample.dtype)

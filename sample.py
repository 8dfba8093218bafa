"""Command-line sampler with the reference CLI's flags (sample.py:20-33 of the
reference), headless: the text encoders and the VAE of the reference pipeline are
outside the accelerated path, so conditioning is synthetic (seeded N(0,1)) unless
tensors are given with --embeds, weights are seeded random unless a state dict is
given with --unet-state, and the output is the final latent (saved with
torch.save) instead of a PNG.

    python sample.py [--num-inference-steps 50] [--width 1024] [--height 1024]
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 sample.py
"""
from __future__ import annotations

import argparse
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402


def main(
    prompt: str = "",
    negative_prompt: str = "",
    seed: int = 42,
    guidance_scale: float = 5.0,
    num_inference_steps: int = 50,
    width: int = 1024,
    height: int = 1024,
    compile_unet: bool = False,
    fp16_acc_matmul: bool = False,
    patch_parallelism: bool = True,
    distrifusion_warmup_steps: int = 4,
    out_path: str = "sample_latents.pt",
    verbose: bool = False,
    embeds: str | None = None,
    unet_state: str | None = None,
    cuda_graph: bool = True,
):
    from basedxl_b200 import BasedXLPipeline
    from basedxl_b200.utils import BasedXLConfig

    assert not (compile_unet and fp16_acc_matmul), "compile_unet and fp16_acc_matmul are mutually exclusive, as in the reference"
    cfg = BasedXLConfig(
        width=width, height=height, compile_unet=compile_unet, fp16_acc_matmul=fp16_acc_matmul,
        patch_parallelism=patch_parallelism, warmup_steps=distrifusion_warmup_steps, verbose=verbose,
    )
    pipeline = BasedXLPipeline.from_config(cfg, seed=0)
    if unet_state:
        pipeline.unet.model.load_state_dict(torch.load(unet_state, map_location=cfg.device))
    if cuda_graph:
        pipeline.unet.enable_cuda_graph()
    if embeds:
        e = torch.load(embeds)
        pe, ppe, npe, nppe = e["prompt_embeds"], e["pooled_prompt_embeds"], e.get("negative_prompt_embeds"), e.get("negative_pooled_prompt_embeds")
    else:
        g = torch.Generator().manual_seed(seed)
        pe, npe = torch.randn(1, 77, 2048, generator=g), torch.randn(1, 77, 2048, generator=g)
        ppe, nppe = torch.randn(1, 1280, generator=g), torch.randn(1, 1280, generator=g)
    # warm-up image, as the reference does (sample.py:60-65)
    pipeline(pe, ppe, npe, nppe, num_inference_steps=10, guidance_scale=guidance_scale, generator=torch.Generator().manual_seed(seed))
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStart()
    t0 = time.perf_counter()
    out = pipeline(pe, ppe, npe, nppe, num_inference_steps=num_inference_steps, guidance_scale=guidance_scale,
                   generator=torch.Generator().manual_seed(seed))
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    torch.cuda.cudart().cudaProfilerStop()
    if cfg.rank == 0:
        torch.save(out.latents.cpu(), out_path)
        print(f"{num_inference_steps} steps at {width}x{height} on {cfg.world_size} GPU(s): {dt:.3f} s; latents -> {out_path}")
    pipeline.unet.release_graph()
    if cfg.world_size > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    for name, default in [("prompt", ""), ("negative-prompt", ""), ("out-path", "sample_latents.pt"), ("embeds", None), ("unet-state", None)]:
        ap.add_argument(f"--{name}", default=default)
    for name, default in [("seed", 42), ("num-inference-steps", 50), ("width", 1024), ("height", 1024), ("distrifusion-warmup-steps", 4)]:
        ap.add_argument(f"--{name}", type=int, default=default)
    ap.add_argument("--guidance-scale", type=float, default=5.0)
    for name, default in [("compile-unet", False), ("fp16-acc-matmul", False), ("patch-parallelism", True), ("verbose", False), ("cuda-graph", True)]:
        ap.add_argument(f"--{name}", type=lambda s: s.lower() in ("1", "true", "yes"), default=default, nargs="?", const=True)
    main(**{k.replace("-", "_"): v for k, v in vars(ap.parse_args()).items()})

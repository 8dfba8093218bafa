"""Golden fixture for the whole displaced-patch-parallel loop, produced by the
reference's OWN wrappers, UNet wrapper and comm manager running unmodified on
CPU ranks (gloo).

    python tests/golden/make_golden_loop.py --reference /path/to/basedxl-checkout

Host graph: the miniature SDXL-shaped UNet of ``basedxl_b200.sdxl_unet`` over
stock ``torch.nn`` layers (``oracle.torch_layers``), standing in for the
third-party UNet class the reference wraps (it is injected under the import
names the reference uses).  The reference never wires up its comm manager;
the script supplies the missing sequence: construct the manager, hand it to the
UNet wrapper, run one registration forward, create the buffers, reset the
counters.

For each configuration (world size, CFG on/off) every rank runs the same
seeded 8-step Euler loop (5 synchronous steps, then 3 displaced ones); rank 0's
per-step UNet outputs and final latents are stored in
``tests/golden/unet_pp_loop.npz`` together with the inputs.  The 8-rank
configuration (CFG halves x 4 strips) is the layout of an 8-GPU run; one
configuration is also run for all 50 steps of the schedule (final latents and
the UNet outputs of a few steps are kept).  ``comm_checkpoint``
is set to 10 so that the miniature's 37 exchanged tensors are gathered in
several chunks plus a tail, as the full network's 155 are with the default 60.
"""
from __future__ import annotations

import argparse
import importlib.util
import os
import sys
import types

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

STEPS, TOTAL_STEPS, GUIDANCE, LATENT, CKPT = 8, 50, 5.0, 32, 10
# (tag, world size, CFG split, steps run)
CONFIGS = [("ws2_nocfg", 2, False, STEPS), ("ws4_cfg", 4, True, STEPS), ("ws4_nocfg", 4, False, STEPS),
           ("ws8_cfg", 8, True, STEPS), ("ws4_cfg_50", 4, True, TOTAL_STEPS)]
KEPT_STEPS_LONG = [0, 4, 5, 6, 24, 49]  # UNet outputs kept from the 50-step run


def loop_inputs(cfg):
    g = torch.Generator().manual_seed(2024)
    pooled = cfg.projection_class_embeddings_input_dim - 6 * cfg.addition_time_embed_dim
    return {
        "latents": torch.randn(1, 4, LATENT, LATENT, generator=g),
        "ehs": torch.randn(2, 9, cfg.cross_attention_dim, generator=g),
        "text_embeds": torch.randn(2, pooled, generator=g),
        "time_ids": torch.tensor([[256.0, 256, 0, 0, 256, 256]] * 2),
    }


def euler_loop(unet_call, inp, sched, steps=STEPS):
    """The headless loop both sides run: CFG batch of 2, guidance, Euler update."""
    sched.set_timesteps(TOTAL_STEPS)
    lat = inp["latents"].clone().float() * sched.init_noise_sigma
    added = {"text_embeds": inp["text_embeds"], "time_ids": inp["time_ids"]}
    outs = []
    for i in range(steps):
        x = sched.scale_model_input(lat, i)
        x2 = torch.cat([x, x])
        eps = unet_call(x2, sched.timesteps[i], inp["ehs"], added).float()
        outs.append(eps.clone())
        e = eps[0:1] + GUIDANCE * (eps[1:2] - eps[0:1])
        lat = sched.step(e, i, lat)
    return lat, outs


def load_reference(root):
    from basedxl_b200.sdxl_unet import UNet2DConditionModel
    from oracle.torch_layers import Attention

    def mod(name, **attrs):
        m = types.ModuleType(name)
        m.__path__ = []
        for k, v in attrs.items():
            setattr(m, k, v)
        sys.modules[name] = m
        return m

    class ConfigMixin:  # plain marker base, as far as the reference uses it
        pass

    mod("diffusers"); mod("diffusers.models"); mod("diffusers.models.unets"); mod("diffusers.utils")
    mod("diffusers.models.unets.unet_2d_condition", UNet2DConditionModel=UNet2DConditionModel)
    mod("diffusers.models.modeling_utils", ModelMixin=nn.Module)
    mod("diffusers.configuration_utils", ConfigMixin=ConfigMixin)
    mod("diffusers.models.attention_processor", Attention=Attention)
    mod("diffusers.utils.constants", USE_PEFT_BACKEND=True)
    mod("basedxl"); mod("basedxl.modules"); mod("basedxl.triton")
    # the Triton matmul is not on this path; lowp_linear imports it at module scope
    mod("basedxl.triton.cascaded_lowp_matmul", cascaded_lowp_matmul=None)

    def load(modname, rel):
        spec = importlib.util.spec_from_file_location(modname, os.path.join(root, rel))
        m = importlib.util.module_from_spec(spec)
        sys.modules[modname] = m
        spec.loader.exec_module(m)
        return m

    utils = load("basedxl.utils", "basedxl/utils.py")
    for f in ("base_module", "conv2d", "groupnorm", "attn", "lowp_linear"):
        load(f"basedxl.modules.{f}", f"basedxl/modules/{f}.py")
    unet = load("basedxl.unet", "basedxl/unet.py")
    return utils, unet


def worker(rank, world, use_cfg, steps, ref_root, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    from basedxl_b200.scheduler import EulerDiscreteScheduler
    from basedxl_b200.sdxl_unet import UNet2DConditionModel, tiny_config
    from oracle.torch_layers import TorchLayers

    utils, unet_mod = load_reference(ref_root)
    # the reference config tries NCCL and falls into its single-device branch; patch the plain attributes
    cfg = utils.BasedXLConfig(use_cfg=use_cfg, patch_parallelism=True, warmup_steps=4, comm_checkpoint=CKPT, dtype=torch.float32)
    cfg.rank, cfg.world_size, cfg.device = rank, world, "cpu"
    cfg.n_device_per_batch = world // 2 if use_cfg else world
    cfg.batch_group = None
    if use_cfg:
        half = world // 2
        groups = [dist.new_group(list(range(i * half, (i + 1) * half))) for i in range(2)]
        cfg.batch_group = groups[cfg.batch_idx()]
    torch.manual_seed(0)
    ucfg = tiny_config()
    model = UNet2DConditionModel(ucfg, layers=TorchLayers).eval()
    state = {k: v.clone() for k, v in model.state_dict().items()}
    wrapped = unet_mod.BasedXLUnet(model, cfg)
    inp = loop_inputs(ucfg)
    added = {"text_embeds": inp["text_embeds"], "time_ids": inp["time_ids"]}
    with torch.no_grad():
        cm = utils.PatchParallelismCommManager(cfg)
        wrapped.set_comm_manager(cm)
        wrapped(torch.cat([inp["latents"]] * 2), torch.tensor(999.0), inp["ehs"], added_cond_kwargs=added)
        cm.create_buffer()
        wrapped.set_counter(0)
        call = lambda x, t, e, a: wrapped(x, t, e, added_cond_kwargs=a)[0]
        lat, outs = euler_loop(call, inp, EulerDiscreteScheduler(), steps=steps)
        cm.clear()
    if rank == 0:
        ret["latents"] = lat.numpy()
        ret["outs"] = torch.stack(outs).numpy()
        ret["n_registered"] = len(cm.starts)
        ret["numel"] = cm.numel
        ret["state"] = {k: v.numpy() for k, v in state.items()}
        ret["inputs"] = {k: v.numpy() for k, v in inp.items()}
    dist.barrier()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--out", default=os.path.join(HERE, "unet_pp_loop.npz"))
    args = ap.parse_args()
    blob = {}
    mgr = mp.Manager()
    for n, (tag, world, use_cfg, steps) in enumerate(CONFIGS):
        ret = mgr.dict()
        mp.spawn(worker, args=(world, use_cfg, steps, args.reference, 29540 + n, ret), nprocs=world, join=True)
        blob[f"{tag}_latents"] = ret["latents"]
        outs = ret["outs"].astype(np.float32)
        if steps > STEPS:
            outs = outs[KEPT_STEPS_LONG]
            blob[f"{tag}_kept_steps"] = np.array(KEPT_STEPS_LONG)
        blob[f"{tag}_outs"] = outs
        blob[f"{tag}_n_registered"] = np.int64(ret["n_registered"])
        blob[f"{tag}_numel"] = np.int64(ret["numel"])
        if n == 0:
            for k, v in ret["inputs"].items():
                blob[f"in_{k}"] = v
            # weights are reproducible from the seed; a checksum pins them
            blob["state_checksum"] = np.float64(sum(float(np.abs(v).sum()) for v in ret["state"].values()))
        print(tag, "registered", ret["n_registered"], "latents |.|", float(np.abs(ret["latents"]).mean()))
    # single-rank run of the same loop, for scale: how far displaced parallelism moves the result
    from basedxl_b200.scheduler import EulerDiscreteScheduler
    from basedxl_b200.sdxl_unet import UNet2DConditionModel, tiny_config
    from oracle.torch_layers import TorchLayers

    torch.manual_seed(0)
    model = UNet2DConditionModel(tiny_config(), layers=TorchLayers).eval()
    with torch.no_grad():
        lat, outs = euler_loop(lambda x, t, e, a: model(x, t, e, added_cond_kwargs=a)[0], loop_inputs(tiny_config()), EulerDiscreteScheduler())
    blob["ws1_latents"] = lat.numpy()
    blob["ws1_outs"] = torch.stack(outs).numpy()
    np.savez_compressed(args.out, **blob)
    print("written", args.out)


if __name__ == "__main__":
    main()

"""Generate the golden fixtures in this directory by executing the reference's
own modules, unmodified, on CPU.

Usage (only where a checkout of the reference is available):

    python tests/golden/make_golden.py --reference /path/to/basedxl-checkout

The reference files are loaded by path under a stub ``basedxl`` namespace
package (its ``__init__`` imports the third-party ``diffusers`` pipeline, which
is not needed here).  ``basedxl/modules/attn.py`` imports two names from
``diffusers``; a minimal stand-in module provides them.  Collectives issued by
the reference's synchronous path are served by an in-process fake
``all_gather`` that delivers what the peers would have sent, so each fixture is
produced by a single process and is deterministic.

The fixtures are small ``.npz`` files holding the seeded inputs, the exchange
buffers handed to the module, and the module's output.
"""
from __future__ import annotations

import argparse
import importlib.util
import os
import sys
import types

import numpy as np
import torch
import torch.nn as nn

HERE = os.path.dirname(os.path.abspath(__file__))


# ---------------------------------------------------------------------------
# loading the reference
# ---------------------------------------------------------------------------
def load_reference(root: str) -> types.SimpleNamespace:
    if not os.path.isdir(os.path.join(root, "basedxl")):
        raise SystemExit(f"no reference checkout at {root}")

    # stand-in for the two diffusers names attn.py imports
    class Attention(nn.Module):
        def __init__(self, dim, heads, ctx_dim=None, out_bias=True):
            super().__init__()
            ctx_dim = ctx_dim or dim
            self.heads = heads
            self.to_q = nn.Linear(dim, dim, bias=False)
            self.to_k = nn.Linear(ctx_dim, dim, bias=False)
            self.to_v = nn.Linear(ctx_dim, dim, bias=False)
            self.to_out = nn.ModuleList([nn.Linear(dim, dim, bias=out_bias), nn.Dropout(0.0)])
            self.residual_connection = False
            self.rescale_output_factor = 1.0

    d = types.ModuleType("diffusers")
    dm = types.ModuleType("diffusers.models")
    dap = types.ModuleType("diffusers.models.attention_processor")
    du = types.ModuleType("diffusers.utils")
    duc = types.ModuleType("diffusers.utils.constants")
    dap.Attention = Attention
    duc.USE_PEFT_BACKEND = True
    for name, mod in [
        ("diffusers", d),
        ("diffusers.models", dm),
        ("diffusers.models.attention_processor", dap),
        ("diffusers.utils", du),
        ("diffusers.utils.constants", duc),
    ]:
        sys.modules[name] = mod

    def ns(name):
        m = types.ModuleType(name)
        m.__path__ = []  # namespace-like package
        sys.modules[name] = m
        return m

    ns("basedxl")
    ns("basedxl.modules")
    ns("basedxl.triton")

    def load(modname, rel):
        spec = importlib.util.spec_from_file_location(modname, os.path.join(root, rel))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[modname] = mod
        spec.loader.exec_module(mod)
        return mod

    utils = load("basedxl.utils", "basedxl/utils.py")
    base = load("basedxl.modules.base_module", "basedxl/modules/base_module.py")
    conv = load("basedxl.modules.conv2d", "basedxl/modules/conv2d.py")
    gn = load("basedxl.modules.groupnorm", "basedxl/modules/groupnorm.py")
    attn = load("basedxl.modules.attn", "basedxl/modules/attn.py")
    return types.SimpleNamespace(utils=utils, base=base, conv=conv, gn=gn, attn=attn, Attention=Attention, root=root)


def make_cfg(ref, n_split: int, split_idx: int, warmup_steps: int = 4):
    """A reference config object describing one strip of ``n_split`` on CPU.
    The constructor falls into its single-device branch (no NCCL here); the
    plain attributes are then overwritten."""
    cfg = ref.utils.BasedXLConfig(use_cfg=False, warmup_steps=warmup_steps)
    cfg.rank = split_idx
    cfg.world_size = n_split
    cfg.n_device_per_batch = n_split
    cfg.device = "cpu"
    cfg.batch_group = None
    return cfg


class FakeManager:
    """Stands in for the comm manager: buffers are handed to the module
    directly, ``enqueue`` only records what the module publishes."""

    def __init__(self):
        self.handles = None
        self.buffer_list = [None]
        self.published = {}

    def enqueue(self, idx, tensor):
        self.published[idx] = tensor.detach().clone()


class FakeAllGather:
    """Context manager that replaces ``torch.distributed.all_gather`` while a
    reference module runs: the output list is filled with the tensors every
    peer contributes (own = the one passed in)."""

    def __init__(self, peers, split_idx):
        self.peers, self.split_idx = peers, split_idx

    def __call__(self, out_list, tensor, group=None, async_op=False):
        for j, o in enumerate(out_list):
            o.copy_(tensor if j == self.split_idx else self.peers[j])

    def __enter__(self):
        import torch.distributed as dist

        self._real = dist.all_gather
        dist.all_gather = self
        return self

    def __exit__(self, *exc):
        import torch.distributed as dist

        dist.all_gather = self._real


def strips(x, n, dim=2):
    return list(torch.chunk(x, n, dim=dim))


# ---------------------------------------------------------------------------
# fixtures
# ---------------------------------------------------------------------------
def golden_conv(ref, out):
    torch.manual_seed(0)
    cases = {}
    for tag, (cin, cout, h, w, stride) in {
        "s1": (32, 48, 16, 16, 1),
        "s2": (32, 32, 16, 16, 2),
    }.items():
        conv = nn.Conv2d(cin, cout, 3, stride=stride, padding=1)
        x = torch.randn(2, cin, h, w)
        x_prev = x + 0.01 * torch.randn_like(x)  # previous-step activations
        cases[f"{tag}_x"] = x.numpy()
        cases[f"{tag}_x_prev"] = x_prev.numpy()
        cases[f"{tag}_w"] = conv.weight.detach().numpy()
        cases[f"{tag}_b"] = conv.bias.detach().numpy()
        cases[f"{tag}_stride"] = np.int64(stride)
        for n in (2, 4):
            xs, xps = strips(x, n), strips(x_prev, n)
            bnd = lambda t: torch.stack([t[:, :, :1, :], t[:, :, -1:, :]], dim=0)
            for idx in range(n):
                cfg = make_cfg(ref, n, idx)
                # displaced (stale halo) path
                m = ref.conv.BasedConv2dPP(conv, cfg)
                m.comm_manager = FakeManager()
                m.idx = 0
                m.buffer_list = [bnd(t).clone() for t in xps]
                m.counter = cfg.warmup_steps + 1
                with torch.no_grad():
                    y = m(xs[idx])
                cases[f"{tag}_n{n}_i{idx}_stale_y"] = y.numpy()
                cases[f"{tag}_n{n}_i{idx}_published"] = m.comm_manager.published[0].numpy()
                # synchronous path
                m = ref.conv.BasedConv2dPP(conv, cfg)
                m.comm_manager = FakeManager()
                m.idx = 0
                m.buffer_list = [torch.zeros_like(bnd(t)) for t in xs]
                m.counter = 0
                with torch.no_grad(), FakeAllGather([bnd(t) for t in xs], idx):
                    y = m(xs[idx])
                cases[f"{tag}_n{n}_i{idx}_sync_y"] = y.numpy()
                # first-layer path: full input in, strip out
                m = ref.conv.BasedConv2dPP(conv, cfg, is_first_layer=True)
                with torch.no_grad():
                    y = m(x)
                cases[f"{tag}_n{n}_i{idx}_first_y"] = y.numpy()
    np.savez_compressed(os.path.join(out, "conv2d_pp.npz"), **cases)


def golden_groupnorm(ref, out):
    torch.manual_seed(1)
    cases = {}
    c, g, h, w = 64, 32, 16, 8
    gn = nn.GroupNorm(g, c, eps=1e-5)
    with torch.no_grad():
        gn.weight.normal_(1.0, 0.2)
        gn.bias.normal_(0.0, 0.2)
    x = torch.randn(2, c, h, w) * 1.5 + 0.3
    x_prev = x + 0.01 * torch.randn_like(x)
    cases.update(x=x.numpy(), x_prev=x_prev.numpy(), gamma=gn.weight.detach().numpy(), beta=gn.bias.detach().numpy())
    cases["eps"] = np.float64(gn.eps)
    cases["groups"] = np.int64(g)

    def moments(t):
        n_, c_, h_, w_ = t.shape
        tg = t.view(n_, g, c_ // g, h_, w_)
        return torch.stack([tg.mean(dim=[2, 3, 4], keepdim=True), (tg**2).mean(dim=[2, 3, 4], keepdim=True)], dim=0)

    for n in (2, 4):
        xs, xps = strips(x, n), strips(x_prev, n)
        for idx in range(n):
            cfg = make_cfg(ref, n, idx)
            m = ref.gn.BasedXLGroupNorm(gn, cfg)  # no manager: strip statistics only
            with torch.no_grad():
                cases[f"n{n}_i{idx}_local_y"] = m(xs[idx]).numpy()
            m = ref.gn.BasedXLGroupNorm(gn, cfg)
            m.comm_manager = FakeManager()
            m.idx = 0
            m.buffer_list = [moments(t).clone() for t in xps]
            m.counter = cfg.warmup_steps + 1
            with torch.no_grad():
                cases[f"n{n}_i{idx}_stale_y"] = m(xs[idx]).numpy()
            cases[f"n{n}_i{idx}_published"] = m.comm_manager.published[0].numpy()
            m = ref.gn.BasedXLGroupNorm(gn, cfg)
            m.comm_manager = FakeManager()
            m.idx = 0
            m.buffer_list = [torch.zeros_like(moments(t)) for t in xs]
            m.counter = 0
            with torch.no_grad(), FakeAllGather([moments(t) for t in xs], idx):
                cases[f"n{n}_i{idx}_sync_y"] = m(xs[idx]).numpy()
    np.savez_compressed(os.path.join(out, "groupnorm_pp.npz"), **cases)


def golden_attention(ref, out):
    torch.manual_seed(2)
    cases = {}
    dim, heads, L = 128, 2, 64
    attn = ref.Attention(dim, heads)
    x = torch.randn(2, L, dim)
    x_prev = x + 0.01 * torch.randn_like(x)
    for n in (2, 4):
        for idx in range(n):
            cfg = make_cfg(ref, n, idx)
            xs, xps = strips(x, n, dim=1), strips(x_prev, n, dim=1)
            m = ref.attn.BasedXLSelfAttentionPP(attn, cfg)
            if "wq" not in cases:
                cases.update(
                    x=x.numpy(),
                    x_prev=x_prev.numpy(),
                    wq=attn.to_q.weight.detach().numpy(),
                    wkv=m.to_kv.weight.detach().numpy(),
                    wo=attn.to_out[0].weight.detach().numpy(),
                    bo=attn.to_out[0].bias.detach().numpy(),
                    heads=np.int64(heads),
                )
            with torch.no_grad():
                kv_prev = [m.to_kv(t) for t in xps]
                kv_now = [m.to_kv(t) for t in xs]
            # no buffers yet: own K/V repeated
            m.comm_manager = FakeManager()
            m.comm_manager.buffer_list = None

            def no_register(shape, torch_dtype, layer_type=None):
                return 0

            m.comm_manager.register_tensor = no_register
            with torch.no_grad():
                cases[f"n{n}_i{idx}_local_y"] = m(xs[idx]).numpy()
            # displaced path
            m = ref.attn.BasedXLSelfAttentionPP(attn, cfg)
            m.comm_manager = FakeManager()
            m.idx = 0
            m.buffer_list = [t.clone() for t in kv_prev]
            m.counter = cfg.warmup_steps + 1
            with torch.no_grad():
                cases[f"n{n}_i{idx}_stale_y"] = m(xs[idx]).numpy()
            cases[f"n{n}_i{idx}_published"] = m.comm_manager.published[0].numpy()
            # synchronous path
            m = ref.attn.BasedXLSelfAttentionPP(attn, cfg)
            m.comm_manager = FakeManager()
            m.idx = 0
            m.buffer_list = [torch.zeros_like(t) for t in kv_now]
            m.counter = 0
            with torch.no_grad(), FakeAllGather(kv_now, idx):
                cases[f"n{n}_i{idx}_sync_y"] = m(xs[idx]).numpy()
    # cross attention (no communication)
    ctx_dim, ctx_len = 96, 77
    attn2 = ref.Attention(dim, heads, ctx_dim=ctx_dim)
    ctx = torch.randn(2, ctx_len, ctx_dim)
    m = ref.attn.BasedXLCrossAttentionPP(attn2, make_cfg(ref, 1, 0))
    with torch.no_grad():
        y0 = m(x, encoder_hidden_states=ctx)
        y1 = m(x_prev, encoder_hidden_states=torch.zeros_like(ctx))  # cached K/V must be reused
    cases.update(
        cross_ctx=ctx.numpy(),
        cross_wq=attn2.to_q.weight.detach().numpy(),
        cross_wkv=m.to_kv.weight.detach().numpy(),
        cross_wo=attn2.to_out[0].weight.detach().numpy(),
        cross_bo=attn2.to_out[0].bias.detach().numpy(),
        cross_y=y0.numpy(),
        cross_y_cached=y1.numpy(),
    )
    np.savez_compressed(os.path.join(out, "attention_pp.npz"), **cases)


def golden_comm_schedule(ref, out):
    """Trace of the flat ranges the reference manager gathers, for a toy stack
    of 7 tensors with a checkpoint of 3, over three steps."""
    import torch.distributed as dist

    if not dist.is_initialized():
        dist.init_process_group("gloo", rank=0, world_size=1, init_method="tcp://127.0.0.1:29431")
    cfg = make_cfg(ref, 1, 0)
    cfg.comm_checkpoint = 3
    cm = ref.utils.PatchParallelismCommManager(cfg)
    sizes = [(2, 3), (5,), (4, 2), (7,), (1, 1, 6), (3,), (8,)]
    for s in sizes:
        cm.register_tensor(s, torch.float32, layer_type="t")
    cm.create_buffer()
    launches = []
    real = ref.utils.dist.all_gather

    def spy(buffer_list, tensor, group=None, async_op=False):
        base = cm.buffer_list[0]
        start = (tensor.data_ptr() - base.data_ptr()) // tensor.element_size()
        launches.append((start, start + tensor.numel()))
        return real(buffer_list, tensor, group=group, async_op=async_op)

    ref.utils.dist.all_gather = spy
    per_step = []
    for step in range(3):
        before = len(launches)
        for i, s in enumerate(sizes):
            cm.enqueue(i, torch.full(s, float(step * 10 + i)))
        per_step.append(len(launches) - before)
    cm.clear()
    ref.utils.dist.all_gather = real
    np.savez_compressed(
        os.path.join(out, "comm_schedule.npz"),
        sizes=np.array([int(np.prod(s)) for s in sizes]),
        checkpoint=np.int64(3),
        starts=np.array(cm.starts),
        ends=np.array(cm.ends),
        launches=np.array(launches),
        launches_per_step=np.array(per_step),
        final_buffer=cm.buffer_list[0].numpy(),
    )


def golden_matmul(ref, out):
    """The reference's Triton kernel body, run under Triton's CPU interpreter
    at one shape that reaches the kernel (M >= 512, N >= 256).  The autotuner
    needs a GPU driver, so the jitted function underneath it is launched with
    the kernel's own block configuration."""
    os.environ["TRITON_INTERPRET"] = "1"
    spec = importlib.util.spec_from_file_location(
        "basedxl.triton.cascaded_lowp_matmul", os.path.join(ref.root, "basedxl/triton/cascaded_lowp_matmul.py")
    )
    mod = importlib.util.module_from_spec(spec)
    sys.modules["basedxl.triton.cascaded_lowp_matmul"] = mod
    spec.loader.exec_module(mod)
    import triton

    kern = mod._matmul_kernel
    while not isinstance(kern, triton.runtime.interpreter.InterpretedFunction) and hasattr(kern, "fn"):
        kern = kern.fn
    torch.manual_seed(0)
    M, K, N = 512, 640, 256
    a = torch.randn(M, K).half()
    b = torch.randn(K, N).half()
    cases = {"a": a.numpy(), "b": b.numpy()}
    for bk in (16, 32):
        c = torch.empty(M, N, dtype=torch.float16)
        grid = (triton.cdiv(M, 256) * triton.cdiv(N, 128),)
        kern[grid](
            a, b, c, M, N, K, a.stride(0), a.stride(1), b.stride(0), b.stride(1), c.stride(0), c.stride(1),
            BLOCK_M=256, BLOCK_N=128, BLOCK_K=bk, GROUP_M=8, K_ACC_DIV=1, K_IS_DIVISIBLE=True,
        )
        cases[f"c_bk{bk}"] = c.numpy()
    np.savez_compressed(os.path.join(out, "lowp_matmul.npz"), **cases)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--out", default=HERE)
    ap.add_argument("--skip-matmul", action="store_true")
    args = ap.parse_args()
    ref = load_reference(args.reference)
    golden_conv(ref, args.out)
    golden_groupnorm(ref, args.out)
    golden_attention(ref, args.out)
    golden_comm_schedule(ref, args.out)
    if not args.skip_matmul:
        golden_matmul(ref, args.out)
    print("fixtures written to", args.out)


if __name__ == "__main__":
    main()

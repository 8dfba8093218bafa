"""The patch-parallel WRAPPERS (``BasedConv2dPP``, ``BasedXLGroupNorm``,
``BasedXLSelfAttentionPP``) on one GPU, driven through the real comm manager
with hand-filled peer buffers: register -> ``create_buffer`` -> ``buffer_list``
views -> ``own_slot`` -> ``enqueue``.  Peers are not running; what they would
have sent is written into their staging ranges (displaced steps) or delivered by
a stand-in for ``torch.distributed.all_gather`` (synchronous steps), exactly as
the script that produced the fixtures did with the reference's modules.
Outputs and published tensors are compared with those fixtures
(tests/golden/conv2d_pp.npz, groupnorm_pp.npz, attention_pp.npz)."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist

from tests._util import assert_close, cuda_or_skip

pytestmark = pytest.mark.gpu
T = torch.from_numpy


def _cfg(n, idx, warmup_steps=4):
    """Single-process config describing strip ``idx`` of ``n`` (no CFG split): the plain
    attributes are overwritten, as the fixture script does with the reference's config."""
    from basedxl_b200.utils import BasedXLConfig

    cfg = BasedXLConfig(use_cfg=False, patch_parallelism=True, warmup_steps=warmup_steps)
    cfg.rank, cfg.world_size, cfg.n_device_per_batch, cfg.batch_group = idx, n, n, None
    return cfg


class FakeAllGather:
    """Stands in for ``torch.distributed.all_gather`` while a wrapper runs its synchronous
    path: fills the output list with what every peer contributes (own = the tensor passed)."""

    def __init__(self, peers, own):
        self.peers, self.own, self.calls = peers, own, 0

    def __call__(self, out_list, tensor, group=None, async_op=False):
        self.calls += 1
        for j, o in enumerate(out_list):
            src = tensor if j == self.own else self.peers[j]
            o.copy_(src.reshape(o.shape) if src.dtype == o.dtype else src.reshape(-1).view(o.dtype).reshape(o.shape))

    def __enter__(self):
        self._real = dist.all_gather
        dist.all_gather = self
        return self

    def __exit__(self, *exc):
        dist.all_gather = self._real


def _wire(wrapper, cfg, *first_call_args):
    """The prepare sequence for one layer: comm manager, registration pass, buffers, counter 0."""
    from basedxl_b200.utils import PatchParallelismCommManager

    cm = PatchParallelismCommManager(cfg)
    wrapper.set_comm_manager(cm)
    with torch.no_grad():
        wrapper(*first_call_args)
    assert wrapper.idx == 0 and len(cm.starts) == 1
    cm.create_buffer()
    wrapper.set_counter(0)
    return cm


def _pad64(t, dim):
    """Zero-pad ``dim`` to 64 channels (the tensor-core convolution takes C_in in multiples of 64;
    the fixtures use 32)."""
    pad = [0, 0] * (t.dim() - 1 - dim) + [0, 64 - t.shape[dim]]
    return torch.nn.functional.pad(t, pad)


def _boundary_nhwc(t):
    """[B, C, h, W] strip -> what the strip publishes, in the staging layout [2, B, 1, W, C]."""
    th = t.permute(0, 2, 3, 1)
    return torch.stack([th[:, :1], th[:, -1:]], dim=0).contiguous()


@pytest.mark.parametrize("tag", ["s1", "s2"])
@pytest.mark.parametrize("n", [2, 4])
def test_conv_wrapper_sync_and_displaced(golden_dir, tag, n):
    dev = cuda_or_skip()
    from basedxl_b200 import _lib, layers
    from basedxl_b200.modules.conv2d import BasedConv2dPP

    g = np.load(os.path.join(golden_dir, "conv2d_pp.npz"))
    x, xp, w, b = T(g[f"{tag}_x"]), T(g[f"{tag}_x_prev"]), T(g[f"{tag}_w"]), T(g[f"{tag}_b"])
    stride = int(g[f"{tag}_stride"])
    xz, xpz, wz = _pad64(x, 1), _pad64(xp, 1), _pad64(w, 1)
    conv = layers.Conv2d(64, w.shape[0], 3, stride=stride, padding=1)
    conv.load_state_dict({"weight": wz, "bias": b})
    conv = conv.half().to(dev)
    cl = lambda t: t.half().to(dev).contiguous(memory_format=torch.channels_last)
    xs, xps = torch.chunk(xz, n, 2), torch.chunk(xpz, n, 2)
    for idx in range(n):
        cfg = _cfg(n, idx)
        m = BasedConv2dPP(conv, cfg)
        cm = _wire(m, cfg, cl(xs[idx]))
        # ---- synchronous step: the gather delivers every strip's fresh boundary
        with torch.no_grad(), FakeAllGather([_boundary_nhwc(t).half().to(dev) for t in xs], idx) as ag:
            y = m(cl(xs[idx]))
        assert ag.calls == 1 and m.counter == 1
        assert_close(y, T(g[f"{tag}_n{n}_i{idx}_sync_y"]), what=f"conv wrapper sync {tag} n={n} i={idx}")
        # ---- displaced step: peers' ranges hold last step's boundaries
        m.set_counter(cfg.warmup_steps + 1)
        for j in range(n):
            cm.buffer_list[j][cm.starts[0] : cm.ends[0]].copy_(_boundary_nhwc(xps[j]).half().to(dev).reshape(-1))
        with torch.no_grad():
            y = m(cl(xs[idx]))
        _lib.device_status()
        assert_close(y, T(g[f"{tag}_n{n}_i{idx}_stale_y"]), what=f"conv wrapper displaced {tag} n={n} i={idx}")
        # what the layer published: its own fresh boundary, queued for the next gather
        assert cm.idx_queue == [0]
        pub = cm.own_slot(0).view(2, 2, 1, x.shape[3], 64).float().cpu()
        ref = T(g[f"{tag}_n{n}_i{idx}_published"])  # reference layout [2, B, C, 1, W], 32 channels
        assert torch.equal(pub[..., :32].permute(0, 1, 4, 2, 3), ref.half().float())
        assert float(pub[..., 32:].abs().max()) == 0.0


@pytest.mark.parametrize("n", [2, 4])
def test_groupnorm_wrapper_sync_and_displaced(golden_dir, n):
    dev = cuda_or_skip()
    from basedxl_b200 import _lib, layers
    from basedxl_b200.modules.groupnorm import BasedXLGroupNorm
    from oracle import patched_ops as po

    g = np.load(os.path.join(golden_dir, "groupnorm_pp.npz"))
    x, xp = T(g["x"]), T(g["x_prev"])
    groups, eps = int(g["groups"]), float(g["eps"])
    gn = layers.GroupNorm(groups, x.shape[1], eps=eps)
    gn.load_state_dict({"weight": T(g["gamma"]), "bias": T(g["beta"])})
    gn = gn.half().to(dev)
    cl = lambda t: t.half().to(dev).contiguous(memory_format=torch.channels_last)
    xs, xps = torch.chunk(x, n, 2), torch.chunk(xp, n, 2)
    # fp32 moments [2, B, G] of the fp16-rounded strips, as the kernels see them
    mom = lambda t: po.groupnorm_moments(t.half().float(), groups).reshape(-1).float().to(dev)
    for idx in range(n):
        cfg = _cfg(n, idx)
        m = BasedXLGroupNorm(gn, cfg)
        cm = _wire(m, cfg, cl(xs[idx]))
        # one fp32 moment occupies two fp16 staging elements
        assert cm.ends[0] - cm.starts[0] == 2 * 2 * groups * 2
        with torch.no_grad(), FakeAllGather([mom(t) for t in xs], idx) as ag:
            y = m(cl(xs[idx]))
        assert ag.calls == 1
        assert_close(y, T(g[f"n{n}_i{idx}_sync_y"]), what=f"gn wrapper sync n={n} i={idx}")
        m.set_counter(cfg.warmup_steps + 1)
        for j in range(n):
            cm.buffer_list[j][cm.starts[0] : cm.ends[0]].view(torch.float32).copy_(mom(xps[j]))
        with torch.no_grad():
            y = m(cl(xs[idx]))
        _lib.device_status()
        assert_close(y, T(g[f"n{n}_i{idx}_stale_y"]), what=f"gn wrapper displaced n={n} i={idx}")
        assert cm.idx_queue == [0]
        pub = cm.own_slot(0).reshape(-1).view(torch.float32).cpu()
        assert_close(pub, T(g[f"n{n}_i{idx}_published"]).reshape(-1), tol=1e-3, what="gn published moments")


@pytest.mark.parametrize("n", [2, 4])
def test_self_attention_wrapper_sync_and_displaced(golden_dir, n):
    dev = cuda_or_skip()
    from basedxl_b200 import _lib, layers
    from basedxl_b200.modules.attn import BasedXLSelfAttentionPP

    g = np.load(os.path.join(golden_dir, "attention_pp.npz"))
    x, xp = T(g["x"]), T(g["x_prev"])
    dim, heads = x.shape[2], int(g["heads"])
    attn = layers.Attention(dim, heads)
    wkv = T(g["wkv"])
    attn.load_state_dict({"to_q.weight": T(g["wq"]), "to_k.weight": wkv[:dim], "to_v.weight": wkv[dim:],
                          "to_out.0.weight": T(g["wo"]), "to_out.0.bias": T(g["bo"])})
    attn = attn.half().to(dev)
    d = lambda t: t.half().to(dev)
    xs, xps = torch.chunk(x, n, 1), torch.chunk(xp, n, 1)
    kv_of = lambda t: (t.half().float() @ wkv.half().float().t())  # [B, l, 2C]
    for idx in range(n):
        cfg = _cfg(n, idx)
        m = BasedXLSelfAttentionPP(attn, cfg)
        cm = _wire(m, cfg, d(xs[idx]))
        with torch.no_grad(), FakeAllGather([d(kv_of(t)) for t in xs], idx) as ag:
            y = m(d(xs[idx]))
        assert ag.calls == 1
        assert_close(y, T(g[f"n{n}_i{idx}_sync_y"]), tol=4e-3, what=f"attention wrapper sync n={n} i={idx}")
        m.set_counter(cfg.warmup_steps + 1)
        for j in range(n):
            cm.buffer_list[j][cm.starts[0] : cm.ends[0]].copy_(d(kv_of(xps[j])).reshape(-1))
        with torch.no_grad():
            y = m(d(xs[idx]))
        _lib.device_status()
        assert_close(y, T(g[f"n{n}_i{idx}_stale_y"]), tol=4e-3, what=f"attention wrapper displaced n={n} i={idx}")
        # the fused projection wrote this strip's fresh K/V straight into its own staging range
        assert cm.idx_queue == [0]
        assert_close(cm.own_slot(0), T(g[f"n{n}_i{idx}_published"]), what="published K/V")

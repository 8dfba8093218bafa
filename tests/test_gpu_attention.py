"""Flash-style attention kernel through the C ABI against the CPU oracle and the
fixtures produced by the reference module."""
import os

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import patched_ops as po
from tests._util import assert_close, cuda_or_skip, h16

pytestmark = pytest.mark.gpu
T = torch.from_numpy


def _ops():
    from basedxl_b200 import _lib, ops

    return _lib, ops


@pytest.mark.parametrize(
    "B,heads,Lq,Lslot,nslots",
    [
        (1, 1, 128, 128, 1),
        (2, 2, 128, 256, 1),
        (1, 2, 256, 128, 3),
        (2, 10, 77, 77, 1),       # ragged query and key tiles
        (2, 10, 512, 77, 1),      # cross-attention: 77 text tokens
        (2, 20, 1024, 128, 2),    # 160 work units on 148 SMs: the under-filled second round runs as half units
        (2, 20, 1024, 77, 1),     # the same count for cross-attention
        (1, 3, 200, 72, 4),       # ragged slots
        (2, 10, 512, 512, 8),     # benchmark shape at world size 8: L = 4096
        (2, 20, 256, 256, 4),     # 1280-level blocks, 4 strips
        (2, 10, 4096, 77, 1),     # 320 units of 256 queries: every CTA walks two or three units
        (2, 20, 1024, 256, 1),    # 160 units on 148 SMs: some CTAs walk two units of two tiles
        (4, 20, 384, 100, 2),     # 160 units, every second one with a single query tile, ragged slots
    ],
)
def test_attention_core_vs_oracle(B, heads, Lq, Lslot, nslots):
    dev = cuda_or_skip()
    _lib, ops = _ops()
    C = heads * 64
    gen = torch.Generator().manual_seed(B + heads + Lq + Lslot + nslots)
    q = h16(torch.randn(B, Lq, C, generator=gen))
    slots = [h16(torch.randn(B, Lslot, 2 * C, generator=gen)) for _ in range(nslots)]
    ref = po._sdpa_heads(q, torch.cat(slots, dim=1), heads)
    y = ops.attention(q.half().to(dev), [s.half().to(dev) for s in slots], heads)
    _lib.device_status()
    assert_close(y, ref, what=f"attention B{B} h{heads} Lq{Lq} Ls{Lslot} n{nslots}")


def test_attention_large_logits_are_stable():
    dev = cuda_or_skip()
    _lib, ops = _ops()
    gen = torch.Generator().manual_seed(1)
    q = h16(6 * torch.randn(1, 128, 64, generator=gen))
    kv = h16(torch.cat([6 * torch.randn(1, 384, 64, generator=gen), torch.randn(1, 384, 64, generator=gen)], dim=2))
    ref = po._sdpa_heads(q, kv, 1)
    y = ops.attention(q.half().to(dev), [kv.half().to(dev)], 1)
    _lib.device_status()
    assert torch.isfinite(y).all()
    assert_close(y, ref, tol=4e-3, what="attention with large logits")


@pytest.mark.parametrize("n", [2, 4])
def test_self_attention_block_golden(golden_dir, n):
    """Whole patched self-attention block (to_q, fused to_kv, slots read in place,
    to_out) assembled from the library's GEMM and attention kernels."""
    dev = cuda_or_skip()
    _lib, ops = _ops()
    g = np.load(os.path.join(golden_dir, "attention_pp.npz"))
    x, xp = T(g["x"]), T(g["x_prev"])
    wq, wkv, wo, bo, heads = T(g["wq"]), T(g["wkv"]), T(g["wo"]), T(g["bo"]), int(g["heads"])
    d = lambda t: t.half().to(dev)
    xs, xps = torch.chunk(x, n, 1), torch.chunk(xp, n, 1)
    kv_prev = [ops.linear(d(t), d(wkv)) for t in xps]
    kv_now = [ops.linear(d(t), d(wkv)) for t in xs]
    for i in range(n):
        q = ops.linear(d(xs[i]), d(wq))
        for tag, slots in (("stale", [kv_now[j] if j == i else kv_prev[j] for j in range(n)]), ("sync", kv_now), ("local", [kv_now[i]] * n)):
            o = ops.attention(q, slots, heads)
            y = ops.linear(o, d(wo), d(bo))
            assert_close(y, T(g[f"n{n}_i{i}_{tag}_y"]), tol=4e-3, what=f"self-attention block {tag}")
        assert_close(kv_now[i], T(g[f"n{n}_i{i}_published"]), what="published kv")
    _lib.device_status()


def test_cross_attention_block_golden(golden_dir):
    dev = cuda_or_skip()
    _lib, ops = _ops()
    g = np.load(os.path.join(golden_dir, "attention_pp.npz"))
    d = lambda t: t.half().to(dev)
    x, ctx = T(g["x"]), T(g["cross_ctx"])
    q = ops.linear(d(x), d(T(g["cross_wq"])))
    kv = ops.linear(d(ctx), d(T(g["cross_wkv"])))
    o = ops.attention(q, [kv], int(g["heads"]))
    y = ops.linear(o, d(T(g["cross_wo"])), d(T(g["cross_bo"])))
    _lib.device_status()
    assert_close(y, T(g["cross_y"]), tol=4e-3, what="cross-attention block")


def test_benchmark_shape_self_attention():
    """10 heads x 64 on 2 x 4096 x 640 tokens; stale K/V = current + N(0, 0.01); world sizes 2/4/8."""
    dev = cuda_or_skip()
    _lib, ops = _ops()
    gen = torch.Generator().manual_seed(0)
    C, heads, L = 640, 10, 4096
    kv = h16(torch.randn(2, L, 2 * C, generator=gen))
    kv_prev = h16(kv + 0.01 * torch.randn(2, L, 2 * C, generator=gen))
    q = h16(torch.randn(2, L, C, generator=gen))
    for n in (2, 4, 8):
        ls = L // n
        for i in sorted({0, n // 2, n - 1}):  # first, middle and last strip: the fresh slot in every position
            slots = [(kv if j == i else kv_prev)[:, j * ls : (j + 1) * ls] for j in range(n)]
            ref = po._sdpa_heads(q[:, i * ls : (i + 1) * ls], torch.cat(slots, dim=1), heads)
            y = ops.attention(q[:, i * ls : (i + 1) * ls].half().to(dev), [s.half().to(dev).contiguous() for s in slots], heads)
            _lib.device_status()
            assert_close(y, ref, what=f"self-attention strip {i} of n={n}")


@pytest.mark.parametrize("split", [1, 2, 4])
@pytest.mark.parametrize("B,heads,Lq,Lslot,nslots", [(1, 2, 256, 128, 4), (2, 3, 200, 72, 5), (1, 20, 256, 256, 4), (2, 10, 512, 77, 1), (1, 4, 640, 512, 2)])
def test_attention_kv_split_over_a_cluster(B, heads, Lq, Lslot, nslots, split):
    """The K/V range split over 1, 2 or 4 CTAs per query block and merged through distributed
    shared memory gives the same result (ragged tiles, several slots, odd query-tile counts)."""
    dev = cuda_or_skip()
    _lib, ops = _ops()
    if split > nslots * ((Lslot + 127) // 128):
        pytest.skip("more splits than key/value tiles")
    C = heads * 64
    gen = torch.Generator().manual_seed(B + heads + Lq + Lslot + nslots)
    q = h16(torch.randn(B, Lq, C, generator=gen))
    slots = [h16(torch.randn(B, Lslot, 2 * C, generator=gen) * (1.0 + 2.0 * i)) for i in range(nslots)]  # very different maxima per slot
    ref = po._sdpa_heads(q, torch.cat(slots, dim=1), heads)
    l = _lib.lib()
    _lib.check(l.bxl_debug_force_attn_split(split), l, kernels=0)
    try:
        y = ops.attention(q.half().to(dev), [s.half().to(dev) for s in slots], heads)
        _lib.device_status()
    finally:
        _lib.check(l.bxl_debug_force_attn_split(0), l, kernels=0)
    assert_close(y, ref, tol=3e-3, what=f"attention split={split}")


def test_self_attention_at_16384_tokens():
    """The 2048 x 2048 image's highest-resolution attention (L = 16384 keys): one head, the
    last of 4 strips (4096 queries), stale K/V in the other three slots."""
    dev = cuda_or_skip()
    _lib, ops = _ops()
    gen = torch.Generator().manual_seed(5)
    C, heads, L, n = 64, 1, 16384, 4
    kv = h16(torch.randn(1, L, 2 * C, generator=gen))
    kv_prev = h16(kv + 0.01 * torch.randn(1, L, 2 * C, generator=gen))
    q = h16(torch.randn(1, L, C, generator=gen))
    ls, i = L // n, n - 1
    slots = [(kv if j == i else kv_prev)[:, j * ls : (j + 1) * ls] for j in range(n)]
    ref = po._sdpa_heads(q[:, i * ls : (i + 1) * ls], torch.cat(slots, dim=1), heads)
    y = ops.attention(q[:, i * ls : (i + 1) * ls].half().to(dev), [s.half().to(dev).contiguous() for s in slots], heads)
    _lib.device_status()
    assert_close(y, ref, what="self-attention L=16384")

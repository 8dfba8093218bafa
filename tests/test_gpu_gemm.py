"""tcgen05 GEMM through the C ABI against the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import matmul as om
from tests._util import assert_close, cuda_or_skip, h16

pytestmark = pytest.mark.gpu


def _ops():
    from basedxl_b200 import _lib, ops

    return _lib, ops


@pytest.mark.parametrize(
    "M,K,N",
    [
        (128, 64, 128),      # one tile, one k-block
        (128, 256, 256),     # 256-wide tile
        (256, 320, 320),     # N not a tile multiple, K = 5 blocks
        (300, 200, 136),     # ragged M, K tail (200 = 3*64 + 8), ragged N
        (2, 320, 1280),      # the time-embedding linear
        (154, 2048, 640),    # cross-attention K/V projection of 2 x 77 tokens
        (1024, 2048, 1024),  # the reference unit test's kernel-reaching shape
        (8192, 640, 640),
        (2048, 1280, 10240),
    ],
)
@pytest.mark.parametrize("b_is_kn", [False, True])
def test_gemm_matches_oracle(M, K, N, b_is_kn):
    dev = cuda_or_skip()
    _lib, ops = _ops()
    g = torch.Generator().manual_seed(M * 7 + K * 3 + N)
    a = torch.randn(M, K, generator=g)
    w = torch.randn(N, K, generator=g) / K**0.5
    bias = torch.randn(N, generator=g)
    ref = h16(a) @ h16(w).t() + h16(bias)
    b_dev = (w.t().contiguous() if b_is_kn else w).half().to(dev)
    y = ops.gemm(a.half().to(dev), b_dev, bias=bias.half().to(dev), b_is_kn=b_is_kn)
    _lib.device_status()
    assert_close(y, ref, what=f"gemm {M}x{K}x{N} kn={b_is_kn}")


def test_gemm_residual_and_strided_output():
    dev = cuda_or_skip()
    _lib, ops = _ops()
    g = torch.Generator().manual_seed(5)
    M, K, N = 384, 640, 1280
    a, w, r = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g) / K**0.5, torch.randn(M, N, generator=g)
    ref = h16(a) @ h16(w).t() + h16(r)
    big = torch.zeros(M, 2 * N, device=dev, dtype=torch.float16)
    out = big[:, N:]  # row stride 2N: the K/V slot case
    ops.gemm(a.half().to(dev), w.half().to(dev), residual=r.half().to(dev), out=out)
    _lib.device_status()
    assert_close(out, ref, what="gemm residual/strided")
    assert float(big[:, :N].abs().max()) == 0.0


def test_gemm_reference_unit_test_tolerance():
    # tests/test_cascaded_lowp_matmul.py:26 of the reference: rtol 1e-3, atol 0.35 vs torch.matmul
    dev = cuda_or_skip()
    _lib, ops = _ops()
    g = torch.Generator().manual_seed(11)
    a, b = torch.randn(1024, 2048, generator=g).half(), torch.randn(2048, 1024, generator=g).half()
    y = ops.gemm(a.to(dev), b.to(dev), b_is_kn=True)
    _lib.device_status()
    expected = (a.float() @ b.float()).half()
    assert torch.allclose(y.cpu(), expected, rtol=1e-3, atol=0.35)


@pytest.mark.parametrize("M,K,N", [(8192, 640, 640), (8192, 640, 5120), (2048, 1280, 1280), (2048, 1280, 10240), (16384, 320, 320)])
def test_error_vs_fp64_no_worse_than_reference_kernel(M, K, N):
    """Method of the reference's error study: fp64 product as truth."""
    dev = cuda_or_skip()
    _lib, ops = _ops()
    torch.manual_seed(0)
    a32, b32 = torch.randn(M, K), torch.randn(K, N)
    a16, b16 = a32.half(), b32.half()
    # (i) fp16 operands: new kernel vs the optimistic model of the reference kernel
    exp16 = om.matmul_fp64(a16, b16)
    y16 = ops.gemm(a16.to(dev), b16.to(dev), b_is_kn=True).cpu()
    _lib.device_status()
    e_new = om.error_table(exp16, y16)
    sub = slice(0, 512)  # the model is slow: bound it on a row block
    e_ref = om.error_table(exp16[sub], om.matmul_fp16_accumulate(a16[sub], b16, block_k=32, model="block"))
    e_new_sub = om.error_table(exp16[sub], y16[sub])
    assert e_new_sub["l1"] <= e_ref["l1"] and e_new_sub["mse"] <= e_ref["mse"]
    assert e_new_sub["rel_median"] <= e_ref["rel_median"]
    # (ii) fp32 operands through the split-operand product: far below fp16-operand rounding
    exp32 = om.matmul_fp64(a32, b32)
    y32 = ops.gemm_split_f32(a32.to(dev), b32.to(dev)).cpu()
    _lib.device_status()
    e_split = om.error_table(exp32, y32)
    e_half = om.error_table(exp32, y16)
    assert e_split["max"] < 1e-3 * max(1.0, K**0.5)
    assert e_split["l1"] < 0.05 * e_half["l1"]  # tensor-core fp32 accumulation truncates; still ~50x below fp16 operands
    assert e_new["max"] < 0.35


def test_bad_arguments_are_rejected():
    dev = cuda_or_skip()
    _lib, ops = _ops()
    a = torch.zeros(128, 68, device=dev, dtype=torch.float16)  # K = 68: row stride not 16-byte granular
    w = torch.zeros(128, 68, device=dev, dtype=torch.float16)
    with pytest.raises(_lib.BxlError):
        ops.gemm(a, w)


@pytest.mark.parametrize("bn,split", [(32, 1), (64, 1), (96, 1), (160, 1), (192, 1), (224, 1), (256, 1), (64, 2), (128, 2), (128, 4), (256, 2), (256, 4)])
@pytest.mark.parametrize("M,K,N,b_is_kn", [(300, 1280, 1280, False), (1024, 640, 5120, False), (256, 5120, 1280, False), (384, 704, 640, True)])
def test_forced_tile_width_and_k_split(M, K, N, b_is_kn, bn, split):
    """Every tile width and cluster K split gives the same product (several tiles per
    cluster, so the exchange buffers are reused)."""
    dev = cuda_or_skip()
    _lib, ops = _ops()
    if b_is_kn and bn % 64:
        pytest.skip("[K,N] operands are loaded in 64-column boxes")
    g = torch.Generator().manual_seed(M + K + N + bn + split)
    a = torch.randn(M, K, generator=g)
    w = torch.randn(N, K, generator=g) / K**0.5
    bias, res = torch.randn(N, generator=g), torch.randn(M, N, generator=g)
    ref = h16(a) @ h16(w).t() + h16(bias) + h16(res)
    l = _lib.lib()
    _lib.check(l.bxl_debug_force_tiles(bn, split, -1), l, kernels=0)
    try:
        y = ops.gemm(a.half().to(dev), (w.t().contiguous() if b_is_kn else w).half().to(dev), bias=bias.half().to(dev),
                     residual=res.half().to(dev), b_is_kn=b_is_kn)
        _lib.device_status()
    finally:
        _lib.check(l.bxl_debug_force_tiles(0, 0, -1), l, kernels=0)
    assert_close(y, ref, what=f"gemm bn={bn} split={split}")


@pytest.mark.parametrize("order", [0, 1])
@pytest.mark.parametrize("bn,split", [(64, 1), (128, 2), (256, 1)])
def test_gemm_tile_order(order, bn, split):
    """Both orders in which output tiles are handed to the CTAs (rows first / columns first, the
    latter chosen by the library for activations that do not stay in L2) give the same result,
    row statistics of the output included."""
    dev = cuda_or_skip()
    _lib, ops = _ops()
    g = torch.Generator().manual_seed(5 + bn + split)
    M, K, N = 640, 320, 768
    a = torch.randn(M, K, generator=g)
    w = torch.randn(N, K, generator=g) / K**0.5
    bias = torch.randn(N, generator=g)
    ref = h16(a) @ h16(w).t() + h16(bias)
    l = _lib.lib()
    _lib.check(l.bxl_debug_force_tiles(bn, split, -1), l, kernels=0)
    _lib.check(l.bxl_debug_force_tile_order(order), l, kernels=0)
    try:
        y = ops.gemm(a.half().to(dev), w.half().to(dev), bias=bias.half().to(dev))
        y2, stats = ops.gemm_fused(a.half().to(dev), w.half().to(dev), bias=bias.half().to(dev), want_stats=True)
        _lib.device_status()
    finally:
        _lib.check(l.bxl_debug_force_tiles(0, 0, -1), l, kernels=0)
        _lib.check(l.bxl_debug_force_tile_order(-1), l, kernels=0)
    assert_close(y, ref, what=f"gemm order={order} bn={bn} split={split}")
    assert torch.equal(y, y2)
    mean, _ = stats.moments(N)
    assert_close(mean, y.float().cpu().mean(dim=1), tol=1e-4, what="row mean of the stored values")


@pytest.mark.parametrize("tokens", [8192, 4096, 2048, 1024, 512, 256])
def test_auto_tiling_on_every_per_rank_linear_shape(tokens):
    """The linear-layer shapes of the UNet at the token counts a rank sees with 1, 2, 4
    or 8 GPUs, each with the tiling the library chooses by itself (tile width, K split),
    against an fp32 matmul on the device."""
    dev = cuda_or_skip()
    _lib, ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(tokens)
    for (K, N) in [(640, 640), (640, 1280), (640, 5120), (2560, 640), (1280, 1280), (1280, 2560), (1280, 10240), (5120, 1280),
                   (2048, 1280), (2048, 2560), (320, 1280), (2816, 1280)]:
        a = torch.randn(tokens, K, device=dev, generator=g).half()
        w = (torch.randn(N, K, device=dev, generator=g) / K**0.5).half()
        bias = torch.randn(N, device=dev, generator=g).half()
        y = ops.gemm(a, w, bias=bias)
        ref = a.float() @ w.float().t() + bias.float()
        err = float((y.float() - ref).norm() / ref.norm())
        assert torch.isfinite(y).all() and err < 2e-3, f"tokens={tokens} K={K} N={N}: rel-L2 {err:.3e}"
    _lib.device_status()


@pytest.mark.parametrize("pair", [-1, 1])
@pytest.mark.parametrize("M,K,F", [(300, 640, 2560), (2048, 1280, 5120), (64, 128, 512)])
def test_gemm_with_fused_geglu(M, K, F, pair):
    dev = cuda_or_skip()
    _lib, ops = _ops()
    l = _lib.lib()
    g = torch.Generator().manual_seed(M + F)
    x = h16(torch.randn(M, K, generator=g))
    w = h16(torch.randn(2 * F, K, generator=g) / K**0.5)
    b = h16(torch.randn(2 * F, generator=g))
    h = x @ w.t() + b
    ref = h[:, :F] * torch.nn.functional.gelu(h[:, F:])
    wi, bi = ops.geglu_interleave(w.half().to(dev), b.half().to(dev))
    _lib.check(l.bxl_debug_force_tiles(0, 1 if pair == 1 else 0, pair), l, kernels=0)
    try:
        y = ops.gemm_geglu(x.half().to(dev), wi, bi)
        _lib.device_status()
    finally:
        _lib.check(l.bxl_debug_force_tiles(0, 0, -1), l, kernels=0)
    assert y.shape == (M, F)
    assert_close(y, ref, what=f"gemm+geglu {M}x{K}x{F}")


@pytest.mark.parametrize("pair", [-1, 1])
@pytest.mark.parametrize("M,K,C", [(300, 640, 640), (2048, 1280, 1280), (512, 128, 128)])
def test_gemm_with_two_destinations(M, K, C, pair):
    """q | k|v projection in one launch, k|v into a wider (strided) destination."""
    dev = cuda_or_skip()
    _lib, ops = _ops()
    l = _lib.lib()
    g = torch.Generator().manual_seed(M + C)
    x = h16(torch.randn(M, K, generator=g))
    w = h16(torch.randn(3 * C, K, generator=g) / K**0.5)
    ref = x @ w.t()
    slot = torch.zeros(M, 2 * C + 64, device=dev, dtype=torch.float16)
    _lib.check(l.bxl_debug_force_tiles(0, 1 if pair == 1 else 0, pair), l, kernels=0)
    try:
        q, _ = ops.gemm_dual(x.half().to(dev), w.half().to(dev), C, out2=slot[:, : 2 * C])
        _lib.device_status()
    finally:
        _lib.check(l.bxl_debug_force_tiles(0, 0, -1), l, kernels=0)
    assert_close(q, ref[:, :C], what="q part")
    assert_close(slot[:, : 2 * C], ref[:, C:], what="k|v part")
    assert float(slot[:, 2 * C :].abs().max()) == 0.0


@pytest.mark.parametrize("bn", [128, 256])
@pytest.mark.parametrize("M,K,N", [(300, 320, 384), (2048, 1280, 1280)])
def test_cta_pair_tiles(M, K, N, bn):
    """256-row tiles computed by two CTAs with one MMA stream (cta_group::2), each CTA staging
    half of the B tile and reporting its copies to the leader's barrier."""
    dev = cuda_or_skip()
    _lib, ops = _ops()
    g = torch.Generator().manual_seed(M + bn)
    a = torch.randn(M, K, generator=g)
    w = torch.randn(N, K, generator=g) / K**0.5
    bias = torch.randn(N, generator=g)
    ref = h16(a) @ h16(w).t() + h16(bias)
    l = _lib.lib()
    _lib.check(l.bxl_debug_force_tiles(bn, 1, 1), l, kernels=0)
    try:
        y = ops.gemm(a.half().to(dev), w.half().to(dev), bias=bias.half().to(dev))
        _lib.device_status()
    finally:
        _lib.check(l.bxl_debug_force_tiles(0, 0, -1), l, kernels=0)
    assert_close(y, ref, what=f"pair gemm bn={bn}")


def test_static_weights_mode_chain():
    """With the static-weights promise the B copies of a GEMM start before the kernel waits for
    its predecessor; a chain in which every A is the previous output must still be exact."""
    dev = cuda_or_skip()
    _lib, ops = _ops()
    g = torch.Generator().manual_seed(11)
    x = h16(torch.randn(512, 640, generator=g))
    ws = [h16(torch.randn(640, 640, generator=g) / 640**0.5) for _ in range(4)]
    ref = x
    for w in ws:
        ref = h16(ref @ w.t())
    l = _lib.lib()
    xd, wd = x.half().to(dev), [w.half().to(dev) for w in ws]
    torch.cuda.synchronize()
    _lib.check(l.bxl_set_static_weights(1), l, kernels=0)
    try:
        y = xd
        for w in wd:
            y = ops.gemm(y, w)
        _lib.device_status()
    finally:
        _lib.check(l.bxl_set_static_weights(0), l, kernels=0)
    assert_close(y, ref, what="gemm chain with static weights")


# ---------------------------------------------------------------------------------------------
# LayerNorm folded into the consumer GEMM, row statistics emitted by the producer GEMM
# ---------------------------------------------------------------------------------------------
def _ln_case(M, K, seed):
    g = torch.Generator().manual_seed(seed)
    x = h16(torch.randn(M, K, generator=g) * 1.7 + 0.4)
    gamma, beta = h16(1.0 + 0.2 * torch.randn(K, generator=g)), h16(0.2 * torch.randn(K, generator=g))
    return g, x, gamma, beta


@pytest.mark.parametrize("bn,split,pair", [(0, 0, -1), (64, 1, 0), (128, 2, 0), (256, 4, 0), (128, 1, 1), (160, 1, 0)])
@pytest.mark.parametrize("M,K,N", [(300, 1280, 1280), (1024, 640, 640)])
def test_row_statistics_of_the_output(M, K, N, bn, split, pair):
    """Producer side: per-row (sum, sum of squares) partials of the fp16 output, whatever the tiling."""
    dev = cuda_or_skip()
    _lib, ops = _ops()
    g, a, _, _ = _ln_case(M, K, M + N + bn + split)
    w = h16(torch.randn(N, K, generator=g) / K**0.5)
    bias, res = h16(torch.randn(N, generator=g)), h16(torch.randn(M, N, generator=g))
    l = _lib.lib()
    _lib.check(l.bxl_debug_force_tiles(bn, split, pair), l, kernels=0)
    try:
        y, st = ops.gemm_fused(a.half().to(dev), w.half().to(dev), bias=bias.half().to(dev), residual=res.half().to(dev), want_stats=True)
        _lib.device_status()
    finally:
        _lib.check(l.bxl_debug_force_tiles(0, 0, -1), l, kernels=0)
    assert_close(y, a @ w.t() + bias + res, what="gemm with statistics")
    mean, var = st.moments(N)
    yf = y.float().cpu()
    assert_close(mean, yf.mean(dim=1), tol=1e-4, what="row mean of the stored values")
    assert_close(var, yf.var(dim=1, unbiased=False), tol=1e-3, what="row variance of the stored values")


@pytest.mark.parametrize("bn,split,pair", [(0, 0, -1), (96, 1, 0), (128, 2, 0), (256, 4, 0), (128, 1, 1)])
@pytest.mark.parametrize("kind", ["plain", "dual", "geglu"])
def test_layernorm_folded_into_gemm(kind, bn, split, pair):
    """Linear(LayerNorm(x)) computed from the un-normalised x: weight pre-scaled by the gain,
    rstd * (acc - mean * colsum) + (W beta + b) in the epilogue; the three epilogue forms that
    follow a LayerNorm in a transformer block."""
    dev = cuda_or_skip()
    _lib, ops = _ops()
    M, K, N = 520, 1280, 1280
    g, x, gamma, beta = _ln_case(M, K, 17 + bn + split)
    # x itself is produced by a GEMM with a residual, which also emits its row statistics
    a0 = h16(torch.randn(M, 320, generator=g))
    w0 = h16(torch.randn(K, 320, generator=g) / 320**0.5)
    xd, st = ops.gemm_fused(a0.half().to(dev), w0.half().to(dev), residual=x.half().to(dev), want_stats=True)
    x_ref = xd.float().cpu()  # the fp16 values the consumer reads
    n_w = 2 * N if kind == "geglu" else (3 * N if kind == "dual" else N)
    w = h16(torch.randn(n_w, K, generator=g) / K**0.5)
    b = h16(0.3 * torch.randn(n_w, generator=g))
    ln = torch.nn.functional.layer_norm(x_ref, (K,), gamma, beta, 1e-5)
    l = _lib.lib()
    _lib.check(l.bxl_debug_force_tiles(bn, split, pair), l, kernels=0)
    try:
        if kind == "geglu":
            wi, bi = ops.geglu_interleave(w.half().to(dev), b.half().to(dev))
            fold = ops.FoldedLayerNorm(wi, bi, gamma.half().to(dev), beta.half().to(dev), 1e-5)
            y = ops.gemm_fused(xd, None, geglu=True, ln=(st, fold))
            h = ln @ w.t() + b
            ref = h[:, :N] * torch.nn.functional.gelu(h[:, N:])
        elif kind == "dual":
            fold = ops.FoldedLayerNorm(w.half().to(dev), b.half().to(dev), gamma.half().to(dev), beta.half().to(dev), 1e-5)
            big = torch.zeros(M, 3 * N, device=dev, dtype=torch.float16)
            q, kv = ops.gemm_fused(xd, None, n_split=N, out2=big[:, N:], ln=(st, fold))
            y = torch.cat([q, big[:, N:]], dim=1)
            ref = ln @ w.t() + b
        else:
            fold = ops.FoldedLayerNorm(w.half().to(dev), b.half().to(dev), gamma.half().to(dev), beta.half().to(dev), 1e-5)
            y = ops.gemm_fused(xd, None, ln=(st, fold))
            ref = ln @ w.t() + b
        _lib.device_status()
    finally:
        _lib.check(l.bxl_debug_force_tiles(0, 0, -1), l, kernels=0)
    assert_close(y, ref, what=f"LayerNorm folded into {kind} GEMM (bn={bn} split={split} pair={pair})")

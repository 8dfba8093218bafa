"""Host-side arithmetic of the folded LayerNorm (no GPU): the weight / column-sum / bias triple that
``ops.FoldedLayerNorm`` prepares, combined the way the GEMM epilogue combines it, equals
Linear(LayerNorm(x)); and the row moments recovered from per-tile partial sums equal the moments
of the row."""
import torch

from basedxl_b200 import ops


def test_folded_layernorm_identity():
    g = torch.Generator().manual_seed(0)
    M, K, N = 37, 96, 64
    x = torch.randn(M, K, generator=g) * 1.5 + 0.7
    w, b = torch.randn(N, K, generator=g) / K**0.5, torch.randn(N, generator=g)
    gamma, beta = 1 + 0.3 * torch.randn(K, generator=g), 0.2 * torch.randn(K, generator=g)
    fold = ops.FoldedLayerNorm(w, b, gamma, beta, 1e-5)
    mean = x.mean(dim=1, keepdim=True)
    rstd = (x.var(dim=1, unbiased=False, keepdim=True) + 1e-5).rsqrt()
    acc = x @ fold.weight.t()                      # what the tensor core accumulates: UN-normalised rows
    y = rstd * (acc - mean * fold.colsum[None, :]) + fold.bias_f32[None, :]
    ref = torch.nn.functional.linear(torch.nn.functional.layer_norm(x, (K,), gamma, beta, 1e-5), w, b)
    assert torch.allclose(y, ref, atol=1e-4, rtol=1e-4)
    # no gain / shift (elementwise_affine=False) and no bias
    fold = ops.FoldedLayerNorm(w, None, None, None, 1e-5)
    y = rstd * (x @ fold.weight.t() - mean * fold.colsum[None, :]) + fold.bias_f32[None, :]
    ref = torch.nn.functional.linear(torch.nn.functional.layer_norm(x, (K,), None, None, 1e-5), w)
    assert torch.allclose(y, ref, atol=1e-4, rtol=1e-4)


def test_row_moments_from_partial_sums():
    g = torch.Generator().manual_seed(1)
    M, N, parts = 19, 160, 5
    y = torch.randn(M, N, generator=g) * 2 - 0.3
    tiles = y.view(M, parts, N // parts)
    buf = torch.zeros(M, 8, 2)
    buf[:, :parts, 0] = tiles.sum(dim=2)
    buf[:, :parts, 1] = (tiles**2).sum(dim=2)
    st = ops.RowStats(buf.view(-1)[: M * 8 * 2].view(M, 8, 2)[:, :parts].contiguous(), parts)
    mean, var = st.moments(N)
    assert torch.allclose(mean, y.mean(dim=1), atol=1e-5)
    assert torch.allclose(var, y.var(dim=1, unbiased=False), atol=1e-4)

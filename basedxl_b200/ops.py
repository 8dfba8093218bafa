"""Tensor-level wrappers over the C ABI: torch tensors in, torch tensors out.

PyTorch is used for device memory and streams only; every function here
launches kernels of libbasedxl_b200 on the current CUDA stream.  Activations
are NHWC-contiguous ``[B, H, W, C]`` fp16 tensors or ``[..., C]`` matrices.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib

_vp = C.c_void_p


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _req(cond: bool, msg: str) -> None:
    if not cond:
        raise ValueError(msg)


def _f16_cuda(t: torch.Tensor, name: str) -> None:
    _req(t.is_cuda and t.dtype == torch.float16, f"{name}: expected a CUDA fp16 tensor, got {t.device} {t.dtype}")


# --------------------------------------------------------------------------- matmul
def gemm(a, b, bias=None, residual=None, out=None, b_is_kn=False, out_f32=False):
    """``a[M,K] @ B`` with ``b`` given as [N,K] (default) or [K,N] (``b_is_kn``)."""
    _f16_cuda(a, "a"), _f16_cuda(b, "b")
    _req(a.dim() == 2 and b.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1, "gemm: 2-D row-major operands")
    M, K = a.shape
    N = b.shape[1] if b_is_kn else b.shape[0]
    _req((b.shape[0] if b_is_kn else b.shape[1]) == K, "gemm: inner dimensions differ")
    if out is None:
        out = torch.empty((M, N), device=a.device, dtype=torch.float32 if out_f32 else torch.float16)
    _req(out.shape == (M, N) and out.stride(1) == 1, "gemm: bad output")
    if residual is not None:
        _req(residual.shape == (M, N) and residual.stride(1) == 1, "gemm: bad residual")
    l = _lib.lib()
    _lib.check(
        l.bxl_gemm_f16(
            _p(a), a.stride(0), _p(b), b.stride(0), int(b_is_kn), _p(bias), _p(residual),
            0 if residual is None else residual.stride(0), _p(out), out.stride(0), int(out_f32), M, N, K, _stream(),
        ),
        l,
    )
    return out


def linear(x, weight, bias=None, residual=None):
    """``x[..., K] @ weight[N, K]^T (+ bias) (+ residual[..., N])``."""
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    r2 = None if residual is None else residual.reshape(-1, weight.shape[0])
    y = gemm(x2, weight, bias=bias, residual=r2)
    return y.view(*lead, weight.shape[0])


def gemm_dual(a, w, n1: int, bias=None, out1=None, out2=None):
    """``a @ w^T (+ bias)`` with the first ``n1`` output columns written to ``out1`` and the
    rest to ``out2`` (each with its own row stride)."""
    _f16_cuda(a, "a"), _f16_cuda(w, "w")
    M, K = a.shape
    N = w.shape[0]
    _req(w.shape[1] == K and a.stride(1) == 1 and w.stride(1) == 1, "gemm_dual: bad operands")
    if out1 is None:
        out1 = torch.empty((M, n1), device=a.device, dtype=torch.float16)
    if out2 is None:
        out2 = torch.empty((M, N - n1), device=a.device, dtype=torch.float16)
    _req(out1.shape == (M, n1) and out2.shape == (M, N - n1) and out1.stride(1) == 1 and out2.stride(1) == 1, "gemm_dual: bad outputs")
    l = _lib.lib()
    _lib.check(
        l.bxl_gemm_dual_f16(_p(a), a.stride(0), _p(w), w.stride(0), _p(bias), _p(out1), out1.stride(0), n1, _p(out2),
                            out2.stride(0), M, N, K, _stream()),
        l,
    )
    return out1, out2


def geglu_interleave(weight: torch.Tensor, bias: torch.Tensor | None):
    """Reorder the rows of a GEGLU projection ([2F, K]: F value rows then F gate rows) into
    groups of 16 value rows followed by their 16 gate rows, the order ``gemm_geglu`` expects."""
    F2 = weight.shape[0]
    F = F2 // 2
    assert F % 16 == 0
    idx = torch.arange(F, device=weight.device).view(F // 16, 16)
    perm = torch.cat([idx, idx + F], dim=1).reshape(-1)
    return weight[perm].contiguous(), (None if bias is None else bias[perm].contiguous())


def gemm_geglu(a, w_interleaved, bias_interleaved=None, out=None):
    """``geglu(a @ W^T + b)`` in one kernel; ``w_interleaved`` from :func:`geglu_interleave`."""
    _f16_cuda(a, "a"), _f16_cuda(w_interleaved, "w")
    M, K = a.shape
    N = w_interleaved.shape[0]
    _req(w_interleaved.shape[1] == K and a.stride(1) == 1 and w_interleaved.stride(1) == 1, "gemm_geglu: bad operands")
    if out is None:
        out = torch.empty((M, N // 2), device=a.device, dtype=torch.float16)
    l = _lib.lib()
    _lib.check(
        l.bxl_gemm_geglu_f16(_p(a), a.stride(0), _p(w_interleaved), w_interleaved.stride(0), _p(bias_interleaved), _p(out),
                             out.stride(0), M, N, K, _stream()),
        l,
    )
    return out


class RowStats:
    """Per-row partial sums (sum, sum of squares) of a matrix a GEMM has just written:
    ``buf[m, part, 2]`` fp32 with ``parts`` partials per row.  Input of a LayerNorm folded into
    the next GEMM."""

    __slots__ = ("buf", "parts")

    def __init__(self, buf: torch.Tensor, parts: int):
        self.buf, self.parts = buf, parts

    def moments(self, k: int):
        """(mean, variance) per row, for checking."""
        s = self.buf[:, : self.parts].sum(dim=1)
        mean = s[:, 0] / k
        return mean, s[:, 1] / k - mean * mean


class FoldedLayerNorm:
    """What a GEMM needs to apply ``Linear(LayerNorm(x))`` to the UN-normalised ``x``: the weight
    with the LayerNorm gain multiplied into its columns, its row sums, and the bias W beta + b."""

    __slots__ = ("weight", "colsum", "bias_f32", "eps")

    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None, gamma: torch.Tensor | None, beta: torch.Tensor | None, eps: float):
        w32 = weight.detach().float()
        wg = (w32 * gamma.detach().float()[None, :]) if gamma is not None else w32
        self.weight = wg.to(weight.dtype).contiguous()
        # sums of the ROUNDED weights: the mean term then cancels exactly against the accumulator
        self.colsum = self.weight.float().sum(dim=1).contiguous()
        b = torch.zeros(weight.shape[0], device=weight.device, dtype=torch.float32) if bias is None else bias.detach().float().clone()
        if beta is not None:
            b += w32 @ beta.detach().float()
        self.bias_f32 = b.contiguous()
        self.eps = float(eps)


_MAX_STAT_PARTS = 256


def gemm_fused(a, w, *, bias=None, bias_f32=None, residual=None, out=None, out2=None, n_split=0, geglu=False,
               ln: tuple | None = None, want_stats=False):
    """``a[M,K] @ w[N,K]^T`` through the general entry point.  ``ln = (RowStats of a, FoldedLayerNorm)``
    folds a LayerNorm over ``a``'s rows into the product (``w`` is then ignored in favour of the
    folded weight); ``want_stats`` returns the RowStats of the fp16 output as a second value."""
    _f16_cuda(a, "a")
    M, K = a.shape
    fold = None
    if ln is not None:
        stats_in, fold = ln
        w, bias, bias_f32 = fold.weight, None, fold.bias_f32
        _req(stats_in.buf.shape[0] == M and stats_in.buf.is_contiguous(), "gemm_fused: row statistics do not match a")
    _f16_cuda(w, "w")
    N = w.shape[0]
    _req(a.dim() == 2 and w.shape[1] == K and a.stride(1) == 1 and w.stride(1) == 1, "gemm_fused: bad operands")
    n_out = N // 2 if geglu else (n_split if n_split else N)
    if out is None:
        out = torch.empty((M, n_out), device=a.device, dtype=torch.float16)
    _req(out.shape == (M, n_out) and out.stride(1) == 1, "gemm_fused: bad output")
    if n_split:
        if out2 is None:
            out2 = torch.empty((M, N - n_split), device=a.device, dtype=torch.float16)
        _req(out2.shape == (M, N - n_split) and out2.stride(1) == 1, "gemm_fused: bad second output")
    if residual is not None:
        _req(residual.shape == (M, N) and residual.stride(1) == 1, "gemm_fused: bad residual")
    args = _lib.GemmFusedArgs()
    args.A, args.lda, args.B, args.ldb = _p(a), a.stride(0), _p(w), w.stride(0)
    args.bias, args.bias_f32 = _p(bias), _p(bias_f32)
    args.residual, args.ldr = _p(residual), 0 if residual is None else residual.stride(0)
    args.C, args.ldc = _p(out), out.stride(0)
    args.C2, args.ldc2, args.n_split = (_p(out2), out2.stride(0), n_split) if n_split else (None, 0, 0)
    args.geglu = int(geglu)
    if ln is not None:
        args.ln_partials, args.ln_parts = _p(stats_in.buf), stats_in.parts
        args.ln_colsum, args.ln_eps = _p(fold.colsum), fold.eps
    stats = None
    if want_stats:
        buf = torch.empty((M, min(_MAX_STAT_PARTS, 4 * max(1, N // 32)), 2), device=a.device, dtype=torch.float32)
        args.row_stats, args.row_stats_capacity = _p(buf), buf.numel()
    args.M, args.N, args.K = M, N, K
    parts = C.c_int(0)
    l = _lib.lib()
    _lib.check(l.bxl_gemm_fused_f16(C.byref(args), C.byref(parts), _stream()), l)
    if want_stats:
        # the partials of row m live at buf.view(-1)[m * parts * 2 ...]: re-view with the real count
        stats = RowStats(buf.view(-1)[: M * parts.value * 2].view(M, parts.value, 2), parts.value)
    if n_split:
        return (out, out2, stats) if want_stats else (out, out2)
    return (out, stats) if want_stats else out


def gemm_split_f32(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """fp32 ``a[M,K] @ b[K,N]`` through the split-operand tensor-core product."""
    _req(a.is_cuda and a.dtype == torch.float32 and b.dtype == torch.float32, "gemm_split_f32: CUDA fp32 operands")
    a, b = a.contiguous(), b.contiguous()
    M, K = a.shape
    N = b.shape[1]
    l = _lib.lib()
    ws_bytes = l.bxl_gemm_split_workspace_bytes(M, N, K)
    ws = torch.empty(ws_bytes, device=a.device, dtype=torch.uint8)
    out = torch.empty((M, N), device=a.device, dtype=torch.float32)
    _lib.check(l.bxl_gemm_split_f32(_p(a), _p(b), _p(out), M, N, K, _p(ws), ws_bytes, _stream()), l, kernels=3)
    return out


# --------------------------------------------------------------------------- convolution
def conv_weight_pack(w_oihw: torch.Tensor) -> torch.Tensor:
    _f16_cuda(w_oihw, "weight")
    co, ci, kh, kw = w_oihw.shape
    _req(kh == 3 and kw == 3, "conv_weight_pack: 3x3 kernels only")
    w = w_oihw.contiguous()
    out = torch.empty((co, 9 * ci), device=w.device, dtype=torch.float16)
    l = _lib.lib()
    _lib.check(l.bxl_conv_weight_pack_f16(_p(w), _p(out), co, ci, _stream()), l)
    return out


def _halo_args(x, top, bot):
    B, H, W, Ci = x.shape
    halo_stride = 0
    for h in (top, bot):
        if h is not None:
            _f16_cuda(h, "halo")
            _req(h.shape == (B, 1, W, Ci) and h.stride(3) == 1 and h.stride(2) == Ci, "halo rows must be [B,1,W,C]")
            _req(halo_stride in (0, h.stride(0)), "top and bottom halo must share one image stride")
            halo_stride = h.stride(0)
    return halo_stride


def _nhwc_strip(x, name):
    _f16_cuda(x, name)
    _req(x.dim() == 4, f"{name}: expected [B,H,W,C]")
    B, H, W, Ci = x.shape
    _req(x.stride(3) == 1 and x.stride(2) == Ci and x.stride(1) == W * Ci, f"{name}: rows of one image must be NHWC-contiguous")


def conv3x3(x, w_packed, bias=None, stride=1, top=None, bot=None, bias_rows=None, residual=None, out=None):
    """3x3 / pad 1 convolution of an NHWC strip with optional halo rows."""
    _nhwc_strip(x, "x")
    B, H, W, Ci = x.shape
    Co = w_packed.shape[0]
    _req(w_packed.shape[1] == 9 * Ci, "conv3x3: packed weight does not match C_in")
    halo_stride = _halo_args(x, top, bot)
    if out is None:
        out = torch.empty((B, H // stride, W // stride, Co), device=x.device, dtype=torch.float16)
    _req(out.is_contiguous(), "conv3x3: output must be contiguous")
    if residual is not None:
        _req(residual.shape == out.shape and residual.is_contiguous(), "conv3x3: bad residual")
    bias_rows_stride = 0
    if bias_rows is not None:
        # [B, C_out], possibly a column slice of a wider matrix (rows bias_rows.stride(0) apart)
        _req(bias_rows.shape == (B, Co) and bias_rows.stride(1) == 1 and bias_rows.dtype == torch.float16,
             "conv3x3: bias_rows must be fp16 [B,C_out] with unit column stride")
        bias_rows_stride = bias_rows.stride(0) if B > 1 else Co
    l = _lib.lib()
    if Ci % 64 == 0 and Co % 4 == 0:
        _lib.check(
            l.bxl_conv3x3_halo_f16(
                _p(x), x.stride(0), _p(top), _p(bot), halo_stride, _p(w_packed), _p(bias), _p(bias_rows), bias_rows_stride,
                _p(residual), _p(out), B, Ci, Co, H, W, stride, _stream(),
            ),
            l,
        )
    else:
        _req(stride == 1 and bias_rows is None and residual is None, "conv3x3: thin convolutions are plain stride-1")
        _lib.check(
            l.bxl_conv3x3_direct_f16(
                _p(x), x.stride(0), _p(top), _p(bot), halo_stride, _p(w_packed), _p(bias), _p(out), B, Ci, Co, H, W, _stream()
            ),
            l,
        )
    return out


def halo_pack(x, pad=1, out=None):
    """``[2, B, pad, W, C]``: the strip's first and last ``pad`` rows."""
    _nhwc_strip(x, "x")
    B, H, W, Ci = x.shape
    if out is None:
        out = torch.empty((2, B, pad, W, Ci), device=x.device, dtype=torch.float16)
    _req(out.numel() == 2 * B * pad * W * Ci and out.is_contiguous(), "halo_pack: bad output")
    l = _lib.lib()
    _lib.check(l.bxl_halo_pack_f16(_p(x), x.stride(0), _p(out), B, H, W, Ci, pad, _stream()), l)
    return out


# --------------------------------------------------------------------------- GroupNorm
_gn_scratch: dict[int, torch.Tensor] = {}


def _scratch(device, nbytes: int) -> torch.Tensor:
    """Per-device scratch for the GroupNorm statistics kernel (zeroed once; the
    kernel leaves its ticket word at zero).  Calls that share it must be ordered
    on one stream, which holds for the single compute stream the library runs on."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    t = _gn_scratch.get(key)
    if t is None or t.numel() < nbytes:
        t = torch.zeros(max(nbytes, 1 << 20), device=device, dtype=torch.uint8)
        _gn_scratch[key] = t
    return t


def groupnorm_stats(x, groups: int, out=None):
    """fp32 moments ``[2, B, G]`` of an NHWC strip (mean, mean of squares per group)."""
    _nhwc_strip(x, "x")
    B, H, W, Ci = x.shape
    if out is None:
        out = torch.empty((2, B, groups), device=x.device, dtype=torch.float32)
    _req(out.dtype == torch.float32 and out.numel() == 2 * B * groups and out.is_contiguous(), "groupnorm_stats: bad output")
    l = _lib.lib()
    nbytes = l.bxl_groupnorm_scratch_bytes(B, groups)
    s = _scratch(x.device, nbytes)
    _lib.check(l.bxl_groupnorm_stats_f16(_p(x), x.stride(0), B, H * W, Ci, groups, _p(out), _p(s), s.numel(), _stream()), l)
    return out


MODE_LOCAL, MODE_SYNC, MODE_STALE = 0, 1, 2


def groupnorm_apply(x, groups, eps, gamma, beta, fresh, peers=None, own=0, mode=MODE_LOCAL, silu=False, out=None):
    _nhwc_strip(x, "x")
    B, H, W, Ci = x.shape
    if out is None:
        out = torch.empty_like(x)
    _req(out.shape == x.shape and out.stride() == x.stride(), "groupnorm_apply: output must match x")
    n = 0 if peers is None else len(peers)
    arr = (_vp * max(n, 1))(*[(_p(t) if t is not None else None) for t in (peers or [None])])
    l = _lib.lib()
    _lib.check(
        l.bxl_groupnorm_apply_f16(
            _p(x), _p(out), x.stride(0), B, H * W, Ci, groups, _p(fresh), arr, n, own, mode, float(eps), _p(gamma), _p(beta),
            int(silu), _stream(),
        ),
        l,
    )
    return out


def groupnorm_fused(x, groups, eps, gamma, beta, peers=None, own=0, mode=MODE_LOCAL, silu=False, fresh_out=None, halo_out=None, out=None):
    """GroupNorm (+ SiLU) of an NHWC strip in one launch (``MODE_LOCAL`` or ``MODE_STALE``).
    ``fresh_out`` ([2, B, G] fp32) receives the strip's moments - it may be the strip's own entry of
    ``peers``; ``halo_out`` ([2, B, 1, W, C] fp16) receives the first and last row of the result."""
    _nhwc_strip(x, "x")
    _req(mode in (MODE_LOCAL, MODE_STALE), "groupnorm_fused: local or stale moments only")
    B, H, W, Ci = x.shape
    if out is None:
        out = torch.empty_like(x)
    _req(out.shape == x.shape and out.stride() == x.stride(), "groupnorm_fused: output must match x")
    if fresh_out is not None:
        _req(fresh_out.dtype == torch.float32 and fresh_out.numel() == 2 * B * groups and fresh_out.is_contiguous(), "groupnorm_fused: bad fresh_out")
    if halo_out is not None:
        _f16_cuda(halo_out, "halo_out")
        _req(halo_out.numel() == 2 * B * W * Ci and halo_out.is_contiguous(), "groupnorm_fused: bad halo_out")
    n = 0 if peers is None or mode == MODE_LOCAL else len(peers)
    arr = (_vp * max(n, 1))(*([_p(t) for t in peers] if n else [None]))
    l = _lib.lib()
    _lib.check(
        l.bxl_groupnorm_fused_f16(_p(x), _p(out), x.stride(0), B, H, W, Ci, groups, _p(fresh_out), arr, n, own, mode, float(eps),
                                  _p(gamma), _p(beta), int(silu), _p(halo_out), _stream()),
        l,
    )
    return out


# --------------------------------------------------------------------------- attention
def attention(q, kv_slots, heads: int, scale: float | None = None, out=None):
    """``q [B, L_q, C]`` against the concatenation of ``kv_slots`` (each
    ``[B, L_slot, 2C]``: K then V along the last axis).  Head dim 64."""
    _f16_cuda(q, "q")
    B, Lq, Cq = q.shape
    _req(Cq == heads * 64 and q.stride(2) == 1, "attention: head dimension must be 64")
    s0 = kv_slots[0]
    Bk, Ls, C2 = s0.shape
    _req(Bk == B and C2 == 2 * Cq, "attention: slot shape does not match q")
    for s in kv_slots:
        _f16_cuda(s, "kv slot")
        _req(s.shape == s0.shape and s.stride() == s0.stride() and s.stride(2) == 1, "attention: slots must share shape and strides")
    if out is None:
        out = torch.empty((B, Lq, Cq), device=q.device, dtype=torch.float16)
    if scale is None:
        scale = 64**-0.5
    arr = (_vp * len(kv_slots))(*[_p(s) for s in kv_slots])
    l = _lib.lib()
    _lib.check(
        l.bxl_attn_fwd_f16(
            _p(q), q.stride(0), q.stride(1), arr, len(kv_slots), s0.stride(0), s0.stride(1), Cq, _p(out), out.stride(0),
            out.stride(1), B, heads, Lq, Ls, float(scale), _stream(),
        ),
        l,
    )
    return out


# --------------------------------------------------------------------------- host-graph helpers
def upsample2x(x):
    _nhwc_strip(x, "x")
    _req(x.is_contiguous(), "upsample2x: contiguous input")
    B, H, W, Ci = x.shape
    out = torch.empty((B, 2 * H, 2 * W, Ci), device=x.device, dtype=torch.float16)
    l = _lib.lib()
    _lib.check(l.bxl_upsample2x_f16(_p(x), _p(out), B, H, W, Ci, _stream()), l)
    return out


def layernorm(x, gamma, beta, eps):
    _f16_cuda(x, "x")
    _req(x.is_contiguous(), "layernorm: contiguous input")
    Ci = x.shape[-1]
    out = torch.empty_like(x)
    l = _lib.lib()
    _lib.check(l.bxl_layernorm_f16(_p(x), _p(out), _p(gamma), _p(beta), x.numel() // Ci, Ci, float(eps), _stream()), l)
    return out


def geglu(h):
    _f16_cuda(h, "h")
    _req(h.is_contiguous() and h.shape[-1] % 16 == 0, "geglu: contiguous input with an even number of 8-vectors")
    F = h.shape[-1] // 2
    out = torch.empty((*h.shape[:-1], F), device=h.device, dtype=torch.float16)
    l = _lib.lib()
    _lib.check(l.bxl_geglu_f16(_p(h), _p(out), h.numel() // (2 * F), F, _stream()), l)
    return out


def cfg_euler_step(eps, latents, next_input, guidance: float, sigma: float, sigma_next: float):
    """Guidance combine, Euler update of ``latents`` (fp32, in place) and the scaled fp16 input
    of the next step (both CFG rows) in one launch.  The three tensors are dense and share one
    memory order (all row-major, or all channels-last)."""
    _f16_cuda(eps, "eps"), _f16_cuda(next_input, "next_input")
    _req(latents.is_cuda and latents.dtype == torch.float32, "cfg_euler_step: fp32 latents")
    n = latents.numel()
    fmt = torch.contiguous_format if latents.is_contiguous() else torch.channels_last
    _req(all(t.is_contiguous(memory_format=fmt) for t in (eps, latents, next_input)) and eps.numel() == 2 * n
         and next_input.numel() == 2 * n and eps.shape[1:] == latents.shape[1:] and next_input.shape[1:] == latents.shape[1:],
         "cfg_euler_step: eps and next_input must be dense [2, ...] tensors in the memory order of the latents")
    l = _lib.lib()
    _lib.check(l.bxl_cfg_euler_step(_p(eps), _p(latents), _p(next_input), n, float(guidance), float(sigma), float(sigma_next), _stream()), l)
    return latents, next_input

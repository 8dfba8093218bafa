"""``cascaded_lowp_matmul(a, b, *, out=None)``: drop-in for the reference's Triton
matmul (basedxl/triton/cascaded_lowp_matmul.py:139-173).

Same contract: ``a [..., K]`` with any leading dimensions, ``b [K, N]``
contiguous, result ``[..., N]`` in ``a.dtype``.  The arithmetic differs on
purpose: fp16 products are accumulated in fp32 tensor memory (the reference
accumulates in fp16), and fp32 operands go through the split-operand product.
Every shape runs on the library kernel; there is no ``torch.matmul`` fallback
for small shapes (the reference falls back below 512 x 256,
cascaded_lowp_matmul.py:154-156), except for a batched ``b``, which only that
fallback ever supported and which is evaluated one matrix at a time here.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops


def cascaded_lowp_matmul(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    out: Optional[torch.Tensor] = None,
    dump_ptx: bool = False,
    bias: Optional[torch.Tensor] = None,
    residual: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    assert a.shape[-1] == b.shape[-2], "Incompatible dimensions"
    assert b.is_contiguous(), "Matrix B must be contiguous"
    if dump_ptx:
        raise NotImplementedError("dump_ptx: this implementation is ahead-of-time compiled CUDA, there is no PTX to dump")
    if b.dim() > 2:
        # batched right operand: one product per matrix, broadcasting like torch.matmul
        batch = torch.broadcast_shapes(a.shape[:-2], b.shape[:-2])
        a_b = a.expand(*batch, *a.shape[-2:]).reshape(-1, *a.shape[-2:])
        b_b = b.expand(*batch, *b.shape[-2:]).reshape(-1, *b.shape[-2:])
        res = torch.stack([cascaded_lowp_matmul(x, y.contiguous()) for x, y in zip(a_b, b_b)])
        res = res.view(*batch, a.shape[-2], b.shape[-1])
        if out is not None:
            out.copy_(res)
            return out
        return res
    batch_dims, K = a.shape[:-1], a.shape[-1]
    N = b.shape[-1]
    a2 = a.reshape(-1, K)
    if a2.stride(-1) != 1:
        a2 = a2.contiguous()
    if a.dtype == torch.float32:
        assert bias is None and residual is None
        res = ops.gemm_split_f32(a2, b)
        if out is not None:
            out.copy_(res.view(out.shape))
            return out
        return res.reshape(*batch_dims, N)
    if K % 8 or N % 8:
        # rows must be whole 16-byte vectors for the copy engine: zero-pad K and N
        Kp, Np = (K + 7) // 8 * 8, (N + 7) // 8 * 8
        a_p = torch.zeros(a2.shape[0], Kp, device=a.device, dtype=a.dtype)
        a_p[:, :K] = a2
        b_p = torch.zeros(Kp, Np, device=b.device, dtype=b.dtype)
        b_p[:K, :N] = b
        res = ops.gemm(a_p, b_p, b_is_kn=True)[:, :N]
        if bias is not None:
            res = res + bias
        res = res.reshape(*batch_dims, N)
        if out is not None:
            out.copy_(res)
            return out
        return res.contiguous()
    o2 = None if out is None else out.view(-1, N)
    r2 = None if residual is None else residual.reshape(-1, N)
    res = ops.gemm(a2, b, bias=bias, residual=r2, out=o2, b_is_kn=True)
    return res.reshape(*batch_dims, N)

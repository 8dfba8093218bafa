"""CPU restatement of the reference's low-precision matmul and of its error
measurement method.  Test infrastructure (see ``oracle/__init__.py``).
"""
from __future__ import annotations

import numpy as np
import torch

EPS = 1e-6  # extras/measure_cascaded_lowp_matmul_error.py:8
QUANTILES = [0.01, 0.2, 0.5, 0.8, 0.99]  # extras/measure_cascaded_lowp_matmul_error.py:9


def matmul_fp64(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """The "expected" product of the reference's error study: operands widened
    to fp64 (extras/measure_cascaded_lowp_matmul_error.py:21)."""
    return a.double() @ b.double()


def matmul_fp16_accumulate(a: torch.Tensor, b: torch.Tensor, block_k: int = 32, model: str = "block") -> torch.Tensor:
    """Model of the reference kernel's arithmetic
    (basedxl/triton/cascaded_lowp_matmul.py:105-126 with K_ACC_DIV = 1, :8-9):
    fp16 operands, one fp16 accumulator carried over all of K in steps of
    ``block_k`` (the kernel's BLOCK_K, 16 or 32, :13), result cast
    fp16 -> fp32 -> fp16.

    Two roundings models bracket what tensor cores do with an fp16 accumulator:

    ``"interpreter"``: every multiply-add inside a block is rounded to fp16
        (numpy's fp16 matmul).  This is bit-for-bit what the kernel computes
        under Triton's CPU interpreter, which is how the golden fixture was
        produced.
    ``"block"``: each ``block_k``-wide partial product is formed exactly and
        rounded once into the fp16 accumulator.  No hardware rounds less often
        than this, so its error is a lower bound on the reference kernel's.
    """
    a16, b16 = a.half(), b.half()
    m, k = a16.shape
    n = b16.shape[1]
    if model == "interpreter":
        an, bn = a16.numpy(), b16.numpy()
        acc = np.zeros((m, n), dtype=np.float16)
        for k0 in range(0, k, block_k):
            acc = np.matmul(an[:, k0 : k0 + block_k], bn[k0 : k0 + block_k, :], dtype=np.float16) + acc
        return torch.from_numpy(acc.astype(np.float32).astype(np.float16))
    assert model == "block"
    acc = torch.zeros(m, n, dtype=torch.float16)
    af, bf = a16.float(), b16.float()
    for k0 in range(0, k, block_k):
        part = af[:, k0 : k0 + block_k] @ bf[k0 : k0 + block_k, :]
        acc = (acc.float() + part).half()
    return acc.float().half()


def error_table(expected: torch.Tensor, out: torch.Tensor) -> dict:
    """Error figures of the reference's study
    (extras/measure_cascaded_lowp_matmul_error.py:26-41): mean absolute error,
    mean squared error, max absolute error and quantiles of
    |expected - out| / (|expected| + EPS)."""
    e = expected.double()
    o = out.double()
    diff = (e - o).abs()
    rel = (diff / (e.abs() + EPS)).numpy()
    return {
        "l1": float(diff.mean()),
        "mse": float((diff**2).mean()),
        "max": float(diff.max()),
        "rel_quantiles": [float(q) for q in np.quantile(rel, QUANTILES)],
        "rel_median": float(np.median(rel)),
    }


def wrapper_shape(a_shape: tuple[int, ...], b_shape: tuple[int, ...]) -> tuple[int, ...]:
    """Result shape of the reference wrapper
    (basedxl/triton/cascaded_lowp_matmul.py:146-173 and torch.matmul broadcasting
    for the small-shape fallback at :154-156)."""
    assert a_shape[-1] == b_shape[-2]
    batch = torch.broadcast_shapes(a_shape[:-2], b_shape[:-2])
    return tuple(batch) + (a_shape[-2], b_shape[-1])

"""Helpers shared by the GPU parity tests."""
import pytest
import torch

from oracle.patched_ops import rel_l2

TOL_FP16 = 2e-3  # per-op bar: relative L2 against the fp32 oracle on the same fp16-rounded inputs


def cuda_or_skip():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


def nhwc(x_nchw: torch.Tensor) -> torch.Tensor:
    """NCHW host tensor -> NHWC-contiguous tensor (same device)."""
    return x_nchw.permute(0, 2, 3, 1).contiguous()


def nchw(x_nhwc: torch.Tensor) -> torch.Tensor:
    return x_nhwc.permute(0, 3, 1, 2)


def h16(t: torch.Tensor) -> torch.Tensor:
    """Round to fp16 and return as fp32 (what the oracle consumes)."""
    return t.half().float()


def assert_close(y_gpu: torch.Tensor, y_ref: torch.Tensor, tol: float = TOL_FP16, what: str = ""):
    err = rel_l2(y_gpu.detach().float().cpu(), y_ref.float())
    assert err <= tol, f"{what}: rel-L2 {err:.3e} > {tol:.1e}"
    return err

"""Common state of the patch-parallel wrappers (reference:
basedxl/modules/base_module.py:6-29)."""
from __future__ import annotations

import torch
from torch import nn

from ..utils import BasedXLConfig, PatchParallelismCommManager


class BaseModule(nn.Module):
    # wrappers (and the host graph's own layers) that fuse bias rows, residuals or
    # SiLU into their kernels advertise it, so the host graph knows it may pass
    # the extra keyword arguments
    supports_fused_epilogue = True

    def __init__(self, module: nn.Module, basedxl_config: BasedXLConfig):
        super().__init__()
        self.module = module
        self.basedxl_config = basedxl_config
        self.comm_manager: PatchParallelismCommManager | None = None
        self.counter = 0
        self.buffer_list = None
        self.idx = None

    def forward(self, *args, **kwargs):
        raise NotImplementedError

    def set_counter(self, counter: int = 0):
        self.counter = counter

    def set_comm_manager(self, comm_manager: PatchParallelismCommManager):
        self.comm_manager = comm_manager

    def _wait_pending(self):
        """Order the current stream after the in-flight gather that delivers this
        layer's peer data (basedxl/modules/conv2d.py:48-51)."""
        if self.comm_manager is not None:
            self.comm_manager.wait(self.idx)


def as_nhwc(x: torch.Tensor) -> torch.Tensor:
    """[B,C,H,W]-shaped tensor -> NHWC-contiguous [B,H,W,C] view.  Tensors that
    are already channels-last are viewed, others are converted once."""
    y = x.permute(0, 2, 3, 1)
    if not y.is_contiguous():
        y = y.contiguous()
    return y


def as_nchw(y_nhwc: torch.Tensor) -> torch.Tensor:
    """NHWC-contiguous tensor -> [B,C,H,W]-shaped channels-last view."""
    return y_nhwc.permute(0, 3, 1, 2)

"""Linear layer on the tensor-core matmul (reference:
basedxl/modules/lowp_linear.py:7-20).  Keeps the reference's attributes: the
weight is stored transposed, ``[in_features, out_features]`` contiguous; the
bias add is fused into the kernel's epilogue."""
from __future__ import annotations

import torch
import torch.nn as nn

from ..cascaded_lowp_matmul import cascaded_lowp_matmul


class BasedXLLowPLinear(nn.Module):
    supports_fused_epilogue = True

    def __init__(self, submodule: nn.Linear):
        super().__init__()
        self.in_features = submodule.in_features
        self.out_features = submodule.out_features
        self.weight = submodule.weight.T.contiguous().clone()
        self.bias = submodule.bias.clone() if submodule.bias is not None else None

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        return cascaded_lowp_matmul(x, self.weight, bias=self.bias, residual=residual)

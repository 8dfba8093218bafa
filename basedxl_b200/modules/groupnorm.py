"""Patch-parallel GroupNorm (reference: basedxl/modules/groupnorm.py:9-72),
optionally fused with the SiLU that follows it in the host graph (the wrapped
module carries ``fuse_silu = True`` in that case).

Moments are kept in fp32.  The reference registers ``[2, B, G, 1, 1, 1]`` values
in the activation dtype per layer; here each fp32 moment occupies two fp16
slots of the shared staging buffer, i.e. the registered shape is
``[2, B, G, 1, 1, 2]``.
"""
from __future__ import annotations

import torch
from torch import nn

from .. import ops
from ..utils import BasedXLConfig
from .base_module import BaseModule, as_nchw, as_nhwc


class BasedXLGroupNorm(BaseModule):
    def __init__(self, module: nn.GroupNorm, basedxl_config: BasedXLConfig):
        assert isinstance(module, nn.GroupNorm)
        super().__init__(module, basedxl_config)

    # forward() can also write the first and last row of its result into the staging range of the
    # convolution that consumes it (what that convolution publishes to the neighbouring strips)
    supports_halo_out = True

    def forward(self, x: torch.Tensor, silu: bool | None = None, halo_out: torch.Tensor | None = None) -> torch.Tensor:
        torch.cuda.nvtx.range_push("group_norm::forward")
        m = self.module
        cfg = self.basedxl_config
        self._wait_pending()
        assert x.ndim == 4
        n, c, h, w = x.shape
        groups = m.num_groups
        if silu is None:
            silu = bool(getattr(m, "fuse_silu", False))

        if self.buffer_list is None and self.comm_manager is not None:
            if self.comm_manager.buffer_list is None:
                # one fp32 moment = 4 // itemsize staging elements (2 for fp16 activations)
                self.idx = self.comm_manager.register_tensor(
                    shape=[2, n, groups, 1, 1, 4 // x.element_size()], torch_dtype=x.dtype, layer_type="gn"
                )
            else:
                self.buffer_list = [t.view(-1).view(torch.float32) for t in self.comm_manager.get_buffer_list(self.idx)]

        xh = as_nhwc(x)
        gamma = m.weight if m.affine else None
        beta = m.bias if m.affine else None
        if self.buffer_list is None:
            # strip statistics only: one launch
            y = ops.groupnorm_fused(xh, groups, m.eps, gamma, beta, silu=silu, halo_out=halo_out)
        elif self.counter <= cfg.warmup_steps:
            # synchronous step: the fresh moments of all strips are gathered between the two passes
            assert self.comm_manager is not None
            fresh = ops.groupnorm_stats(xh, groups, out=self.buffer_list[cfg.split_idx()].view(2, n, groups))  # own range, fp32
            self.comm_manager.sync_exchange(self.idx)
            y = ops.groupnorm_apply(xh, groups, m.eps, gamma, beta, fresh, self.buffer_list, cfg.split_idx(), ops.MODE_SYNC, silu=silu)
            if halo_out is not None:
                ops.halo_pack(y, 1, out=halo_out)
        else:
            # displaced step: one launch; the kernel reads every strip's stale moments (its own
            # included) and then stores its fresh moments straight into its own staging range
            assert self.comm_manager is not None
            own = self.buffer_list[cfg.split_idx()]
            y = ops.groupnorm_fused(xh, groups, m.eps, gamma, beta, self.buffer_list, cfg.split_idx(), ops.MODE_STALE, silu=silu,
                                    fresh_out=own.view(2, n, groups), halo_out=halo_out)
            self.comm_manager.enqueue(self.idx, own)
        self.counter += 1
        torch.cuda.nvtx.range_pop()
        return as_nchw(y)

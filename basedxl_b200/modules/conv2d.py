"""Patch-parallel 3x3 convolution (reference: basedxl/modules/conv2d.py:10-112).

The wrapped ``nn.Conv2d`` keeps owning the parameters.  Activations are
``[B, C, H_local, W]``-shaped channels-last tensors; the kernel reads the fresh
local strip and the neighbours' boundary rows from their own buffers, so the
padded input of the reference (its ``torch.cat`` / ``F.pad``) is never built.

Staging layout: the reference registers ``[2, B, C, pad, W]`` per layer; the
same number of elements is registered here but stored as ``[2, B, pad, W, C]``
(channels last), index 0 = the strip's top rows, 1 = its bottom rows.
"""
from __future__ import annotations

import torch
from torch import nn

from .. import ops
from ..utils import BasedXLConfig
from .base_module import BaseModule, as_nchw, as_nhwc


def packed_weight(module: nn.Conv2d) -> torch.Tensor:
    """[C_out, 9*C_in] tap-major copy of the weight, cached on the module
    (inference: parameters are frozen)."""
    w = module.weight
    cache = getattr(module, "_bxl_packed", None)
    if cache is None or cache[0] != (w.data_ptr(), w._version):
        module._bxl_packed = ((w.data_ptr(), w._version), ops.conv_weight_pack(w.detach()))
    return module._bxl_packed[1]


def check_conv(module: nn.Conv2d):
    ks, st, pd = module.kernel_size, module.stride, module.padding
    if tuple(ks) != (3, 3) or tuple(pd) != (1, 1) or st[0] != st[1] or st[0] not in (1, 2) or module.groups != 1:
        raise NotImplementedError(f"patched convolution supports 3x3 / padding 1 / stride 1 or 2, got {module}")
    if tuple(module.dilation) != (1, 1):
        raise NotImplementedError("dilated convolutions are not supported")


class BasedConv2dPP(BaseModule):
    def __init__(self, module: nn.Conv2d, basedxl_config: BasedXLConfig, is_first_layer: bool = False):
        super().__init__(module, basedxl_config)
        check_conv(module)
        self.is_first_layer = is_first_layer

    def naive_forward(self, x: torch.Tensor, **fused) -> torch.Tensor:
        m = self.module
        y = ops.conv3x3(as_nhwc(x), packed_weight(m), m.bias, stride=m.stride[0], **fused)
        return as_nchw(y)

    def sliced_forward(self, x: torch.Tensor, **fused) -> torch.Tensor:
        """Full-height input in, this strip's output rows out
        (basedxl/modules/conv2d.py:20-41): the rows above and below the slice are
        taken straight from the full input, the image edges are zero rows."""
        cfg = self.basedxl_config
        m = self.module
        b, c, h, w = x.shape
        assert h % cfg.n_device_per_batch == 0
        stride = m.stride[0]
        idx = cfg.split_idx()
        rows = h // cfg.n_device_per_batch
        r0, r1 = rows * idx, rows * (idx + 1)
        xh = as_nhwc(x)
        body = xh[:, r0:r1]
        top = xh[:, r0 - 1 : r0] if r0 > 0 else None
        bot = xh[:, r1 : r1 + 1] if r1 < h else None
        y = ops.conv3x3(body, packed_weight(m), m.bias, stride=stride, top=top, bot=bot, **fused)
        return as_nchw(y)

    def halo_staging(self) -> torch.Tensor | None:
        """This strip's staging range ``[2, B, pad, W, C]`` when the next call is a displaced step, so
        that the producer of the input can write the boundary rows there itself (``forward`` is then
        called with ``halo_packed=True``); None when the layer packs them itself."""
        cfg = self.basedxl_config
        if (cfg.n_device_per_batch == 1 or self.is_first_layer or self.comm_manager is None or self.idx is None
                or self.comm_manager.buffer_list is None or self.counter <= cfg.warmup_steps or self.module.padding[0] != 1):
            return None
        # the gather of the previous step that still reads this range must have finished
        self._wait_pending()
        shape = self.comm_manager.shapes[self.idx]  # registered as [2, B, C, pad, W]
        return self.comm_manager.own_slot(self.idx).view(2, shape[1], shape[3], shape[4], shape[2])

    def forward(self, x: torch.Tensor, *args, bias_rows=None, residual=None, halo_packed: bool = False, **kwargs) -> torch.Tensor:
        torch.cuda.nvtx.range_push("conv2d::forward")
        cfg = self.basedxl_config
        m = self.module
        fused = {}
        if bias_rows is not None:
            fused["bias_rows"] = bias_rows
        if residual is not None:
            fused["residual"] = as_nhwc(residual)
        self._wait_pending()

        if cfg.n_device_per_batch == 1:
            output = self.naive_forward(x, **fused)
        elif self.is_first_layer:
            output = self.sliced_forward(x, **fused)
        else:
            pad = m.padding[0]
            if self.buffer_list is None and self.comm_manager is not None:
                if self.comm_manager.buffer_list is None:
                    self.idx = self.comm_manager.register_tensor(
                        shape=[2, x.shape[0], x.shape[1], pad, x.shape[3]], torch_dtype=x.dtype, layer_type="conv2d"
                    )
                else:
                    self.buffer_list = self.comm_manager.get_buffer_list(self.idx)
            if self.buffer_list is None:
                output = self.naive_forward(x, **fused)
            else:
                xh = as_nhwc(x)
                b, hl, w, c = xh.shape
                idx, n = cfg.split_idx(), cfg.n_device_per_batch
                sync = self.counter <= cfg.warmup_steps
                if sync:
                    # fresh boundary rows into the own staging range, then to every peer
                    assert self.comm_manager is not None
                    ops.halo_pack(xh, pad, out=self.comm_manager.own_slot(self.idx).view(2, b, pad, w, c))
                    self.comm_manager.sync_exchange(self.idx)
                # strip above publishes its bottom rows (index 1), strip below its top rows (index 0)
                top = self.buffer_list[idx - 1].view(2, b, pad, w, c)[1] if idx > 0 else None
                bot = self.buffer_list[idx + 1].view(2, b, pad, w, c)[0] if idx < n - 1 else None
                y = ops.conv3x3(xh, packed_weight(m), m.bias, stride=m.stride[0], top=top, bot=bot, **fused)
                output = as_nchw(y)
                if not sync:
                    assert self.comm_manager is not None
                    # pack straight into the own staging range, then queue it
                    own = self.comm_manager.own_slot(self.idx)
                    if not halo_packed:
                        ops.halo_pack(xh, pad, out=own.view(2, b, pad, w, c))
                    self.comm_manager.enqueue(self.idx, own)

        self.counter += 1
        torch.cuda.nvtx.range_pop()
        return output

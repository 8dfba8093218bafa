"""UNet wrapper: patched-module swap, CFG / strip dispatch, output gather
(reference: basedxl/unet.py:18-199).

``BasedXLUnet(model, cfg)`` takes a host UNet graph (``basedxl_b200.sdxl_unet``
or anything with the same child-module naming) and, when patch parallelism is
on, replaces in place every non-1x1 ``nn.Conv2d``, every ``nn.GroupNorm`` and
every attention child named ``attn1`` / ``attn2`` by its patch-parallel wrapper
(basedxl/unet.py:89-114); with ``fp16_acc_matmul`` every ``nn.Linear`` is
replaced by ``BasedXLLowPLinear`` (:81-87).

The reference never constructs its comm manager (nothing calls
``set_comm_manager`` / ``create_buffer``); ``prepare`` below supplies that
sequence and ``forward`` calls it on first use.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from .modules.attn import BasedXLCrossAttentionPP, BasedXLSelfAttentionPP
from .modules.base_module import BaseModule
from .modules.conv2d import BasedConv2dPP
from .modules.groupnorm import BasedXLGroupNorm
from .modules.lowp_linear import BasedXLLowPLinear
from .utils import BasedXLConfig, PatchParallelismCommManager


def _is_attention(m: nn.Module) -> bool:
    return all(hasattr(m, a) for a in ("to_q", "to_k", "to_v", "to_out", "heads"))


class BaseModel(nn.Module):
    def __init__(self, model: nn.Module, basedxl_config: BasedXLConfig):
        super().__init__()
        self.model = model
        self.basedxl_config = basedxl_config
        self.comm_manager = None
        self.buffer_list = None
        self.output_buffer = None
        self.world_peer = None
        self.output_views = None
        self.counter = 0

    def forward(self, *args, **kwargs):
        raise NotImplementedError

    def set_counter(self, counter: int = 0):
        self.counter = counter
        for module in self.model.modules():
            if isinstance(module, BaseModule):
                module.set_counter(counter)

    def set_comm_manager(self, comm_manager: PatchParallelismCommManager):
        self.comm_manager = comm_manager
        for module in self.model.modules():
            if isinstance(module, BaseModule):
                module.set_comm_manager(comm_manager)

    @property
    def config(self):
        return self.model.config

    def synchronize(self):
        if self.comm_manager is not None and self.comm_manager.handles is not None:
            for i in range(len(self.comm_manager.handles)):
                if self.comm_manager.handles[i] is not None:
                    self.comm_manager.handles[i].wait()
                    self.comm_manager.handles[i] = None


class BasedXLUnet(BaseModel):
    def __init__(self, model: nn.Module, basedxl_config: BasedXLConfig):
        cfg = basedxl_config
        self.patched = bool(cfg.patch_parallelism and cfg.world_size > 1 and cfg.n_device_per_batch > 1)
        if self.patched:
            self.patch_pp_layers(model, cfg)
        if cfg.fp16_acc_matmul:
            self.patch_linear_layers(model)
        if cfg.compile_unet:
            raise NotImplementedError(
                "compile_unet: there is no tracing compiler in this implementation; launch overhead is removed with "
                "CUDA graphs (BasedXLPipeline(..., cuda_graph=True)) instead"
            )
        super().__init__(model, cfg)
        self.prepack_weights()
        self.cuda_graph = False
        self._graphed = None        # displaced steps (single GPU: every step)
        self._graphed_sync = None   # synchronous warm-up steps of a patch-parallel run

    def enable_cuda_graph(self, enabled: bool = True):
        """Replay one captured CUDA graph per denoising step instead of launching
        ~1200 kernels from Python.  Single-GPU runs capture the whole forward."""
        self.cuda_graph = enabled
        self.release_graph()
        for m in self.model.modules():
            if isinstance(m, BasedXLCrossAttentionPP):
                m.kv_managed = bool(enabled)

    def release_graph(self):
        """Drop the captured step graph (call before destroying the process group)."""
        for slot in ("_graphed", "_graphed_sync"):
            if getattr(self, slot, None) is not None:
                getattr(self, slot).release()
            setattr(self, slot, None)

    @torch.no_grad()
    def prepack_weights(self):
        """Build the tap-major copies of the 3x3 convolution weights now rather than at each
        layer's first call, so that no packing kernel is launched in the middle of a step.
        (Weights loaded later are re-packed at the layer's next call.)"""
        from .modules.conv2d import packed_weight

        for m in self.model.modules():
            if isinstance(m, nn.Conv2d) and tuple(m.kernel_size) == (3, 3) and m.weight.is_cuda and m.weight.dtype == torch.float16:
                packed_weight(m)

    def patch_linear_layers(self, model: nn.Module):
        for _name, module in model.named_modules():
            for subname, submodule in module.named_children():
                if isinstance(submodule, nn.Linear):
                    setattr(module, subname, BasedXLLowPLinear(submodule))

    def patch_pp_layers(self, model: nn.Module, cfg: BasedXLConfig):
        for _name, module in model.named_modules():
            if isinstance(module, BaseModule):
                continue
            for subname, submodule in module.named_children():
                if isinstance(submodule, nn.Conv2d):
                    ks = submodule.kernel_size
                    if ks == (1, 1) or ks == 1:
                        continue
                    setattr(module, subname, BasedConv2dPP(submodule, cfg, is_first_layer=subname == "conv_in"))
                elif _is_attention(submodule):
                    if subname == "attn1":
                        wrapped = BasedXLSelfAttentionPP(submodule, cfg)
                    elif subname == "attn2":
                        wrapped = BasedXLCrossAttentionPP(submodule, cfg)
                    else:
                        raise ValueError(f"Unknown attention layer: {subname}")
                    setattr(module, subname, wrapped)
                elif isinstance(submodule, nn.GroupNorm):
                    setattr(module, subname, BasedXLGroupNorm(submodule, cfg))

    def reset(self):
        """Start a new image: drain the exchange queue and every pending gather,
        then re-enter the synchronous warm-up phase."""
        if self.comm_manager is not None:
            self.comm_manager.clear()
        self.set_counter(0)

    @property
    def add_embedding(self):
        return self.model.add_embedding

    # ------------------------------------------------------------------ set-up
    @torch.no_grad()
    def prepare(self, sample, timestep, encoder_hidden_states, added_cond_kwargs=None):
        """Create the comm manager, let every patched layer register its exchange
        tensor in one forward pass over its strip, allocate the staging buffers
        and reset the step counter."""
        if not self.patched:
            return
        cm = PatchParallelismCommManager(self.basedxl_config)
        self.set_comm_manager(cm)
        self._run_local(sample, timestep, encoder_hidden_states, added_cond_kwargs or {})
        cm.create_buffer()
        self.set_counter(0)

    @torch.no_grad()
    def _refresh_context(self, sample, timestep, encoder_hidden_states, added_cond_kwargs):
        """Recompute, in place, the K/V of the conditioning that cross-attention layers cache (the
        step graphs read it but do not recompute it)."""
        _, _, ehs, _ = self._slice_batch(sample, timestep, encoder_hidden_states, added_cond_kwargs)
        ctx = ehs.to(next(self.model.parameters()).dtype)
        wrapped = set()
        for m in self.model.modules():
            if isinstance(m, BasedXLCrossAttentionPP):
                m.refresh_context_kv(ctx)
                wrapped.add(id(m.module))
        for m in self.model.modules():
            if hasattr(m, "context_kv") and getattr(m, "is_cross", False) and id(m) not in wrapped:
                m.context_kv(ctx, force=True)

    def _slice_batch(self, sample, timestep, encoder_hidden_states, added_cond_kwargs):
        cfg = self.basedxl_config
        if not (cfg.use_cfg and cfg.world_size > 1):
            return sample, timestep, encoder_hidden_states, added_cond_kwargs
        assert sample.shape[0] == 2
        i = cfg.batch_idx()
        sample = sample[i : i + 1]
        if isinstance(timestep, torch.Tensor) and timestep.ndim > 0:
            timestep = timestep[i : i + 1]
        encoder_hidden_states = encoder_hidden_states[i : i + 1]
        added_cond_kwargs = {k: v[i : i + 1] for k, v in added_cond_kwargs.items()}
        return sample, timestep, encoder_hidden_states, added_cond_kwargs

    def _run_local(self, sample, timestep, encoder_hidden_states, added_cond_kwargs):
        s, t, e, a = self._slice_batch(sample, timestep, encoder_hidden_states, added_cond_kwargs)
        return self.model(s, t, e, added_cond_kwargs=a, return_dict=False)[0]

    def _prepare_output(self, sample):
        """The full-size output every rank assembles each step, channels-last (a strip's rows are then
        one contiguous range), and - where the ranks can write each other's memory - its mapping in
        every peer, so that the strips are stored straight into place."""
        cfg = self.basedxl_config
        b, c, h, w = sample.shape
        dt = next(self.model.parameters()).dtype
        self.output_buffer = torch.empty((b, c, h, w), device=cfg.device, dtype=dt, memory_format=torch.channels_last)
        self.world_peer = None
        self.output_views = None
        if self.output_buffer.is_cuda:
            from .peer import make_peer_group

            self.world_peer = make_peer_group(None, cfg.rank, cfg.world_size, cfg.device, verbose=cfg.verbose and cfg.rank == 0)
            if self.world_peer is not None:
                flat = self.output_buffer.permute(0, 2, 3, 1).reshape(-1)  # NHWC memory order, a view
                assert flat.data_ptr() == self.output_buffer.data_ptr()
                self.output_views = self.world_peer.share(flat)  # address of every rank's output
                if self.world_peer.failed is not None:
                    raise RuntimeError(f"mapping the peers' output buffers failed: {self.world_peer.failed!r}")

    def _step_multi(self, sample, timestep, encoder_hidden_states, added_cond_kwargs, drain: bool = True):
        """One step on this rank's strip / CFG half, then the assembly of all ranks' output strips
        (basedxl/unet.py:166-175,185-195).  With ``drain`` the tail of the exchange queue is flushed
        and every pending gather joined before returning, which makes the step self-contained
        (what graph replay needs); without it the tail is flushed by the next step's first layer,
        as in the reference.  Either way every layer sees exactly the previous step's data."""
        cfg = self.basedxl_config
        b, c, h, w = sample.shape
        n = cfg.n_device_per_batch
        hs = h // n
        local = self._run_local(sample, timestep, encoder_hidden_states, added_cond_kwargs)
        local = local.permute(0, 2, 3, 1).contiguous()  # [b_local, h/n, w, c]: the kernels' own order, no copy
        if drain and self.comm_manager is not None:
            self.comm_manager.clear()
        if self.output_buffer is None:
            self._prepare_output(sample)
        out = self.output_buffer.permute(0, 2, 3, 1)  # [b, h, w, c] view
        # rank r serves image batch_idx(r) (CFG split) or all images, rows split_idx(r)*hs ...
        images = [cfg.batch_idx()] if cfg.use_cfg else list(range(b))
        r0 = cfg.split_idx() * hs
        if self.world_peer is not None:
            # every rank stores its strip into every rank's output (its own included): one kernel,
            # peer stores + flag barrier; the handshake keeps a fast rank from overwriting an output
            # that a slower rank still reads
            for k, img in enumerate(images):
                off = ((img * h + r0) * w * c) * local.element_size()  # rows r0.. of image img, NHWC
                self.world_peer.exchange(local[k], [p + off for p in self.output_views], handshake=True)
        else:
            if self.buffer_list is None:
                self.buffer_list = [torch.empty_like(local) for _ in range(cfg.world_size)]
            dist.all_gather(self.buffer_list, local, async_op=False)
            for r, t in enumerate(self.buffer_list):
                rr = cfg.split_idx(r) * hs
                if cfg.use_cfg:
                    out[cfg.batch_idx(r), rr : rr + hs].copy_(t[0])
                else:
                    out[:, rr : rr + hs].copy_(t)
        return self.output_buffer

    # ------------------------------------------------------------------ one denoising step
    def forward(self, sample, timestep, encoder_hidden_states, added_cond_kwargs={}, **kwargs):
        # Inside a UNet step the B operand of every GEMM and convolution is a model weight:
        # the library may fetch it before a kernel waits for its predecessor.
        self._static_weights(True)
        try:
            return self._forward(sample, timestep, encoder_hidden_states, added_cond_kwargs, **kwargs)
        finally:
            self._static_weights(False)

    def _static_weights(self, on: bool):
        if torch.device(self.basedxl_config.device).type != "cuda":
            return
        from . import _lib

        l = _lib.lib()
        _lib.check(l.bxl_set_static_weights(1 if on else 0), l, kernels=0)

    def _forward(self, sample, timestep, encoder_hidden_states, added_cond_kwargs={}, **kwargs):
        torch.cuda.nvtx.range_push("unet::forward")
        cfg = self.basedxl_config
        b, c, h, w = sample.shape
        if self.patched and self.comm_manager is None:
            self.prepare(sample, timestep, encoder_hidden_states, added_cond_kwargs)
        if cfg.world_size > 1 and self.output_buffer is None:
            self._prepare_output(sample)  # collectives and memory mapping: never inside a graph capture

        if cfg.world_size == 1:
            if self.cuda_graph and isinstance(timestep, torch.Tensor):
                if self._graphed is None:
                    from .graph import GraphedStep

                    self._graphed = GraphedStep(
                        lambda s, t, e, a: self.model(s, t, e, added_cond_kwargs=a, return_dict=False)[0],
                        on_condition_change=self._refresh_context,
                    )
                output = self._graphed(sample, timestep, encoder_hidden_states, added_cond_kwargs)
            else:
                output = self.model(sample, timestep, encoder_hidden_states, added_cond_kwargs=added_cond_kwargs, return_dict=False)[0]
        else:
            # Every step of an image repeats one of two launch sequences: the synchronous one (steps
            # 0..warmup_steps: blocking per-layer collectives) and the displaced one (later steps).
            # Each is captured once - kernels and collectives - and replayed.  The K/V of the
            # conditioning, which the reference recomputes in the first step of an image, is
            # refreshed outside the graphs whenever the conditioning changes.
            c = self.counter
            graphable = self.cuda_graph and isinstance(timestep, torch.Tensor)
            if graphable:
                from .graph import GraphedStep

                displaced = (not self.patched) or c > cfg.warmup_steps
                slot = "_graphed" if displaced else "_graphed_sync"
                if getattr(self, slot) is None:
                    # capture does not execute anything, so no step is rehearsed (a rehearsal
                    # would publish this step's tensors a step early); the layers' own step
                    # counters select the path that is recorded
                    for module in self.model.modules():
                        if isinstance(module, BaseModule):
                            module.set_counter(c)
                    drain = displaced
                    # patched layers: no rehearsal (see above; their registration pass has already
                    # built every cached weight copy).  CFG split alone: one eager run first, which
                    # builds those copies outside the capture and changes no state.
                    setattr(self, slot, GraphedStep(lambda s_, t_, e_, a_, d=drain: self._step_multi(s_, t_, e_, a_, drain=d),
                                                    warmup_runs=0 if self.patched else 1, on_condition_change=self._refresh_context))
                output = getattr(self, slot)(sample, timestep, encoder_hidden_states, added_cond_kwargs)
            else:
                output = self._step_multi(sample, timestep, encoder_hidden_states, added_cond_kwargs, drain=False)
        self.counter += 1
        torch.cuda.nvtx.range_pop()
        return (output,)

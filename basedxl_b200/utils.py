"""Run configuration, process groups and the asynchronous exchange manager.

Same public surface as the reference's ``basedxl/utils.py`` (``BasedXLConfig``
at :8-73, ``PatchParallelismCommManager`` at :76-169): field names, attribute
names, method names and the gather schedule are kept, so code written against
the reference runs against this module unchanged.

Differences, all deliberate:
  * distributed mode is entered only when a launcher set WORLD_SIZE > 1; a
    failure to initialise is an error, not a silent fall-back to one device
    (reference: blanket ``except`` at basedxl/utils.py:29-33);
  * the backend follows the device: NCCL on GPUs, gloo for host tensors (used
    by the CPU tests of the multi-rank logic).
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass
class BasedXLConfig:
    pretrained_model_name_or_path: str = "stabilityai/stable-diffusion-xl-base-1.0"
    dtype: torch.dtype = torch.float16
    fp16_acc_matmul: bool = False
    patch_parallelism: bool = False
    compile_unet: bool = False
    width: int = 1024
    height: int = 1024
    use_cfg: bool = True
    warmup_steps: int = 4
    comm_checkpoint: int = 60
    verbose: bool = False
    # not in the reference: "cuda" (default) or "cpu" (host-logic tests only)
    device_type: str = "cuda"

    def __post_init__(self):
        world = int(os.environ.get("WORLD_SIZE", "1"))
        if world > 1:
            if not dist.is_initialized():
                if self.device_type == "cuda":
                    local = int(os.environ.get("LOCAL_RANK", os.environ.get("RANK", "0")))
                    torch.cuda.set_device(local)
                    dist.init_process_group(backend="nccl", device_id=torch.device("cuda", local))
                else:
                    dist.init_process_group(backend="gloo")
            self.rank = dist.get_rank()
            self.world_size = dist.get_world_size()
            if self.device_type == "cuda":
                local = int(os.environ.get("LOCAL_RANK", self.rank))
                self.device = f"cuda:{local}"
                torch.cuda.set_device(local)
            else:
                self.device = "cpu"
        else:
            self.rank = 0
            self.world_size = 1
            self.device = "cuda" if self.device_type == "cuda" else "cpu"

        # basedxl/utils.py:35-42
        if self.use_cfg:
            n_device_per_batch = self.world_size // 2
            if n_device_per_batch == 0:
                n_device_per_batch = 1
        else:
            n_device_per_batch = self.world_size
        self.n_device_per_batch = n_device_per_batch

        batch_group = None
        split_group = None
        # basedxl/utils.py:47-57: ranks of one CFG half / the same strip in both halves
        if self.use_cfg and self.world_size >= 2:
            half = self.world_size // 2
            batch_groups = [dist.new_group(list(range(i * half, (i + 1) * half))) for i in range(2)]
            batch_group = batch_groups[self.batch_idx()]
            split_groups = [dist.new_group([i, i + half]) for i in range(half)]
            split_group = split_groups[self.split_idx()]
        self.batch_group = batch_group
        self.split_group = split_group

    def batch_idx(self, rank: int | None = None) -> int:
        """Which CFG half a rank serves (basedxl/utils.py:62-68)."""
        if rank is None:
            rank = self.rank
        if self.use_cfg:
            return 1 - int(rank < (self.world_size // 2))
        return 0

    def split_idx(self, rank: int | None = None) -> int:
        """Which H-strip a rank serves (basedxl/utils.py:70-73)."""
        if rank is None:
            rank = self.rank
        return rank % self.n_device_per_batch


class PatchParallelismCommManager:
    """Flat per-peer staging buffers and the one-step-stale chunked gather.

    Every patched layer registers one tensor (its halo rows, group moments or
    K/V); ``create_buffer`` then allocates, per peer of the batch group, one flat
    buffer covering all registered tensors.  During the displaced phase a layer
    ``enqueue``s its fresh tensor into the own-rank buffer; every
    ``comm_checkpoint`` tensors (and when layer 0 comes round again with a
    non-empty queue) ONE asynchronous all-gather over the contiguous flat range
    of the queued tensors is launched on the process group's communication
    stream, overlapping the following layers' compute.  The layer waits on that
    gather at its next forward, one step later.  (basedxl/utils.py:94-169)
    """

    def __init__(self, basedxl_config: BasedXLConfig):
        self.basedxl_config = basedxl_config
        self.torch_dtype = None
        self.numel = 0
        self.numel_dict: dict[str, int] = {}
        self.buffer_list: list[torch.Tensor] | None = None
        self.starts: list[int] = []
        self.ends: list[int] = []
        self.shapes: list = []
        self.idx_queue: list[int] = []
        self.handles: list | None = None
        # bytes handed to the collectives since creation (own contribution only); calls recorded into
        # a CUDA graph count once, at capture
        self.bytes_sent = 0
        self.sync_bytes = 0
        self.flat = None
        self.peer = None
        self.peer_flat = None

    def register_tensor(self, shape, torch_dtype: torch.dtype, layer_type: str | None = None) -> int:
        if self.torch_dtype is None:
            self.torch_dtype = torch_dtype
        else:
            assert self.torch_dtype == torch_dtype
        self.starts.append(self.numel)
        numel = 1
        for dim in shape:
            numel *= dim
        # every registered range starts on a 16-byte boundary (TMA base alignment)
        assert (numel * torch.empty((), dtype=torch_dtype).element_size()) % 16 == 0, (
            f"registered tensor of shape {tuple(shape)} is not a whole number of 16-byte vectors"
        )
        self.numel += numel
        if layer_type is not None:
            self.numel_dict[layer_type] = self.numel_dict.get(layer_type, 0) + numel
        self.ends.append(self.numel)
        self.shapes.append(shape)
        return len(self.starts) - 1

    def create_buffer(self):
        cfg = self.basedxl_config
        if cfg.rank == 0 and cfg.verbose:
            print(f"Create buffer with {self.numel / 1e6:.3f}M parameters for {len(self.starts)} tensors on each device.")
            for layer_type, numel in self.numel_dict.items():
                print(f"  {layer_type}: {numel / 1e6:.3f}M parameters")
        n = cfg.n_device_per_batch
        # one allocation, one slot of `numel` elements per strip (16-byte aligned slots)
        assert (self.numel * torch.empty((), dtype=self.torch_dtype).element_size()) % 16 == 0
        self.flat = torch.zeros(n * self.numel, dtype=self.torch_dtype, device=cfg.device)
        self.buffer_list = [self.flat[j * self.numel : (j + 1) * self.numel] for j in range(n)]
        self.handles = [None for _ in range(len(self.starts))]
        # Peers that can write each other's memory exchange the synchronous steps' tensors with one
        # kernel per layer (peer stores + flag barrier) instead of a blocking collective.
        self.peer = None
        self.peer_flat = None
        if n > 1 and self.flat.is_cuda and dist.is_initialized():
            from .peer import make_peer_group

            self.peer = make_peer_group(cfg.batch_group, cfg.split_idx(), n, cfg.device, verbose=cfg.verbose and cfg.rank == 0)
            if self.peer is not None:
                self.peer_flat = self.peer.share(self.flat)
                if self.peer.failed is not None:
                    raise RuntimeError(f"mapping the peers' staging buffers failed: {self.peer.failed!r}")

    def get_buffer_list(self, idx: int) -> list[torch.Tensor]:
        assert self.buffer_list is not None
        return [t[self.starts[idx] : self.ends[idx]].view(self.shapes[idx]) for t in self.buffer_list]

    def own_slot(self, idx: int) -> torch.Tensor:
        """This rank's staging range for tensor ``idx`` (what ``enqueue`` fills)."""
        assert self.buffer_list is not None
        own = self.basedxl_config.split_idx()
        return self.buffer_list[own][self.starts[idx] : self.ends[idx]].view(self.shapes[idx])

    def sync_exchange(self, idx: int):
        """Synchronous steps: this rank's fresh tensor ``idx`` (already written into its own slot)
        goes to every peer, and the call returns with the stream ordered after the arrival of all
        the peers' tensors ``idx`` (the blocking all-gathers of basedxl/modules/conv2d.py:95,
        groupnorm.py:47, attn.py:135)."""
        assert self.buffer_list is not None
        cfg = self.basedxl_config
        own, n = cfg.split_idx(), cfg.n_device_per_batch
        start, end = self.starts[idx], self.ends[idx]
        src = self.buffer_list[own][start:end]
        self.sync_bytes += src.numel() * src.element_size()
        if self.peer is not None:
            off = (own * self.numel + start) * src.element_size()  # this rank's slot in every member's buffer
            dsts = [None if p == own else self.peer_flat[p] + off for p in range(n)]
            self.peer.exchange(src, dsts)
        else:
            outs = [t[start:end] for t in self.buffer_list]
            dist.all_gather(outs, src if src.is_cuda else src.clone(), group=cfg.batch_group, async_op=False)

    def communicate(self):
        assert self.buffer_list is not None and self.handles is not None
        cfg = self.basedxl_config
        start = self.starts[self.idx_queue[0]]
        end = self.ends[self.idx_queue[-1]]
        tensor = self.buffer_list[cfg.split_idx()][start:end]
        buffer_list = [t[start:end] for t in self.buffer_list]
        handle = dist.all_gather(buffer_list, tensor, group=cfg.batch_group, async_op=True)
        self.bytes_sent += tensor.numel() * tensor.element_size()
        for i in self.idx_queue:
            self.handles[i] = handle
        self.idx_queue = []

    def enqueue(self, idx: int, tensor: torch.Tensor):
        """Stage ``tensor`` as this rank's contribution for layer ``idx``.  A
        tensor that already *is* the own staging range (a producer wrote it in
        place) is not copied again."""
        assert self.buffer_list is not None
        cfg = self.basedxl_config
        if idx == 0 and len(self.idx_queue) > 0:
            self.communicate()
        assert len(self.idx_queue) == 0 or self.idx_queue[-1] == idx - 1
        self.idx_queue.append(idx)
        dst = self.buffer_list[cfg.split_idx()][self.starts[idx] : self.ends[idx]]
        if tensor.data_ptr() != dst.data_ptr():
            dst.copy_(tensor.reshape(-1) if tensor.dtype == dst.dtype else tensor.reshape(-1).view(dst.dtype))
        if len(self.idx_queue) == cfg.comm_checkpoint:
            self.communicate()

    def wait(self, idx: int | None):
        """Make the current stream wait for the pending gather of layer ``idx``
        (what every patched layer does first: basedxl/modules/conv2d.py:48-51)."""
        if self.handles is not None and idx is not None and self.handles[idx] is not None:
            self.handles[idx].wait()
            self.handles[idx] = None

    def clear(self):
        if len(self.idx_queue) > 0:
            self.communicate()
        if self.handles is not None:
            for i in range(len(self.handles)):
                if self.handles[i] is not None:
                    self.handles[i].wait()
                    self.handles[i] = None

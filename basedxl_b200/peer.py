"""Peer-memory groups: ranks on one node that write straight into each other's
device memory over NVLink.

The reference exchanges everything with ``torch.distributed.all_gather``
(basedxl/utils.py:135-147, basedxl/modules/conv2d.py:95, groupnorm.py:47,
attn.py:135, basedxl/unet.py:172).  Where every strip needs the others' FRESH
data before it can go on (the synchronous steps, the per-step output), this
module replaces the collective by one kernel of the library that stores the
rank's contribution into each peer's buffer and meets the peers at a flag
barrier (``bxl_comm_exchange``).

PyTorch supplies the plumbing only: buffers are ordinary CUDA tensors; the
allocation that holds one is exported as a CUDA IPC handle, handed to the peers
with ``all_gather_object`` over the group and mapped there by the library
(``bxl_comm_ipc_export`` / ``bxl_comm_ipc_open``).  Peers' buffers are handled as
raw device addresses.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import _lib

_vp = C.c_void_p
# allocations of peer processes already mapped into this process: IPC handle -> base address
_opened: dict[bytes, int] = {}


def _export(t: torch.Tensor):
    l = _lib.lib()
    handle = C.create_string_buffer(64)
    off = C.c_longlong(0)
    _lib.check(l.bxl_comm_ipc_export(t.data_ptr(), handle, C.byref(off)), l, kernels=0)
    return handle.raw, off.value


def _open(handle: bytes) -> int:
    if handle not in _opened:
        l = _lib.lib()
        base = _vp(0)
        _lib.check(l.bxl_comm_ipc_open(handle, C.byref(base)), l, kernels=0)
        _opened[handle] = base.value
    return _opened[handle]


class PeerGroup:
    """The members of one process group (all on this node, one GPU each).

    ``share(t)`` maps every member's tensor ``t`` (same shape on all members) into this
    process and returns its device address in every member, index = position in the group;
    ``exchange`` launches the library's exchange kernel on the current stream."""

    def __init__(self, group, index: int, size: int, device: torch.device, wait_seconds: float = 10.0):
        self.group, self.index, self.size, self.device = group, index, size, device
        self.wait_seconds = wait_seconds
        self.failed: Exception | None = None  # first failure to export or map memory; collectives still run in step
        self._keep = []  # shared tensors stay allocated for the life of the group
        words = _lib.load().bxl_comm_ctl_bytes() // 4
        self.ctl = torch.zeros(words, dtype=torch.int32, device=device)
        self.ctl_ptrs = self.share(self.ctl)
        # nobody signals before every member has zeroed and mapped the control words
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def share(self, t: torch.Tensor) -> list[int]:
        """Device address of every member's ``t`` as seen from this process.  Every member takes part
        in the one collective below even if exporting or mapping fails on it; the failure is kept in
        ``self.failed``."""
        assert t.is_cuda and t.is_contiguous()
        self._keep.append(t)
        meta = None
        try:
            with torch.cuda.device(self.device):
                meta = (*_export(t), tuple(t.shape), str(t.dtype))
        except Exception as e:
            self.failed = self.failed or e
        metas = [None] * self.size
        dist.all_gather_object(metas, meta, group=self.group)
        ptrs = [t.data_ptr()] * self.size
        if any(m is None for m in metas):
            self.failed = self.failed or RuntimeError("a member of the group could not export its memory")
            return ptrs
        try:
            with torch.cuda.device(self.device):
                for j, (handle, offset, shape, dtype) in enumerate(metas):
                    if j == self.index:
                        continue
                    assert tuple(shape) == tuple(t.shape) and dtype == str(t.dtype), "members must share tensors of one shape and dtype"
                    ptrs[j] = _open(handle) + offset
        except Exception as e:
            self.failed = self.failed or e
        return ptrs

    def exchange(self, src: torch.Tensor, dst_ptrs: list, handshake: bool = False):
        """Copy ``src`` (this rank's contribution, local) to address ``dst_ptrs[p]`` in member p's
        memory for every member with an entry (None = nothing to copy), then wait until every
        member's contribution has arrived here."""
        n = self.size
        nbytes = src.numel() * src.element_size()
        assert src.is_contiguous() and len(dst_ptrs) == n
        dst = (_vp * n)(*dst_ptrs)
        ctl = (_vp * n)(*self.ctl_ptrs)
        l = _lib.lib()
        _lib.check(
            l.bxl_comm_exchange(src.data_ptr(), dst, nbytes, self.ctl.data_ptr(), ctl, n, self.index, int(handshake),
                                float(self.wait_seconds), torch.cuda.current_stream().cuda_stream),
            l,
        )


def make_peer_group(group, index: int, size: int, device, verbose: bool = False) -> PeerGroup | None:
    """A ``PeerGroup`` if every member can map the others' memory, else None (all members agree).
    BXL_PEER_EXCHANGE=0 in the environment keeps the collectives on NCCL."""
    import os

    pg = None
    if os.environ.get("BXL_PEER_EXCHANGE", "1") != "0":
        pg = PeerGroup(group, index, size, torch.device(device))
    ok = int(pg is not None and pg.failed is None)
    flag = torch.tensor([ok], device=device, dtype=torch.int32)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    if int(flag.item()) == 1:
        return pg
    if verbose and pg is not None:
        print(f"peer-memory exchange unavailable ({pg.failed!r}); using NCCL all-gathers")
    return None

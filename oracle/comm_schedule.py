"""Pure-Python model of the reference's asynchronous exchange schedule.
Test infrastructure (see ``oracle/__init__.py``).

Models the bookkeeping of ``PatchParallelismCommManager``
(basedxl/utils.py:76-169) without any tensors or collectives: which flat
ranges are registered, and which contiguous ranges are gathered at which
point of a step.
"""
from __future__ import annotations


class CommScheduleModel:
    def __init__(self, comm_checkpoint: int = 60):
        self.comm_checkpoint = comm_checkpoint
        self.numel = 0
        self.starts: list[int] = []
        self.ends: list[int] = []
        self.shapes: list[tuple[int, ...]] = []
        self.numel_dict: dict[str, int] = {}
        self.idx_queue: list[int] = []
        # every launched gather: (first_idx, last_idx, flat_start, flat_end)
        self.launches: list[tuple[int, int, int, int]] = []
        # per registered tensor: index into ``launches`` of its pending gather
        self.pending: list[int | None] = []

    def register_tensor(self, shape, layer_type: str | None = None) -> int:
        """basedxl/utils.py:94-113."""
        self.starts.append(self.numel)
        n = 1
        for d in shape:
            n *= d
        self.numel += n
        if layer_type is not None:
            self.numel_dict[layer_type] = self.numel_dict.get(layer_type, 0) + n
        self.ends.append(self.numel)
        self.shapes.append(tuple(shape))
        self.pending.append(None)
        return len(self.starts) - 1

    def communicate(self) -> None:
        """One gather over the contiguous range covered by the queue
        (basedxl/utils.py:135-147)."""
        first, last = self.idx_queue[0], self.idx_queue[-1]
        self.launches.append((first, last, self.starts[first], self.ends[last]))
        for i in self.idx_queue:
            self.pending[i] = len(self.launches) - 1
        self.idx_queue = []

    def enqueue(self, idx: int) -> None:
        """basedxl/utils.py:149-159: a non-empty queue is flushed when layer 0
        comes round again; a gather is launched every ``comm_checkpoint``
        tensors."""
        if idx == 0 and self.idx_queue:
            self.communicate()
        assert not self.idx_queue or self.idx_queue[-1] == idx - 1
        self.idx_queue.append(idx)
        if len(self.idx_queue) == self.comm_checkpoint:
            self.communicate()

    def clear(self) -> None:
        """basedxl/utils.py:161-169."""
        if self.idx_queue:
            self.communicate()
        self.pending = [None] * len(self.pending)

    def run_step(self) -> list[tuple[int, int, int, int]]:
        """Enqueue every registered tensor once, in order; return the gathers
        launched during that step."""
        before = len(self.launches)
        for i in range(len(self.starts)):
            self.enqueue(i)
        return self.launches[before:]

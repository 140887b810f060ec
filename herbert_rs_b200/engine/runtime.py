"""What every part gets to run with: device, dtypes, page size, a workspace arena."""

from __future__ import annotations

import torch

from ..errors import BackendError


class _Lane:
    """One bump allocator over one device buffer."""

    def __init__(self, device, nbytes: int):
        self.device = device
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        self.offset = 0
        self.wanted = 0
        self.overflow: list = []
        self.views: dict = {}           # (offset, shape, dtype) -> the tensor over that place


class Workspace:
    """Scratch memory of a step: bump allocators over device buffers, rewound at the start of every step.

    The same sequence of requests yields the same addresses in every step, which is what a
    captured CUDA graph of the step needs; nothing is allocated while a step runs once the
    buffers have grown to the largest step seen (growth happens between steps, never during capture).

    There are three lanes.  Lane 0 holds what lives for the whole step (the residual stream, the
    logits).  Lanes 1 and 2 alternate between the layers: `use(lane)` makes a lane current and
    empties it, so a layer's scratch is gone when the layer after the next begins, while what a
    layer hands to its successor (a norm it has begun) survives that successor.  A step's scratch
    is therefore two layers' worth, not the sum over all layers.
    """

    LANES = 3

    def __init__(self, device, nbytes: int = 1 << 20):
        self.device = device
        self.lanes = [_Lane(device, nbytes) for _ in range(self.LANES)]
        self.current = self.lanes[0]
        self.frozen = False
        self._overflow_seen = False     # a buffer was replaced since this flag was last cleared

    def rewind(self) -> None:
        for lane in self.lanes:
            if lane.wanted > lane.buf.numel() and not self.frozen:
                lane.buf = torch.empty(int(lane.wanted * 1.25) + 4096, dtype=torch.uint8, device=self.device)
                lane.views.clear()      # they point into the old buffer
                self._overflow_seen = True
            lane.offset = 0
            lane.wanted = 0
            lane.overflow.clear()
        self.current = self.lanes[0]

    def use(self, lane: int) -> None:
        """Make `lane` current; lanes 1 and 2 start empty again (what they held is dead by now)."""
        self.current = self.lanes[lane]
        if lane != 0:
            self.current.offset = 0

    def take(self, shape, dtype: torch.dtype) -> torch.Tensor:
        lane = self.current
        shape = tuple(shape)
        n = 1
        for s in shape:
            n *= int(s)
        es = dtype.itemsize
        nbytes = (n * es + 255) & ~255
        start = lane.offset
        lane.offset += nbytes
        if lane.offset > lane.wanted:
            lane.wanted = lane.offset
        if lane.offset > lane.buf.numel():
            if self.frozen:
                raise BackendError("workspace is frozen (a graph was captured) and too small for this step")
            t = torch.empty(shape, dtype=dtype, device=self.device)  # this step only; grows at rewind
            lane.overflow.append(t)
            return t
        # the same requests come again every step and every layer: the view of a place is made once
        key = (start, shape, dtype)
        t = lane.views.get(key)
        if t is None:
            if len(lane.views) > 4096:
                lane.views.clear()
            t = lane.views[key] = lane.buf[start:start + n * es].view(dtype).view(shape)
        return t


# Positions per cache page unless a caller asks otherwise: the tile of keys that the attention
# kernels fetch at a time.
DEFAULT_PAGE_SIZE = 64


class Runtime:
    def __init__(self, device, dtype: torch.dtype, page_size: int | None = None):
        page_size = DEFAULT_PAGE_SIZE if page_size is None else int(page_size)
        if dtype not in (torch.float32, torch.bfloat16):
            raise BackendError(f"compute dtype must be float32 or bfloat16, got {dtype}")
        self.device = torch.device(device)
        self.dtype = dtype
        self.page_size = page_size
        self.workspace = Workspace(self.device) if self.device.type == "cuda" else None

"""What every part gets to run with: device, dtypes, page size, a workspace arena."""

from __future__ import annotations

import torch

from ..errors import BackendError


class Workspace:
    """A bump allocator over one device buffer, rewound at the start of every step.

    The same sequence of requests yields the same addresses in every step, which is what a
    captured CUDA graph of the step needs; nothing is allocated while a step runs once the
    buffer has grown to the largest step seen (growth happens between steps, never during capture).
    """

    def __init__(self, device, nbytes: int = 1 << 20):
        self.device = device
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        self.offset = 0
        self.frozen = False
        self._overflow: list = []
        self._overflow_seen = False     # the buffer was replaced since this flag was last cleared
        self._wanted = 0

    def rewind(self) -> None:
        if self._wanted > self.buf.numel() and not self.frozen:
            self.buf = torch.empty(int(self._wanted * 1.25) + 4096, dtype=torch.uint8, device=self.device)
            self._overflow_seen = True
        self.offset = 0
        self._wanted = 0
        self._overflow.clear()

    def take(self, shape, dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        es = torch.empty((), dtype=dtype).element_size()
        nbytes = (n * es + 255) & ~255
        start = self.offset
        self.offset += nbytes
        self._wanted = max(self._wanted, self.offset)
        if self.offset > self.buf.numel():
            if self.frozen:
                raise BackendError("workspace is frozen (a graph was captured) and too small for this step")
            t = torch.empty(tuple(shape), dtype=dtype, device=self.device)  # this step only; grows at rewind
            self._overflow.append(t)
            return t
        return self.buf[start:start + n * es].view(dtype).view(tuple(shape))


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

"""The step's workspace: one device allocation that every activation of a step lives in.

adarsh-sgh/edgelm plans an arena from the live ranges of its graph's tensors
(src/passes.cpp:160-208).  Here layers are put together from parts, and live ranges nest: a
buffer lives for a whole step (the residual stream), for one layer (the normalised input) or
for one part (projections, the feed-forward's middle).  So the arena is a stack: `frame()`
marks the top, `alloc` pushes, leaving the frame pops everything pushed inside it.  Its size is
the sum that the parts declare for the largest step (`workspace_bytes`), fixed when the
engine is built; a step that would need more is a bug and raises.  Equal steps get equal
addresses, which is what CUDA graph replay needs.
"""
import contextlib

import torch

ALIGN = 256


class WorkspaceError(RuntimeError):
    pass


class Workspace:
    def __init__(self, capacity_bytes, device):
        self.capacity = (int(capacity_bytes) + ALIGN - 1) // ALIGN * ALIGN
        self.buffer = torch.empty(self.capacity, dtype=torch.uint8, device=device)
        self.top = 0
        self.peak = 0

    @contextlib.contextmanager
    def frame(self):
        mark = self.top
        try:
            yield
        finally:
            self.top = mark

    def alloc(self, shape, dtype):
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty(0, dtype=dtype).element_size()
        start = self.top
        end = start + (nbytes + ALIGN - 1) // ALIGN * ALIGN
        if end > self.capacity:
            raise WorkspaceError(f"the step's workspace holds {self.capacity} bytes; a buffer of shape {tuple(shape)} "
                                 f"({nbytes} bytes) at offset {start} does not fit (a part declared too little)")
        self.top = end
        self.peak = max(self.peak, end)
        return self.buffer[start:start + nbytes].view(dtype).view(tuple(shape))

    def reset(self):
        self.top = 0

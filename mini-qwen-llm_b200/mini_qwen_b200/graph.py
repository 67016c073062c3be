"""CUDA-graph capture of a block's forward pass for a fixed input shape.

A layer call is a dozen short kernels; launched one by one from Python the host can fall behind the
GPU, and with expert parallelism every late launch on one rank is a wait at the next rank barrier on
all the others.  The forward pass has no host synchronisation (routing, plan and exchange are all
device-side), so it captures into one graph and a step becomes one launch.
"""
from __future__ import annotations

import torch

from . import _cabi


class CapturedForward:
    """``block(x)`` for inputs of ``example``'s shape, captured once and replayed.

    ``self.x`` is the graph's input buffer (copy or upload the step's input into it), ``replay()``
    launches the graph on the current stream and returns the graph's output buffer, which the next
    replay overwrites.  With expert parallelism every rank of the group must construct and replay its
    capture the same number of times (the calls are collective, as the eager forward is).
    Pass another capture's ``pool`` to share its memory pool.
    """

    def __init__(self, block, example: torch.Tensor, warmup: int = 3, pool=None):
        if not example.is_cuda:
            raise ValueError("graph capture needs a CUDA tensor")
        self.block = block
        self.x = example.clone()
        side = torch.cuda.Stream(example.device)
        side.wait_stream(torch.cuda.current_stream(example.device))
        with torch.no_grad(), torch.cuda.stream(side):
            for _ in range(max(1, warmup)):          # first calls allocate buffers and set kernel attributes
                block(self.x)
        torch.cuda.current_stream(example.device).wait_stream(side)
        torch.cuda.synchronize(example.device)
        self.graph = torch.cuda.CUDAGraph()
        before = _cabi.launch_count
        with torch.no_grad(), torch.cuda.graph(self.graph, pool=pool):
            self.out = block(self.x)
        self.launches = _cabi.launch_count - before   # kernels of this library inside one replay

    def pool(self):
        return self.graph.pool()

    def replay(self) -> torch.Tensor:
        self.graph.replay()
        _cabi.count_launches(self.launches)
        return self.out

"""CUDA-graph capture of a fixed sequence of operator calls.

One pass of the selection path is seven short kernels (pooling, scoring + top-k, forward,
inverted index, dQ, dK/dV); launched one by one from Python the host needs longer per launch
than the small ones run, so the device idles between them.  `CapturedStep` records the launches
of `fn()` once - all operator entry points are asynchronous on the current stream, allocate
nothing outside torch's allocator and make no synchronising call, so they can be captured -
and replays them with a single launch.  The tensors `fn` reads must stay at the same addresses
(copy new inputs into them); its results are returned by `replay()` and are overwritten by the
next replay.
"""
from __future__ import annotations

from typing import Any, Callable

import torch


class CapturedStep:
    def __init__(self, fn: Callable[[], Any], warmup: int = 3):
        self._fn = fn
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):        # first calls resolve symbols / set attributes: not capturable
                fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.outputs = fn()

    def replay(self):
        self.graph.replay()
        return self.outputs

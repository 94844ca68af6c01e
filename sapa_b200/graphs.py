"""CUDA-graph capture of an inference callable built from this library's ops (for example a decoder pyramid of chained
``SAPA`` modules): the launches of one forward pass are recorded once and replayed, which removes the per-launch host
cost that dominates small feature levels.  The reference has no counterpart (its extensions launch on the legacy default
stream, which cannot be captured).
"""
from __future__ import annotations

import torch


class GraphedForward:
    """Record ``fn(*example_inputs)`` into a CUDA graph and replay it on new inputs of the same shapes and dtypes.

    ``fn`` must be an inference function of CUDA tensors with static shapes (it runs under ``torch.no_grad()``); every op
    of this library qualifies, and so do torch's own kernels.  ``__call__`` copies the arguments into the captured input
    buffers, replays the graph and returns the captured output tensor(s) - the same storage on every call, so clone what
    must outlive the next call.  Replays of graphs that hold this library's kernels must not overlap each other on one
    device (they keep their tile-scheduler slots): replay on one stream at a time.
    """

    def __init__(self, fn, example_inputs, warmup: int = 3):
        if not all(isinstance(t, torch.Tensor) and t.is_cuda for t in example_inputs):
            raise ValueError("GraphedForward takes CUDA tensors")
        self._inputs = [t.clone() for t in example_inputs]
        self._graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream(device=self._inputs[0].device)
        side.wait_stream(torch.cuda.current_stream(self._inputs[0].device))
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(max(1, warmup)):          # first calls load kernels and size caches: keep them out of the capture
                fn(*self._inputs)
        torch.cuda.current_stream(self._inputs[0].device).wait_stream(side)
        torch.cuda.synchronize(self._inputs[0].device)
        with torch.no_grad(), torch.cuda.graph(self._graph):
            self._output = fn(*self._inputs)

    def __call__(self, *inputs):
        if len(inputs) != len(self._inputs):
            raise ValueError(f"expected {len(self._inputs)} inputs, got {len(inputs)}")
        for dst, src in zip(self._inputs, inputs):
            if dst.shape != src.shape or dst.dtype != src.dtype:
                raise ValueError(f"captured with {tuple(dst.shape)} {dst.dtype}, called with {tuple(src.shape)} {src.dtype}")
            if dst.data_ptr() != src.data_ptr():
                dst.copy_(src)
        self._graph.replay()
        return self._output

    @property
    def inputs(self):
        """The captured input buffers: write into them directly to skip the copy in ``__call__``."""
        return self._inputs

"""CUDA-graph replay of a forward pass.

At small latent sizes (512 px images: 1 024 tokens) a block's kernels finish faster than the
host can launch them - a dozen launches per block, each through Python and ctypes - so the GPU
idles between kernels.  Capturing the whole forward once and replaying the graph removes the
host from the loop.  Every kernel of the library launches on the current stream with
arguments fixed at launch time (tensor maps are passed by value), and its one-time set-up
(function attributes, occupancy queries) happens during the warm-up calls, so the modules
capture as they are.

    fwd = GraphedForward(model, x, timestep, y)        # warm-up + capture with these shapes
    out = fwd(x2, timestep2, y2)                       # copies into the static inputs, replays

The returned tensor is the graph's static output buffer: it is overwritten by the next call.
"""
from __future__ import annotations

from typing import Any, Sequence

import torch


class GraphedForward:
    """Captures ``module(*args, **kwargs)`` into a CUDA graph.  Tensor positional arguments
    become static input buffers (same shapes and dtypes on every call); everything else
    (None, tuples, numbers, keyword arguments) is frozen at capture time."""

    def __init__(self, module, *args: Any, warmup: int = 3, **kwargs: Any):
        if not torch.cuda.is_available():
            raise RuntimeError("GraphedForward needs a CUDA device")
        self.module = module
        self.kwargs = kwargs
        self.static_args = [a.clone() if torch.is_tensor(a) else a for a in args]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(max(1, warmup)):
                module(*self.static_args, **kwargs)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph), torch.no_grad():
            self.static_out = module(*self.static_args, **kwargs)

    def __call__(self, *args: Any):
        if len(args) != len(self.static_args):
            raise ValueError(f"expected {len(self.static_args)} positional arguments, got {len(args)}")
        for dst, src in zip(self.static_args, args):
            if torch.is_tensor(dst):
                if not torch.is_tensor(src) or src.shape != dst.shape or src.dtype != dst.dtype:
                    raise ValueError("graphed forward called with a tensor of another shape or dtype")
                if src.data_ptr() != dst.data_ptr():
                    dst.copy_(src, non_blocking=True)
        self.graph.replay()
        return self.static_out


def static_inputs(fwd: GraphedForward) -> Sequence[Any]:
    """The graph's input buffers (write into them directly to skip the copy in ``__call__``)."""
    return fwd.static_args

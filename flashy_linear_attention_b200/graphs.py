"""CUDA-graph capture of calls into the library.

Every entry point of libflashlinear_sm100 only enqueues kernels on the caller's stream (no
allocation, no synchronisation), so a forward + backward step over fixed buffers can be captured
once and replayed: the launches of a step then cost one graph launch instead of several Python /
ctypes round trips, which matters when a GPU holds few heads (a step of 0.07-0.15 ms).

    step = capture_step(lambda: ops.causal_dot_product_bwd(dy, q, k, v))
    grads = step()        # replays; returns the tensors the captured call returned

Calls whose arguments change between launches cannot be replayed. The peer state exchange is not
one of them when its exchange count lives on the device (`PeerStateExchange` does that), so a
sequence-sharded step can be captured as well.
"""
from __future__ import annotations

from typing import Any, Callable

import torch


class CapturedStep:
    """A captured callable: calling it replays the graph and returns the captured outputs (the
    same tensor objects every time; their contents are overwritten by each replay)."""

    def __init__(self, graph: torch.cuda.CUDAGraph, outputs: Any):
        self.graph = graph
        self.outputs = outputs

    def __call__(self) -> Any:
        self.graph.replay()
        return self.outputs


def capture_step(fn: Callable[[], Any], warmup: int = 2) -> CapturedStep:
    """Runs `fn` `warmup` times on a side stream (so that one-time initialisation and the caching
    allocator's first allocations happen outside the capture), then captures one call."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(max(1, warmup)):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outputs = fn()
    return CapturedStep(graph, outputs)

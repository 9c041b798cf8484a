"""CUDA-graph capture of a whole training step.

One MoE-layer step is ~300 kernel launches; issued eagerly from Python the host needs about as
long as the GPU, so any hiccup on one rank's CPU becomes a bubble on every rank at the next
cross-rank barrier.  Capturing forward + backward + optimizer into one graph removes the host
from the loop.  All kernels of this library can be captured: launches are plain or cooperative
kernel nodes, cross-rank synchronisation happens on the device, shapes are static and the
communication stream is forked from / joined to the capturing stream.  (The reference's benches
time CUDA graphs of its kernels too, benchmarks/bench_comm.py:118-163.)
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch


class GraphedStep:
    """``fn(*static_inputs) -> tensor(s)`` captured once; ``__call__(*inputs)`` copies the inputs
    into the static buffers, replays the graph and returns the static outputs."""

    def __init__(self, fn: Callable, example_inputs: Sequence[torch.Tensor], warmup: int = 3):
        self.static_inputs = [t.clone() for t in example_inputs]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):                       # warm-up off the default stream
            for _ in range(warmup):
                fn(*self.static_inputs)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.static_outputs = fn(*self.static_inputs)

    def __call__(self, *inputs: torch.Tensor):
        for dst, src in zip(self.static_inputs, inputs):
            if dst.data_ptr() != src.data_ptr():
                dst.copy_(src, non_blocking=True)
        self.graph.replay()
        return self.static_outputs

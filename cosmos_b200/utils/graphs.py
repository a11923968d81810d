"""CUDA-graph capture of launch-bound inner loops (the reference runs "with CUDA Graphs enabled
where supported", inference_benchmarks.md:39).

`GraphedCallable` captures one call of a function whose arguments are fixed-shape tensors and
replays it with new data copied into static input buffers. It is meant for the Reasoner's decode
step (dozens of tiny kernels per token) and for small-resolution denoise steps; the 720p denoise
step is compute bound and gains nothing from it.

Capture rules: warm the function up first (lazy initialisation such as workspace allocation,
symmetric-memory set-up or `cudaGetSymbolAddress` look-ups must have happened), no host
synchronisation inside the function, and every kernel on the capturing stream.
"""
from __future__ import annotations

from typing import Callable, List, Sequence

import torch


class GraphedCallable:
    def __init__(self, fn: Callable, example_inputs: Sequence[torch.Tensor], warmup: int = 2):
        assert torch.cuda.is_available(), "CUDA graphs need a GPU"
        self.fn = fn
        self.static_in: List[torch.Tensor] = [t.clone() for t in example_inputs]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(warmup):
                fn(*self.static_in)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(self.graph):
            self.static_out = fn(*self.static_in)

    def __call__(self, *inputs: torch.Tensor):
        for dst, src in zip(self.static_in, inputs):
            dst.copy_(src, non_blocking=True)
        self.graph.replay()
        return self.static_out

"""CUDA-graph replay of a fixed sequence of launches.

A decode step of a stack of MoE layers is dozens of small launches per layer (norm, routing, the fused mat-vec
kernel, the exchange of an expert-parallel rank, the combine); issued one by one from the host they cost more host
time than the GPU needs to run them.  `GraphedCall` records such a sequence once - every launch of this package goes
to torch's current stream, collectives of `torch.distributed` (NCCL) included - and replays it with one call.

The reference has no counterpart: its encoder batches Metal commands per token (src/model.rs:300-410).
"""
from __future__ import annotations

import torch


class GraphedCall:
    """Capture ``fn()`` into a CUDA graph.  ``fn`` takes no arguments, reads and writes tensors that stay where they
    are, allocates only through torch, and makes no host decision that depends on device data.  It is run
    ``warmup`` times first, on the stream the capture uses (lazy initialisations - kernel attributes, communicators,
    workspaces - must not happen inside the capture).  ``replay()`` returns what ``fn`` returned in the capture:
    the same tensors every time, overwritten by each replay."""

    def __init__(self, fn, warmup: int = 2):
        self.stream = torch.cuda.Stream()
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            for _ in range(warmup):
                fn()
        self.stream.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, stream=self.stream, capture_error_mode="thread_local"):
            self.out = fn()

    def replay(self):
        self.graph.replay()
        return self.out

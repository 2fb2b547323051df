"""CUDA graphs for pure-decode steps.

A step in which every request brings one token launches the same kernels with
the same shapes whatever the context lengths are: the kernels read lengths,
positions and block tables from the step's device buffer.  So one graph per
batch bucket (1, 2, 4, ... requests) is captured once and replayed; a replay
costs one upload of the step's metadata and one graph launch instead of a few
hundred kernel launches from Python.  A batch smaller than its bucket is padded
with lanes that read nothing and write nothing: position 0, an all-padding-page
block-table row (the append kernel skips page 0, the attention kernels mask it)
and the spare state slot.  The reference pads its decode graphs the same way
(``runner/paged_runner.py:595-683``) and keeps the sampler outside the graph
(``:556-570``), as here.
"""

from __future__ import annotations

import torch

from .. import ops
from .step import StepEntry


class DecodeGraphs:
    def __init__(self, runner, model, max_requests: int):
        self.runner, self.model = runner, model
        self.max_requests = max_requests
        self.graphs: dict[int, tuple] = {}
        self.launches = 0          # kernels replayed so far
        self.h2d_bytes = 0         # upload of the last replayed step
        self.generation = runner.generation

    def bucket_for(self, n: int) -> int:
        b = 1
        while b < n:
            b *= 2
        return min(b, self.max_requests) if n <= self.max_requests else n

    def _capture(self, bucket: int):
        ctx = self.runner.prepare([], pad_to=bucket)
        self.runner.forward(ctx)                     # eager once: first-use set-up, scratch buffers
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        before = ops.launches
        with torch.cuda.graph(graph):
            logits = self.runner.forward(ctx)
        kernels = ops.launches - before
        entry = (graph, logits, kernels)
        self.graphs[bucket] = entry
        return entry

    def run(self, entries: list[StepEntry], tokens_from: torch.Tensor | None = None, take_rows=None) -> torch.Tensor:
        """Logits [len(entries), V] of a step whose entries all bring one token
        and want its logits.  ``tokens_from``: int32 on the device, the entries'
        tokens in order (their host copies are not known yet): they are copied into
        the step's buffer after its upload."""
        if self.generation != self.runner.generation:     # the step buffer moved: graphs point at the old one
            self.graphs.clear()
            self.generation = self.runner.generation
        n = len(entries)
        bucket = self.bucket_for(n)
        entry = self.graphs.get(bucket) or self._capture(bucket)
        graph, logits, kernels = entry
        ctx = self.runner.prepare(entries, pad_to=bucket, take_rows=take_rows)
        if tokens_from is not None:
            self.runner.place_tokens(ctx, n, tokens_from, take_rows)
        self.h2d_bytes = self.runner.h2d_bytes
        graph.replay()
        self.launches += kernels
        return logits[:n]

"""A decode step driven from host buffers as one CUDA graph.

The serving loop of the reference's host (one writer append + one decode launch per layer and step, workspace allocated
before capture: reference kernels.py:314-327) is launch-bound from Python: three copies, two C calls and one copy back
cost more CPU time than the kernels take.  `HostStep` records that sequence once on a capture stream and replays it with
a single launch; the host buffers stay where they are (pinned), the caller rewrites their contents between replays.
"""
from __future__ import annotations

import torch


class HostStep:
    """copies_in: [(device tensor, pinned host tensor)], body: callable launching the library calls on the current stream,
    copies_out: [(pinned host tensor, device tensor)].  The body must not allocate device memory or synchronise (use a
    Workspace made beforehand) and must have run once before capture (first calls set kernel attributes)."""

    def __init__(self, copies_in, body, copies_out):
        for dst, src in copies_in:
            assert dst.is_cuda and src.is_pinned(), "host -> device copies need pinned host memory"
        for dst, src in copies_out:
            assert dst.is_pinned() and src.is_cuda, "device -> host copies need pinned host memory"
        self.h2d_bytes = sum(s.numel() * s.element_size() for _, s in copies_in)
        self.d2h_bytes = sum(s.numel() * s.element_size() for _, s in copies_out)
        self.graph = torch.cuda.CUDAGraph()
        torch.cuda.synchronize()
        with torch.cuda.graph(self.graph):
            for dst, src in copies_in:
                dst.copy_(src, non_blocking=True)
            body()
            for dst, src in copies_out:
                dst.copy_(src, non_blocking=True)

    def launch(self):
        """asynchronous replay on the current stream"""
        self.graph.replay()

    def run(self):
        """replay and wait until the outputs are in host memory"""
        self.graph.replay()
        torch.cuda.current_stream().synchronize()

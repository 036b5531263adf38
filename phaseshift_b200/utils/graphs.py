"""CUDA graph capture that is safe against Python's cycle collector.

Destroying an old ``torch.cuda.CUDAGraph`` releases its executable graph and memory pool with calls that are
illegal while ANY stream of the process is capturing; if the cycle collector happens to free a dead engine (its
graphs, its tensors) in the middle of a capture, the capture is invalidated and the next launch fails with
cudaErrorStreamCaptureImplicit.  So: collect before the capture, and keep the collector off while it runs.
"""
from __future__ import annotations

import gc
from typing import Callable, Tuple

import torch


def capture(device, fn: Callable[[], object]) -> Tuple["torch.cuda.CUDAGraph", object]:
    """Capture ``fn()`` (launches on the current stream) into a new graph; returns (graph, fn's result)."""
    gc.collect()
    was_enabled = gc.isenabled()
    gc.disable()
    try:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=torch.cuda.Stream(device)):
            out = fn()
    finally:
        if was_enabled:
            gc.enable()
    return g, out

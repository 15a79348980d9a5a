"""Recording a step's launches into a CUDA graph.

While a stream is capturing, destroying another CUDA graph is not permitted and invalidates the capture.  Graphs
of engines that are no longer used sit in dead reference cycles until Python's cycle collector runs, and it runs
whenever enough objects have been allocated, so it can run in the middle of a capture.  Hence: collect first,
and keep the collector paused until the capture has ended.
"""
from __future__ import annotations

import contextlib
import gc

import torch


@contextlib.contextmanager
def capture(graph: torch.cuda.CUDAGraph):
    gc.collect()
    was_enabled = gc.isenabled()
    gc.disable()
    try:
        with torch.cuda.graph(graph):
            yield
    finally:
        if was_enabled:
            gc.enable()

"""CUDA-graph capture that the garbage collector cannot invalidate.

Destroying a ``torch.cuda.CUDAGraph`` is a CUDA call that is not permitted while ANY stream of the process captures
(the default capture mode is global).  Graph holders that sit in reference cycles - a module whose ``forward`` was
replaced by a bound method of its own graph container, an engine kept alive by a closure - are freed by the cyclic
collector at an arbitrary later allocation, which may fall inside somebody else's capture and invalidates it.
``graph_capture`` collects such garbage BEFORE the capture starts and keeps the cyclic collector off until it ends."""
from __future__ import annotations

import contextlib
import gc

import torch


@contextlib.contextmanager
def graph_capture(graph: torch.cuda.CUDAGraph, pool=None, **kwargs):
    was_enabled = gc.isenabled()
    gc.collect()
    gc.disable()
    try:
        with torch.cuda.graph(graph, pool, **kwargs):
            yield
    finally:
        if was_enabled:
            gc.enable()

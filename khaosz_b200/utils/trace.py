"""NVTX ranges around the phases of a step (reference: none - ``astrai`` has no tracing hooks).

Off by default; ``KHAOSZ_B200_NVTX=1`` (or ``enable_tracing()``) turns the ranges on so that a
timeline profiler shows micro-steps, optimizer steps, prefill and decode calls by name.  A
disabled range costs one attribute lookup.
"""

from __future__ import annotations

import contextlib
import os

_ENABLED = os.environ.get("KHAOSZ_B200_NVTX", "0") == "1"


def enable_tracing(flag: bool = True) -> None:
    global _ENABLED
    _ENABLED = bool(flag)


def tracing_enabled() -> bool:
    return _ENABLED


@contextlib.contextmanager
def _nvtx(name: str):
    import torch

    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


_NULL = contextlib.nullcontext()


def trace_range(name: str):
    """Context manager: an NVTX range when tracing is enabled and CUDA is present, else a no-op."""
    if not _ENABLED:
        return _NULL
    import torch

    return _nvtx(name) if torch.cuda.is_available() else _NULL

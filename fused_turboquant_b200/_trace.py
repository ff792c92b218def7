"""Optional NVTX ranges around the library's launches, and the package loggers.

The reference times with wall clocks / CUDA events only and logs through
``logging.getLogger(__name__)`` (src/fused_turboquant/hf/fused_cache.py:42,
vllm_plugin/v1_backend.py:67).  Here every module logs under its own name in the
``fused_turboquant_b200`` hierarchy, and setting ``FTQ_NVTX=1`` before the import
wraps store / decode / all-gather calls in NVTX ranges (``ftq.store``,
``ftq.decode``, ``ftq.all_gather``), which a system profiler shows on the
launching thread.  Off by default: the ranges are host-side calls on the launch
path.
"""
from __future__ import annotations

import contextlib
import logging
import os

ENABLED = os.environ.get("FTQ_NVTX", "0") not in ("", "0")


def get_logger(name: str) -> logging.Logger:
    return logging.getLogger(name)


@contextlib.contextmanager
def _nvtx_range(name: str):
    import torch

    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


_NULL = contextlib.nullcontext()


def nvtx(name: str):
    """Context manager: an NVTX range when FTQ_NVTX is set, else nothing."""
    return _nvtx_range(name) if ENABLED else _NULL

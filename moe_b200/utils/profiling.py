"""NVTX ranges per phase of a training step (attention, experts, loss head, gradient reduce, optimizer).

Off by default: `enable()` is called by `train.py --profile`; `phase(name)` is then a context manager that
pushes / pops an NVTX range on CUDA and does nothing otherwise.  The ranges are for a timeline viewer; numbers
reported by this repository are always taken with CUDA events outside of any profiler."""
from __future__ import annotations

import contextlib

_ENABLED = False


def enable(on: bool = True) -> None:
    global _ENABLED
    _ENABLED = bool(on)


def enabled() -> bool:
    return _ENABLED


@contextlib.contextmanager
def phase(name: str):
    if not _ENABLED:
        yield
        return
    import torch

    if not torch.cuda.is_available():
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()

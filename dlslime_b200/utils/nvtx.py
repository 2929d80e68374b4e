"""NVTX ranges for host-side API calls (shows up in Nsight timelines); no-ops without CUDA.

Counterpart of the reference's ``NvtxScope`` / ``NVTX_RANGE`` helper (``dlslime/csrc/device/cuda/nvtx_helper.h:17-38``
in the reference), for the Python layer that launches the kernels here.
"""

from __future__ import annotations

import contextlib
import functools

import torch


@contextlib.contextmanager
def nvtx_range(name: str):
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


def nvtx_annotate(name: str | None = None):
    """Decorator form: the call is wrapped in a range named after the function."""

    def wrap(fn):
        label = name or fn.__qualname__

        @functools.wraps(fn)
        def inner(*a, **k):
            with nvtx_range(label):
                return fn(*a, **k)

        return inner

    return wrap

"""Profiler ranges around the stages of a lowered optimizer step.

Off by default (a no-op costing one attribute test per stage).  ``HB200_NVTX=1`` in the environment, or
``tracing.enable()``, pushes an NVTX range per stage - ``momentum``, ``ns/<rows>x<cols>``, ``update``, ``soap.project``,
``soap.refresh``, ``psgd.apply``, ``psgd.fit``, ``peer.begin``, ``peer.end`` - so a timeline shows where a step spends its
time.  The ranges are also recorded by ``torch.profiler`` (as user annotations) when it is active.
"""

from __future__ import annotations

import contextlib
import os

import torch

enabled = os.environ.get("HB200_NVTX") == "1"
seen = []  # names of the ranges opened since the last ``seen.clear()`` (tests, and a cheap textual trace)
record_names = False


def enable(on: bool = True, record: bool = False):
    global enabled, record_names
    enabled, record_names = on, record


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NULL = _Null()


@contextlib.contextmanager
def _range(name: str):
    if record_names:
        seen.append(name)
    use_nvtx = torch.cuda.is_available()
    if use_nvtx:
        torch.cuda.nvtx.range_push(name)
    try:
        with torch.profiler.record_function(f"hb200::{name}"):
            yield
    finally:
        if use_nvtx:
            torch.cuda.nvtx.range_pop()


def stage(name: str):
    """Context manager for one stage of a step; free when tracing is off."""
    return _range(name) if enabled else _NULL

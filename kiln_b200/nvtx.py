"""NVTX ranges around the library's GPU calls, the counterpart of kiln's `kiln-nvtx` crate
(kiln-nvtx/src/lib.rs:26-84; call sites such as kiln-model/src/forward.rs:2772, 2801, 2830).

Off by default, like the crate's cargo feature: `range(name)` is then an empty context manager.  Setting the
environment variable KILN_NVTX=1 before the first call turns the ranges on (they show up as named spans in a profiler
timeline)."""
from __future__ import annotations

import contextlib
import os

_enabled = os.environ.get("KILN_NVTX", "0") not in ("", "0")
_push = _pop = None


def enable(on: bool = True, push=None, pop=None) -> None:
    """Switches the ranges on or off at run time; `push` / `pop` replace torch.cuda.nvtx (tests pass recorders)."""
    global _enabled, _push, _pop
    _enabled = bool(on)
    _push, _pop = push, pop


@contextlib.contextmanager
def range(name: str):  # noqa: A001 - named after the crate's `range!` macro
    if not _enabled:
        yield
        return
    push, pop = _push, _pop
    if push is None:
        import torch

        push, pop = torch.cuda.nvtx.range_push, torch.cuda.nvtx.range_pop
    push(name)
    try:
        yield
    finally:
        pop()

"""Tracing hooks: NVTX ranges and CUDA-event phase timers.

Off by default (a range then costs one attribute test). `BDH_NVTX=1` or `enable(nvtx=True)` wraps
every kernel launch of this library and every phase of the fused model path (embedding, each
layer's forward / backward, head + loss, optimizer, collectives) in an NVTX range, so a timeline
tool shows the step structure. `enable(timers=True)` additionally brackets the phases with CUDA
events on the launching stream; `report()` synchronises once and returns device milliseconds and
call counts per phase (nested phases are reported under their own names; nothing is subtracted).
The reference only logs lines and an analytic FLOP count (src/bin/train.rs:635-659).
"""
from __future__ import annotations

import os
from contextlib import contextmanager
from typing import Dict, List, Tuple

import torch

_cfg = {"nvtx": os.environ.get("BDH_NVTX", "0") == "1", "timers": False}
_events: List[Tuple[str, "torch.cuda.Event", "torch.cuda.Event"]] = []


def enable(nvtx: bool = None, timers: bool = None) -> None:
    if nvtx is not None:
        _cfg["nvtx"] = bool(nvtx)
    if timers is not None:
        _cfg["timers"] = bool(timers)
        if not timers:
            _events.clear()


def active() -> bool:
    return _cfg["nvtx"] or _cfg["timers"]


def nvtx_on() -> bool:
    return _cfg["nvtx"]


@contextmanager
def phase(name: str):
    """Mark a phase of the step. No-op unless tracing is enabled and a CUDA device is in use."""
    if not active() or not torch.cuda.is_available():
        yield
        return
    ev = None
    if _cfg["timers"]:
        ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        ev[0].record()
    if _cfg["nvtx"]:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if _cfg["nvtx"]:
            torch.cuda.nvtx.range_pop()
        if ev is not None:
            ev[1].record()
            _events.append((name, ev[0], ev[1]))


def report(reset: bool = True) -> Dict[str, Dict[str, float]]:
    """{phase: {"ms": total device time, "calls": n}} for everything recorded since the last reset."""
    out: Dict[str, Dict[str, float]] = {}
    if _events:
        torch.cuda.synchronize()
    for name, a, b in _events:
        d = out.setdefault(name, {"ms": 0.0, "calls": 0})
        d["ms"] += a.elapsed_time(b)
        d["calls"] += 1
    if reset:
        _events.clear()
    return out

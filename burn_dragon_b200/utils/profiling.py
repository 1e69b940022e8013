"""Tracing hooks: NVTX ranges and CUDA-event phase timers.

Off by default (a range then costs one attribute test). `BDH_NVTX=1` or `enable(nvtx=True)` wraps
every kernel launch of this library and every phase of the fused model path (embedding, each
layer's forward / backward, head + loss, optimizer, collectives) in an NVTX range, so a timeline
tool shows the step structure. `enable(timers=True)` additionally brackets the phases with CUDA
events on the launching stream; `report()` synchronises once and returns device milliseconds and
call counts per phase (nested phases are reported under their own names; nothing is subtracted).
Without a CUDA device the timers fall back to the host clock (CPU ops are synchronous), so that
the phase structure of a step can be read on gloo ranks too. Phases named `comm.*` (and
`grad_reduce`) are the collectives that are NOT hidden inside a compute kernel: `comm_ms()` adds
them up for the "exposed communication" column of the metrics log.
The reference only logs lines and an analytic FLOP count (src/bin/train.rs:635-659).
"""
from __future__ import annotations

import os
import time
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
    """Mark a phase of the step. No-op unless tracing is enabled."""
    if not active():
        yield
        return
    if not torch.cuda.is_available():
        if not _cfg["timers"]:
            yield
            return
        t0 = time.perf_counter()
        try:
            yield
        finally:
            _events.append((name, t0, time.perf_counter()))
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
    if _events and torch.cuda.is_available():
        torch.cuda.synchronize()
    for name, a, b in _events:
        d = out.setdefault(name, {"ms": 0.0, "calls": 0})
        d["ms"] += (b - a) * 1e3 if isinstance(a, float) else a.elapsed_time(b)
        d["calls"] += 1
    if reset:
        _events.clear()
    return out


def timers_on() -> bool:
    return _cfg["timers"]


def comm_ms(rep: Dict[str, Dict[str, float]]) -> float:
    """Exposed communication of a report: the collectives that run as launches of their own (gradient
    all-reduce, reduce-scatter + AdamW + all-gather, the gather half of a tensor-parallel reduction,
    NCCL calls). Communication done by a GEMM epilogue is inside the compute phases by design."""
    return sum(v["ms"] for k, v in rep.items() if k == "grad_reduce" or k.startswith("comm."))

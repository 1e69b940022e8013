"""Loader for the compiled sm_100a extension (`torch.ops.bdh.*`).

`available()` is True only when a CUDA device is present and the library loaded. On a machine
with a GPU a missing or unloadable library is an error, never a silent fallback: the torch
definitions in `ops.reference` exist for CPU runs and as numerical oracles, not as a GPU path.
"""
from __future__ import annotations

import os
import threading

import torch

from ..utils import profiling as prof

_lock = threading.Lock()
_state = {"loaded": False, "error": None}


def load(build_if_missing: bool = True) -> bool:
    """Load `_C.so` into the process (idempotent). Returns True when torch.ops.bdh is usable."""
    with _lock:
        if _state["loaded"]:
            return True
        from .. import build as _build

        try:
            checked = os.environ.get("BDH_CHECKED_KERNELS", "0") == "1"     # the bounds-checked build
            if build_if_missing:
                path = _build.ensure_built(checked=checked)
            else:
                path = _build.LIB_CHECKED if checked else _build.LIB
                if not path.exists():
                    raise FileNotFoundError(path)
            torch.ops.load_library(str(path))
            _state["loaded"] = True
        except Exception as e:  # noqa: BLE001 - reported to the caller below
            _state["error"] = e
            if torch.cuda.is_available() and os.environ.get("BDH_ALLOW_NO_NATIVE", "0") != "1":
                raise RuntimeError(
                    "burn_dragon_b200: the sm_100a extension could not be loaded on a machine with a GPU; "
                    "run `python -m burn_dragon_b200.build`"
                ) from e
            return False
        return True


def available() -> bool:
    """True when kernels can actually run: a CUDA device exists and the extension is loaded."""
    if not torch.cuda.is_available():
        return False
    return load()


def status_code() -> int:
    """Read the device status word (synchronises). Non-zero means an in-kernel wait gave up."""
    if not available():
        return 0
    return int(torch.ops.bdh.status()[0].item())


def clear_status() -> None:
    if available():
        torch.ops.bdh.status().zero_()


BOUNDS_SITES = {1: "embed_ln_fwd: token id", 2: "embed_ln_bwd: token id", 3: "cross_entropy: target id",
                4: "graph_spmm_relu: column block"}


def bounds_violations(clear: bool = True) -> list:
    """Checked build (`BDH_CHECKED_KERNELS=1`): the first out-of-range data-dependent index each group
    of kernels has seen since the last clear, as dicts {site, index, extent, where}; empty when the
    run was clean. Raises when the loaded library was built without the checks. Synchronises."""
    if not available():
        return []
    rec = torch.ops.bdh.bounds_records(bool(clear)).tolist()
    if not all(r[0] for r in rec):
        raise RuntimeError("this process loaded the unchecked library; set BDH_CHECKED_KERNELS=1 before the first kernel call")
    return [dict(site=BOUNDS_SITES.get(r[1], str(r[1])), index=r[2], extent=r[3], where=r[4]) for r in rec if r[1]]


class _CountingOps:
    """`torch.ops.bdh` with a launch counter: every call through this proxy launches exactly one of
    this library's kernels, so `launch_count()` is the number of own kernels launched so far."""

    def __init__(self):
        self.count = 0

    def __getattr__(self, name):
        load()
        fn = getattr(torch.ops.bdh, name)

        def call(*a, **k):
            self.count += 1
            if prof.nvtx_on():
                torch.cuda.nvtx.range_push("bdh." + name)
                try:
                    return fn(*a, **k)
                finally:
                    torch.cuda.nvtx.range_pop()
            return fn(*a, **k)

        self.__dict__[name] = call
        return call


ops = _CountingOps()


def launch_count() -> int:
    return ops.count

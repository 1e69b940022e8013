"""A memory pool of compressible device memory for the kernel path's [tokens, neurons] activations.

`BDH_COMPRESS_ACT=1` makes `ops/fused_bdh.py` allocate its large bf16 activation tensors from a
`torch.cuda.MemPool` whose segments are created with generic compute-data compression
(`csrc/comp_alloc.cu`): the memory system then compresses the ReLU-sparse streams between L2 and HBM.
Off by default; `stats()` reports how much of the pool the driver accepted as compressible. The reference has
no counterpart (its tensors live in Burn's backend allocator).
"""
from __future__ import annotations

import contextlib
import ctypes
import os
from typing import Optional

import torch

_state = {"tried": False, "pool": None, "lib": None, "alloc": None}
MIN_BYTES = 32 << 20          # only streams much larger than a cache line's worth of bookkeeping go to the pool


def enabled() -> bool:
    return os.environ.get("BDH_COMPRESS_ACT", "0") == "1"


def pool() -> Optional["torch.cuda.MemPool"]:
    """The pool, or None when the switch is off, there is no GPU, or the device offers no compression."""
    if _state["tried"]:
        return _state["pool"]
    _state["tried"] = True
    if not enabled() or not torch.cuda.is_available():
        return None
    from .. import build as _build
    from ..ops import native
    if not native.load():
        return None
    lib = ctypes.CDLL(str(_build.LIB))
    lib.bdh_comp_supported.argtypes = [ctypes.c_int]
    if lib.bdh_comp_supported(torch.cuda.current_device()) != 1:
        return None
    alloc = torch.cuda.memory.CUDAPluggableAllocator(str(_build.LIB), "bdh_comp_alloc", "bdh_comp_free")
    _state["lib"], _state["alloc"] = lib, alloc
    _state["pool"] = torch.cuda.MemPool(alloc.allocator())
    return _state["pool"]


def allocate(nbytes: int):
    """Context manager: allocations of the current thread inside it come from the compressible pool when it
    is available and the tensor is large enough, else from the ordinary allocator."""
    p = pool() if nbytes >= MIN_BYTES else None
    return torch.cuda.use_mem_pool(p) if p is not None else contextlib.nullcontext()


def stats() -> dict:
    """{'bytes': held by the pool, 'compressible_bytes': of them accepted as compressible by the driver}."""
    lib = _state["lib"]
    if lib is None:
        return dict(bytes=0, compressible_bytes=0)
    out = (ctypes.c_longlong * 2)()
    lib.bdh_comp_stats(out)
    return dict(bytes=int(out[0]), compressible_bytes=int(out[1]))

"""Symmetric memory (peer-mapped buffers + NVSwitch multicast) and the collectives built on it.

Allocation and rendezvous use torch's symmetric-memory manager (CUDA VMM handles exchanged over
the process group's store); everything that touches the memory afterwards is this library's own
kernels (`csrc/collectives.cu`): the data-parallel gradient all-reduce fused with the 1/world
scale, and the reduce-scatter + AdamW + parameter all-gather used by the sharded optimizer.

`BDH_NO_MULTIMEM=1` forces plain peer loads/stores even when the fabric offers multicast (used by
the rank-failure tests, where a dying rank must not be bound to a multicast object).
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import native

COLL_CTAS = 64
_FLAG_WORDS = 8192


class SymmetricBuffer:
    """A tensor allocated in symmetric memory plus every rank's mapping of it."""

    def __init__(self, numel: int, dtype: torch.dtype, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        try:
            symm_mem.enable_symm_mem_for_group(self.group.group_name)
        except Exception:  # noqa: BLE001 - newer torch versions do not need (or have) this call
            pass
        self.tensor = symm_mem.empty(numel, dtype=dtype, device=device)
        self.handle = symm_mem.rendezvous(self.tensor, self.group)
        self.rank = int(self.handle.rank)
        self.world = int(self.handle.world_size)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        mc = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        if os.environ.get("BDH_NO_MULTIMEM", "0") == "1":
            mc = 0
        self.multicast_ptr = mc

    def barrier(self) -> None:
        torch.cuda.synchronize()
        dist.barrier(group=self.group)


class _Flags:
    """Zero-initialised symmetric flag words and the call epoch shared by every collective on a group."""

    _cache = {}

    @classmethod
    def get(cls, device, group):
        key = (str(device), getattr(group, "group_name", "world"))
        if key not in cls._cache:
            buf = SymmetricBuffer(_FLAG_WORDS, torch.int32, device, group)
            buf.tensor.zero_()
            buf.barrier()
            cls._cache[key] = dict(buf=buf, epoch=0)
        return cls._cache[key]


class SymmetricAllReduce:
    """In-place `t <- scale * sum_ranks t` for an fp32 buffer that lives in symmetric memory.

    Construction allocates a symmetric buffer of the same size as `like`; callers re-point their
    gradient views at `self.tensor` (see `parallel.ddp.DataParallel`)."""

    def __init__(self, like: torch.Tensor, group=None):
        if not native.available():
            raise RuntimeError("symmetric all-reduce needs the sm_100a extension")
        world = dist.get_world_size(group)
        n = like.numel()
        pad = (-n) % (4 * world)
        self.numel = n + pad
        self.buf = SymmetricBuffer(self.numel, torch.float32, like.device, group)
        self.tensor = self.buf.tensor
        self.tensor.zero_()
        self.flags = _Flags.get(like.device, self.buf.group)
        self.buf.barrier()

    def all_reduce_(self, scale: float = 1.0) -> None:
        f = self.flags
        f["epoch"] += 1
        b = self.buf
        native.ops.allreduce_scale(self.tensor, b.ptrs, f["buf"].ptrs, b.multicast_ptr, b.rank, b.world,
                                   self.numel, float(scale), f["epoch"], COLL_CTAS)


class ShardedAdamW:
    """Optimizer-state sharding over a data-parallel group (ZeRO style), one kernel per step:
    gradients are reduce-scattered over NVLink inside the kernel, the owner of each slice applies
    AdamW to its fp32 master slice, and the refreshed bf16 parameters are written to every rank.

    `grad` (fp32) and `shadow` (bf16) are full-size symmetric buffers; `master`, `m`, `v` hold the
    local slice only."""

    def __init__(self, master_full: torch.Tensor, group=None, lr=1e-3, weight_decay=0.1, beta1=0.9, beta2=0.999,
                 eps=1e-5):
        world = dist.get_world_size(group)
        rank = dist.get_rank(group)
        dev = master_full.device
        n = master_full.numel()
        pad = (-n) % (4 * world)
        self.numel = n + pad
        self.grad_buf = SymmetricBuffer(self.numel, torch.float32, dev, group)
        self.shadow_buf = SymmetricBuffer(self.numel, torch.bfloat16, dev, group)
        self.grad, self.shadow = self.grad_buf.tensor, self.shadow_buf.tensor
        self.grad.zero_()
        per = self.numel // world
        self.lo = per * rank
        self.hi = self.numel if rank == world - 1 else self.lo + per
        full = torch.zeros(self.numel, dtype=torch.float32, device=dev)
        full[:n].copy_(master_full.reshape(-1))
        self.master = full[self.lo:self.hi].clone()
        self.shadow.copy_(full)
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self.lr, self.weight_decay, self.beta1, self.beta2, self.eps = lr, weight_decay, beta1, beta2, eps
        self.step_count = 0
        self.world, self.rank = world, rank
        self.flags = _Flags.get(dev, self.grad_buf.group)
        self.grad_buf.barrier()

    @torch.no_grad()
    def step(self, lr: Optional[float] = None) -> None:
        self.step_count += 1
        f = self.flags
        f["epoch"] += 1
        g, s = self.grad_buf, self.shadow_buf
        native.ops.rs_adamw_ag(self.grad, g.ptrs, f["buf"].ptrs, g.multicast_ptr, s.ptrs, g.rank, g.world,
                               self.numel, self.master, self.m, self.v, float(self.lr if lr is None else lr),
                               self.beta1, self.beta2, self.eps, self.weight_decay, self.step_count,
                               1.0 / self.world, f["epoch"], COLL_CTAS)

    def zero_grad(self) -> None:
        self.grad.zero_()

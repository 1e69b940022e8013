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
import weakref
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import native

COLL_CTAS = 64
_FLAG_WORDS = 8192


GUARD_BYTES = 256 if os.environ.get("BDH_CHECKED_KERNELS", "0") == "1" else 0
CANARY = 0x5AFEC0DE
_LIVE = weakref.WeakSet()


class SymmetricBuffer:
    """A tensor allocated in symmetric memory plus every rank's mapping of it.

    In the checked configuration (`BDH_CHECKED_KERNELS=1`) the allocation is `GUARD_BYTES` larger
    at both ends and the guards hold a canary pattern: a peer (or a local kernel) that writes
    outside the window it was given lands in a guard instead of in a neighbouring allocation, and
    `check_canaries()` finds it afterwards. `tensor`, `ptrs` and `multicast_ptr` all address the
    interior, so nothing else knows about the guards; with a zero guard the layout is the plain one."""

    def __init__(self, numel: int, dtype: torch.dtype, device, group=None, guard_bytes: Optional[int] = None):
        self.group = group if group is not None else dist.group.WORLD
        guard = GUARD_BYTES if guard_bytes is None else int(guard_bytes)
        item = torch.empty((), dtype=dtype).element_size()
        if guard % 16 or guard % item:
            raise ValueError("guard_bytes must be a multiple of 16 and of the element size")
        ge = guard // item
        if guard:
            numel_alloc = numel + (-numel * item % 16) // item      # the upper guard starts on a 16-byte boundary
        else:
            numel_alloc = numel
        raw, ptrs, mc, self.rank, self.world = self._allocate(numel_alloc + 2 * ge, dtype, device)
        self.raw, self.guard_bytes = raw, guard
        self.tensor = raw[ge:ge + numel]
        self.ptrs = [int(p) + guard for p in ptrs]
        if os.environ.get("BDH_NO_MULTIMEM", "0") == "1":
            mc = 0
        self.multicast_ptr = int(mc) + guard if mc else 0
        if guard:
            for g in self._guards():
                g.fill_(CANARY)
            _LIVE.add(self)

    def _allocate(self, numel: int, dtype: torch.dtype, device):
        """-> (tensor in symmetric memory, every rank's pointer to it, multicast pointer or 0, rank, world)."""
        import torch.distributed._symmetric_memory as symm_mem
        import warnings
        try:
            with warnings.catch_warnings():
                warnings.simplefilter("ignore", FutureWarning)      # (deprecated where it is no longer needed)
                symm_mem.enable_symm_mem_for_group(self.group.group_name)
        except Exception:  # noqa: BLE001 - newer torch versions do not need (or have) this call
            pass
        raw = symm_mem.empty(numel, dtype=dtype, device=device)
        self.handle = symm_mem.rendezvous(raw, self.group)
        return (raw, [int(p) for p in self.handle.buffer_ptrs], int(getattr(self.handle, "multicast_ptr", 0) or 0),
                int(self.handle.rank), int(self.handle.world_size))

    def _guards(self):
        ge = self.guard_bytes // self.raw.element_size()
        if ge == 0:
            return []
        return [self.raw[:ge].view(torch.int32), self.raw[self.raw.numel() - ge:].view(torch.int32)]

    def check_canaries(self) -> list:
        """Guard words of THIS rank's copy that no longer hold the pattern, as (side, word index, value)."""
        bad = []
        for side, g in zip(("below", "above"), self._guards()):
            for i in (g != CANARY).nonzero().flatten().tolist():
                bad.append((side, i, int(g[i]) & 0xFFFFFFFF))
        return bad

    def barrier(self) -> None:
        torch.cuda.synchronize()
        dist.barrier(group=self.group)


def check_all_canaries() -> int:
    """Checked configuration: verify the guards of every live symmetric buffer of this process (after
    a device synchronise, so that every collective launched so far has finished). Returns how many
    buffers were checked; raises when one has been written outside its window."""
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    n = 0
    for buf in list(_LIVE):
        bad = buf.check_canaries()
        if bad:
            raise RuntimeError(f"symmetric buffer of {buf.tensor.numel()} x {buf.tensor.dtype} on rank {buf.rank}: "
                               f"{len(bad)} guard words overwritten, first {bad[0]}")
        n += 1
    return n


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

    def all_reduce_(self, scale: float = 1.0, offset: int = 0, numel: Optional[int] = None) -> None:
        """The whole buffer, or the window [offset, offset + numel) of it (both multiples of 4 * world floats
        and of 4 floats respectively): small replicated tensors inside a larger gradient buffer."""
        f = self.flags
        f["epoch"] += 1
        b = self.buf
        n = self.numel if numel is None else int(numel)
        ptrs = b.ptrs if not offset else [p + 4 * offset for p in b.ptrs]
        mc = b.multicast_ptr + 4 * offset if (b.multicast_ptr and offset) else b.multicast_ptr
        native.ops.allreduce_scale(self.tensor, ptrs, f["buf"].ptrs, mc, b.rank, b.world, n, float(scale), f["epoch"],
                                   COLL_CTAS if n >= (1 << 20) else 8)


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
    def step(self, lr: Optional[float] = None, grad_scale: float = 1.0) -> None:
        """`grad_scale` multiplies the 1/world of the reduction (1/n after n accumulated micro-batches)."""
        self.step_count += 1
        f = self.flags
        f["epoch"] += 1
        g, s = self.grad_buf, self.shadow_buf
        native.ops.rs_adamw_ag(self.grad, g.ptrs, f["buf"].ptrs, g.multicast_ptr, s.ptrs, g.rank, g.world,
                               self.numel, self.master, self.m, self.v, float(self.lr if lr is None else lr),
                               self.beta1, self.beta2, self.eps, self.weight_decay, self.step_count,
                               float(grad_scale) / self.world, f["epoch"], COLL_CTAS)

    def zero_grad(self) -> None:
        self.grad.zero_()

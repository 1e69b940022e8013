"""Data parallelism over a flat gradient buffer.

The reference trains on a single device only (src/bin/train.rs:395); this is new capability.
Because every parameter's gradient lives in one contiguous fp32 buffer (engine.optim.FlatParams)
and the BDH weights are shared by all layers (their gradients are complete only when the whole
backward has finished), gradient reduction is one collective over one pointer, followed by the
AdamW kernel that folds in the 1/world scale.

Two reductions are available:
  nccl   torch.distributed all_reduce (the measured baseline)
  fused  the in-kernel NVLink reduction of parallel.symm (peer loads, or multimem through NVSwitch)
         fused with the 1/world scale; falls back to nccl when symmetric memory is unavailable
"""
from __future__ import annotations


import torch.distributed as dist

from . import dist_utils


class DataParallel:
    def __init__(self, flat, mode: str = "fused", group=None):
        self.flat = flat
        self.group = group
        self.world = dist_utils.world_size()
        self.mode = mode if self.world > 1 else "none"
        self._symm = None
        self.fallback_reason = None
        if self.mode == "fused":
            try:
                from . import symm
                self._symm = symm.SymmetricAllReduce(flat.grad, group=group)
            except Exception as e:  # noqa: BLE001 - recorded, baseline path is used instead
                self.fallback_reason = repr(e)
            # the mode is a collective decision: one rank without symmetric memory sends every rank to NCCL
            if dist_utils.all_agree(self._symm is not None, group, flat.grad.device):
                # gradients now accumulate directly in symmetric memory, so the reduction needs no copy
                flat.grad = self._symm.tensor[:flat.numel]
                flat.zero_grad()
            else:
                self.fallback_reason = self.fallback_reason or "a peer rank could not set up symmetric memory"
                self._symm = None
                self.mode = "nccl"
                if dist_utils.rank() == 0:
                    print(f"DataParallel: fused NVLink all-reduce unavailable, using NCCL ({self.fallback_reason})",
                          flush=True)

    def broadcast_parameters(self) -> None:
        """Make every rank start from rank 0's weights."""
        if self.world > 1:
            dist.broadcast(self.flat.master, src=0, group=self.group)
            self.flat.refresh_shadow()

    def reduce_gradients(self) -> float:
        """Sum gradients over ranks in place. Returns the scale the optimizer must apply (1/world)."""
        if self.world == 1:
            return 1.0
        if self.mode == "fused" and self._symm is not None:
            self._symm.all_reduce_(scale=1.0 / self.world)
            return 1.0
        dist.all_reduce(self.flat.grad, op=dist.ReduceOp.SUM, group=self.group)
        return 1.0 / self.world

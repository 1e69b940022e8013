"""Data parallelism over a flat gradient buffer.

The reference trains on a single device only (src/bin/train.rs:395); this is new capability.
Because every parameter's gradient lives in one contiguous fp32 buffer (engine.optim.FlatParams)
and the BDH weights are shared by all layers (their gradients are complete only when the whole
backward has finished), gradient reduction is one collective over one pointer, followed by the
AdamW kernel that folds in the 1/world scale.

Three reductions are available:
  nccl      torch.distributed all_reduce (the measured baseline)
  fused     the in-kernel NVLink all-reduce of parallel.symm (peer loads, or multimem through NVSwitch) fused with
            the 1/world scale, one launch after the backward pass
  epilogue  (BDH models whose [H*N, D] weights split into 128-row blocks per rank; what `fused` becomes when it
            can) the reduce-scatter half happens INSIDE the backward pass: the weights are shared by the layers, so
            their gradients are complete at layer 0, the last layer of the backward pass; its three weight-gradient
            GEMMs take up the local sum of the other layers in their epilogues and add the tiles into the slice of
            the gradient their owner rank holds (`red.add` over NVLink, the sink of parallel/fsdp.py), overlapped
            tile by tile with the rest of layer 0's backward pass; afterwards one kernel (`shard_bcast`) scales each owner's slice by 1/world and writes it into every
            rank's gradient buffer (multimem.st), and the two small replicated tensors are all-reduced in place.
Falls back to nccl when symmetric memory is unavailable (decided collectively).
"""
from __future__ import annotations


import torch
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
                self._try_epilogue_reduction()
            else:
                self.fallback_reason = self.fallback_reason or "a peer rank could not set up symmetric memory"
                self._symm = None
                self.mode = "nccl"
                if dist_utils.rank() == 0:
                    print(f"DataParallel: fused NVLink all-reduce unavailable, using NCCL ({self.fallback_reason})",
                          flush=True)

    def _try_epilogue_reduction(self) -> None:
        """Switch to the reduction that runs inside the weight-gradient epilogues when the model allows it."""
        import os
        from .fsdp import SHARDED, REPLICATED, GradSink
        f = self.flat
        self.sink = None
        if os.environ.get("BDH_DDP_EPILOGUE", "1") != "1" or set(f.names) != set(SHARDED) | set(REPLICATED):
            return
        big = [f.params[f.names.index(n)] for n in SHARDED]
        R, D = big[0].shape
        ok = all(tuple(p.shape) == (R, D) for p in big) and R % (128 * self.world) == 0
        if not dist_utils.all_agree(ok, self.group, f.grad.device):
            return
        from . import symm
        rank = dist.get_rank(self.group)
        rpr = R // self.world
        self._acc_buf = symm.SymmetricBuffer(3 * rpr * D, torch.float32, f.grad.device, self.group)
        acc = self._acc_buf.tensor.view(3, rpr, D)
        acc.zero_()
        sink = GradSink(R, D, self.world, rank)
        sink.last_layer_only = True          # the layers accumulate locally; layer 0's epilogues send the sums
        sink.acc = acc
        sink.ptrs = {n: [p + 4 * i * rpr * D for p in self._acc_buf.ptrs] for i, n in enumerate(SHARDED)}
        n_loc = rpr * D
        self._seg_lo = [0, n_loc, 2 * n_loc, 3 * n_loc]
        self._seg_dst = [f.offsets[f.names.index(n)] + rank * n_loc for n in SHARDED]
        self._small = [(f.offsets[f.names.index(n)], f.params[f.names.index(n)].numel()) for n in REPLICATED]
        if any(o % 4 or k % (4 * self.world) for o, k in self._small) or any(o % 4 for o in self._seg_dst):
            return
        self._acc_buf.barrier()
        self.sink = sink
        f.module._grad_sink = sink           # ops.fused_bdh sends the big weights' gradients there
        self.mode = "epilogue"

    def broadcast_parameters(self) -> None:
        """Make every rank start from rank 0's weights."""
        if self.world > 1:
            dist.broadcast(self.flat.master, src=0, group=self.group)
            self.flat.refresh_shadow()

    def reduce_gradients(self) -> float:
        """Sum gradients over ranks in place. Returns the scale the optimizer must apply (1/world)."""
        if self.world == 1:
            return 1.0
        if self.mode == "epilogue":
            from ..ops import native
            sy, fl = self._symm, self._symm.flags
            fl["epoch"] += 1
            # the owners' slices are complete once every rank has finished its backward pass (the barrier inside):
            # scale, send to every rank's gradient buffer, clear
            native.ops.shard_bcast(fl["buf"].ptrs, sy.buf.ptrs, sy.buf.multicast_ptr, sy.buf.rank, self.world,
                                   self.sink.acc, self._seg_lo, self._seg_dst, 1.0 / self.world, fl["epoch"],
                                   _coll_ctas())
            for off, n in self._small:       # embedding and LM head: small in-place all-reduces
                sy.all_reduce_(scale=1.0 / self.world, offset=off, numel=n)
            return 1.0
        if self.mode == "fused" and self._symm is not None:
            self._symm.all_reduce_(scale=1.0 / self.world)
            return 1.0
        dist.all_reduce(self.flat.grad, op=dist.ReduceOp.SUM, group=self.group)
        return 1.0 / self.world


def _coll_ctas() -> int:
    from . import symm
    return symm.COLL_CTAS

"""Token-sharded activations gathered inside the consuming GEMM (all-gather -> GEMM as one kernel).

Under tensor parallelism the width-D activations between two sharded regions can live as token shards:
rank r holds rows [r*M/W, (r+1)*M/W) of a [M, K] matrix, and the next sharded GEMM (the encoder: every rank
multiplies ALL token rows by its own slice of the neurons) needs all of them. `GatheredOperand` keeps the
matrix in symmetric memory; `gemm()` launches this library's tcgen05 GEMM with the gather inside: the kernel's
epilogue warps pull the other ranks' row blocks over NVLink with plain peer loads into the local copy, in
ring order, the TMA producer starts a row block's tiles when its counter says the block has arrived, and the
tiles of the local rows run while the transfer is in flight (csrc/gemm_sm100.cuh: GatherArgs). Every tensor
map points at local memory and no load is multicast. `gemm_nccl()` is the same product behind an NCCL
all-gather, kept as the measured baseline.

The reference has no tensor parallelism (single device, src/model/bdh.rs); this serves the neuron-sharded
wrapper of this package (parallel/tp.py).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import gemm as G
from ..ops import native
from . import symm


class GatheredOperand:
    def __init__(self, M: int, K: int, device, group=None):
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if M % (128 * self.world) or K % 64:
            raise ValueError("M must be a multiple of 128 * world and K of 64")
        self.M, self.K, self.rows = M, K, M // self.world
        self.sym = symm.SymmetricBuffer(M * K, torch.bfloat16, device, group)
        self.full = self.sym.tensor[:M * K].view(M, K)
        self.full.zero_()
        self.arrived = torch.zeros(M // 128, device=device, dtype=torch.int32)
        self.flags = symm._Flags.get(device, self.sym.group)
        self.sym.barrier()

    @property
    def shard(self) -> torch.Tensor:
        """This rank's rows: the producing kernel writes here."""
        return self.full[self.rank * self.rows:(self.rank + 1) * self.rows]

    def _barrier(self) -> None:
        f = self.flags
        f["epoch"] += 1
        native.ops.rank_barrier(self.full, f["buf"].ptrs, self.rank, self.world, f["epoch"])

    def gemm(self, b: torch.Tensor, *, N: int, **kw) -> None:
        """out = epilogue(A_all . B^T) with A_all gathered inside the kernel. Afterwards the local copy holds
        every rank's rows. `release()` must follow before any rank writes its shard again."""
        self.arrived.zero_()
        self._barrier()                     # every rank's shard is complete
        G.gemm(self.full, b, M=self.M, N=N, K=self.K, gather_ptrs=self.sym.ptrs, gather_rows=self.rows,
               gather_rank=self.rank, gather_arrived=self.arrived, **kw)

    def release(self) -> None:
        self._barrier()                     # every rank's kernel has read what it needed

    def gemm_nccl(self, b: torch.Tensor, *, N: int, **kw) -> None:
        dist.all_gather_into_tensor(self.full, self.shard.clone(), group=self.group)
        G.gemm(self.full, b, M=self.M, N=N, K=self.K, **kw)

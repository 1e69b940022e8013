"""`relu_lowrank` on the sm_100a GEMM: relu(x . W^T + bias - theta), restricted to the active blocks of a
latent `BlockPattern1d` (reference: src/kernel/relu_lowrank.rs:7-37, src/kernel/block_sparse.rs:12-64).

The bias is an epilogue add; the block mask is not a multiplication: inactive neuron blocks are never
computed. Their rows are left out of the weight operand (one gather of the active rows), the GEMM runs
on the compacted neuron axis, and the output columns of inactive blocks are zeros.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import gemm as G
from .block_sparse import BlockPattern1d


def active_index(pattern: Optional[BlockPattern1d], n_per_head: int, device) -> Optional[torch.Tensor]:
    """Indices (inside a head) of the neurons in active blocks, ascending; None for a dense pattern."""
    if pattern is None or not pattern.is_sparse():
        return None
    bs = max(1, pattern.block_size)
    keep = [i for b in sorted(pattern.active_blocks) for i in range(b * bs, min((b + 1) * bs, n_per_head))]
    return torch.tensor(keep, dtype=torch.long, device=device)


def head_rows(idx: torch.Tensor, n_head: int, n_per_head: int) -> torch.Tensor:
    """Rows of a [H*N, D] weight that belong to the active neurons `idx` of every head."""
    return (torch.arange(n_head, device=idx.device)[:, None] * n_per_head + idx[None, :]).reshape(-1)


def relu_lowrank(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, theta: float = 0.0,
                 pattern: Optional[BlockPattern1d] = None, n_head: int = 1) -> torch.Tensor:
    """x [M, D] bf16, weight [H*N, D] bf16 (neuron-major), bias [H*N] fp32 or None -> [M, H*N] bf16."""
    M, D = x.shape
    HN = weight.shape[0]
    N = HN // n_head
    idx = active_index(pattern, N, x.device)
    if idx is None:
        out = torch.empty(M, HN, device=x.device, dtype=torch.bfloat16)
        G.gemm(x, weight, M=M, N=HN, K=D, epi=G.EPI_RELU, out0=out, theta=theta, bias=bias)
        return out
    rows = head_rows(idx, n_head, N)
    w = weight.index_select(0, rows)
    b = bias.index_select(0, rows).contiguous() if bias is not None else None
    Na = rows.numel()
    if Na % 8:
        raise ValueError("the active neurons per head must come to a multiple of 8 columns")
    compact = torch.empty(M, Na, device=x.device, dtype=torch.bfloat16)
    G.gemm(x, w, M=M, N=Na, K=D, epi=G.EPI_RELU, out0=compact, theta=theta, bias=b)
    out = torch.zeros(M, HN, device=x.device, dtype=torch.bfloat16)
    out[:, rows] = compact
    return out

"""Block-sparsity patterns over the latent (neuron) axis and over (time x time) attention blocks.

Behavioural restatement of the reference's pattern structs (src/kernel/block_sparse.rs:12-134):
a 1-D pattern is a block size plus an optional set of active block indices (None = dense); a 2-D
pattern is a block size plus an optional set of active (row, col) block pairs, where the dense
default is the causal lower triangle `col <= row`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import FrozenSet, Iterable, Iterator, Optional, Tuple

import torch


@dataclass(frozen=True)
class BlockPattern1d:
    block_size: int = 1
    active_blocks: Optional[FrozenSet[int]] = None

    @staticmethod
    def dense(block_size: int) -> "BlockPattern1d":
        return BlockPattern1d(max(1, int(block_size)), None)

    @staticmethod
    def from_blocks(block_size: int, blocks: Iterable[int]) -> "BlockPattern1d":
        return BlockPattern1d(int(block_size), frozenset(int(b) for b in blocks))

    def is_sparse(self) -> bool:
        return self.active_blocks is not None

    def is_block_active(self, idx: int) -> bool:
        return True if self.active_blocks is None else idx in self.active_blocks

    def mask(self, elements: int, device=None, dtype=torch.float32) -> torch.Tensor:
        """0/1 mask of shape [1, 1, 1, elements]: 1 inside active blocks (block_sparse.rs:48-64)."""
        bs = max(1, self.block_size)
        m = torch.zeros(elements, dtype=dtype, device=device)
        for b in range((elements + bs - 1) // bs):
            if self.is_block_active(b):
                m[b * bs:min((b + 1) * bs, elements)] = 1
        return m.view(1, 1, 1, elements)


@dataclass(frozen=True)
class BlockPattern2d:
    block_size: int = 1
    active_pairs: Optional[FrozenSet[Tuple[int, int]]] = None

    @staticmethod
    def dense(block_size: int) -> "BlockPattern2d":
        return BlockPattern2d(max(1, int(block_size)), None)

    @staticmethod
    def from_pairs(block_size: int, pairs: Iterable[Tuple[int, int]]) -> "BlockPattern2d":
        return BlockPattern2d(int(block_size), frozenset((int(r), int(c)) for r, c in pairs))

    def is_sparse(self) -> bool:
        return self.active_pairs is not None

    def is_active(self, row: int, col: int) -> bool:
        """Dense default = causal block triangle (block_sparse.rs:96-101)."""
        if self.active_pairs is None:
            return col <= row
        return (row, col) in self.active_pairs

    def iter_cols(self, row: int, total_cols: int) -> Iterator[int]:
        """Active column blocks of a row block, never beyond the diagonal (block_sparse.rs:103-118)."""
        for c in range(min(row + 1, total_cols)):
            if self.is_active(row, c):
                yield c

    def pairs(self, n_blocks: int):
        return [(r, c) for r in range(n_blocks) for c in self.iter_cols(r, n_blocks)]


@dataclass(frozen=True)
class BlockSparseConfig:
    latent: BlockPattern1d = field(default_factory=lambda: BlockPattern1d.dense(1))
    time: BlockPattern2d = field(default_factory=lambda: BlockPattern2d.dense(1))

    @staticmethod
    def dense(latent_block: int, time_block: int) -> "BlockSparseConfig":
        return BlockSparseConfig(BlockPattern1d.dense(latent_block), BlockPattern2d.dense(time_block))

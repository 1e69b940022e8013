"""BDH with sparse neuron graphs (the "local graph" form of the Dragon Hatchling).

The reference only has the ingredients: block masks over the latent axis and over (time x time)
attention blocks (src/kernel/block_sparse.rs:12-134) and README to-do items; `model/router.rs` is
empty. This model path makes the neuron <-> embedding couplings E, E_v and D block-sparse: each
block of `graph_block` neurons is wired to a subset of `graph_block`-wide groups of embedding
channels (a block-ELL pattern drawn once from `graph_density` and stored in the checkpoint), and
optionally restricts the neurons themselves with a `BlockPattern1d`. With density 1.0 and no latent
pattern it is exactly BDH-GPU, which is what the tests pin.

Dense kernels run on the masked weights (masked entries stay exactly zero: they start at zero,
their gradient is masked, and decoupled weight decay keeps zero at zero); `encode_sparse` runs the
encoder through the block-ELL SpMM kernel that touches only the wired blocks.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..ops import native
from .bdh import BDH, BDHConfig, build_model_config


@dataclass
class BDHGraphConfig(BDHConfig):
    graph_block: int = 64
    graph_density: float = 0.25
    graph_seed: int = 0


def build_graph_config(overrides, training_block_size: int, vocab_size: Optional[int] = None) -> BDHGraphConfig:
    base = build_model_config(overrides, training_block_size, vocab_size)
    return BDHGraphConfig(**base.__dict__, graph_block=getattr(overrides, "graph_block", None) or 64,
                          graph_density=getattr(overrides, "graph_density", None) or 0.25)


def random_block_mask(n_row_blocks: int, n_col_blocks: int, density: float, seed: int) -> torch.Tensor:
    """[row blocks, col blocks] bool; every row block keeps at least one column block."""
    g = torch.Generator().manual_seed(seed)
    keep = max(1, min(n_col_blocks, int(round(density * n_col_blocks))))
    mask = torch.zeros(n_row_blocks, n_col_blocks, dtype=torch.bool)
    for r in range(n_row_blocks):
        mask[r, torch.randperm(n_col_blocks, generator=g)[:keep]] = True
    return mask


def block_mask_to_ell(mask: torch.Tensor) -> torch.Tensor:
    """Bool block mask -> int32 [row blocks, width] of active column-block indices, -1 padded."""
    width = int(mask.sum(dim=1).max().item())
    ell = torch.full((mask.shape[0], max(width, 1)), -1, dtype=torch.int32)
    for r in range(mask.shape[0]):
        idx = torch.nonzero(mask[r]).flatten()
        ell[r, :len(idx)] = idx.to(torch.int32)
    return ell


class BDHGraph(BDH):
    def __init__(self, config: BDHGraphConfig):
        super().__init__(config)
        c = config
        blk = c.graph_block
        if c.latent_total % blk or c.n_embd % blk:
            raise ValueError("graph_block must divide both the neuron count and n_embd")
        nrb, ncb = c.latent_total // blk, c.n_embd // blk
        for i, name in enumerate(("encoder", "encoder_v", "decoder")):
            bm = random_block_mask(nrb, ncb, c.graph_density, c.graph_seed + i)
            self.register_buffer(f"{name}_blocks", bm)
            self.register_buffer(f"{name}_ell", block_mask_to_ell(bm))
            p = getattr(self, name)
            with torch.no_grad():
                p.mul_(self._expand(bm).to(p.dtype))
            p.register_hook(self._mask_grad(name))

    def _expand(self, block_mask: torch.Tensor) -> torch.Tensor:
        b = self.config.graph_block
        return block_mask.repeat_interleave(b, 0).repeat_interleave(b, 1)

    def _mask_grad(self, name):
        def hook(g):
            return g * self._expand(getattr(self, f"{name}_blocks")).to(g.dtype)
        return hook

    def graph_density(self) -> float:
        return float(self.encoder_blocks.float().mean())

    def edge_count(self) -> int:
        """Number of neuron <-> channel edges kept in the three graphs."""
        b = self.config.graph_block
        return int(sum(getattr(self, f"{n}_blocks").sum() for n in ("encoder", "encoder_v", "decoder"))) * b * b

    @torch.no_grad()
    def encode_sparse(self, cur: torch.Tensor) -> torch.Tensor:
        """x = relu(cur E^T - theta) for cur [M, D] through the block-ELL kernel (bf16)."""
        c = self.config
        w = self.encoder.detach().to(torch.bfloat16).contiguous()
        x = cur.to(torch.bfloat16).contiguous()
        if x.is_cuda and native.available():
            y = torch.empty(x.shape[0], c.latent_total, device=x.device, dtype=torch.bfloat16)
            native.ops.graph_spmm_relu(x, w, self.encoder_ell.to(x.device), y, float(c.relu_threshold))
            return y
        return torch.relu(x.float() @ w.float().t() - c.relu_threshold).to(torch.bfloat16)

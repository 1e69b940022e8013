"""Build a model from a TrainingConfig (`[model].kind` selects the family). The reference builds its
one model inline (`BDH::new(config, &device)`, src/bin/train.rs:261-274, src/bin/infer.rs:168-176);
the Mamba and sparse-graph families have no counterpart there."""
from __future__ import annotations

from typing import Optional

import torch

from .bdh import BDH, build_model_config


def build_model(cfg, vocab_size: Optional[int] = None) -> torch.nn.Module:
    """cfg: config.TrainingConfig. `vocab_size` (from the tokenizer) overrides `[model].vocab_size`."""
    kind = cfg.model.kind
    if kind == "bdh":
        return BDH(build_model_config(cfg.model, cfg.training.block_size, vocab_size))
    if kind == "bdh_graph":
        from .bdh_graph import BDHGraph, build_graph_config
        return BDHGraph(build_graph_config(cfg.model, cfg.training.block_size, vocab_size))
    if kind in ("mamba2", "mamba3"):
        from .mamba import MambaConfig, MambaLM
        m = cfg.model
        mc = MambaConfig(
            version=2 if kind == "mamba2" else 3,
            n_layer=m.n_layer or 6, d_model=m.n_embd or 256, d_state=m.d_state or 128, headdim=m.headdim or 64,
            expand=m.expand or 2, chunk_size=m.chunk_size or 64, d_conv=m.d_conv or 4, mimo_rank=m.mimo_rank or 1,
            vocab_size=vocab_size or m.vocab_size or 256, dropout=m.dropout or 0.0)
        return MambaLM(mc)
    raise ValueError(f"unknown model kind {kind}")

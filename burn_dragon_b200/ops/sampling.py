"""Next-token sampling for a batch of streams.

Definition: `ops.reference.sample_logits` (temperature, top-k with ties kept, fp32 softmax, uniform
fallback; reference src/generation.rs:26-72). On a GPU the batched sampling kernel does the same
in one launch with one warp per stream and a counter-based RNG, so no logits leave the device.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import native
from . import reference as R

_counter = [0]


def sample(logits: torch.Tensor, temperature: float = 1.0, top_k: Optional[int] = None, greedy: bool = False,
           generator: Optional[torch.Generator] = None, seed: Optional[int] = None) -> torch.Tensor:
    """logits [B, V] -> token ids [B] (int64)."""
    if (logits.is_cuda and native.available() and logits.shape[-1] <= 1024 and generator is None
            and hasattr(torch.ops.bdh, "sample_tokens")):
        B, V = logits.shape
        out = torch.empty(B, dtype=torch.int64, device=logits.device)
        _counter[0] += 1
        native.ops.sample_tokens(logits.float().contiguous(), out, float(temperature), int(top_k or 0), bool(greedy),
                                 int(seed if seed is not None else 0x9E3779B9), _counter[0], None)
        return out
    return R.sample_logits(logits, temperature, top_k, greedy, generator)

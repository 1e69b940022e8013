"""Elementwise parts of a Mamba-2 block around the SSD scan: causal depthwise conv1d + SiLU in front,
gated RMSNorm behind. On a GPU both run as one fp32 kernel per direction (`csrc/mamba_ops.cu`) with their
backward passes written out; elsewhere the torch statement of the same function runs under autograd.
The reference has no Mamba path; these serve the Mamba-2 model family of this package (models/mamba.py).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from . import native


def _on_kernels(*ts) -> bool:
    return (native.available() and all(t is None or (t.is_cuda and t.dtype == torch.float32) for t in ts))


# ---- conv1d + SiLU -----------------------------------------------------------------------------------
def conv1d_silu_reference(seq: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
    """seq [B, T + k - 1, C] (the k - 1 leading rows are the previous segment's tail or zeros), w [C, k],
    bias [C] -> silu(depthwise causal conv) [B, T, C]."""
    out = F.conv1d(seq.transpose(1, 2), w.unsqueeze(1), bias, groups=w.shape[0]).transpose(1, 2)
    return F.silu(out)


class _ConvSilu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, seq, w, bias):
        seq, w = seq.contiguous(), w.contiguous()
        B, Tin, C = seq.shape
        k = w.shape[1]
        out = torch.empty(B, Tin - k + 1, C, device=seq.device, dtype=torch.float32)
        native.ops.conv1d_silu_fwd(seq, w, bias, out)
        ctx.save_for_backward(seq, w, bias)
        return out

    @staticmethod
    def backward(ctx, dout):
        seq, w, bias = ctx.saved_tensors
        dout = dout.contiguous()
        dpre = torch.empty_like(dout)
        dseq = torch.empty_like(seq)
        dw = torch.zeros_like(w)
        db = torch.zeros_like(bias) if bias is not None else None
        native.ops.conv1d_silu_bwd(seq, w, bias, dout, dpre, dseq, dw, db)
        return dseq, dw, db


def conv1d_silu(seq: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
    if _on_kernels(seq, w, bias) and w.shape[1] <= 8:
        return _ConvSilu.apply(seq, w, bias)
    return conv1d_silu_reference(seq, w, bias)


# ---- gated RMSNorm -----------------------------------------------------------------------------------
def gated_rmsnorm_reference(v: torch.Tensor, z: torch.Tensor, w: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    g = v * F.silu(z)
    return g * torch.rsqrt(g.pow(2).mean(-1, keepdim=True) + eps) * w


class _GatedRmsNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, v, z, w, eps):
        v, z, w = v.contiguous(), z.contiguous(), w.contiguous()
        out = torch.empty_like(v)
        rstd = torch.empty(v.numel() // v.shape[-1], device=v.device, dtype=torch.float32)
        native.ops.gated_rmsnorm_fwd(v, z, w, out, rstd, float(eps))
        ctx.save_for_backward(v, z, w, rstd)
        return out

    @staticmethod
    def backward(ctx, dout):
        v, z, w, rstd = ctx.saved_tensors
        dout = dout.contiguous()
        dv, dz = torch.empty_like(v), torch.empty_like(z)
        dw = torch.zeros_like(w)
        native.ops.gated_rmsnorm_bwd(v, z, w, rstd, dout, dv, dz, dw)
        return dv, dz, dw, None


def gated_rmsnorm(v: torch.Tensor, z: torch.Tensor, w: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """rmsnorm(v * silu(z)) * w over the last dimension."""
    if _on_kernels(v, z, w) and v.shape == z.shape and v.shape[-1] <= 12288:
        return _GatedRmsNorm.apply(v, z, w, eps)
    return gated_rmsnorm_reference(v, z, w, eps)

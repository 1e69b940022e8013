"""`forward_fast` attention on the sm_100a kernels: additive distance bias + L1 row normalisation.

    S = tril(q q^T, -1) + m_h * tril(j - i, -1);  S <- S / (sum_j |S_ij| + 1e-6);  a = S v

(reference: src/model/attention.rs:142-175, 300-303; parallel entry src/model/bdh.rs:96-168). The
scores come from the tcgen05 GEMM with the causal epilogue (bias added in the epilogue, tiles above
the diagonal skipped), the normalisation is a warp-per-row kernel that keeps the row sums for the
backward pass, and `a = S v` contracts only over s < t. The backward pass reuses the same GEMMs:
G = tril(dA v^T), the row kernel turns it into dS, dv = S^T dA, dq = dS q + dS^T q.

The reference has a block-pair mask for this path (src/kernel/linear_attention.rs:54-112); masked
patterns stay on the torch statement `ops.reference.attention_rownorm`.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import gemm as G
from . import native


def can_run(q: torch.Tensor, v: torch.Tensor) -> bool:
    from . import emulate
    if not emulate.active() and not (q.is_cuda and native.available()):
        return False
    B, H, T, N = q.shape
    D = v.shape[-1]
    return T % 128 == 0 and N % 64 == 0 and D % 64 == 0 and v.shape[1] == 1


class _RowNormAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, v, slopes):
        B, H, T, N = q.shape
        D = v.shape[-1]
        dev = q.device
        q16 = q.to(torch.bfloat16).contiguous().view(B * H * T, N)
        v16 = v.to(torch.bfloat16).contiguous().view(B * T, D)
        # tiles above the diagonal are never written and later read as zeros
        S = torch.zeros(B * H * T, T, device=dev, dtype=torch.bfloat16)
        flags = G.F_BIAS if slopes is not None else 0
        sl = slopes.float().contiguous() if slopes is not None else None
        G.gemm(q16, q16, M=T, N=T, K=N, nz=(H, B), a_off=(T, H * T, 0, 0), b_off=(T, H * T, 0, 0),
               c_off=(T, H * T, 0, 0), epi=G.EPI_CAUSAL, flags=flags, slopes=sl, causal_tiles=1, out0=S)
        rnorm = torch.empty(B * H * T, device=dev, dtype=torch.float32)
        native.ops.rownorm_fwd(S, rnorm, T)
        a = torch.empty(B * H * T, D, device=dev, dtype=torch.float32)
        G.gemm(S, v16, M=T, N=D, K=T, b_mn=True, nz=(H, B), a_off=(T, H * T, 0, 0), b_off=(0, 0, 0, T),
               c_off=(T, H * T, 0, 0), causal_k=1, flags=G.F_OUT_F32, out0=a)
        ctx.save_for_backward(q16, v16, S, rnorm)
        ctx.shape = (B, H, T, N, D)
        ctx.dtypes = (q.dtype, v.dtype)
        return a.view(B, H, T, D).to(q.dtype)

    @staticmethod
    def backward(ctx, da):
        q16, v16, S, rnorm = ctx.saved_tensors
        B, H, T, N, D = ctx.shape
        dev = da.device
        da16 = da.to(torch.bfloat16).contiguous().view(B * H * T, D)
        # dv[b, s] = sum_h sum_t Sn[t, s] dA[t]: every (head, batch) problem adds into the rows of its batch
        dv = torch.zeros(B * T, D, device=dev, dtype=torch.float32)
        G.gemm(S, da16, M=T, N=D, K=T, a_mn=True, b_mn=True, nz=(H, B), a_off=(0, 0, T, H * T),
               b_off=(0, 0, T, H * T), c_off=(0, T, 0, 0), flags=G.F_OUT_F32 | G.F_ATOMIC, out0=dv)
        # G = tril(dA v^T, -1), then through the normalisation
        Gm = torch.zeros(B * H * T, T, device=dev, dtype=torch.bfloat16)
        G.gemm(da16, v16, M=T, N=T, K=D, nz=(H, B), a_off=(T, H * T, 0, 0), b_off=(0, T, 0, 0), c_off=(T, H * T, 0, 0),
               epi=G.EPI_CAUSAL, causal_tiles=1, out0=Gm)
        native.ops.rownorm_bwd(Gm, S, rnorm, T)
        # q is both the query and the key: dq = dS q + dS^T q
        dq = torch.empty(B * H * T, N, device=dev, dtype=torch.float32)
        G.gemm(Gm, q16, M=T, N=N, K=T, b_mn=True, nz=(H, B), a_off=(T, H * T, 0, 0), b_off=(0, 0, T, H * T),
               c_off=(T, H * T, 0, 0), causal_k=1, flags=G.F_OUT_F32, out0=dq)
        G.gemm(Gm, q16, M=T, N=N, K=T, a_mn=True, b_mn=True, nz=(H, B), a_off=(0, 0, T, H * T), b_off=(0, 0, T, H * T),
               c_off=(T, H * T, 0, 0), flags=G.F_OUT_F32 | G.F_ACCUM, out0=dq)
        qd, vd = ctx.dtypes
        return dq.view(B, H, T, N).to(qd), dv.view(B, 1, T, D).to(vd), None


def attention_rownorm(q: torch.Tensor, v: torch.Tensor, slopes: Optional[torch.Tensor]) -> torch.Tensor:
    """q [B, H, T, N], v [B, 1, T, D] (shared by the heads), slopes [H] or None -> a [B, H, T, D]."""
    return _RowNormAttention.apply(q, v, slopes)

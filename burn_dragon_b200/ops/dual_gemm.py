"""Front end of the chained-GEMM kernel (`csrc/dual_gemm_sm100.cuh`): two GEMMs with the
[tokens, neurons] intermediate produced, transformed and consumed on chip.

    Y   = A1 . B1^T                    per (128-token tile, head, 128-neuron chunk), contraction K1
    P   = epilogue(Y; in0, in1)        written once to `p` [M, H*N] (bf16) - and `out1` for the gate backward
    out = P . B2                       [M, N2] summed over all heads, or one [M, N2] block per head

`dual(...)` launches the kernel and the fixed-order reduction of its fp32 partial tiles;
`dual_reference(...)` is the same contract in fp32 torch ops (any device), used by the GPU tests and
by the emulated kernel path. The three epilogues are the layer's gate (reference:
src/model/bdh.rs:359-441), its backward, and the backward of the rotary rotation.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import gemm as G
from . import native

_PARTIALS = {}
_FLOATS = {}


def eligible(M: int, T: int, N: int, D: int) -> bool:
    """Shapes the chained kernel covers: whole 128-token tiles inside a sequence, 128-neuron chunks,
    an output of at most 256 columns (it stays in TMEM next to two first-GEMM accumulators)."""
    return M % 128 == 0 and T % 128 == 0 and M % T == 0 and N % 128 == 0 and D % 64 == 0 and D <= 256


def _partials(dev, floats: int) -> torch.Tensor:
    """Scratch for the fp32 partial tiles, one buffer per device, grown on demand and reused: every
    launch is followed by its reduction on the same stream before the next launch writes it."""
    buf = _PARTIALS.get(dev)
    if buf is None or buf.numel() < floats:
        buf = _PARTIALS[dev] = torch.empty(floats, device=dev, dtype=torch.float32)
    return buf


def dual(a1: torch.Tensor, b1: torch.Tensor, b2: torch.Tensor, p: torch.Tensor, out: torch.Tensor, *, M: int, H: int,
         n_per_head: int, K1: int, N2: int, T: int, epi: int, flags: int = 0, group_per_head: bool = False,
         a1_b: int = 0, a1_h: int = 0, b1_mn: bool = False, b1_b: int = 0, in0: Optional[torch.Tensor] = None,
         in1: Optional[torch.Tensor] = None, out1: Optional[torch.Tensor] = None, alpha: float = 1.0,
         theta: float = 0.0, pos0: int = 0, drop_p: float = 0.0, drop_seed: int = 0, accumulate: bool = False,
         out_h_stride: int = 0, max_ctas: int = 0) -> None:
    if not native.available():
        raise RuntimeError("bdh dual gemm: the sm_100a extension is not available")
    ops = native.ops
    gph = 1 if group_per_head else 0
    key = (a1.device, M, H, n_per_head, N2, gph, max_ctas)
    floats = _FLOATS.get(key)
    if floats is None:
        floats = _FLOATS[key] = int(torch.ops.bdh.dual_gemm_partial_floats(M, H, n_per_head, N2, gph, max_ctas))
    part = _partials(a1.device, floats)
    ops.dual_gemm(a1, b1, bool(b1_mn), b2, p, M, H, n_per_head, K1, N2, T, epi, flags, gph, int(a1_b), int(a1_h),
                  int(b1_b), in0, in1, out1, float(alpha), float(theta), int(pos0), float(drop_p),
                  int(drop_seed) & 0x7FFFFFFF, part, max_ctas)
    ops.dual_gemm_reduce(part, M, H, n_per_head, N2, gph, max_ctas, out, bool(accumulate), int(out_h_stride))


def dual_reference(a1, b1, b2, p, out, *, M, H, n_per_head, K1, N2, T, epi, flags=0, group_per_head=False, a1_b=0,
                   a1_h=0, b1_mn=False, b1_b=0, in0=None, in1=None, out1=None, alpha=1.0, theta=0.0, pos0=0,
                   drop_p=0.0, drop_seed=0, accumulate=False, out_h_stride=0, max_ctas=0) -> None:
    """Writes the same outputs as `dual`, head by head, in fp32 torch ops."""
    from . import emulate
    dev = a1.device
    N = n_per_head
    m = torch.arange(M, device=dev)
    rows_b, rows_t = m // T, m % T
    total = torch.zeros(M, N2, device=dev, dtype=torch.float32)
    for h in range(H):
        cols = slice(h * N, (h + 1) * N)
        A = a1[rows_b * a1_b + rows_t + h * a1_h, :K1].float()                       # [M, K1]
        if b1_mn:
            # B1 is indexed [k, neuron]; the k rows of a token's sequence start at its batch index * b1_b
            Y = torch.empty(M, N, device=dev)
            for b in range(M // T):
                Bk = b1[b * b1_b:b * b1_b + K1, cols].float()                        # [K1, N]
                Y[b * T:(b + 1) * T] = A[b * T:(b + 1) * T] @ Bk
        else:
            Y = A @ b1[cols, :K1].float().t()
        if epi == G.EPI_RELU_GATE:
            P = torch.relu(Y - theta) * in0[:M, cols].float()
            if drop_p > 0:
                keep = G.dropout_keep_mask(int(drop_seed) & 0x7FFFFFFF, h, M, N, drop_p, dev)
                P = torch.where(keep, P / (1.0 - drop_p), torch.zeros_like(P))
        elif epi == G.EPI_GATE_BWD:
            x, xy = in0[:M, cols].float(), in1[:M, cols].float()
            P = torch.where(xy > 0, Y * x * alpha, torch.zeros_like(Y))
            y = torch.where(x > 0, xy / x.clamp(min=1e-30), torch.zeros_like(x))
            gx = Y * y
            gx = torch.where(gx == 0, torch.zeros_like(gx), gx)
            out1[:M, cols] = torch.where(x > 0, gx, torch.full_like(gx, -0.0)).to(out1.dtype)
        elif epi == G.EPI_DQ_BWD:
            g_raw = in0[:M, cols]
            closed = g_raw.contiguous().view(torch.int16) == -32768
            v = Y
            if flags & G.F_ROPE:
                # inverse rotation with the table's (cos, sin): rotate by the negated angle
                tab = in1.view(torch.float16).float().clone()
                tab[:, 1::2] = -tab[:, 1::2]
                v = emulate._rotate_by_table(v, tab.to(torch.float16).view(torch.bfloat16), T, N)
            v = v * alpha + g_raw.float()
            P = torch.where(closed, torch.zeros_like(v), v)
        else:
            raise ValueError(f"dual: unsupported epilogue {epi}")
        Pb = P.to(torch.bfloat16)
        p[:M, cols] = Pb
        contrib = Pb.float() @ b2[cols, :N2].float()
        if group_per_head:
            r = slice(h * out_h_stride, h * out_h_stride + M)
            out[r, :N2] = (out[r, :N2].float() + contrib if accumulate else contrib).to(out.dtype)
        else:
            total += contrib
    if not group_per_head:
        out[:M, :N2] = (out[:M, :N2].float() + total if accumulate else total).to(out.dtype)

"""State-space duality (SSD) scan used by the Mamba-2 / Mamba-3 model paths.

    h_t = exp(loga_t) * h_{t-1} + B_t (x) xw_t          h: [N, P] per (batch, head)
    y_t = C_t . h_t                                      (the current input is included)

`xw` is the input already multiplied by its step weight (dt for Mamba-2; the two trapezoidal
weights for Mamba-3). B and C are shared by all heads of a group (one group here).

Three statements of the same function: the literal recurrence (oracle), the chunked form in torch
(differentiable), and the CUDA chunk-scan kernels: chunk outputs on the tensor cores (tcgen05, bf16
operands) or in fp32 FMA arithmetic; `ssd_dual` runs training on them (forward and the dual scan of
the backward pass).
The reference has no Mamba path; the spec is Mamba-2's SSD algorithm (Dao & Gu, 2024).
"""
from __future__ import annotations

import os
from typing import Optional, Tuple

import torch

from . import native


def ssd_sequential(xw: torch.Tensor, loga: torch.Tensor, Bm: torch.Tensor, Cm: torch.Tensor,
                   h0: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """xw [B,T,H,P], loga [B,T,H], Bm/Cm [B,T,N], h0 [B,H,N,P] -> (y [B,T,H,P], hT [B,H,N,P])."""
    Bsz, T, H, P = xw.shape
    N = Bm.shape[-1]
    h = h0 if h0 is not None else torch.zeros(Bsz, H, N, P, dtype=xw.dtype, device=xw.device)
    ys = []
    for t in range(T):
        h = h * torch.exp(loga[:, t]).view(Bsz, H, 1, 1) + Bm[:, t].view(Bsz, 1, N, 1) * xw[:, t].view(Bsz, H, 1, P)
        ys.append(torch.einsum("bn,bhnp->bhp", Cm[:, t], h))
    return torch.stack(ys, dim=1), h


def ssd_backward_sequential(xw: torch.Tensor, loga: torch.Tensor, Bm: torch.Tensor, Cm: torch.Tensor,
                            dy: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Gradients of `ssd_sequential` (zero initial state) for an output gradient dy [B,T,H,P], written
    out instead of differentiated: the oracle a backward kernel is compared against. The scan is dual
    to itself:
      d xw     = the same scan run backwards in time with B and C exchanged and the decays shifted
                 by one step, fed with dy;
      d log a  = reverse cumulative sum over time of (dy_t . y_t - d xw_t . xw_t), per head;
      d C_t[n] = sum_{h,p} dy_t[h,p] h_t[h,n,p]             (forward state, step t included);
      d B_s[n] = sum_{h,p} xw_s[h,p] G_s[h,n,p]             (reverse state G_s = C_s (x) dy_s + a_{s+1} G_{s+1}).
    Returns (d xw, d log a, d B, d C)."""
    Bsz, T, H, P = xw.shape
    N = Bm.shape[-1]
    flip = lambda t: t.flip(1)
    y, _ = ssd_sequential(xw, loga, Bm, Cm)
    shifted = torch.cat([torch.zeros_like(loga[:, :1]), flip(loga)[:, :-1]], dim=1)
    dxw = flip(ssd_sequential(flip(dy), shifted, flip(Cm), flip(Bm))[0])
    dloga = flip(torch.cumsum(flip((dy * y).sum(-1) - (dxw * xw).sum(-1)), dim=1))
    h = torch.zeros(Bsz, H, N, P, dtype=xw.dtype, device=xw.device)
    G = torch.zeros_like(h)
    dC, dB = [None] * T, [None] * T
    for t in range(T):
        h = h * torch.exp(loga[:, t]).view(Bsz, H, 1, 1) + Bm[:, t].view(Bsz, 1, N, 1) * xw[:, t].view(Bsz, H, 1, P)
        dC[t] = torch.einsum("bhp,bhnp->bn", dy[:, t], h)
    for s in range(T - 1, -1, -1):
        if s + 1 < T:
            G = G * torch.exp(loga[:, s + 1]).view(Bsz, H, 1, 1)
        G = G + Cm[:, s].view(Bsz, 1, N, 1) * dy[:, s].view(Bsz, H, 1, P)
        dB[s] = torch.einsum("bhp,bhnp->bn", xw[:, s], G)
    return dxw, dloga, torch.stack(dB, dim=1), torch.stack(dC, dim=1)


def ssd_chunked(xw: torch.Tensor, loga: torch.Tensor, Bm: torch.Tensor, Cm: torch.Tensor,
                h0: Optional[torch.Tensor] = None, chunk: int = 64) -> Tuple[torch.Tensor, torch.Tensor]:
    """Same function, O(T*chunk) work per head: quadratic inside a chunk, state hand-off between."""
    Bsz, T, H, P = xw.shape
    N = Bm.shape[-1]
    pad = (-T) % chunk
    if pad:
        xw = torch.nn.functional.pad(xw, (0, 0, 0, 0, 0, pad))
        loga = torch.nn.functional.pad(loga, (0, 0, 0, pad))
        Bm = torch.nn.functional.pad(Bm, (0, 0, 0, pad))
        Cm = torch.nn.functional.pad(Cm, (0, 0, 0, pad))
    Tp = T + pad
    C = Tp // chunk
    x_ = xw.view(Bsz, C, chunk, H, P)
    a_ = loga.view(Bsz, C, chunk, H).permute(0, 3, 1, 2)              # [B,H,C,Q]
    B_ = Bm.view(Bsz, C, chunk, N)
    C_ = Cm.view(Bsz, C, chunk, N)
    cum = torch.cumsum(a_, dim=-1)                                     # inclusive: sum_{r<=i} loga_r
    # intra-chunk: y_i += sum_{j<=i} exp(cum_i - cum_j) (C_i . B_j) xw_j
    diff = cum.unsqueeze(-1) - cum.unsqueeze(-2)                       # [B,H,C,Q,Q]  (i, j)
    tri = torch.tril(torch.ones(chunk, chunk, dtype=torch.bool, device=xw.device))
    L = torch.where(tri, torch.exp(diff.masked_fill(~tri, 0.0)), torch.zeros_like(diff))
    CB = torch.einsum("bcin,bcjn->bcij", C_, B_)                       # [B,C,Q,Q]
    y = torch.einsum("bhcij,bcij,bcjhp->bcihp", L, CB, x_)
    # chunk states: S_c = sum_j exp(cum_last - cum_j) B_j (x) xw_j
    decay_to_end = torch.exp(cum[..., -1:] - cum)                      # [B,H,C,Q]
    S = torch.einsum("bhcj,bcjn,bcjhp->bchnp", decay_to_end, B_, x_)   # [B,C,H,N,P]
    chunk_decay = torch.exp(cum[..., -1])                              # [B,H,C]
    h = h0 if h0 is not None else torch.zeros(Bsz, H, N, P, dtype=xw.dtype, device=xw.device)
    prev = []
    for c in range(C):
        prev.append(h)
        h = h * chunk_decay[:, :, c].view(Bsz, H, 1, 1) + S[:, c]
    prev = torch.stack(prev, dim=1)                                    # [B,C,H,N,P] state entering each chunk
    # inter-chunk: y_i += exp(cum_i) C_i . prev
    y = y + torch.einsum("bhci,bcin,bchnp->bcihp", torch.exp(cum), C_, prev)
    y = y.reshape(Bsz, Tp, H, P)[:, :T]
    if pad:
        # the padded steps have loga = 0 and zero input, so the state after T is h unchanged
        pass
    return y, h


def ssd_step(xw: torch.Tensor, loga: torch.Tensor, Bm: torch.Tensor, Cm: torch.Tensor,
             h: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """One decode step. xw [B,H,P], loga [B,H], Bm/Cm [B,N], h [B,H,N,P] (updated in place)."""
    h.mul_(torch.exp(loga).view(*loga.shape, 1, 1)).add_(Bm.view(Bm.shape[0], 1, -1, 1) * xw.unsqueeze(2))
    return torch.einsum("bn,bhnp->bhp", Cm, h), h


def _bc_grads_chunked(xw, loga, Bm, Cm, dy, chunk: int):
    """d B and d C of the scan (zero initial state) in chunked form: the intra-chunk part through
    W_ij = sum_h L_ij (dy_i . xw_j), the inter-chunk part through the forward states entering each
    chunk (for d C) and the reverse states leaving it towards the past (for d B)."""
    Bsz, T, H, P = xw.shape
    N = Bm.shape[-1]
    pad = (-T) % chunk
    if pad:
        f = torch.nn.functional.pad
        xw, dy = f(xw, (0, 0, 0, 0, 0, pad)), f(dy, (0, 0, 0, 0, 0, pad))
        loga, Bm, Cm = f(loga, (0, 0, 0, pad)), f(Bm, (0, 0, 0, pad)), f(Cm, (0, 0, 0, pad))
    C = (T + pad) // chunk
    x_, d_ = xw.view(Bsz, C, chunk, H, P), dy.view(Bsz, C, chunk, H, P)
    B_, C_ = Bm.view(Bsz, C, chunk, N), Cm.view(Bsz, C, chunk, N)
    cum = torch.cumsum(loga.view(Bsz, C, chunk, H).permute(0, 3, 1, 2), dim=-1)          # [B,H,C,Q]
    tri = torch.tril(torch.ones(chunk, chunk, dtype=torch.bool, device=xw.device))
    diff = cum.unsqueeze(-1) - cum.unsqueeze(-2)
    L = torch.where(tri, torch.exp(diff.masked_fill(~tri, 0.0)), torch.zeros_like(diff))
    # (two-operand contractions throughout: each is one batched matmul)
    W = (L * torch.einsum("bcihp,bcjhp->bhcij", d_, x_)).sum(dim=1)                       # [B,C,Q,Q]
    dC = torch.matmul(W, B_)
    dB = torch.matmul(W.transpose(-1, -2), C_)
    to_end = torch.exp(cum[..., -1:] - cum)                                               # [B,H,C,Q]
    chunk_decay = torch.exp(cum[..., -1])                                                 # [B,H,C]
    at_i = torch.exp(cum).permute(0, 2, 3, 1).unsqueeze(-1)                               # [B,C,Q,H,1]
    x_end = x_ * to_end.permute(0, 2, 3, 1).unsqueeze(-1)                                 # xw_j decayed to its chunk's end
    d_at = d_ * at_i                                                                      # dy_i scaled by exp(cum_i)
    S = torch.einsum("bcjn,bcjhp->bchnp", B_, x_end)                                      # state each chunk adds
    dprev = torch.einsum("bcin,bcihp->bchnp", C_, d_at)                                   # d (state entering chunk)
    h = torch.zeros(Bsz, H, N, P, dtype=xw.dtype, device=xw.device)
    prev = []
    for c in range(C):
        prev.append(h)
        h = h * chunk_decay[:, :, c].view(Bsz, H, 1, 1) + S[:, c]
    R = torch.zeros_like(h)
    dS = [None] * C
    for c in range(C - 1, -1, -1):
        dS[c] = R                                        # gradient of the state chunk c adds (seen by later chunks)
        R = dprev[:, c] + R * chunk_decay[:, :, c].view(Bsz, H, 1, 1)
    dC = dC + torch.einsum("bcihp,bchnp->bcin", d_at, torch.stack(prev, dim=1))
    dB = dB + torch.einsum("bcjhp,bchnp->bcjn", x_end, torch.stack(dS, dim=1))
    return dB.reshape(Bsz, T + pad, N)[:, :T], dC.reshape(Bsz, T + pad, N)[:, :T]


class _SSDDual(torch.autograd.Function):
    """The scan with its backward written out (see `ssd_backward_sequential`): nothing but the inputs
    and y is kept for the backward pass, and both y and d xw come from the forward implementation
    (the CUDA chunk-scan kernels on a GPU), d xw through the time-reversed dual scan. Zero initial
    state; the final state is returned without a gradient."""

    @staticmethod
    def forward(ctx, xw, loga, Bm, Cm, chunk):
        with torch.no_grad():
            y, hT = ssd(xw, loga, Bm, Cm, None, chunk)
        ctx.save_for_backward(xw, loga, Bm, Cm, y)
        ctx.chunk = chunk
        ctx.mark_non_differentiable(hT)
        return y.to(xw.dtype), hT

    @staticmethod
    def backward(ctx, dy, _dh):
        xw, loga, Bm, Cm, y = ctx.saved_tensors
        dy = dy.to(y.dtype)
        flip = lambda t: t.flip(1).contiguous()
        with torch.no_grad():
            shifted = torch.cat([torch.zeros_like(loga[:, :1]), flip(loga)[:, :-1]], dim=1)
            dxw = flip(ssd(flip(dy), shifted, flip(Cm), flip(Bm), None, ctx.chunk)[0]).to(y.dtype)
            dloga = ((dy * y).sum(-1) - (dxw * xw).sum(-1)).flip(1).cumsum(1).flip(1)
            dB, dC = _bc_grads_chunked(xw.to(y.dtype), loga.to(y.dtype), Bm.to(y.dtype), Cm.to(y.dtype), dy, ctx.chunk)
        return dxw.to(xw.dtype), dloga.to(loga.dtype), dB.to(Bm.dtype), dC.to(Cm.dtype), None


def ssd_dual(xw, loga, Bm, Cm, chunk: int = 64):
    """Differentiable scan from a zero state whose backward is the written-out dual form (what `ssd` uses for
    training calls without an initial state on a GPU; `BDH_SSD_DUAL=1` / `0` forces it on / off everywhere)."""
    return _SSDDual.apply(xw, loga, Bm, Cm, chunk)


_DUAL = os.environ.get("BDH_SSD_DUAL")        # "1": always, "0": never, unset: wherever the kernels run


def ssd(xw, loga, Bm, Cm, h0=None, chunk: int = 64):
    """Dispatch: CUDA chunk-scan kernels when no gradient is needed, else the torch chunked form."""
    ct = torch.promote_types(torch.promote_types(xw.dtype, loga.dtype), torch.promote_types(Bm.dtype, Cm.dtype))
    xw, loga, Bm, Cm = xw.to(ct), loga.to(ct), Bm.to(ct), Cm.to(ct)
    if h0 is not None:
        h0 = h0.to(ct)
    need_grad = torch.is_grad_enabled() and any(t.requires_grad for t in (xw, loga, Bm, Cm))
    kernels = (xw.is_cuda and native.available() and hasattr(torch.ops.bdh, "ssd_chunk_scan")
               and xw.shape[-1] == 64 and Bm.shape[-1] == 128 and chunk == 64)
    # training from a zero state: on a GPU the written-out dual form, whose forward scan and backward (dual) scan
    # both run on the chunk-scan kernels; elsewhere autograd of the torch chunked form
    if need_grad and h0 is None and (_DUAL == "1" or (_DUAL is None and kernels)):
        return ssd_dual(xw, loga, Bm, Cm, chunk)
    if xw.shape[1] == 1 and h0 is not None and not need_grad:
        # single-token decode: one recurrence step on a private copy of the state
        if kernels and ct == torch.float32:
            h = h0.clone().contiguous()
            y = torch.empty_like(xw[:, 0])
            native.ops.ssd_decode_step(xw[:, 0].contiguous(), loga[:, 0].contiguous(), Bm[:, 0].contiguous(),
                                       Cm[:, 0].contiguous(), h, y)
            return y.unsqueeze(1), h
        y, h = ssd_step(xw[:, 0], loga[:, 0], Bm[:, 0], Cm[:, 0], h0.clone())
        return y.unsqueeze(1), h
    if kernels and not need_grad:
        return ssd_cuda(xw, loga, Bm, Cm, h0)
    return ssd_chunked(xw, loga, Bm, Cm, h0, chunk)


def ssd_cuda(xw, loga, Bm, Cm, h0=None, tensor_cores: Optional[bool] = None):
    """Chunk-scan kernels. `tensor_cores` (default: on, `BDH_SSD_FMA=1` turns it off): the chunk outputs - the
    quadratic part and the carried-state product - run as tcgen05 MMAs over pairs of chunks with bf16 operands and
    fp32 accumulation (`csrc/ssd_tc.cu`); off: the fp32 FMA kernels (`csrc/ssd.cu`), exact to fp32 rounding."""
    if tensor_cores is None:
        tensor_cores = os.environ.get("BDH_SSD_FMA", "0") != "1"
    Bsz, T, H, P = xw.shape
    N = Bm.shape[-1]
    chunk = 64
    pad = (-T) % chunk
    f = lambda t: t.float().contiguous()
    if pad:
        xw = torch.nn.functional.pad(xw, (0, 0, 0, 0, 0, pad))
        loga = torch.nn.functional.pad(loga, (0, 0, 0, pad))
        Bm = torch.nn.functional.pad(Bm, (0, 0, 0, pad))
        Cm = torch.nn.functional.pad(Cm, (0, 0, 0, pad))
    xw, loga, Bm, Cm = f(xw), f(loga), f(Bm), f(Cm)
    Tp = T + pad
    C = Tp // chunk
    y = torch.empty(Bsz, Tp, H, P, device=xw.device, dtype=torch.float32)
    states = torch.empty(Bsz, C, H, N, P, device=xw.device, dtype=torch.float32)   # scratch: per-chunk states
    h = h0.float().clone().contiguous() if h0 is not None else torch.zeros(Bsz, H, N, P, device=xw.device)
    decay = torch.empty(Bsz, C, H, device=xw.device, dtype=torch.float32)                 # scratch: per-chunk decay
    native.ops.ssd_chunk_scan(xw, loga, Bm, Cm, h, states, decay, y, bool(tensor_cores))
    return y[:, :T], h

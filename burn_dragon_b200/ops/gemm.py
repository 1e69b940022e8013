"""Front end of the tcgen05 GEMM with fused epilogues (`csrc/gemm_sm100.cuh`).

`gemm(...)` launches the kernel; `gemm_reference(...)` is the same contract written with plain
fp32 torch ops (any device) and is what the GPU tests compare against.

Contract:  for z0 < nz[0], z1 < nz[1]:
    C[z][m, n] = epilogue( sum_k A[z][m, k] * B[z][n, k] ),  m < M, n < N, k < K
Operands are 2-D bf16 matrices. A K-major operand is indexed [mn, k], an MN-major one [k, mn].
`a_off = (mn per z0, mn per z1, k per z0, k per z1)` shifts the window inside the 2-D matrix for
each batch index; `c_off = (row per z0, row per z1, col per z0, col per z1)` does the same for
the outputs and the auxiliary inputs (which share C's coordinates).
"""
from __future__ import annotations

import math
import os
from typing import Optional, Sequence

import torch

from . import native

EPI_STORE, EPI_RELU, EPI_RELU_GATE, EPI_CAUSAL, EPI_GATE_BWD, EPI_DQ_BWD = range(6)
F_OUT_F32, F_ACCUM, F_ROPE, F_POPE, F_UPPER, F_NO_OUT0, F_TABLE, F_MC_RED, F_ATOMIC = 1, 2, 4, 8, 16, 32, 128, 256, 512
F_PEER_RS = 1024
F_BIAS = 64
F_ROWDECAY = 2048
F_KEEP_MARK = 4096        # EPI_DQ_BWD: closed gates keep the -0.0 marker in out0 (a second launch adds to it)
F_ROWDECAY_REV = 8192     # EPI_STORE: row m scaled by exp(-slope * (T - m))

_SUPPORTED = {
    (256, False, False, EPI_STORE), (256, False, False, EPI_RELU), (256, False, False, EPI_RELU_GATE),
    (256, False, False, EPI_CAUSAL), (256, False, False, EPI_GATE_BWD), (256, False, True, EPI_STORE),
    (256, False, True, EPI_DQ_BWD), (256, True, True, EPI_STORE), (256, True, False, EPI_STORE),
    (128, False, False, EPI_STORE), (128, False, False, EPI_CAUSAL), (128, False, True, EPI_STORE),
    (128, True, True, EPI_STORE),
}


def supported(bn: int, a_mn: bool, b_mn: bool, epi: int) -> bool:
    return (bn, bool(a_mn), bool(b_mn), epi) in _SUPPORTED


def operand_ok(t: torch.Tensor) -> bool:
    """TMA requirements for a 2-D bf16 operand: unit column stride, 16-byte aligned rows."""
    return (t.dim() == 2 and t.dtype == torch.bfloat16 and t.stride(1) == 1 and t.stride(0) % 8 == 0
            and t.data_ptr() % 16 == 0)


def check_extents(a, b, *, M, N, K, a_mn=False, b_mn=False, nz=(1, 1), a_off=(0, 0, 0, 0), b_off=(0, 0, 0, 0),
                  epi=EPI_STORE, flags=0, out0=None, out1=None, in0=None, in1=None, c_off=(0, 0, 0, 0),
                  o1_off=(0, 0, 0), T=1, n_per_head=1, **_) -> None:
    """Host-side bounds check of one launch: for the last batch index (the offsets are linear and
    must be non-negative) every operand window [mn_lo, mn_lo + M|N) x [k_lo, k_lo + K) and every
    output / auxiliary window [r0, r0 + M) x [c0, c0 + N) has to lie inside its 2-D tensor. The
    kernel itself would not fault on most of these (TMA clips and zero-fills), it would compute on
    the wrong data; a plain-store epilogue would write outside its tensor. Runs for every launch of
    the emulated kernel path and, with `BDH_CHECKED_KERNELS=1`, before every real launch."""
    z0, z1 = int(nz[0]) - 1, int(nz[1]) - 1
    if z0 < 0 or z1 < 0 or min(M, N, K) < 1:
        raise ValueError(f"gemm: empty problem M={M} N={N} K={K} nz={tuple(nz)}")

    def inside(name, t, rows_lo, rows_n, cols_lo, cols_n):
        if t is None:
            raise ValueError(f"gemm: epilogue {epi} needs `{name}`")
        if t.dim() != 2:
            raise ValueError(f"gemm: `{name}` must be 2-D, got {tuple(t.shape)}")
        if rows_lo + rows_n > t.shape[0] or cols_lo + cols_n > t.shape[1]:
            raise ValueError(f"gemm: window of `{name}` rows [{rows_lo}, {rows_lo + rows_n}) x cols [{cols_lo}, "
                             f"{cols_lo + cols_n}) leaves its tensor {tuple(t.shape)} (last batch index {z0}, {z1})")

    for name, off in (("a_off", a_off), ("b_off", b_off), ("c_off", c_off), ("o1_off", o1_off)):
        if any(int(o) < 0 for o in off):
            raise ValueError(f"gemm: negative {name} {tuple(off)}")
    for name, t, mn_major, off, n in (("a", a, a_mn, a_off, M), ("b", b, b_mn, b_off, N)):
        mn_lo, k_lo = off[0] * z0 + off[1] * z1, off[2] * z0 + off[3] * z1
        if mn_major:
            inside(name, t, k_lo, K, mn_lo, n)
        else:
            inside(name, t, mn_lo, n, k_lo, K)
    r0, c0 = c_off[0] * z0 + c_off[1] * z1, c_off[2] * z0 + c_off[3] * z1
    if not (flags & (F_NO_OUT0 | F_PEER_RS | F_MC_RED)):
        inside("out0", out0, r0, M, c0, N)
    if epi == EPI_RELU and flags & (F_ROPE | F_POPE):
        c1 = o1_off[0] * z0 + o1_off[1] * z1
        inside("out1", out1, r0, M, c1, N + (o1_off[2] if flags & F_POPE else 0))
        if flags & F_TABLE:
            inside("in0 (rotary table)", in0, 0, T, 0, n_per_head)
    elif epi == EPI_RELU_GATE:
        inside("in0", in0, r0, M, c0, N)
        inside("out1", out1, r0, M, c0, N)
    elif epi == EPI_GATE_BWD:
        inside("in0", in0, r0, M, c0, N)
        inside("in1", in1, r0, M, c0, N)
        inside("out1", out1, r0, M, c0, N)
    elif epi == EPI_DQ_BWD:
        inside("in0", in0, r0, M, c0, N)
        if flags & F_TABLE:
            inside("in1 (rotary table)", in1, 0, T, 0, n_per_head)


_CHECKED = os.environ.get("BDH_CHECKED_KERNELS", "0") == "1"


def gemm(a: torch.Tensor, b: torch.Tensor, *, M: int, N: int, K: int, a_mn: bool = False, b_mn: bool = False,
         nz: Sequence[int] = (1, 1), a_off: Sequence[int] = (0, 0, 0, 0), b_off: Sequence[int] = (0, 0, 0, 0),
         epi: int = EPI_STORE, flags: int = 0, out0: Optional[torch.Tensor] = None,
         out1: Optional[torch.Tensor] = None, in0: Optional[torch.Tensor] = None,
         in1: Optional[torch.Tensor] = None, c_off: Sequence[int] = (0, 0, 0, 0),
         o1_off: Sequence[int] = (0, 0, 0), alpha: float = 1.0, theta: float = 0.0, T: int = 1, pos0: int = 0,
         n_per_head: int = 1, freqs: Optional[torch.Tensor] = None, slopes: Optional[torch.Tensor] = None,
         causal_tiles: int = 0, causal_k: int = 0, bn: int = 256, max_ctas: int = 0,
         tma_epilogue: bool = True, mc_out: int = 0, drop_p: float = 0.0, drop_seed: int = 0,
         peer_ptrs: Sequence[int] = (), peer_rows: int = 0, peer_rank: int = 0,
         bias: Optional[torch.Tensor] = None, gather_ptrs: Sequence[int] = (), gather_rows: int = 0,
         gather_rank: int = 0, gather_arrived: Optional[torch.Tensor] = None,
         tile_skip: Optional[torch.Tensor] = None) -> None:
    if not native.available():
        raise RuntimeError("bdh gemm: the sm_100a extension is not available")
    if _CHECKED:
        check_extents(a, b, M=M, N=N, K=K, a_mn=a_mn, b_mn=b_mn, nz=nz, a_off=a_off, b_off=b_off, epi=epi, flags=flags,
                      out0=out0, out1=out1, in0=in0, in1=in1, c_off=c_off, o1_off=o1_off, T=T, n_per_head=n_per_head)
    native.ops.gemm(a, a_mn, b, b_mn, M, N, K, nz[0], nz[1], list(a_off), list(b_off), epi, flags, out0, out1,
                       in0, in1, list(c_off), list(o1_off), float(alpha), float(theta), T, pos0, n_per_head, freqs,
                       slopes, causal_tiles, causal_k, bn, max_ctas, tma_epilogue, int(mc_out), float(drop_p),
                    int(drop_seed) & 0x7FFFFFFF, [int(p) for p in peer_ptrs], int(peer_rows), int(peer_rank), bias,
                    [int(p) for p in gather_ptrs], int(gather_rows), int(gather_rank), gather_arrived, tile_skip)


# ------------------------------------------------------------------------------------------------
# fp32 torch statement of the same contract
# ------------------------------------------------------------------------------------------------
def _window(t, mn_major, mn_lo, mn_n, k_lo, k_n):
    if mn_major:
        return t[k_lo:k_lo + k_n, mn_lo:mn_lo + mn_n].float().t()
    return t[mn_lo:mn_lo + mn_n, k_lo:k_lo + k_n].float()


def rot_phases(pos: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    """2*pi*frac(pos*freq) (reference: src/model/attention.rs:342-343). pos [T], freqs [N] -> [T, N]."""
    raw = pos.float()[:, None] * freqs.float()[None, :]
    return (raw - raw.floor()) * (2.0 * math.pi)


def rope_table(pos0: int, T: int, pair_freqs: torch.Tensor) -> torch.Tensor:
    """(cos, sin) of the rotary phase as fp16 pairs, returned bit-cast to a bf16 [T, 2*len(pair_freqs)]
    tensor (the layout the kernels read with TMA): element 2i = cos, 2i+1 = sin of pair i."""
    pos = torch.arange(pos0, pos0 + T, device=pair_freqs.device)
    ph = rot_phases(pos, pair_freqs)
    tab = torch.stack((ph.cos(), ph.sin()), dim=-1).to(torch.float16).reshape(T, -1)
    return tab.view(torch.bfloat16)


def rope_table_rows(positions: torch.Tensor, pair_freqs: torch.Tensor) -> torch.Tensor:
    """`rope_table` for an arbitrary position per row (positions [R] -> bf16-viewed fp16 [R, 2*pairs]):
    a decode step over streams that sit at different positions passes one row per stream."""
    ph = rot_phases(positions, pair_freqs)
    tab = torch.stack((ph.cos(), ph.sin()), dim=-1).to(torch.float16).reshape(positions.shape[0], -1)
    return tab.view(torch.bfloat16)


def _hash32(h: torch.Tensor) -> torch.Tensor:
    m = 0xFFFFFFFF
    h = h ^ (h >> 16)
    h = (h * 0x7feb352d) & m
    h = h ^ (h >> 15)
    h = (h * 0x846ca68b) & m
    return h ^ (h >> 16)


def dropout_keep_mask(seed: int, z0: int, M: int, N: int, p: float, device) -> torch.Tensor:
    """The kernel's counter-based dropout mask for rows m < M, columns n < N of batch index z0:
    one 32-bit hash per (row, column pair), low / high 16 bits for the even / odd column."""
    m32 = 0xFFFFFFFF
    rows = torch.arange(M, device=device, dtype=torch.int64)
    pairs = torch.arange((N + 1) // 2, device=device, dtype=torch.int64)
    base = (seed ^ ((rows * 0x9E3779B1) & m32) ^ ((z0 * 0xC2B2AE3D) & m32)) & m32
    h = _hash32(base[:, None] ^ ((pairs[None, :] * 0x85EBCA77) & m32))
    u = torch.stack((h & 0xFFFF, h >> 16), dim=-1).reshape(M, -1)[:, :N]
    return u >= int(p * 65536.0)


def rope_rotate(x: torch.Tensor, phases: torch.Tensor, inverse: bool = False) -> torch.Tensor:
    """Interleaved-pair rotation (reference: src/model/attention.rs:305-321). x, phases [..., N]."""
    cos, sin = phases.cos(), phases.sin()
    if inverse:
        sin = -sin
    pairs = x.reshape(*x.shape[:-1], -1, 2)
    rotated = torch.stack((-pairs[..., 1], pairs[..., 0]), dim=-1).reshape(x.shape)
    return x * cos + rotated * sin


def gemm_reference(a, b, *, M, N, K, a_mn=False, b_mn=False, nz=(1, 1), a_off=(0, 0, 0, 0), b_off=(0, 0, 0, 0),
                   epi=EPI_STORE, flags=0, out0=None, out1=None, in0=None, in1=None, c_off=(0, 0, 0, 0),
                   o1_off=(0, 0, 0), alpha=1.0, theta=0.0, T=1, pos0=0, n_per_head=1, freqs=None, slopes=None,
                   causal_tiles=0, causal_k=0, bn=256, max_ctas=0, tma_epilogue=True, mc_out=0, drop_p=0.0,
                   drop_seed=0, bias=None, tile_skip=None) -> None:
    """Writes the same outputs as `gemm`, computed in fp32 with torch ops."""
    dev = a.device
    for z1 in range(nz[1]):
        for z0 in range(nz[0]):
            A = _window(a, a_mn, a_off[0] * z0 + a_off[1] * z1, M, a_off[2] * z0 + a_off[3] * z1, K)
            B = _window(b, b_mn, b_off[0] * z0 + b_off[1] * z1, N, b_off[2] * z0 + b_off[3] * z1, K)
            if causal_k == 1:
                # row block mb only contracts k < mb*128 + 128
                acc = torch.zeros(M, N, device=dev)
                for m0 in range(0, M, 128):
                    ke = min(K, m0 + 128)
                    acc[m0:m0 + 128] = A[m0:m0 + 128, :ke] @ B[:, :ke].t()
            elif causal_k == 2:
                # row block mb only contracts k >= mb*128
                acc = torch.zeros(M, N, device=dev)
                for m0 in range(0, M, 128):
                    acc[m0:m0 + 128] = A[m0:m0 + 128, m0:] @ B[:, m0:].t()
            else:
                acc = A @ B.t()
            r0 = c_off[0] * z0 + c_off[1] * z1
            c0 = c_off[2] * z0 + c_off[3] * z1
            rs, cs = slice(r0, r0 + M), slice(c0, c0 + N)
            mm = torch.arange(M, device=dev)
            nn = torch.arange(N, device=dev)
            if epi == EPI_STORE:
                v = acc * alpha
                if flags & F_ROWDECAY:
                    slope = float(slopes[z0]) if slopes is not None else 0.0
                    v = v * torch.exp(-slope * mm.float())[:, None]
                if flags & F_ROWDECAY_REV:
                    slope = float(slopes[z0]) if slopes is not None else 0.0
                    v = v * torch.exp(-slope * (T - mm).float())[:, None]
                if flags & (F_ACCUM | F_ATOMIC):
                    v = v + out0[rs, cs].float()
                out0[rs, cs] = v.to(out0.dtype)
            elif epi == EPI_RELU:
                if bias is not None:
                    acc = acc + bias[c0:c0 + N].float()[None, :]
                x = torch.relu(acc - theta)
                out0[rs, cs] = x.to(out0.dtype)
                if flags & (F_ROPE | F_POPE):
                    pos = pos0 + (mm % T)
                    # RoPE passes one frequency per column pair, PoPE one per column
                    fr = freqs.repeat_interleave(2) if flags & F_ROPE else freqs
                    ph = rot_phases(pos, fr[(nn % n_per_head)])
                    c1 = o1_off[0] * z0 + o1_off[1] * z1
                    if flags & F_ROPE:
                        out1[rs, c1:c1 + N] = rope_rotate(x, ph).to(out1.dtype)
                    else:
                        mag = torch.nn.functional.softplus(x)
                        out1[rs, c1:c1 + N] = (mag * ph.cos()).to(out1.dtype)
                        out1[rs, c1 + o1_off[2]:c1 + o1_off[2] + N] = (mag * ph.sin()).to(out1.dtype)
            elif epi == EPI_RELU_GATE:
                if bias is not None:
                    acc = acc + bias[c0:c0 + N].float()[None, :]
                y = torch.relu(acc - theta)
                if not (flags & F_NO_OUT0):
                    out0[rs, cs] = y.to(out0.dtype)
                xy = y * in0[rs, cs].float()
                if drop_p > 0:
                    keep = dropout_keep_mask(int(drop_seed) & 0x7FFFFFFF, z0, M, N, drop_p, dev)
                    xy = torch.where(keep, xy / (1.0 - drop_p), torch.zeros_like(xy))
                out1[rs, cs] = xy.to(out1.dtype)
            elif epi == EPI_CAUSAL:
                slope = float(slopes[z0]) if slopes is not None else 0.0
                dist = (mm[:, None] - nn[None, :]).float()
                if flags & F_UPPER:
                    mask = dist < 0
                    val = acc * alpha * torch.exp(-slope * dist.abs())
                    cur = out0[rs, cs].float()
                    if causal_tiles == 2:
                        # tiles entirely below the diagonal are never visited
                        pass
                    out0[rs, cs] = torch.where(mask, val, cur).to(out0.dtype)
                else:
                    if flags & F_BIAS:
                        val = torch.where(dist > 0, acc * alpha - slope * dist, torch.zeros_like(acc))
                    else:
                        val = torch.where(dist > 0, acc * alpha * torch.exp(-slope * dist.abs()), torch.zeros_like(acc))
                    if causal_tiles == 1:
                        # tiles with n0 >= m0 + 128 are never written: keep what is there
                        m0 = (mm // 128) * 128
                        n0 = (nn // bn) * bn
                        visited = n0[None, :] <= (m0[:, None] + 127)
                        val = torch.where(visited, val, out0[rs, cs].float())
                    if tile_skip is not None:
                        # skipped tiles (inactive pairs of time blocks) are not written either
                        sk = tile_skip.to(dev).bool()[(mm // 128)[:, None], (nn // bn)[None, :]]
                        val = torch.where(sk, out0[rs, cs].float(), val)
                    out0[rs, cs] = val.to(out0.dtype)
            elif epi == EPI_GATE_BWD:
                # in0 = x, in1 = x*y. y is recovered as xy/x where x > 0; closed x gates get -0.0
                x = in0[rs, cs].float()
                xy = in1[rs, cs].float()
                out0[rs, cs] = torch.where(xy > 0, acc * x * alpha, torch.zeros_like(acc)).to(out0.dtype)
                y = torch.where(x > 0, xy / x.clamp(min=1e-30), torch.zeros_like(x))
                g = acc * y
                g = torch.where(g == 0, torch.zeros_like(g), g)          # +0.0 for open gates
                out1[rs, cs] = torch.where(x > 0, g, torch.full_like(g, -0.0)).to(out1.dtype)
            elif epi == EPI_DQ_BWD:
                # in0 = gate gradient whose -0.0 entries mark closed ReLU gates
                g_raw = in0[rs, cs]
                closed = g_raw.contiguous().view(torch.int16) == -32768
                v = acc
                if flags & F_ROPE:
                    pos = pos0 + ((r0 + mm) % T)           # position of the output row (table mode of the kernel)
                    ph = rot_phases(pos, freqs.repeat_interleave(2)[(nn % n_per_head)])
                    v = rope_rotate(v, ph, inverse=True)
                v = v * alpha + g_raw.float() + 0.0
                mark = -0.0 if flags & F_KEEP_MARK else 0.0
                out0[rs, cs] = torch.where(closed, torch.full_like(v, mark), v).to(out0.dtype)
            else:
                raise ValueError(f"unknown epilogue {epi}")

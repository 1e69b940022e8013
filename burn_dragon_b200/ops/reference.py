"""Plain torch (fp32-friendly, any device) statements of every BDH op.

These are the definitions the CUDA kernels are tested against and the path that runs on CPU.
Citations point at the reference implementation whose behaviour each function restates.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

LN_EPS = 1e-5          # src/model/bdh.rs:17
ROW_NORM_EPS = 1e-6    # src/model/attention.rs:11


def layer_norm(x: torch.Tensor) -> torch.Tensor:
    """Affine-free LayerNorm over the last dim, biased variance (src/model/bdh.rs:86-89)."""
    mean = x.mean(dim=-1, keepdim=True)
    var = (x - mean).pow(2).mean(dim=-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + LN_EPS)


def alibi_slopes(n_head: int, device=None) -> torch.Tensor:
    """m_h = 2^(-h/H), h = 0..H-1 (src/kernel/linear_attention.rs:152-163)."""
    h = torch.arange(n_head, dtype=torch.float32, device=device)
    return torch.pow(2.0, -h / n_head)


def build_freqs(latent: int, theta: float, kind: str, device=None) -> torch.Tensor:
    """Rotary frequencies in cycles per position (src/model/attention.rs:351-373)."""
    idx = torch.arange(latent, dtype=torch.float32, device=device)
    if kind == "rope":
        exponent = torch.floor(idx / 2.0) * 2.0 / latent
    elif kind == "pope":
        exponent = idx / latent
    else:
        return torch.zeros(latent, dtype=torch.float32, device=device)
    return 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float32, device=device), exponent) / (2.0 * math.pi)


def phases(positions: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    """2*pi*frac(pos*freq): [T] x [N] -> [T, N] (src/model/attention.rs:340-343)."""
    raw = positions.to(torch.float32)[:, None] * freqs[None, :]
    return (raw - raw.floor()) * (2.0 * math.pi)


def rope(x: torch.Tensor, ph: torch.Tensor) -> torch.Tensor:
    """Interleaved pair rotation (src/model/attention.rs:305-321). x [..., T, N], ph [T, N]."""
    cos, sin = ph.cos().to(x.dtype), ph.sin().to(x.dtype)
    pairs = x.reshape(*x.shape[:-1], -1, 2)
    rotated = torch.stack((-pairs[..., 1], pairs[..., 0]), dim=-1).reshape(x.shape)
    return x * cos + rotated * sin


def pope(x: torch.Tensor, ph: torch.Tensor) -> torch.Tensor:
    """softplus magnitude times (cos, sin), concatenated: N -> 2N (src/model/attention.rs:323-330)."""
    mag = F.softplus(x)
    return torch.cat((mag * ph.cos().to(x.dtype), mag * ph.sin().to(x.dtype)), dim=-1)


def rotate(x: torch.Tensor, kind: str, freqs: torch.Tensor, start: int) -> torch.Tensor:
    """Apply the configured positional rotation to x [B, H, T, N] (src/model/attention.rs:332-349)."""
    if kind == "alibi":
        return x
    T = x.shape[-2]
    pos = torch.arange(start, start + T, device=x.device)
    ph = phases(pos, freqs.to(x.device))
    return rope(x, ph) if kind == "rope" else pope(x, ph)


# ------------------------------------------------------------------------------------------------
# canonical (recurrent) linear attention and its equivalent forms
# ------------------------------------------------------------------------------------------------
def linear_attention_recurrent(q: torch.Tensor, v: torch.Tensor, decay: Optional[torch.Tensor],
                               rho: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
    """Literal per-timestep recurrence (src/model/bdh.rs:258-307).

    q [B,H,T,N'] (already rotated), v [B,1|H,T,D], decay [H] = exp(-slope) or None, rho [B,H,N',D].
    a_t = q_t . rho ; rho = (rho + q_t^T v_t) * decay. Returns (a [B,H,T,D], rho).
    """
    B, H, T, N = q.shape
    D = v.shape[-1]
    if rho is None or tuple(rho.shape) != (B, H, N, D):
        rho = torch.zeros(B, H, N, D, dtype=q.dtype, device=q.device)
    v = v.expand(B, H, T, D)
    g = decay.to(q.dtype).view(1, H, 1, 1) if decay is not None else None
    outs = []
    for t in range(T):
        qt = q[:, :, t, :]                                   # [B,H,N]
        outs.append(torch.einsum("bhn,bhnd->bhd", qt, rho))
        rho = rho + qt.unsqueeze(-1) * v[:, :, t, :].unsqueeze(-2)
        if g is not None:
            rho = rho * g
    return torch.stack(outs, dim=2), rho


def decay_matrix(T: int, slopes: Optional[torch.Tensor], H: int, device, dtype=torch.float32) -> torch.Tensor:
    """Gamma[h, t, s] = exp(-m_h (t - s)) for s < t, else 0."""
    t = torch.arange(T, device=device)
    dist = (t[:, None] - t[None, :]).to(dtype)
    mask = dist > 0
    if slopes is None:
        return mask.to(dtype).expand(H, T, T)
    g = torch.exp(-slopes.to(dtype).view(H, 1, 1) * dist.clamp(min=0))
    return g * mask


def linear_attention_parallel(q: torch.Tensor, v: torch.Tensor, slopes: Optional[torch.Tensor],
                              rho: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Masked-decay quadratic form, equal to the recurrence:
    a_t = sum_{s<t} g^(t-s) (q_t.q_s) v_s + g^t q_t.rho_in ;  rho_out = g^T rho_in + sum_s g^(T-s) q_s^T v_s."""
    B, H, T, N = q.shape
    D = v.shape[-1]
    v = v.expand(B, H, T, D)
    G = decay_matrix(T, slopes, H, q.device, q.dtype)
    P = torch.matmul(q, q.transpose(-1, -2)) * G
    a = torch.matmul(P, v)
    t = torch.arange(T, device=q.device, dtype=q.dtype)
    if slopes is not None:
        m = slopes.to(q.dtype).view(1, H, 1, 1)
        w_in = torch.exp(-m * t.view(1, 1, T, 1))               # g^t
        w_out = torch.exp(-m * (T - t).view(1, 1, T, 1))        # g^(T-s)
        g_T = torch.exp(-m * T)
    else:
        w_in = w_out = g_T = torch.ones((), dtype=q.dtype, device=q.device)
    if rho is not None and tuple(rho.shape) == (B, H, N, D):
        a = a + w_in * torch.matmul(q, rho)
        rho_out = g_T * rho
    else:
        rho_out = torch.zeros(B, H, N, D, dtype=q.dtype, device=q.device)
    rho_out = rho_out + torch.matmul((q * w_out).transpose(-1, -2), v)
    return a, rho_out


def carry_in(q: torch.Tensor, rho_in: torch.Tensor, slopes: Optional[torch.Tensor]) -> torch.Tensor:
    """What a state carried into the segment adds to the attention output: g^t (q_t . rho_in)."""
    B, H, T, N = q.shape
    a = torch.matmul(q, rho_in.to(q.dtype))
    if slopes is not None:
        t = torch.arange(T, device=q.device, dtype=q.dtype)
        a = a * torch.exp(-slopes.to(q.dtype).view(1, H, 1, 1) * t.view(1, 1, T, 1))
    return a


def linear_attention_chunked(q: torch.Tensor, v: torch.Tensor, slopes: Optional[torch.Tensor],
                             rho: Optional[torch.Tensor] = None, chunk: int = 64) -> Tuple[torch.Tensor, torch.Tensor]:
    """Chunk-state form: quadratic inside a chunk, state hand-off between chunks. Same result as the
    recurrence with O(T*chunk) score memory; this is the long-context algorithm."""
    B, H, T, N = q.shape
    outs = []
    for c0 in range(0, T, chunk):
        a, rho = linear_attention_parallel(q[:, :, c0:c0 + chunk], v[..., c0:c0 + chunk, :], slopes, rho)
        outs.append(a)
    return torch.cat(outs, dim=2), rho


# ------------------------------------------------------------------------------------------------
# `forward_fast` attention: additive ALiBi bias + L1 row normalisation
# ------------------------------------------------------------------------------------------------
def attention_rownorm(q: torch.Tensor, v: torch.Tensor, slopes: Optional[torch.Tensor],
                      block_pairs=None, block: Optional[int] = None, reduce_scores=None) -> torch.Tensor:
    """S = tril(q q^T, -1) (+ m_h * tril(j - i, -1)); S /= sum_j |S_ij| + 1e-6; a = S v
    (src/model/attention.rs:142-175, 300-303). `block_pairs`/`block` restrict the score matrix to the
    active (row-block, col-block) pairs of a BlockPattern2d (src/kernel/linear_attention.rs:54-112).
    `reduce_scores`: when q holds only a shard of the neurons, q q^T is a partial sum; the callable
    sums it over the shards BEFORE the bias and the (non-linear) normalisation."""
    B, H, T, N = q.shape
    D = v.shape[-1]
    v = v.expand(B, H, T, D)
    S = torch.tril(torch.matmul(q, q.transpose(-1, -2)), diagonal=-1)
    if reduce_scores is not None:
        S = reduce_scores(S)
    if slopes is not None:
        t = torch.arange(T, device=q.device, dtype=q.dtype)
        bias = torch.tril(t[None, :] - t[:, None], diagonal=-1)   # (j - i) <= 0 below the diagonal
        S = S + slopes.to(q.dtype).view(1, H, 1, 1) * bias
    if block_pairs is not None and block:
        nb = (T + block - 1) // block
        keep = torch.zeros(nb, nb, dtype=torch.bool, device=q.device)
        for (r, c) in block_pairs:
            if r < nb and c < nb:
                keep[r, c] = True
        keep = keep.repeat_interleave(block, 0).repeat_interleave(block, 1)[:T, :T]
        S = S * keep
    S = S / (S.abs().sum(dim=-1, keepdim=True) + ROW_NORM_EPS)
    return torch.matmul(S, v)


# ------------------------------------------------------------------------------------------------
# encoder / gate / sampling
# ------------------------------------------------------------------------------------------------
def relu_lowrank(inp: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], threshold: float,
                 latent_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """relu(x @ W + b - theta) * block_mask (src/kernel/relu_lowrank.rs:7-37).
    inp [B,1|H,T,D], weight [H,D,N] -> [B,H,T,N]."""
    out = torch.matmul(inp, weight.unsqueeze(0))
    if bias is not None:
        out = out + bias
    out = torch.relu(out - threshold)
    if latent_mask is not None:
        out = out * latent_mask
    return out


def top_k_filter(logits: torch.Tensor, k: Optional[int]) -> torch.Tensor:
    """Keep values >= the k-th largest (ties survive), others -> -inf (src/generation.rs:26-45)."""
    V = logits.shape[-1]
    if k is None or k <= 0 or k >= V:
        return logits
    kth = torch.topk(logits, k, dim=-1).values[..., -1:]
    return torch.where(logits < kth, torch.full_like(logits, float("-inf")), logits)


def sample_logits(logits: torch.Tensor, temperature: float = 1.0, top_k: Optional[int] = None,
                  greedy: bool = False, generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """Next-token draw for logits [..., V] (src/generation.rs:26-72, 106-129): temperature, top-k with
    ties kept, softmax in fp32, uniform fallback when the distribution is degenerate. `greedy` takes
    the arg-max instead (an addition: the reference has no greedy mode)."""
    logits = logits.float()
    if greedy:
        return logits.argmax(dim=-1)
    logits = top_k_filter(logits / max(temperature, 1e-8), top_k)
    probs = torch.softmax(logits, dim=-1)
    bad = ~torch.isfinite(probs).all(dim=-1, keepdim=True) | (probs.sum(dim=-1, keepdim=True) <= 0)
    probs = torch.where(bad, torch.full_like(probs, 1.0 / probs.shape[-1]), probs)
    flat = probs.reshape(-1, probs.shape[-1])
    idx = torch.multinomial(flat, 1, generator=generator).reshape(probs.shape[:-1])
    return idx


def cross_entropy_mean(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Mean CE over all B*T positions (src/model/loss.rs:5-18)."""
    return F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), targets.reshape(-1))

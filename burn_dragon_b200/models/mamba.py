"""Mamba-2 and Mamba-3 language models on the shared trainer / generator / bench interfaces.

The reference has neither (`grep -ri mamba` over it finds nothing); these paths exist because the
framework's scope names them. The specs are frozen here and pinned by the CPU oracles in
`ops.ssd` (literal recurrence == chunked form):

Mamba-2 block (SSD, Dao & Gu 2024), d_inner = expand * d_model, H = d_inner / headdim heads:
    z, xBC, dt = in_proj(u)                      xBC = [x (d_inner) | B (d_state) | C (d_state)]
    xBC = silu(causal_depthwise_conv1d(xBC, width d_conv))
    dt = softplus(dt + dt_bias);  a_t = dt * A,  A = -exp(A_log) per head
    h_t = exp(a_t) h_{t-1} + B_t (x) (dt_t x_t);  y_t = C_t . h_t + D x_t
    out = out_proj( rmsnorm(y * silu(z)) * norm_weight )

Mamba-3 block (this framework's spec of the 2025 design): no convolution; B and C are RMS-normed
with learned per-channel scale and bias and rotated by a data-dependent cumulative angle (complex
state via paired channels); trapezoidal discretisation with a data-dependent mix lambda_t:
    h_t = exp(a_t) h_{t-1} + lambda_t dt_t B_t (x) x_t + (1 - lambda_t) dt_t exp(a_t) B_{t-1} (x) x_{t-1}
optional MIMO rank r (r input and r output maps share one state).

Both are pre-norm residual stacks with un-shared layers, a byte/char embedding and an LM head, and
both expose `forward`, `forward_with_state`, `init_state` and `generate` like the BDH model.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import mamba_ops as MO
from ..ops import reference as R
from ..ops import ssd as SSD


@dataclass
class MambaConfig:
    version: int = 2
    n_layer: int = 6
    d_model: int = 256
    d_state: int = 128
    headdim: int = 64
    expand: int = 2
    chunk_size: int = 64
    d_conv: int = 4
    mimo_rank: int = 1
    vocab_size: int = 256
    dropout: float = 0.0

    @property
    def d_inner(self) -> int:
        return self.expand * self.d_model

    @property
    def n_heads(self) -> int:
        assert self.d_inner % self.headdim == 0
        return self.d_inner // self.headdim

    @property
    def n_embd(self) -> int:
        return self.d_model


def rmsnorm(x: torch.Tensor, weight: Optional[torch.Tensor] = None, eps: float = 1e-5) -> torch.Tensor:
    y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return y * weight if weight is not None else y


@dataclass
class MambaLayerState:
    h: Optional[torch.Tensor] = None          # [B, H, N, P] fp32
    conv: Optional[torch.Tensor] = None       # mamba2: [B, d_conv-1, d_xbc] tail of the conv input
    prev_bx: Optional[tuple] = None           # mamba3: (B_{t-1} [B,r,N], x_{t-1} [B,r,H,P]) of the last step
    angle: Optional[torch.Tensor] = None      # mamba3: cumulative rotation angle [B, N/2]


@dataclass
class MambaState:
    layers: List[MambaLayerState] = field(default_factory=list)
    position: int = 0
    viz = None

    def reset(self):
        for i in range(len(self.layers)):
            self.layers[i] = MambaLayerState()
        self.position = 0

    def trim(self, window: int) -> None:
        return None

    def take_viz(self):
        return None


class Mamba2Block(nn.Module):
    def __init__(self, c: MambaConfig):
        super().__init__()
        self.c = c
        H, N, Di = c.n_heads, c.d_state, c.d_inner
        self.d_xbc = Di + 2 * N
        self.in_proj = nn.Linear(c.d_model, Di + self.d_xbc + H, bias=False)
        self.conv_w = nn.Parameter(torch.randn(self.d_xbc, c.d_conv) * (1.0 / math.sqrt(c.d_conv)))
        self.conv_b = nn.Parameter(torch.zeros(self.d_xbc))
        dt = torch.exp(torch.rand(H) * (math.log(0.1) - math.log(0.001)) + math.log(0.001))
        self.dt_bias = nn.Parameter(dt + torch.log(-torch.expm1(-dt)))        # inverse softplus
        self.A_log = nn.Parameter(torch.log(torch.arange(1, H + 1, dtype=torch.float32)))
        self.D = nn.Parameter(torch.ones(H))
        self.norm_w = nn.Parameter(torch.ones(Di))
        self.out_proj = nn.Linear(Di, c.d_model, bias=False)

    def forward(self, u: torch.Tensor, st: Optional[MambaLayerState]) -> torch.Tensor:
        c = self.c
        Bsz, T, _ = u.shape
        H, N, P, Di = c.n_heads, c.d_state, c.headdim, c.d_inner
        z, xbc, dt = torch.split(self.in_proj(u), [Di, self.d_xbc, H], dim=-1)
        tail = st.conv if st is not None and st.conv is not None else xbc.new_zeros(Bsz, c.d_conv - 1, self.d_xbc)
        seq = torch.cat((tail.to(xbc.dtype), xbc), dim=1)                      # [B, T + k - 1, C]
        if st is not None:
            st.conv = seq[:, -(c.d_conv - 1):].detach()
        xbc = MO.conv1d_silu(seq, self.conv_w, self.conv_b)                    # one kernel per direction on a GPU
        x, Bm, Cm = torch.split(xbc, [Di, N, N], dim=-1)
        dt = F.softplus(dt.float() + self.dt_bias)                             # [B,T,H]
        loga = dt * (-torch.exp(self.A_log.float()))
        xh = x.view(Bsz, T, H, P).float()
        h0 = st.h if st is not None else None
        y, hT = SSD.ssd(xh * dt.unsqueeze(-1), loga, Bm.float(), Cm.float(), h0, c.chunk_size)
        if st is not None:
            st.h = hT.detach()
        y = y + xh * self.D.view(1, 1, H, 1)
        y = MO.gated_rmsnorm(y.reshape(Bsz, T, Di).to(u.dtype), z, self.norm_w)
        return self.out_proj(y)


class Mamba3Block(nn.Module):
    def __init__(self, c: MambaConfig):
        super().__init__()
        self.c = c
        H, N, Di, r = c.n_heads, c.d_state, c.d_inner, c.mimo_rank
        assert N % 2 == 0
        # z | x (r copies) | B (r) | C (r) | dt (H) | lambda (H) | omega (N/2)
        self.sizes = [Di, Di * r, N * r, N * r, H, H, N // 2]
        self.in_proj = nn.Linear(c.d_model, sum(self.sizes), bias=False)
        dt = torch.exp(torch.rand(H) * (math.log(0.1) - math.log(0.001)) + math.log(0.001))
        self.dt_bias = nn.Parameter(dt + torch.log(-torch.expm1(-dt)))
        self.A_log = nn.Parameter(torch.log(torch.arange(1, H + 1, dtype=torch.float32)))
        self.D = nn.Parameter(torch.ones(H))
        self.b_scale = nn.Parameter(torch.ones(r, N))
        self.b_bias = nn.Parameter(torch.zeros(r, N))
        self.c_scale = nn.Parameter(torch.ones(r, N))
        self.c_bias = nn.Parameter(torch.zeros(r, N))
        self.norm_w = nn.Parameter(torch.ones(Di * r))
        self.out_proj = nn.Linear(Di * r, c.d_model, bias=False)

    @staticmethod
    def _rotate(v: torch.Tensor, ang: torch.Tensor) -> torch.Tensor:
        """Rotate channel pairs (2i, 2i+1) of v [..., N] by ang [..., N/2]."""
        cos, sin = ang.cos().unsqueeze(-1), ang.sin().unsqueeze(-1)
        p = v.reshape(*v.shape[:-1], -1, 2)
        out = torch.cat((p[..., :1] * cos - p[..., 1:] * sin, p[..., 1:] * cos + p[..., :1] * sin), dim=-1)
        return out.reshape(v.shape)

    def forward(self, u: torch.Tensor, st: Optional[MambaLayerState]) -> torch.Tensor:
        c = self.c
        Bsz, T, _ = u.shape
        H, N, P, Di, r = c.n_heads, c.d_state, c.headdim, c.d_inner, c.mimo_rank
        z, x, Bm, Cm, dt, lam, om = torch.split(self.in_proj(u).float(), self.sizes, dim=-1)
        dt = F.softplus(dt + self.dt_bias)                                     # [B,T,H]
        loga = dt * (-torch.exp(self.A_log.float()))
        lam = torch.sigmoid(lam)
        Bm = rmsnorm(Bm.view(Bsz, T, r, N)) * self.b_scale + self.b_bias
        Cm = rmsnorm(Cm.view(Bsz, T, r, N)) * self.c_scale + self.c_bias
        # data-dependent rotation: cumulative angle, carried across calls
        step_ang = om * dt.mean(dim=-1, keepdim=True)                          # [B,T,N/2]
        ang0 = st.angle if st is not None and st.angle is not None else om.new_zeros(Bsz, N // 2)
        ang = ang0.unsqueeze(1) + torch.cumsum(step_ang, dim=1)
        if st is not None:
            st.angle = ang[:, -1].detach()
        Bm = self._rotate(Bm, ang.unsqueeze(2))
        Cm = self._rotate(Cm, ang.unsqueeze(2))
        xh = x.view(Bsz, T, r, H, P)
        # trapezoid: current term weight lambda*dt, previous term weight (1-lambda)*dt*exp(a)
        w_cur = (lam * dt)
        w_prev = ((1 - lam) * dt * torch.exp(loga))
        if st is not None and st.prev_bx is not None:
            pB, pX = st.prev_bx
        else:
            pB, pX = Bm.new_zeros(Bsz, r, N), xh.new_zeros(Bsz, r, H, P)
        B_prev = torch.cat((pB.unsqueeze(1), Bm[:, :-1]), dim=1)
        x_prev = torch.cat((pX.unsqueeze(1), xh[:, :-1]), dim=1)
        if st is not None:
            st.prev_bx = (Bm[:, -1].detach(), xh[:, -1].detach())
        h0 = st.h if st is not None else None
        ys = [0.0] * r
        hT = None
        # the state is shared by all r input maps (contributions add) and read by all r output maps
        for ro in range(r):
            acc = 0.0
            for ri in range(r):
                # two input streams per map; the carried state enters exactly once (ri == 0, first stream)
                y1, h1 = SSD.ssd(xh[:, :, ri] * w_cur.unsqueeze(-1), loga, Bm[:, :, ri], Cm[:, :, ro],
                                 h0 if ri == 0 else None, c.chunk_size)
                y2, h2 = SSD.ssd(x_prev[:, :, ri] * w_prev.unsqueeze(-1), loga, B_prev[:, :, ri], Cm[:, :, ro],
                                 None, c.chunk_size)
                acc = acc + y1 + y2
                if ro == 0:
                    hT = (h1 + h2) if hT is None else hT + h1 + h2
            ys[ro] = acc + xh[:, :, ro] * self.D.view(1, 1, H, 1)
        if st is not None:
            st.h = hT.detach()
        y = torch.stack(ys, dim=2).reshape(Bsz, T, r * Di).to(u.dtype)
        y = rmsnorm(y * F.silu(z.to(u.dtype)).repeat(1, 1, r), self.norm_w)
        return self.out_proj(y)


class MambaLM(nn.Module):
    def __init__(self, config: MambaConfig):
        super().__init__()
        self.config = config
        c = config
        self.embed = nn.Embedding(c.vocab_size, c.d_model)
        blk = Mamba2Block if c.version == 2 else Mamba3Block
        self.layers = nn.ModuleList([blk(c) for _ in range(c.n_layer)])
        self.norms = nn.ParameterList([nn.Parameter(torch.ones(c.d_model)) for _ in range(c.n_layer)])
        self.norm_f = nn.Parameter(torch.ones(c.d_model))
        self.lm_head = nn.Linear(c.d_model, c.vocab_size, bias=False)
        self.drop = nn.Dropout(c.dropout)
        nn.init.normal_(self.embed.weight, 0.0, 0.02)
        self.use_native = True

    def init_state(self) -> MambaState:
        return MambaState([MambaLayerState() for _ in range(self.config.n_layer)], 0)

    def _run(self, tokens: torch.Tensor, state: Optional[MambaState]) -> torch.Tensor:
        x = self.embed(tokens)
        for i, layer in enumerate(self.layers):
            st = state.layers[i] if state is not None else None
            x = x + self.drop(layer(rmsnorm(x, self.norms[i]), st))
        if state is not None:
            state.position += tokens.shape[1]
        return self.lm_head(rmsnorm(x, self.norm_f))

    def forward_with_state(self, tokens, state, mode: str = "auto"):
        return self._run(tokens, state)

    def forward(self, tokens, targets=None, mode: str = "auto"):
        logits = self._run(tokens, None)
        if targets is not None:
            return R.cross_entropy_mean(logits, targets)
        return logits

    def forward_fast(self, tokens, targets=None):
        return self.forward(tokens, targets)

    @torch.no_grad()
    def generate(self, idx, max_new_tokens, temperature=1.0, top_k=None, greedy=False, generator=None,
                 on_token: Optional[Callable] = None):
        state = self.init_state()
        logits = self.forward_with_state(idx, state)[:, -1]
        out = [idx]
        for _ in range(max_new_tokens):
            nxt = R.sample_logits(logits, temperature, top_k, greedy, generator).view(-1, 1)
            out.append(nxt)
            if on_token is not None:
                on_token(nxt)
            logits = self.forward_with_state(nxt, state)[:, -1]
        return torch.cat(out, dim=1)

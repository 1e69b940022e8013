"""BDH-GPU language model (Dragon Hatchling).

Behaviour follows the reference model (src/model/bdh.rs:19-450, src/model/attention.rs:102-373,
src/model/config.rs:11-164, src/model/state.rs:5-80): one set of weights shared by all layers,
ReLU-sparse neuron encoders E / E_v, un-normalised causal linear attention over the sparse
activations with RoPE / PoPE rotation or ALiBi state decay, x*y gating, decoder D, affine-free
LayerNorms and an LM head. Two forward functions exist and are different functions:

  forward / forward_with_state   canonical recurrent semantics (training default, inference)
  forward_fast                   quadratic scores + additive ALiBi bias + L1 row normalisation

Weight layout differs from the reference on purpose: the three big matrices are stored
neuron-major, `[H*N, D]` (row = one neuron), which is the K-major operand layout the tcgen05
GEMMs consume directly. `engine.burn_record` converts to and from the reference's `[H, D, N]` /
`[H*N, D]` record layout.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import reference as R
from ..ops.block_sparse import BlockPattern1d, BlockPattern2d, BlockSparseConfig


@dataclass
class BDHConfig:
    """reference: src/model/config.rs:114-164 (defaults) plus `n_latent_per_head` to give N directly."""
    n_layer: int = 6
    n_embd: int = 256
    n_head: int = 4
    mlp_internal_dim_multiplier: int = 4
    n_expert: int = 1
    vocab_size: int = 256
    dropout: float = 0.1
    relu_threshold: float = 0.0
    rotary_embedding: str = "alibi"
    rope_theta: float = 65536.0
    fused_kernels: bool = False          # reference flag: use the blocked op compositions
    block_size: int = 512                # block size of the reference's blocked ops
    n_latent_per_head: Optional[int] = None
    block_sparse: Optional[BlockSparseConfig] = None
    alibi_slopes: Optional[List[float]] = None

    def __post_init__(self):
        if self.n_expert != 1:
            raise ValueError("n_expert must be 1 (expert routing is not part of the model)")
        if self.rotary_embedding not in ("alibi", "rope", "pope"):
            raise ValueError(f"unknown rotary_embedding {self.rotary_embedding}")
        if self.n_latent_per_head is None:
            total = self.mlp_internal_dim_multiplier * self.n_embd
            if total % self.n_head != 0:
                raise ValueError("mlp_internal_dim_multiplier * n_embd must be divisible by n_head")
        if self.rotary_embedding == "rope" and self.latent_per_head % 2:
            raise ValueError("RoPE needs an even latent size per head")

    @property
    def latent_per_head(self) -> int:
        """N (src/model/config.rs:141-155)."""
        if self.n_latent_per_head is not None:
            return int(self.n_latent_per_head)
        return self.mlp_internal_dim_multiplier * self.n_embd // self.n_head

    @property
    def latent_total(self) -> int:
        return self.latent_per_head * self.n_head

    @property
    def state_latent(self) -> int:
        """N' : rows of the recurrent state per head (2N for PoPE)."""
        return self.latent_per_head * (2 if self.rotary_embedding == "pope" else 1)

    def num_params(self) -> int:
        return 3 * self.latent_total * self.n_embd + 2 * self.vocab_size * self.n_embd

    def flops_per_token_forward(self, T: int) -> float:
        """Forward FLOPs per token: both encoder GEMMs, causal attention (half the T^2 products),
        decoder and LM head. (The reference's own model, src/bin/train.rs:635-659, counts one encoder
        and no LM head.)"""
        D, HN, Np, H = self.n_embd, self.latent_total, self.state_latent, self.n_head
        per_layer = 2 * 2 * D * HN + 2 * HN * D + (2 * H * T * Np + 2 * H * T * D) / 2
        return self.n_layer * per_layer + 2 * D * self.vocab_size


@dataclass
class LayerState:
    rho: Optional[torch.Tensor] = None       # [B, H, N', D]


@dataclass
class ModelState:
    """Recurrent state of all layers plus the absolute position (src/model/state.rs:5-57)."""
    layers: List[LayerState] = field(default_factory=list)
    position: int = 0
    viz: Optional[list] = None               # last-token x / y / xy / rho energy per layer when captured

    @staticmethod
    def new(n_layer: int) -> "ModelState":
        return ModelState([LayerState() for _ in range(n_layer)], 0)

    def reset(self) -> None:
        for l in self.layers:
            l.rho = None
        self.position = 0

    def trim(self, window: int) -> None:
        """No-op, as in the reference (src/model/state.rs:55-57): the state has no time axis."""
        return None

    def take_viz(self):
        v, self.viz = self.viz, None
        return v


class BDH(nn.Module):
    def __init__(self, config: BDHConfig):
        super().__init__()
        self.config = config
        c = config
        HN, D, V = c.latent_total, c.n_embd, c.vocab_size
        self.embed = nn.Embedding(V, D)                       # N(0,1), like Burn's default embedding init
        self.encoder = nn.Parameter(torch.empty(HN, D))       # E   : row (h*N + n) = neuron n of head h
        self.encoder_v = nn.Parameter(torch.empty(HN, D))     # E_v
        self.decoder = nn.Parameter(torch.empty(HN, D))       # D
        self.lm_head = nn.Parameter(torch.empty(D, V))
        for p in (self.encoder, self.encoder_v, self.decoder, self.lm_head):
            nn.init.normal_(p, 0.0, 0.02)                     # src/model/bdh.rs:50-67
        self.register_buffer("freqs", R.build_freqs(c.latent_per_head, c.rope_theta, c.rotary_embedding),
                             persistent=False)
        slopes = (torch.tensor(c.alibi_slopes, dtype=torch.float32) if c.alibi_slopes is not None
                  else R.alibi_slopes(c.n_head))
        self.register_buffer("slopes", slopes, persistent=False)
        self.capture_viz = False
        self.use_native = True     # use the sm_100a kernels whenever they apply

    # ---- helpers -------------------------------------------------------------------------------
    @property
    def use_alibi(self) -> bool:
        return self.config.rotary_embedding == "alibi"

    def _slopes(self) -> Optional[torch.Tensor]:
        return self.slopes if self.use_alibi else None

    def _latent_mask(self, device, dtype) -> Optional[torch.Tensor]:
        bs = self.config.block_sparse
        if bs is None or not bs.latent.is_sparse():
            return None
        return bs.latent.mask(self.config.latent_per_head, device=device, dtype=dtype)

    def _enc(self, w: torch.Tensor) -> torch.Tensor:
        """[H*N, D] -> [H, D, N] view for the torch path."""
        c = self.config
        return w.view(c.n_head, c.latent_per_head, c.n_embd).transpose(1, 2)

    def init_state(self) -> ModelState:
        return ModelState.new(self.config.n_layer)

    # ---- torch path (any device; the definition) ------------------------------------------------
    def _layer_torch(self, cur, start, rho, mode: str):
        """One layer. cur [B,1,T,D]. mode: 'recurrent' | 'parallel' | 'chunked' | 'fast'."""
        c = self.config
        mask = self._latent_mask(cur.device, cur.dtype)
        # neuron-sharded tensor parallelism (parallel/tp.py): `cur` and LN(a) are replicated inputs of
        # sharded products (their gradients are summed over the ranks), `a` and the decoder output are
        # partial sums over the neuron shards (summed in the forward pass); the residual uses `cur` as is
        tp = getattr(self, "_tp", None)
        res = cur
        if tp is not None:
            cur = tp.copy(cur)
        x = R.relu_lowrank(cur, self._enc(self.encoder).to(cur.dtype), None, c.relu_threshold, mask)
        new_rho = None
        if mode == "fast":
            q = R.rotate(x, c.rotary_embedding, self.freqs, 0)
            pairs = block = None
            if c.block_sparse is not None and c.block_sparse.time.is_sparse():
                block = c.block_sparse.time.block_size
                pairs = c.block_sparse.time.pairs((cur.shape[2] + block - 1) // block)
            from ..ops import rownorm_attention as RA
            if tp is not None:
                # neuron-sharded: the scores are partial sums over the shards and must be complete before
                # the normalisation; S V is then the same on every rank, so V is the replicated `res`
                # (whose gradient is NOT summed over the ranks) and `a` needs no reduction
                a = R.attention_rownorm(q, res, self._slopes(), pairs, block, reduce_scores=tp.reduce)
            elif pairs is None and getattr(self, "use_native", True) and RA.can_run(q, cur):
                a = RA.attention_rownorm(q, cur, self._slopes())
            else:
                a = R.attention_rownorm(q, cur, self._slopes(), pairs, block)
        else:
            q = R.rotate(x, c.rotary_embedding, self.freqs, start)
            if mode == "recurrent":
                decay = torch.exp(-self.slopes) if self.use_alibi else None
                a, new_rho = R.linear_attention_recurrent(q, cur, decay, rho)
            elif getattr(self, "_cp", None) is not None:
                # context parallel: local part, state exchange between the ranks, then the carried part
                fn = R.linear_attention_chunked if mode == "chunked" else R.linear_attention_parallel
                a, rho_loc = fn(q, cur, self._slopes(), None)
                sl = self._slopes()
                g_T = torch.exp(-sl.to(q.dtype) * q.shape[2]).view(1, -1, 1, 1) if sl is not None else 1.0
                if torch.is_grad_enabled() and rho_loc.requires_grad:
                    # training: the hand-off is part of the autograd graph (no state leaves the call)
                    new_rho = None
                    a = a + R.carry_in(q, self._cp.scan_grad(rho_loc, g_T), sl)
                else:
                    rho_in, new_rho = self._cp.scan(rho_loc, rho, g_T)
                    if rho_in is not None:
                        a = a + R.carry_in(q, rho_in, sl)
            elif mode == "chunked":
                a, new_rho = R.linear_attention_chunked(q, cur, self._slopes(), rho)
            else:
                a, new_rho = R.linear_attention_parallel(q, cur, self._slopes(), rho)
        if tp is not None and mode != "fast":
            a = tp.reduce(a)
        a = R.layer_norm(a)
        if tp is not None:
            a = tp.copy(a)
        y = R.relu_lowrank(a, self._enc(self.encoder_v).to(cur.dtype), None, c.relu_threshold, mask)
        xy = F.dropout(x * y, c.dropout, self.training)
        B, H, T, N = xy.shape
        mlp = xy.transpose(1, 2).reshape(B * T, H * N) @ self.decoder.to(cur.dtype)
        if tp is not None:
            mlp = tp.reduce(mlp)
        mlp = R.layer_norm(mlp.view(B, 1, T, c.n_embd))
        out = R.layer_norm(res + mlp)
        return out, new_rho, (x, y, xy)

    def _forward_torch(self, tokens, state: Optional[ModelState], mode: str, start: int = 0):
        c = self.config
        cur = R.layer_norm(self.embed(tokens)).unsqueeze(1)          # [B,1,T,D]
        start = state.position if state is not None else start
        viz = []
        for l in range(c.n_layer):
            rho = state.layers[l].rho if state is not None else None
            cur, new_rho, acts = self._layer_torch(cur, start, rho, mode)
            if l == c.n_layer - 1 and getattr(self, "measure_sparsity", False):
                self.last_sparsity = dict(x=(acts[0] != 0).float().mean().detach(),
                                          xy=(acts[2] != 0).float().mean().detach())
            if state is not None and mode != "fast":
                state.layers[l].rho = new_rho
                if self.capture_viz:
                    x, y, xy = acts
                    viz.append(dict(x_last=x[:, :, -1].detach(), y_last=y[:, :, -1].detach(),
                                    xy_last=xy[:, :, -1].detach(),
                                    rho_last=new_rho.detach().abs().mean(dim=-1)))
        if state is not None and mode != "fast":
            state.position += tokens.shape[1]
            if self.capture_viz:
                state.viz = viz
        B, _, T, D = cur.shape
        return (cur.reshape(B * T, D) @ self.lm_head.to(cur.dtype)).view(B, T, c.vocab_size)

    # ---- public forward functions ---------------------------------------------------------------
    def forward_with_state(self, tokens: torch.Tensor, state: ModelState, mode: str = "auto") -> torch.Tensor:
        """Canonical semantics with an explicit recurrent state that is read and updated
        (src/model/bdh.rs:309-450). `mode='recurrent'` runs the literal per-step loop; the other
        modes compute the same function in parallel / chunked form."""
        if mode == "auto":
            from ..ops import fused_bdh
            if fused_bdh.can_run(self, tokens, state):
                return fused_bdh.forward_logits(self, tokens, state)
            mode = "parallel" if tokens.shape[1] <= 1024 else "chunked"
        return self._forward_torch(tokens, state, mode)

    def forward(self, tokens: torch.Tensor, targets: Optional[torch.Tensor] = None, mode: str = "auto"):
        """Stateless canonical forward (src/model/bdh.rs:91-94). With `targets`, returns the mean
        cross-entropy loss instead of logits (the training call)."""
        if mode == "auto":
            from ..ops import fused_bdh
            if fused_bdh.can_run(self, tokens, None):
                if targets is not None:
                    return fused_bdh.loss(self, tokens, targets)
                return fused_bdh.forward_logits(self, tokens, None)
            mode = "parallel" if tokens.shape[1] <= 1024 else "chunked"
        logits = self._forward_torch(tokens, None, mode)
        if targets is not None:
            return R.cross_entropy_mean(logits, targets)
        return logits

    def forward_fast(self, tokens: torch.Tensor, targets: Optional[torch.Tensor] = None):
        """Row-normalised parallel path (src/model/bdh.rs:96-168). Produces no state."""
        from ..ops import fused_bdh
        # (under neuron-sharded tensor parallelism this mode runs on the torch path: the scores have to
        # be summed over the shards before they are normalised, which the fused stack does not do)
        if getattr(self, "_tp", None) is None and fused_bdh.can_run(self, tokens, None):
            if targets is not None:
                return fused_bdh.loss(self, tokens, targets, fast=True)
            return fused_bdh.forward_logits(self, tokens, None, fast=True)
        logits = self._forward_torch(tokens, None, "fast")
        if targets is not None:
            return R.cross_entropy_mean(logits, targets)
        return logits

    @torch.no_grad()
    def generate(self, idx: torch.Tensor, max_new_tokens: int, temperature: float = 1.0,
                 top_k: Optional[int] = None, greedy: bool = False,
                 generator: Optional[torch.Generator] = None,
                 on_token: Optional[Callable[[torch.Tensor], None]] = None) -> torch.Tensor:
        """Prefill then cached single-token decode (src/model/bdh.rs:170-252). idx [B, P] -> [B, P+n].
        Unlike the reference (batch 1 only) every row of the batch is an independent stream."""
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


def build_model_config(overrides, training_block_size: int, vocab_size: Optional[int] = None) -> BDHConfig:
    """Apply `[model]` overrides over the defaults (src/inference.rs:4-40). The blocked ops' block
    size defaults to the training block size."""
    c = BDHConfig()
    kw = {}
    for name in ("n_layer", "n_embd", "n_head", "mlp_internal_dim_multiplier", "relu_threshold", "dropout",
                 "fused_kernels", "rotary_embedding", "n_latent_per_head", "rope_theta"):
        v = getattr(overrides, name, None)
        if v is not None:
            kw[name] = v
    block = getattr(overrides, "block_size", None) or training_block_size
    kw["block_size"] = max(1, int(block))
    vs = vocab_size if vocab_size is not None else getattr(overrides, "vocab_size", None)
    if vs is not None:
        kw["vocab_size"] = int(vs)
    active = getattr(overrides, "latent_active_blocks", None)
    cfg = BDHConfig(**{**c.__dict__, **kw})
    latent = (BlockPattern1d.from_blocks(getattr(overrides, "graph_block", None) or cfg.block_size, active)
              if active is not None else BlockPattern1d.dense(cfg.block_size))
    cfg.block_sparse = BlockSparseConfig(latent, BlockPattern2d.dense(cfg.block_size))
    return cfg

"""BDH forward / backward on the sm_100a kernels.

The whole stack (embedding+LN, L shared-weight layers, LM head, cross-entropy) is one
`torch.autograd.Function`; its forward and backward are explicit sequences of tcgen05 GEMM
launches with fused epilogues plus a few row-wise kernels. The math is the canonical recurrent
semantics of the reference (src/model/bdh.rs:309-450) in its exact parallel form
    a_t = sum_{s<t} g^(t-s) (q_t . q_s) v_s
evaluated as  S = causal_decay(Q Q^T),  A = S V  per (batch, head).

Activation layouts (all bf16, row-major 2-D):
  cur  [M, D]          M = B*T tokens, row b*T + t
  x,q,y,xy [M, H*N']   column h*N' + n
  S    [B*H*T, T]      row (b*H + h)*T + t, column s
  a    [H*M, D]        row (h*B + b)*T + t   (head-major so each head's rows are contiguous)
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch

from . import dual_gemm as DG
from . import gemm as G
from . import native
from ..utils import compressed_pool as _CP
from ..utils import profiling as prof

ops = native.ops


# ------------------------------------------------------------------------------------------------
# eligibility
# ------------------------------------------------------------------------------------------------
def can_run(model, tokens: torch.Tensor, state) -> bool:
    """True when the kernel path computes exactly what the torch path defines for this call."""
    if not getattr(model, "use_native", True):
        return False
    if not emulate.active() and (not tokens.is_cuda or not native.available()):
        return False
    c = model.config
    B, T = tokens.shape
    if T % 64 or c.n_embd % 8 or c.n_embd > 2048 or c.latent_per_head % 64:
        return False
    if c.block_sparse is not None and c.block_sparse.latent.is_sparse():
        # a latent block pattern runs on the kernels with the inactive neuron blocks left out of every operand
        # (`_Dims.rows`); PoPE gives a masked neuron the non-zero query softplus(0), the sharded wrappers have
        # their own row bookkeeping: those keep the torch path
        lat = c.block_sparse.latent
        n_act = sum(min((b + 1) * lat.block_size, c.latent_per_head) - b * lat.block_size
                    for b in lat.active_blocks if b * lat.block_size < c.latent_per_head)
        if (c.rotary_embedding == "pope" or lat.block_size % 2 or n_act == 0 or n_act % 64
                or getattr(model, "_dims_hook", None) is not None or getattr(model, "_grad_sink", None) is not None
                or getattr(model, "_cp", None) is not None):
            return False
    if c.vocab_size > 1024:
        return False
    if state is not None:
        has_rho = any(l.rho is not None for l in state.layers)
        if has_rho and any(l.rho is None or l.rho.shape[0] != B for l in state.layers):
            return False
    return True


def _weights(model) -> Dict[str, torch.Tensor]:
    """bf16 working copies of the parameters. An optimizer that keeps a bf16 shadow registers it as
    `model._bf16_shadow`; otherwise the weights are cast here."""
    sh = getattr(model, "_bf16_shadow", None)
    if sh is not None:
        return sh
    return {n: p.detach().to(torch.bfloat16) for n, p in
            (("embed", model.embed.weight), ("encoder", model.encoder), ("encoder_v", model.encoder_v),
             ("decoder", model.decoder), ("lm_head", model.lm_head))}


def _compact(d, W):
    """Weights of the active neurons only (latent block pattern), else W unchanged."""
    if d.rows is None:
        return W
    return {**W, **{k: W[k].index_select(0, d.rows) for k in ("encoder", "encoder_v", "decoder")}}


class _Dims:
    def table(self, pos0: int) -> torch.Tensor:
        """RoPE (cos, sin) table for positions [pos0, pos0 + T), cached per start position."""
        if self._table is None or self._table[0] != pos0:
            self._table = (pos0, G.rope_table(pos0, self.T, self.freqs))
        return self._table[1]

    def __init__(self, model, B, T, fast: bool = False):
        self._table = None
        self.device = model.encoder.device
        self.fast = bool(fast)     # `forward_fast` semantics: additive bias + L1 row normalisation, no state
        self.comm = None           # set by the neuron-sharded tensor-parallel wrapper
        c = model.config
        self.B, self.T, self.M = B, T, B * T
        self.D, self.H, self.N = c.n_embd, c.n_head, c.latent_per_head
        self.Np = c.state_latent
        # latent block pattern: only the neurons of active blocks exist on the kernel path
        self.N_full, self.idx, self.rows = self.N, None, None
        if c.block_sparse is not None and c.block_sparse.latent.is_sparse():
            from . import lowrank
            self.idx = lowrank.active_index(c.block_sparse.latent, self.N, model.encoder.device)
            self.rows = lowrank.head_rows(self.idx, self.H, self.N)
            self.N = self.Np = int(self.idx.numel())
        self.HN, self.HNp = self.H * self.N, self.H * self.Np
        self.V = c.vocab_size
        self.L = c.n_layer
        self.rot = c.rotary_embedding
        self.theta = float(c.relu_threshold)
        # the RoPE epilogues take one frequency per (2i, 2i+1) column pair, PoPE one per column
        if self.rot == "rope":
            fr = model.freqs.float() if self.idx is None else model.freqs.float()[self.idx]
            self.freqs = fr[0::2].contiguous()
            self.freqs_full = fr.contiguous()
        elif self.rot == "pope":
            self.freqs = self.freqs_full = model.freqs.float().contiguous()
        else:
            self.freqs = self.freqs_full = None
        self.slopes = model.slopes.float().contiguous() if self.rot == "alibi" else None
        # time block pattern (row-normalised mode only, as in the reference: src/kernel/linear_attention.rs:54-112):
        # a [T, T] 0/1 matrix of the active (row block, column block) pairs, applied to the scores
        self.time_keep = None
        self.tile_skip = None
        if self.fast and c.block_sparse is not None and c.block_sparse.time.is_sparse():
            tp = c.block_sparse.time
            nb = -(-T // tp.block_size)
            keep = torch.zeros(nb, nb, dtype=torch.bool)
            for (r, cc) in tp.pairs(nb):
                keep[r, cc] = True
            keep = keep.repeat_interleave(tp.block_size, 0).repeat_interleave(tp.block_size, 1)[:T, :T]
            self.time_keep = keep.to(device=model.encoder.device, dtype=torch.bfloat16)
            # output tiles (128 rows x 256 columns) of the score GEMMs that hold no active strictly-causal entry are
            # not computed at all (the tile predicate of the causal walker); the mask still clears partial tiles
            tm, tn = -(-T // 128), -(-T // 256)
            padded = torch.zeros(tm * 128, tn * 256, dtype=torch.bool)
            padded[:T, :T] = keep.bool() & torch.ones(T, T, dtype=torch.bool).tril(-1)
            active = padded.view(tm, 128, tn, 256).any(dim=3).any(dim=1)
            self.tile_skip = (~active).to(torch.uint8).contiguous().to(model.encoder.device)
        self.cp = getattr(model, "_cp", None)        # context-parallel hook (parallel/cp.py)
        # fully sharded data parallelism: the weight gradients of the [H*N, D] weights go to their owners' slices
        # from the GEMM epilogues (parallel/fsdp.py: GradSink) instead of into local full-size tensors
        self.sink = getattr(model, "_grad_sink", None)
        # dropout on x*y (training only): a fresh mask seed per call, one derived seed per layer
        self.drop_p = float(c.dropout) if (model.training and c.dropout > 0) else 0.0
        model._drop_calls = getattr(model, "_drop_calls", 0) + 1
        self.drop_base = (torch.initial_seed() * 0x9E3779B1 + model._drop_calls * 0x85EBCA77) & 0x7FFFFFFF
        hook = getattr(model, "_dims_hook", None)
        if hook is not None:
            hook(self)
        # the chained-GEMM kernels (the [tokens, neurons] intermediates x*y, dy, dx never re-read by the GEMM that
        # contracts them) cover unsharded layers with D <= 256; the backward chains leave PoPE to the separate
        # launches (its rotated copy has twice the width)
        # chunk-state attention: the sequence is cut into J segments of C tokens; inside a segment the scores
        # are the quadratic causal form, between segments the [N', D] state is handed on (and its gradient
        # handed back), so the score matrix is [.., C] wide instead of [.., T]. `model.attention_chunk`: an int,
        # or None = automatic (1024 from T = 4096 on when T > 1024 + 4 D, where the quadratic form costs more than
        # the state products). The row-normalised mode has no state; the neuron-sharded wrapper keeps one segment.
        self.C = T
        chunk = getattr(model, "attention_chunk", None)
        if not self.fast and self.comm is None:
            if chunk is None and T >= 4096 and T % 1024 == 0 and T > 1024 + 4 * self.D:
                # per token and head the quadratic form costs about 3 score-sized products over T/2 columns, the
                # segments 3 over C/2 plus 5 state-sized products over D: segments pay from T > C + ~3.3 D on
                chunk = 1024
            if chunk and 0 < int(chunk) < T and T % int(chunk) == 0 and int(chunk) % 64 == 0:
                self.C = int(chunk)
        self.J = T // self.C
        self.Bs = B * self.J                         # number of (sequence, segment) problems
        self.handoff = self.J > 1 or self.cp is not None   # states (and their gradients) cross segment borders
        ok_fwd = self.comm is None and DG.eligible(self.M, self.T, self.N, self.D)
        ok = ok_fwd and self.rot != "pope"
        which = getattr(model, "use_dual_gemm", None)
        if which is None:
            which = os.environ.get("BDH_DUAL", "fwd")
        which = set(str(which).split(",")) if which else set()
        # (the forward chain - y, gate, decoder - does not touch the rotated query, so PoPE models take it too)
        self.dual_fwd = ok_fwd and bool(which & {"fwd", "all", "True"})
        self.dual_gate = ok and bool(which & {"gate", "all", "True"})
        self.dual_dq = ok and bool(which & {"dq", "all", "True"}) and not self.handoff

    def decay(self, n: int):
        """g^n per head as a [1, H, 1, 1] tensor, or None without ALiBi decay."""
        return torch.exp(-self.slopes * float(n)).view(1, self.H, 1, 1) if self.slopes is not None else None


_SM_COUNT = {}


def _split_k(tiles: int, K: int, dev) -> int:
    """Split factor for a GEMM with few output tiles and a long K: the persistent kernel runs one
    CTA per SM, so `tiles` that are not close to a multiple of the SM count leave SMs idle in the
    last wave. Splitting K multiplies the tile count; partial sums meet through fp32 atomics."""
    sms = _SM_COUNT.get(dev)
    if sms is None:
        # (the emulated path on a CPU plans as for a B200)
        sms = _SM_COUNT[dev] = (torch.cuda.get_device_properties(dev).multi_processor_count
                                if torch.device(dev).type == "cuda" else 148)
    best, best_eff = 1, tiles / (-(-tiles // sms) * sms)
    for s in (2, 3, 4, 6, 8):
        if K % (s * 64) or K // s < 1024:
            continue
        t = tiles * s
        eff = t / (-(-t // sms) * sms)
        if eff > best_eff + 0.03:
            best, best_eff = s, eff
    return best


def _bf16(rows, cols, dev):
    # (large activation streams can live in compressible memory: utils/compressed_pool.py, off by default)
    if _CP.enabled() and torch.device(dev).type == "cuda":
        with _CP.allocate(rows * cols * 2):
            return torch.empty(rows, cols, device=dev, dtype=torch.bfloat16)
    return torch.empty(rows, cols, device=dev, dtype=torch.bfloat16)


# ------------------------------------------------------------------------------------------------
# one layer forward
# ------------------------------------------------------------------------------------------------
def _weighted_values(d: "_Dims", cur) -> torch.Tensor:
    """g^(C-s) v_s per head, bf16 [H*M, D] (row h*M + token): what token s of a segment still contributes to the
    state at the segment's end."""
    H, C, M, D = d.H, d.C, d.M, d.D
    t = torch.arange(C, device=cur.device, dtype=torch.float32)
    w = torch.exp(-d.slopes.view(H, 1) * (C - t).view(1, C))
    return (cur.view(1, d.Bs, C, D).float() * w.view(H, 1, C, 1)).to(torch.bfloat16).reshape(H * M, D)


def _segment_state(d: "_Dims", q, cur) -> torch.Tensor:
    """State each segment adds, sum_s g^(C-s) q_s^T v_s, fp32 [B*J, H, N', D] (one segment per sequence
    unless the attention is chunked)."""
    Bs, H, C, M, D, Np = d.Bs, d.H, d.C, d.M, d.D, d.Np
    rho = torch.empty(Bs, H, Np, D, device=q.device, dtype=torch.float32)
    if d.slopes is not None:
        vw, b_off = _weighted_values(d, cur), (0, 0, M, C)
    else:
        vw, b_off = cur, (0, 0, 0, C)
    G.gemm(q, vw, M=Np, N=D, K=C, a_mn=True, b_mn=True, nz=(H, Bs), a_off=(Np, 0, 0, C), b_off=b_off,
           c_off=(Np, H * Np, 0, 0), flags=G.F_OUT_F32, out0=rho.view(Bs * H * Np, D))
    return rho


def _scan_forward(d: "_Dims", seg: Optional[torch.Tensor], rho0: Optional[torch.Tensor], want_total: bool):
    """Hand the state on from segment to segment (and, under context parallelism, from rank to rank).
    seg: fp32 [B*J, H, N', D], what every segment adds (None when nothing needs it); rho0: the state before
    this call's first token. Returns (rin, total): rin bf16 [B*J*H*N', D], the state every segment starts
    from (None when all of them start from zero), and the fp32 state after the last token (None unless
    wanted). The recurrence over the segments is one elementwise kernel (`state_scan`)."""
    B, J, H, Np, D = d.B, d.J, d.H, d.Np, d.D
    gC = d.decay(d.C)
    gvec = gC.reshape(H).contiguous() if gC is not None else None
    start = rho0.float().contiguous() if rho0 is not None else None
    total = None
    if d.cp is not None:
        # this rank's segments alone (from zero), then the hand-off between the ranks
        scratch = torch.empty(B * J, H, Np, D, device=d.device, dtype=torch.bfloat16)
        local = torch.empty(B, H, Np, D, device=d.device, dtype=torch.float32)
        ops.state_scan(seg, None, gvec, scratch, local, J, H, False)
        del scratch
        gT = d.decay(d.T)
        start, total = d.cp.scan(local, start, gT if gT is not None else 1.0)
        if start is not None:
            start = start.float().contiguous()
    if seg is None or (J == 1 and start is None):
        if seg is not None and want_total and d.cp is None:
            total = seg.view(B, H, Np, D)             # one segment from an empty state: what it adds is the state
        return None, total
    rin = torch.empty(B * J, H, Np, D, device=d.device, dtype=torch.bfloat16)
    out_total = None
    if want_total and d.cp is None:
        out_total = total = torch.empty(B, H, Np, D, device=d.device, dtype=torch.float32)
    ops.state_scan(seg, start, gvec, rin, out_total, J, H, False)
    return rin.view(B * J * H * Np, D), total


def _scan_backward(d: "_Dims", d_rin: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """Reverse of `_scan_forward`: d_rin fp32 [B*J*H*N', D] (gradient of every segment's starting state, None
    when no segment had one) -> gradient of every segment's own state, bf16 [B*J*H*N', D] (None when it is
    exactly zero: a single segment that nobody continues from)."""
    B, J, H, Np, D = d.B, d.J, d.H, d.Np, d.D
    gC = d.decay(d.C)
    gvec = gC.reshape(H).contiguous() if gC is not None else None
    step = (lambda acc: acc) if gC is None else (lambda acc: acc * gC)
    acc = None
    if d.cp is not None:
        # what the later ranks' starting states pass back to this rank's total: they depend on this rank only
        # through its total state, and on it with the weights of the forward scan
        d_start = None
        if d_rin is not None:
            drv = d_rin.view(B, J, H, Np, D)
            for j in reversed(range(J)):
                d_start = drv[:, j] if d_start is None else drv[:, j] + step(d_start)
        if d_start is None:
            d_start = torch.zeros(B, H, Np, D, device=d.device, dtype=torch.float32)
        gT = d.decay(d.T)
        acc = d.cp.scan_backward(d_start.contiguous(), gT if gT is not None else 1.0).float().contiguous()
    if J == 1:
        return acc.to(torch.bfloat16).view(B * H * Np, D) if acc is not None else None
    dseg16 = torch.empty(B * J, H, Np, D, device=d.device, dtype=torch.bfloat16)
    ops.state_scan(d_rin.view(B * J, H, Np, D), acc, gvec, dseg16, None, J, H, True)
    return dseg16.view(B * J * H * Np, D)


def _layer_forward(d: _Dims, W, cur, pos0: int, rho_in: Optional[torch.Tensor], want_rho: bool,
                   drop_seed: int = 0):
    dev = cur.device
    M, D, H, N, Np, T, B = d.M, d.D, d.H, d.N, d.Np, d.T, d.B
    x = _bf16(M, d.HN, dev)
    if d.rot == "rope":
        q = _bf16(M, d.HN, dev)
        G.gemm(cur, W["encoder"], M=M, N=d.HN, K=D, epi=G.EPI_RELU, flags=G.F_ROPE | G.F_TABLE, in0=d.table(pos0),
               out0=x, out1=q, theta=d.theta, T=T, pos0=pos0, n_per_head=N, freqs=d.freqs)
    elif d.rot == "pope":
        q = _bf16(M, d.HNp, dev)
        G.gemm(cur, W["encoder"], M=M, N=N, K=D, nz=(H, 1), b_off=(N, 0, 0, 0), c_off=(0, 0, N, 0),
               o1_off=(Np, 0, N), epi=G.EPI_RELU, flags=G.F_POPE, out0=x, out1=q, theta=d.theta, T=T, pos0=pos0,
               n_per_head=N, freqs=d.freqs)
    else:
        q = x
        G.gemm(cur, W["encoder"], M=M, N=d.HN, K=D, epi=G.EPI_RELU, out0=x, theta=d.theta)

    # tiles above the diagonal are never written; the canonical path never reads them either (S V stops at the
    # diagonal tile, S^T dA starts at it); the row-normalised mode transposes whole matrices and wants zeros.
    # The attention runs per (head, segment): Bs = B*J segments of C tokens (J = 1, C = T unless chunked).
    C, Bs = d.C, d.Bs
    S = (torch.zeros if d.fast else torch.empty)(Bs * H * C, C, device=dev, dtype=torch.bfloat16)
    rnorm = None
    if d.fast:
        # forward_fast (src/model/attention.rs:142-175): S = tril(q q^T, -1) + m_h (s - t), rows L1-normalised
        if d.comm is not None or d.cp is not None or rho_in is not None:
            raise NotImplementedError("the row-normalised path has no state and is not sharded")
        G.gemm(q, q, M=T, N=T, K=Np, nz=(H, B), a_off=(0, T, Np, 0), b_off=(0, T, Np, 0), c_off=(T, H * T, 0, 0),
               epi=G.EPI_CAUSAL, flags=G.F_BIAS if d.slopes is not None else 0, slopes=d.slopes, causal_tiles=1, out0=S,
               tile_skip=d.tile_skip)
        if d.time_keep is not None:
            S.view(B * H, T, T).mul_(d.time_keep)                   # inactive block pairs leave the scores
        rnorm = torch.empty(B * H * T, device=dev, dtype=torch.float32)
        ops.rownorm_fwd(S, rnorm, T)
    else:
        G.gemm(q, q, M=C, N=C, K=Np, nz=(H, Bs), a_off=(0, C, Np, 0), b_off=(0, C, Np, 0), c_off=(C, H * C, 0, 0),
               epi=G.EPI_CAUSAL, slopes=d.slopes, causal_tiles=1, out0=S)
    comm = d.comm
    carry_flags = G.F_ROWDECAY if d.slopes is not None else 0
    # states: what every segment adds, handed on from segment to segment (and rank to rank)
    seg = _segment_state(d, q, cur) if (want_rho or d.handoff) else None
    rin, rho_out = _scan_forward(d, seg, rho_in, want_rho)
    del seg
    if comm is None:
        a = _bf16(H * M, D, dev)
        G.gemm(S, cur, M=C, N=D, K=C, b_mn=True, nz=(H, Bs), a_off=(C, H * C, 0, 0), b_off=(0, 0, 0, C),
               c_off=(M, C, 0, 0), causal_k=1, out0=a)
        if rin is not None:
            # carry-in: a_t += g^t (q_t . rho_in); the row decay g^t is applied in the epilogue
            G.gemm(q, rin, M=C, N=D, K=Np, b_mn=True, nz=(H, Bs), a_off=(0, C, Np, 0), b_off=(0, 0, Np, H * Np),
                   c_off=(M, C, 0, 0), flags=G.F_ACCUM | carry_flags, slopes=d.slopes, out0=a)
    else:
        # neuron-sharded: this rank's scores cover its slice of the neurons, so S V is a partial sum;
        # the GEMM's epilogue is the cross-rank reduction (parallel/tp.py: TPComm)
        buf = comm.begin("a", H * M, D, launches=1 if rin is None else 2)
        G.gemm(S, cur, M=T, N=D, K=T, b_mn=True, nz=(H, B), a_off=(T, H * T, 0, 0), b_off=(0, 0, 0, T),
               c_off=(M, T, 0, 0), causal_k=1, flags=comm.flags, out0=buf.view, **buf.kw)
        if rin is not None:
            G.gemm(q, rin, M=T, N=D, K=Np, b_mn=True, nz=(H, B), a_off=(0, T, Np, 0), b_off=(0, 0, Np, H * Np),
                   c_off=(M, T, 0, 0), flags=comm.flags | carry_flags, slopes=d.slopes, out0=buf.view, **buf.kw)
        a = comm.end(buf, bf16=True)
    lna = torch.empty_like(a)
    ops.layernorm_fwd(a, lna)
    # y is not stored: the backward recovers it as xy / x
    xy = _bf16(M, d.HN, dev)
    if d.dual_fwd:
        # y = relu(LN(a) E_v) -> x*y -> . Dec in one kernel: x*y is written once (for the backward pass) and
        # contracted straight from shared memory
        mlp = _bf16(M, D, dev)
        DG.dual(lna, W["encoder_v"], W["decoder"], xy, mlp, M=M, H=H, n_per_head=N, K1=D, N2=D, T=T,
                epi=G.EPI_RELU_GATE, a1_b=T, a1_h=M, in0=x, theta=d.theta, drop_p=d.drop_p, drop_seed=drop_seed)
    else:
        G.gemm(lna, W["encoder_v"], M=M, N=N, K=D, nz=(H, 1), a_off=(M, 0, 0, 0), b_off=(N, 0, 0, 0),
               c_off=(0, 0, N, 0), epi=G.EPI_RELU_GATE, flags=G.F_NO_OUT0, in0=x, out1=xy, theta=d.theta,
               drop_p=d.drop_p, drop_seed=drop_seed)
    if d.dual_fwd:
        pass
    elif comm is None:
        sk = _split_k(-(-M // 128) * -(-D // 256), d.HN, dev)
        if sk > 1:
            mlp32 = torch.zeros(M, D, device=dev, dtype=torch.float32)
            ks = d.HN // sk
            G.gemm(xy, W["decoder"], M=M, N=D, K=ks, b_mn=True, nz=(sk, 1), a_off=(0, 0, ks, 0), b_off=(0, 0, ks, 0),
                   flags=G.F_OUT_F32 | G.F_ATOMIC, out0=mlp32)
            mlp = mlp32.to(torch.bfloat16)
        else:
            mlp = _bf16(M, D, dev)
            G.gemm(xy, W["decoder"], M=M, N=D, K=d.HN, b_mn=True, out0=mlp)
    else:
        buf = comm.begin("mlp", M, D)
        G.gemm(xy, W["decoder"], M=M, N=D, K=d.HN, b_mn=True, flags=comm.flags, out0=buf.view, **buf.kw)
        mlp = comm.end(buf, bf16=True)
    out = torch.empty_like(cur)
    ops.block_out_fwd(cur, mlp, out)
    saved = dict(cur=cur, x=x, q=q, S=S, a=a, lna=lna, xy=xy, mlp=mlp, drop_seed=drop_seed, rnorm=rnorm, rin=rin)
    return out, saved, rho_out


def _wgrad_target(d: _Dims, grads, name: str, flags: int, final: bool):
    """-> (out0, flags, extra keyword arguments) of the weight-gradient GEMM of `name`."""
    if d.sink is not None:
        return d.sink.launch(name, flags, final, grads[name] if grads is not None else None)
    return grads[name], flags, {}


def _layer_backward(d: _Dims, W, sv, dout, grads, pos0: int, final: bool = False):
    """dout: fp32 [M, D] gradient of the layer output. Returns fp32 [M, D] gradient of the layer input.
    Weight gradients are accumulated into grads['encoder'|'encoder_v'|'decoder'] (fp32)."""
    dev = dout.device
    M, D, H, N, Np, T, B = d.M, d.D, d.H, d.N, d.Np, d.T, d.B
    C, Bs = d.C, d.Bs
    cur, x, q, S, a, lna, xy, mlp = (sv[k] for k in ("cur", "x", "q", "S", "a", "lna", "xy", "mlp"))
    if q is None:
        # this layer did not keep its PoPE query: write it again from x
        q = _bf16(M, d.HNp, dev)
        ops.pope_rotate(x, d.freqs_full, q, H, T, pos0)
    dcur = torch.empty(M, D, device=dev, dtype=torch.float32)
    dmlp = _bf16(M, D, dev)
    ops.block_out_bwd(cur, mlp, dout, dcur, dmlp)
    # gate
    dy = _bf16(M, d.HN, dev)
    dxg = _bf16(M, d.HN, dev)
    # with dropout the stored x*y is already masked and scaled, so only the 1/(1-p) on dy is explicit
    dlna = None
    if d.dual_gate:
        # gate backward and d LN(a) = dy . E_v in one kernel (dy is written once, for the weight gradient)
        dlna = _bf16(H * M, D, dev)
        DG.dual(dmlp, W["decoder"], W["encoder_v"], dy, dlna, M=M, H=H, n_per_head=N, K1=D, N2=D, T=T,
                epi=G.EPI_GATE_BWD, group_per_head=True, a1_b=T, a1_h=0, in0=x, in1=xy, out1=dxg,
                alpha=1.0 / (1.0 - d.drop_p), out_h_stride=M)
    else:
        G.gemm(dmlp, W["decoder"], M=M, N=d.HN, K=D, epi=G.EPI_GATE_BWD, in0=x, in1=xy, out0=dy, out1=dxg,
               alpha=1.0 / (1.0 - d.drop_p))
    wtiles = -(-d.HN // 128) * -(-D // 256)
    sk = _split_k(wtiles, M, dev)
    wflags = G.F_OUT_F32 | (G.F_ATOMIC if sk > 1 else G.F_ACCUM)
    km = M // sk
    o, fl, kw = _wgrad_target(d, grads, "decoder", wflags, final)
    G.gemm(xy, dmlp, M=d.HN, N=D, K=km, a_mn=True, b_mn=True, nz=(1, sk), a_off=(0, 0, 0, km), b_off=(0, 0, 0, km),
           flags=fl, out0=o, **kw)
    # y = relu(LN(a) E_v)
    o, fl, kw = _wgrad_target(d, grads, "encoder_v", wflags, final)
    G.gemm(dy, lna, M=N, N=D, K=km, a_mn=True, b_mn=True, nz=(H, sk), a_off=(N, 0, 0, km), b_off=(0, 0, M, km),
           c_off=(N, 0, 0, 0), flags=fl, out0=o, **kw)
    comm = d.comm
    if dlna is not None:
        pass
    elif comm is None:
        dlna = _bf16(H * M, D, dev)
        G.gemm(dy, W["encoder_v"], M=M, N=D, K=N, b_mn=True, nz=(H, 1), a_off=(0, 0, N, 0), b_off=(0, 0, N, 0),
               c_off=(M, 0, 0, 0), out0=dlna)
    else:
        buf = comm.begin("dlna", H * M, D)
        G.gemm(dy, W["encoder_v"], M=M, N=D, K=N, b_mn=True, nz=(H, 1), a_off=(0, 0, N, 0), b_off=(0, 0, N, 0),
               c_off=(M, 0, 0, 0), flags=comm.flags, out0=buf.view, **buf.kw)
        dlna = comm.end(buf, bf16=True)
    del dy
    da = _bf16(H * M, D, dev)
    ops.layernorm_bwd(a, dlna, da, False)
    if d.fast:
        # through the row normalisation: dS = (tril(dA V^T) - sign(Sn) sum(tril(dA V^T) Sn)) / r, then
        # q is both query and key: Gs = dS + dS^T
        Gl = torch.zeros(B * H * T, T, device=dev, dtype=torch.bfloat16)
        G.gemm(da, cur, M=T, N=T, K=D, nz=(H, B), a_off=(M, T, 0, 0), b_off=(0, T, 0, 0), c_off=(T, H * T, 0, 0),
               epi=G.EPI_CAUSAL, causal_tiles=1, out0=Gl, tile_skip=d.tile_skip)
        ops.rownorm_bwd(Gl, S, sv["rnorm"], T)
        Gl3 = Gl.view(B * H, T, T)
        if d.time_keep is not None:
            Gl3.mul_(d.time_keep)                                   # ... and get no gradient
        Gs = (Gl3 + Gl3.transpose(1, 2)).reshape(B * H * T, T)
        del Gl, Gl3
    else:
        # attention: Gs = causal(dA V^T) + causal(dA V^T)^T with the decay mask, per (head, segment)
        Gs = _bf16(Bs * H * C, C, dev)
        G.gemm(da, cur, M=C, N=C, K=D, nz=(H, Bs), a_off=(M, C, 0, 0), b_off=(0, C, 0, 0), c_off=(C, H * C, 0, 0),
               epi=G.EPI_CAUSAL, slopes=d.slopes, causal_tiles=1, out0=Gs)
        G.gemm(cur, da, M=C, N=C, K=D, nz=(H, Bs), a_off=(0, C, 0, 0), b_off=(M, C, 0, 0), c_off=(C, H * C, 0, 0),
               epi=G.EPI_CAUSAL, flags=G.F_UPPER, slopes=d.slopes, causal_tiles=2, out0=Gs)
    # dV (v = cur for every head): dcur[b] += sum_h S_h^T dA_h
    if comm is None:
        part, pflags, pkw = dcur, G.F_OUT_F32 | G.F_ACCUM, {}
    else:
        pbuf = comm.begin("dcur", M, D, launches=2)        # partial sums over the neuron shards: dV and the encoder path
        part, pflags, pkw = pbuf.view, comm.flags, pbuf.kw
    # all heads in one launch: every (head, segment) problem adds its [C, D] tile into the rows of its segment
    # (row block s only needs t >= s: the contraction starts at the tile's first row; in the row-normalised
    # mode S holds zeros above the diagonal, elsewhere that part is never written and must not be read)
    G.gemm(S, da, M=C, N=D, K=C, a_mn=True, b_mn=True, nz=(H, Bs), a_off=(0, 0, C, H * C), b_off=(0, 0, M, C),
           c_off=(0, C, 0, 0), flags=(pflags & ~G.F_ACCUM) | (G.F_ATOMIC if pflags & G.F_ACCUM else 0), out0=part,
           causal_k=2, **pkw)
    # states across segment borders: a_t also holds g^t q_t . rin (rin = the state its segment starts from), and
    # every segment's own state sum_s g^(C-s) q_s^T v_s feeds the later segments
    x2 = r2 = None            # extra contraction for dq: [g^t dA | g^(C-s) v] . [rin | d seg]^T over 2 D columns
    if d.handoff:
        rin = sv.get("rin")
        if d.slopes is not None:
            t = torch.arange(C, device=dev, dtype=torch.float32)
            w_in = torch.exp(-d.slopes.view(H, 1) * t.view(1, C))
            da_w = (da.view(H, Bs, C, D).float() * w_in.view(H, 1, C, 1)).to(torch.bfloat16).view(H * M, D)
        else:
            da_w = da
        d_rin = None
        if rin is not None:
            # gradient of the starting states: sum_t g^t q_t^T dA_t
            d_rin = torch.empty(Bs * H * Np, D, device=dev, dtype=torch.float32)
            G.gemm(q, da_w, M=Np, N=D, K=C, a_mn=True, b_mn=True, nz=(H, Bs), a_off=(Np, 0, 0, C), b_off=(0, 0, M, C),
                   c_off=(Np, H * Np, 0, 0), flags=G.F_OUT_F32, out0=d_rin)
        dseg = _scan_backward(d, d_rin)
        del d_rin
        xs, rs = [], []
        if rin is not None:
            xs.append(da_w); rs.append(rin)
        if dseg is not None:
            dseg16 = dseg                        # (bf16 [Bs*H*N', D])
            del dseg
            # through the segment state to its values: dv_s += g^(C-s) sum_h q_s . d seg_h
            G.gemm(q, dseg16, M=C, N=D, K=Np, b_mn=True, nz=(H, Bs), a_off=(0, C, Np, 0), b_off=(0, 0, Np, H * Np),
                   c_off=(0, C, 0, 0), flags=G.F_OUT_F32 | G.F_ATOMIC | (G.F_ROWDECAY_REV if d.slopes is not None else 0),
                   slopes=d.slopes, T=C, out0=dcur)
            xs.append(_weighted_values(d, cur) if d.slopes is not None
                      else cur.view(1, M, D).expand(H, M, D).reshape(H * M, D))
            rs.append(dseg16)
        if xs:
            x2 = xs[0] if len(xs) == 1 else torch.cat(xs, 1)
            r2 = rs[0] if len(rs) == 1 else torch.cat(rs, 1)
        del xs, rs, da_w
    # dq = Gs q (+ the state terms), then back through rotation, + gate gradient, ReLU mask
    dx = _bf16(M, d.HN, dev)
    if d.dual_dq:
        # dq = Gs q, rotation undone, + gate gradient, ReLU mask, and d cur += dx . E in one kernel
        rope = d.rot == "rope"
        DG.dual(Gs, q, W["encoder"], dx, dcur, M=M, H=H, n_per_head=N, K1=T, N2=D, T=T, epi=G.EPI_DQ_BWD,
                flags=(G.F_ROPE | G.F_TABLE) if rope else 0, a1_b=H * T, a1_h=T, b1_mn=True, b1_b=T, in0=dxg,
                in1=d.table(pos0) if rope else None, pos0=pos0, accumulate=True)
    elif d.rot == "pope":
        dq = _bf16(M, d.HNp, dev)
        G.gemm(Gs, q, M=C, N=Np, K=C, b_mn=True, nz=(H, Bs), a_off=(C, H * C, 0, 0), b_off=(Np, 0, 0, C),
               c_off=(0, C, Np, 0), out0=dq)
        if x2 is not None:
            G.gemm(x2, r2, M=C, N=Np, K=x2.shape[1], nz=(H, Bs), a_off=(M, C, 0, 0), b_off=(Np, H * Np, 0, 0),
                   c_off=(0, C, Np, 0), flags=G.F_ACCUM, out0=dq)
        ops.pope_bwd(dq, x, dxg, d.freqs_full, dx, H, T, pos0)
    else:
        rope = d.rot == "rope"
        rflags = (G.F_ROPE | G.F_TABLE) if rope else 0
        table = d.table(pos0) if rope else None
        if x2 is not None:
            # two contractions meet in one epilogue: the first launch leaves its rotated-back sum in the gate
            # gradient's place (closed gates keep their marker), the second adds Gs q to it
            dxg2 = _bf16(M, d.HN, dev)
            G.gemm(x2, r2, M=C, N=N, K=x2.shape[1], nz=(H, Bs), a_off=(M, C, 0, 0), b_off=(Np, H * Np, 0, 0),
                   c_off=(0, C, N, 0), epi=G.EPI_DQ_BWD, flags=rflags | G.F_KEEP_MARK, in0=dxg, in1=table, out0=dxg2,
                   T=T, pos0=pos0, n_per_head=N, freqs=d.freqs)
            dxg = dxg2
            del dxg2
        G.gemm(Gs, q, M=C, N=N, K=C, b_mn=True, nz=(H, Bs), a_off=(C, H * C, 0, 0), b_off=(N, 0, 0, C),
               c_off=(0, C, N, 0), epi=G.EPI_DQ_BWD, flags=rflags, in0=dxg, in1=table, out0=dx, T=T, pos0=pos0,
               n_per_head=N, freqs=d.freqs)
    del x2, r2
    del dxg
    o, fl, kw = _wgrad_target(d, grads, "encoder", wflags, final)
    G.gemm(dx, cur, M=d.HN, N=D, K=km, a_mn=True, b_mn=True, nz=(1, sk), a_off=(0, 0, 0, km), b_off=(0, 0, 0, km),
           flags=fl, out0=o, **kw)
    if d.dual_dq:
        pass
    elif comm is None:
        sk2 = _split_k(-(-M // 128) * -(-D // 256), d.HN, dev)
        k2 = d.HN // sk2
        G.gemm(dx, W["encoder"], M=M, N=D, K=k2, b_mn=True, nz=(sk2, 1), a_off=(0, 0, k2, 0), b_off=(0, 0, k2, 0),
               flags=G.F_OUT_F32 | (G.F_ATOMIC if sk2 > 1 else G.F_ACCUM), out0=part)
    else:
        G.gemm(dx, W["encoder"], M=M, N=D, K=d.HN, b_mn=True, flags=pflags, out0=part, **pkw)
    if comm is not None:
        dcur += comm.end(pbuf)
    return dcur


# ------------------------------------------------------------------------------------------------
# whole model
# ------------------------------------------------------------------------------------------------
def _embed(d, W, tokens):
    cur = _bf16(d.M, d.D, tokens.device)
    ops.embed_ln_fwd(tokens.reshape(-1).contiguous(), W["embed"], cur)
    return cur


def _head_logits(d, W, cur):
    dev = cur.device
    if d.V % 8 == 0:
        logits = torch.empty(d.M, d.V, device=dev, dtype=torch.float32)
        G.gemm(cur, W["lm_head"], M=d.M, N=d.V, K=d.D, b_mn=True, flags=G.F_OUT_F32, out0=logits)
        return logits
    return cur.float() @ W["lm_head"].float()


def layer_activation_bytes(d: _Dims) -> int:
    """Bytes one layer keeps for its backward pass when it is not recomputed."""
    wide = d.M * (2 * d.HN + (d.HNp if d.rot != "alibi" else 0)) * 2          # x, x*y, rotated copy
    scores = d.Bs * d.H * d.C * d.C * 2
    narrow = (2 * d.H * d.M * d.D + 3 * d.M * d.D) * 2                        # a, LN(a); cur, mlp, out
    states = (d.Bs * d.H * d.Np * d.D * 2) if d.handoff else 0                # bf16 starting state of every segment
    return wide + scores + narrow + states


def backward_working_bytes(d: _Dims) -> int:
    """Peak of the temporaries one layer's backward pass holds at once: dq (PoPE: over the doubled latent) or dy,
    the gate gradient and its second copy, dx, and the score-sized Gs - plus the fp32 state gradients when states
    cross segment borders."""
    wide = d.M * (max(d.HN, d.HNp) + 3 * d.HN) * 2
    scores = 2 * d.Bs * d.H * d.C * d.C * 2
    # fp32 gradient of the starting states and of the segments' own states, the bf16 copy, the [rin | d seg] operand
    states = (d.Bs * d.H * d.Np * d.D * (4 + 4 + 2 + 4)) if d.handoff else 0
    return wide + scores + states


def recompute_count(model, d: _Dims) -> int:
    """How many of the L layers re-run their forward in the backward pass. `model.recompute`:
    False / True (none / all), an int (that many, counted from the first layer), or "auto": as few as
    fit in 75 % of the free device memory, after setting aside the backward pass's own working set
    (`backward_working_bytes`; the layers that are kept are the last ones, which the backward pass frees
    before it reaches the recomputed ones, so a recomputed layer's activations never add to the peak).
    Measured on the large PoPE configuration (8 sequences of 2048 tokens per GPU): 16.8 GB per kept layer on
    top of 21 GB, against 17.7 and 22.5 GB from these formulas."""
    r = getattr(model, "recompute", False)
    if r is True:
        return d.L
    if r is False or r is None:
        return 0
    if isinstance(r, int):
        return max(0, min(d.L, r))
    if r == "auto":
        if not torch.cuda.is_available():
            return 0                      # (emulated path on a CPU: no device memory to size against)
        free, _ = torch.cuda.mem_get_info()
        free += torch.cuda.memory_reserved() - torch.cuda.memory_allocated()   # cached blocks are reusable
        per = layer_activation_bytes(d)
        keep = int((0.75 * free - backward_working_bytes(d)) // per)
        count = max(0, min(d.L, d.L - keep))
        # a recomputed layer repeats its forward collectives: ranks that shard one model (tensor or context
        # parallel) must agree on the count, whatever their own free memory says
        shared = d.comm if d.comm is not None else d.cp
        if shared is not None and getattr(shared, "world", 1) > 1:
            # (agreed once per shape: the answer is kept on the model)
            cache = model.__dict__.setdefault("_agreed_recompute", {})
            key = (d.B, d.T, d.fast)
            if key not in cache:
                import torch.distributed as dist
                t = torch.tensor([count], device=d.device, dtype=torch.int32)
                dist.all_reduce(t, op=dist.ReduceOp.MAX, group=getattr(shared, "group", None))
                cache[key] = int(t.item())
            count = cache[key]
        return count
    raise ValueError(f"recompute must be a bool, an int or 'auto', not {r!r}")


# a layer's forward pass costs about this many rebuilds of its PoPE query (17.7 ms against 3.3 ms on the large config)
_RECOMPUTE_COST = 5.4


def memory_plan(model, d: _Dims):
    """-> (recomputed layers, layers that drop their rotated query). PoPE stores q = softplus(x) (cos, sin) at twice
    the width of x; a layer that drops it keeps x only and writes q again in its backward pass (one elementwise
    kernel, `pope_rotate`), which is much cheaper than recomputing the layer. With `recompute = "auto"` the plan is
    the cheapest mix of recomputed layers (the first ones), q-dropping layers (the next ones) and fully kept layers
    that fits the memory budget of `recompute_count`; `model.drop_rotated` (an int) overrides the second number."""
    r = recompute_count(model, d)
    k = getattr(model, "drop_rotated", None)
    can_drop = d.rot == "pope" and d.comm is None
    if k is not None:
        return r, (max(0, min(d.L - r, int(k))) if can_drop else 0)
    if getattr(model, "recompute", False) != "auto" or not can_drop or r == 0 or not torch.cuda.is_available():
        return r, 0
    free, _ = torch.cuda.mem_get_info()
    free += torch.cuda.memory_reserved() - torch.cuda.memory_allocated()
    budget = 0.75 * free - backward_working_bytes(d)
    per = layer_activation_bytes(d)
    qbytes = d.M * d.HNp * 2
    best = (r * _RECOMPUTE_COST, r, 0)
    for rr in range(0, r + 1):
        for kk in range(0, d.L - rr + 1):
            mem = kk * (per - qbytes) + (d.L - rr - kk) * per + (qbytes if kk else 0)
            if mem <= budget:
                cost = rr * _RECOMPUTE_COST + kk
                if cost < best[0]:
                    best = (cost, rr, kk)
                break                     # more q-dropping layers only cost more
    return best[1], best[2]


def _stack_forward(model, d: _Dims, W, tokens, state, save: bool, recompute: int, drop_q: int = 0):
    """`recompute` = number of leading layers that keep only their input (and dropout seed); the `drop_q`
    layers after them keep everything but the rotated query."""
    cur = _embed(d, W, tokens)
    # (training of a segment of longer sequences - context parallelism - starts at `model._train_pos0`)
    pos0 = state.position if state is not None else int(getattr(model, "_train_pos0", 0))
    saved: List[dict] = []
    for l in range(d.L):
        rho_in = state.layers[l].rho if state is not None else None
        if rho_in is not None and d.idx is not None:
            rho_in = rho_in.index_select(2, d.idx)           # the state rows of the active neurons
        seed_l = (d.drop_base + 0x632BE5AB * (l + 1)) & 0x7FFFFFFF
        with prof.phase("layer.forward"):
            out, sv, rho_out = _layer_forward(d, W, cur, pos0, rho_in, want_rho=state is not None, drop_seed=seed_l)
        if state is not None:
            if d.idx is not None and rho_out is not None:
                # inactive neurons have zero queries: their state rows stay zero
                full = torch.zeros(d.B, d.H, d.N_full, d.D, device=rho_out.device, dtype=rho_out.dtype)
                full[:, :, d.idx] = rho_out
                rho_out = full
            state.layers[l].rho = rho_out
        if save:
            if l < recompute:
                saved.append(dict(cur=cur, drop_seed=seed_l))
            else:
                if l < recompute + drop_q:
                    sv["q"] = None
                saved.append(sv)
        if l == d.L - 1 and getattr(model, "measure_sparsity", False):
            # fraction of active neurons in the last layer, left on the device for the metrics logger
            model.last_sparsity = dict(x=(sv["x"] != 0).float().mean(), xy=(sv["xy"] != 0).float().mean())
        cur = out
    if state is not None:
        state.position += d.T
    return cur, saved


@torch.no_grad()
def forward_logits(model, tokens: torch.Tensor, state, fast: bool = False) -> torch.Tensor:
    B, T = tokens.shape
    d = _Dims(model, B, T, fast)
    W = _compact(d, _weights(model))
    cur, _ = _stack_forward(model, d, W, tokens, state, save=False, recompute=0)
    return _head_logits(d, W, cur).view(B, T, d.V)


class _FusedLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tokens, targets, embed_w, encoder, encoder_v, decoder, lm_head, model, fast=False):
        B, T = tokens.shape
        d = _Dims(model, B, T, fast)
        W = _compact(d, _weights(model))
        recompute, drop_q = memory_plan(model, d)
        model._recomputed_layers, model._dropped_q_layers = recompute, drop_q
        cur, saved = _stack_forward(model, d, W, tokens, None, save=True, recompute=recompute, drop_q=drop_q)
        with prof.phase("head.loss"):
            logits = _head_logits(d, W, cur)
            row_loss = torch.empty(d.M, device=tokens.device, dtype=torch.float32)
            dlogits = _bf16(d.M, d.V, tokens.device)
            ops.cross_entropy(logits, targets.reshape(-1).contiguous(), row_loss, dlogits, 1.0 / d.M)
        ctx.d, ctx.W, ctx.saved, ctx.final, ctx.dlogits = d, W, saved, cur, dlogits
        ctx.tokens = tokens
        ctx.recompute = recompute
        ctx.pos0 = int(getattr(model, "_train_pos0", 0))
        return row_loss.sum() / d.M

    @staticmethod
    def backward(ctx, grad_out):
        d, W, saved, cur, dlogits = ctx.d, ctx.W, ctx.saved, ctx.final, ctx.dlogits
        dev = cur.device
        # local fp32 accumulation over the shared-weight layers; a sink that takes every launch needs none
        keep_local = d.sink is None or getattr(d.sink, "last_layer_only", False)
        grads = {k: torch.zeros(d.HN, d.D, device=dev, dtype=torch.float32)
                 for k in ("encoder", "encoder_v", "decoder")} if keep_local else None
        # head
        if d.V % 8 == 0:
            g_head = torch.empty(d.D, d.V, device=dev, dtype=torch.float32)
            G.gemm(cur, dlogits, M=d.D, N=d.V, K=d.M, a_mn=True, b_mn=True, flags=G.F_OUT_F32, out0=g_head)
            dcur = torch.empty(d.M, d.D, device=dev, dtype=torch.float32)
            G.gemm(dlogits, W["lm_head"], M=d.M, N=d.D, K=d.V, flags=G.F_OUT_F32, out0=dcur)
        else:
            g_head = cur.float().t() @ dlogits.float()
            dcur = dlogits.float() @ W["lm_head"].float().t()
        for l in reversed(range(d.L)):
            sv = saved[l]
            if "x" not in sv:
                with prof.phase("layer.recompute"):
                    _, sv, _ = _layer_forward(d, W, sv["cur"], ctx.pos0, None, False, sv["drop_seed"])
            with prof.phase("layer.backward"):
                dcur = _layer_backward(d, W, sv, dcur, grads, ctx.pos0, final=(l == 0))
            saved[l] = None
        g_emb = torch.zeros(d.V, d.D, device=dev, dtype=torch.float32)
        ops.embed_ln_bwd(ctx.tokens.reshape(-1).contiguous(), W["embed"], dcur, g_emb)
        s = grad_out.to(torch.float32)
        if grads is None or d.sink is not None:
            # (the sharded weights' gradients are already in their owners' slices; the loss enters with weight 1)
            return (None, None, g_emb * s, None, None, None, g_head * s, None, None)
        if d.rows is not None:
            # latent block pattern: the rows of inactive neurons get no gradient
            for k in grads:
                full = torch.zeros(d.H * d.N_full, d.D, device=dev, dtype=torch.float32)
                full[d.rows] = grads[k]
                grads[k] = full
        return (None, None, g_emb * s, grads["encoder"] * s, grads["encoder_v"] * s, grads["decoder"] * s,
                g_head * s, None, None)


def loss(model, tokens: torch.Tensor, targets: torch.Tensor, fast: bool = False) -> torch.Tensor:
    """Mean cross-entropy of the canonical forward (or, with `fast`, of the row-normalised
    `forward_fast` function), differentiable w.r.t. the model parameters."""
    return _FusedLoss.apply(tokens, targets, model.embed.weight, model.encoder, model.encoder_v, model.decoder,
                            model.lm_head, model, fast)


from . import emulate  # noqa: E402  (last: with BDH_EMULATE_KERNELS=1 it re-points `ops` and `G.gemm` defined above)

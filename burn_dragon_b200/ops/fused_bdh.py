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
        if self.fast and c.block_sparse is not None and c.block_sparse.time.is_sparse():
            tp = c.block_sparse.time
            nb = -(-T // tp.block_size)
            keep = torch.zeros(nb, nb, dtype=torch.bool)
            for (r, cc) in tp.pairs(nb):
                keep[r, cc] = True
            keep = keep.repeat_interleave(tp.block_size, 0).repeat_interleave(tp.block_size, 1)[:T, :T]
            self.time_keep = keep.to(device=model.encoder.device, dtype=torch.bfloat16)
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
        # contracts them) cover unsharded layers with D <= 256; PoPE keeps the separate launches (its rotated
        # copy has twice the width)
        ok = (self.comm is None and self.rot != "pope" and DG.eligible(self.M, self.T, self.N, self.D))
        which = getattr(model, "use_dual_gemm", None)
        if which is None:
            which = os.environ.get("BDH_DUAL", "fwd")
        which = set(str(which).split(",")) if which else set()
        self.dual_fwd = ok and bool(which & {"fwd", "all", "True"})
        self.dual_gate = ok and bool(which & {"gate", "all", "True"})
        self.dual_dq = ok and bool(which & {"dq", "all", "True"})


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
    return torch.empty(rows, cols, device=dev, dtype=torch.bfloat16)


# ------------------------------------------------------------------------------------------------
# one layer forward
# ------------------------------------------------------------------------------------------------
def _segment_state(d: "_Dims", q, cur) -> torch.Tensor:
    """State this segment adds, sum_s g^(T-s) q_s^T v_s, fp32 [B, H, N', D]."""
    B, H, T, M, D, Np = d.B, d.H, d.T, d.M, d.D, d.Np
    dev = q.device
    rho = torch.empty(B, H, Np, D, device=dev, dtype=torch.float32)
    if d.slopes is not None:
        t = torch.arange(T, device=dev, dtype=torch.float32)
        w = torch.exp(-d.slopes.view(H, 1) * (T - t).view(1, T))                     # g^(T-s)
        vw = (cur.view(1, B, T, D).float() * w.view(H, 1, T, 1)).to(torch.bfloat16).reshape(H * M, D)
        b_off = (0, 0, M, T)
    else:
        vw, b_off = cur, (0, 0, 0, T)
    G.gemm(q, vw, M=Np, N=D, K=T, a_mn=True, b_mn=True, nz=(H, B), a_off=(Np, 0, 0, T), b_off=b_off,
           c_off=(Np, H * Np, 0, 0), flags=G.F_OUT_F32, out0=rho.view(B * H * Np, D))
    return rho


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
    # diagonal tile, S^T dA starts at it); the row-normalised mode transposes whole matrices and wants zeros
    S = (torch.zeros if d.fast else torch.empty)(B * H * T, T, device=dev, dtype=torch.bfloat16)
    rnorm = None
    if d.fast:
        # forward_fast (src/model/attention.rs:142-175): S = tril(q q^T, -1) + m_h (s - t), rows L1-normalised
        if d.comm is not None or d.cp is not None or rho_in is not None:
            raise NotImplementedError("the row-normalised path has no state and is not sharded")
        G.gemm(q, q, M=T, N=T, K=Np, nz=(H, B), a_off=(0, T, Np, 0), b_off=(0, T, Np, 0), c_off=(T, H * T, 0, 0),
               epi=G.EPI_CAUSAL, flags=G.F_BIAS if d.slopes is not None else 0, slopes=d.slopes, causal_tiles=1, out0=S)
        if d.time_keep is not None:
            S.view(B * H, T, T).mul_(d.time_keep)                   # inactive block pairs leave the scores
        rnorm = torch.empty(B * H * T, device=dev, dtype=torch.float32)
        ops.rownorm_fwd(S, rnorm, T)
    else:
        G.gemm(q, q, M=T, N=T, K=Np, nz=(H, B), a_off=(0, T, Np, 0), b_off=(0, T, Np, 0), c_off=(T, H * T, 0, 0),
               epi=G.EPI_CAUSAL, slopes=d.slopes, causal_tiles=1, out0=S)
    comm = d.comm
    carry_flags = G.F_ROWDECAY if d.slopes is not None else 0
    cp = d.cp
    rho_total = None
    if cp is not None:
        # context parallel: exchange the segment states, continue from what the earlier ranks left
        g_T = torch.exp(-d.slopes * T).view(1, H, 1, 1) if d.slopes is not None else 1.0
        rho_in, rho_total = cp.scan(_segment_state(d, q, cur), rho_in, g_T)
    if comm is None:
        a = _bf16(H * M, D, dev)
        G.gemm(S, cur, M=T, N=D, K=T, b_mn=True, nz=(H, B), a_off=(T, H * T, 0, 0), b_off=(0, 0, 0, T),
               c_off=(M, T, 0, 0), causal_k=1, out0=a)
        if rho_in is not None:
            # carry-in: a_t += g^t (q_t . rho_in); the row decay g^t is applied in the epilogue
            rin = rho_in.reshape(B * H * Np, D).to(torch.bfloat16)
            G.gemm(q, rin, M=T, N=D, K=Np, b_mn=True, nz=(H, B), a_off=(0, T, Np, 0), b_off=(0, 0, Np, H * Np),
                   c_off=(M, T, 0, 0), flags=G.F_ACCUM | carry_flags, slopes=d.slopes, out0=a)
    else:
        # neuron-sharded: this rank's scores cover its slice of the neurons, so S V is a partial sum;
        # the GEMM's epilogue is the cross-rank reduction (parallel/tp.py: TPComm)
        buf = comm.begin("a", H * M, D, launches=1 if rho_in is None else 2)
        G.gemm(S, cur, M=T, N=D, K=T, b_mn=True, nz=(H, B), a_off=(T, H * T, 0, 0), b_off=(0, 0, 0, T),
               c_off=(M, T, 0, 0), causal_k=1, flags=comm.flags, out0=buf.view, **buf.kw)
        if rho_in is not None:
            rin = rho_in.reshape(B * H * Np, D).to(torch.bfloat16)
            G.gemm(q, rin, M=T, N=D, K=Np, b_mn=True, nz=(H, B), a_off=(0, T, Np, 0), b_off=(0, 0, Np, H * Np),
                   c_off=(M, T, 0, 0), flags=comm.flags | carry_flags, slopes=d.slopes, out0=buf.view, **buf.kw)
        a = comm.end(buf, bf16=True)
    rho_out = None
    if cp is not None:
        rho_out = rho_total
    elif want_rho:
        rho_out = _segment_state(d, q, cur)
        if rho_in is not None:
            # the carried state has decayed by g^T over this segment
            rho_out += rho_in if d.slopes is None else rho_in * torch.exp(-d.slopes * T).view(1, H, 1, 1)
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
    saved = dict(cur=cur, x=x, q=q, S=S, a=a, lna=lna, xy=xy, mlp=mlp, drop_seed=drop_seed, rnorm=rnorm)
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
    cur, x, q, S, a, lna, xy, mlp = (sv[k] for k in ("cur", "x", "q", "S", "a", "lna", "xy", "mlp"))
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
               epi=G.EPI_CAUSAL, causal_tiles=1, out0=Gl)
        ops.rownorm_bwd(Gl, S, sv["rnorm"], T)
        Gl3 = Gl.view(B * H, T, T)
        if d.time_keep is not None:
            Gl3.mul_(d.time_keep)                                   # ... and get no gradient
        Gs = (Gl3 + Gl3.transpose(1, 2)).reshape(B * H * T, T)
        del Gl, Gl3
    else:
        # attention: Gs = causal(dA V^T) + causal(dA V^T)^T with the decay mask
        Gs = _bf16(B * H * T, T, dev)
        G.gemm(da, cur, M=T, N=T, K=D, nz=(H, B), a_off=(M, T, 0, 0), b_off=(0, T, 0, 0), c_off=(T, H * T, 0, 0),
               epi=G.EPI_CAUSAL, slopes=d.slopes, causal_tiles=1, out0=Gs)
        G.gemm(cur, da, M=T, N=T, K=D, nz=(H, B), a_off=(0, T, 0, 0), b_off=(M, T, 0, 0), c_off=(T, H * T, 0, 0),
               epi=G.EPI_CAUSAL, flags=G.F_UPPER, slopes=d.slopes, causal_tiles=2, out0=Gs)
    # dV (v = cur for every head): dcur[b] += sum_h S_h^T dA_h
    if comm is None:
        part, pflags, pkw = dcur, G.F_OUT_F32 | G.F_ACCUM, {}
    else:
        pbuf = comm.begin("dcur", M, D, launches=2)        # partial sums over the neuron shards: dV and the encoder path
        part, pflags, pkw = pbuf.view, comm.flags, pbuf.kw
    # all heads in one launch: every (head, batch) problem adds its [T, D] tile into the rows of its batch
    # (row block s only needs t >= s: the contraction starts at the tile's first row; in the row-normalised
    # mode S holds zeros above the diagonal, elsewhere that part is never written and must not be read)
    G.gemm(S, da, M=T, N=D, K=T, a_mn=True, b_mn=True, nz=(H, B), a_off=(0, 0, T, H * T), b_off=(0, 0, M, T),
           c_off=(0, T, 0, 0), flags=(pflags & ~G.F_ACCUM) | (G.F_ATOMIC if pflags & G.F_ACCUM else 0), out0=part,
           causal_k=2, **pkw)
    # dq = Gs q, then back through rotation, + gate gradient, ReLU mask
    dx = _bf16(M, d.HN, dev)
    if d.dual_dq:
        # dq = Gs q, rotation undone, + gate gradient, ReLU mask, and d cur += dx . E in one kernel
        rope = d.rot == "rope"
        DG.dual(Gs, q, W["encoder"], dx, dcur, M=M, H=H, n_per_head=N, K1=T, N2=D, T=T, epi=G.EPI_DQ_BWD,
                flags=(G.F_ROPE | G.F_TABLE) if rope else 0, a1_b=H * T, a1_h=T, b1_mn=True, b1_b=T, in0=dxg,
                in1=d.table(pos0) if rope else None, pos0=pos0, accumulate=True)
    elif d.rot == "pope":
        dq = _bf16(M, d.HNp, dev)
        G.gemm(Gs, q, M=T, N=Np, K=T, b_mn=True, nz=(H, B), a_off=(T, H * T, 0, 0), b_off=(Np, 0, 0, T),
               c_off=(0, T, Np, 0), out0=dq)
        ops.pope_bwd(dq, x, dxg, d.freqs_full, dx, H, T, pos0)
    else:
        rope = d.rot == "rope"
        G.gemm(Gs, q, M=T, N=N, K=T, b_mn=True, nz=(H, B), a_off=(T, H * T, 0, 0), b_off=(N, 0, 0, T),
               c_off=(0, T, N, 0), epi=G.EPI_DQ_BWD, flags=(G.F_ROPE | G.F_TABLE) if rope else 0, in0=dxg,
               in1=d.table(pos0) if rope else None, out0=dx, T=T, pos0=pos0, n_per_head=N, freqs=d.freqs)
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
    scores = d.B * d.H * d.T * d.T * 2
    narrow = (2 * d.H * d.M * d.D + 3 * d.M * d.D) * 2                        # a, LN(a); cur, mlp, out
    return wide + scores + narrow


def recompute_count(model, d: _Dims) -> int:
    """How many of the L layers re-run their forward in the backward pass. `model.recompute`:
    False / True (none / all), an int (that many, counted from the first layer), or "auto": as few as
    fit in 80 % of the free device memory, after setting aside the backward pass's own working set
    (about five [tokens, H*N'] bf16 tensors and one recomputed layer)."""
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
        working = 5 * d.M * max(d.HN, d.HNp) * 2 + per
        keep = int((0.8 * free - working) // per)
        return max(0, min(d.L, d.L - keep))
    raise ValueError(f"recompute must be a bool, an int or 'auto', not {r!r}")


def _stack_forward(model, d: _Dims, W, tokens, state, save: bool, recompute: int):
    """`recompute` = number of leading layers that keep only their input (and dropout seed)."""
    cur = _embed(d, W, tokens)
    pos0 = state.position if state is not None else 0
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
            saved.append(dict(cur=cur, drop_seed=seed_l) if l < recompute else sv)
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
        recompute = recompute_count(model, d)
        model._recomputed_layers = recompute
        cur, saved = _stack_forward(model, d, W, tokens, None, save=True, recompute=recompute)
        with prof.phase("head.loss"):
            logits = _head_logits(d, W, cur)
            row_loss = torch.empty(d.M, device=tokens.device, dtype=torch.float32)
            dlogits = _bf16(d.M, d.V, tokens.device)
            ops.cross_entropy(logits, targets.reshape(-1).contiguous(), row_loss, dlogits, 1.0 / d.M)
        ctx.d, ctx.W, ctx.saved, ctx.final, ctx.dlogits = d, W, saved, cur, dlogits
        ctx.tokens = tokens
        ctx.recompute = recompute
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
                    _, sv, _ = _layer_forward(d, W, sv["cur"], 0, None, False, sv["drop_seed"])
            with prof.phase("layer.backward"):
                dcur = _layer_backward(d, W, sv, dcur, grads, 0, final=(l == 0))
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

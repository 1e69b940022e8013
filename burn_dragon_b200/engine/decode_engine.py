"""Batched cached decoding for BDH on the sm_100a kernels.

One decode step for B independent streams = sample -> embed+LN -> L x (encoder GEMM with ReLU and
rotation, recurrent state update, LN, gated E_v GEMM, split-K decoder GEMM, layer tail) -> LM head.
Everything stays on the device: the sampled tokens feed the next step's embedding directly (the
reference copies logits to the host and samples there for every token, src/generation.rs:106-129),
and the step is captured once in a CUDA graph and replayed, with the position and the random-stream
counter held in device memory so the graph needs no new arguments.

The recurrent state is fp32 [B, H, N', D] per layer, exactly `LayerState.rho`.
"""
from __future__ import annotations

import os
from typing import Callable, List, Optional

import torch

from ..ops import gemm as G
from ..ops import native
from ..ops.fused_bdh import _Dims, _weights


class DecodeEngine:
    def __init__(self, model, use_graph: bool = True, split_k: int = 32, pope_graph: Optional[bool] = None,
                 lazy_decay: bool = True):
        self.model = model
        self.use_graph = use_graph
        # PoPE: the fused rotation epilogue takes the position as a host argument, so a step that uses
        # it cannot be replayed from a graph. `pope_graph` (or BDH_POPE_DECODE_GRAPH=1) ends the encoder
        # GEMM at the ReLU instead and rotates with elementwise ops that read the position from device
        # memory - the form the stream pool uses - which makes the single-request PoPE step capturable.
        self.pope_graph = (os.environ.get("BDH_POPE_DECODE_GRAPH", "0") == "1") if pope_graph is None else bool(pope_graph)
        self.split_k = split_k
        self.lazy_decay = bool(lazy_decay)
        self._cache = {}       # (streams, device, sampling settings) -> buffers, state storage, captured graph
        self.launches_per_step = None

    # ---- eligibility ---------------------------------------------------------------------------
    def can_run(self, toks: torch.Tensor, settings) -> bool:
        c = self.model.config
        from ..ops import emulate
        if not getattr(self.model, "use_native", True):
            return False
        if not emulate.active() and (not toks.is_cuda or not native.available()):
            return False
        if c.n_embd % 64 or c.n_embd > 1024 or c.latent_per_head % 64 or c.vocab_size > 1024:
            return False
        if c.block_sparse is not None and c.block_sparse.latent.is_sparse():
            return False
        if settings.max_new_tokens is None:
            return False
        return True

    # ---- buffers ---------------------------------------------------------------------------------
    def _alloc(self, B: int, dev):
        c = self.model.config
        d = _Dims(self.model, B, 1)
        S = self.split_k
        while d.HN % (S * 64):
            S //= 2
        S = max(S, 1)
        bf = dict(device=dev, dtype=torch.bfloat16)
        f32 = dict(device=dev, dtype=torch.float32)
        buf = dict(
            d=d, S=S,
            tok=torch.zeros(B, device=dev, dtype=torch.int64),
            logits=torch.zeros(B, d.V, **f32),
            cur=torch.zeros(B, d.D, **bf), nxt=torch.zeros(B, d.D, **bf),
            x=torch.zeros(B, d.HN, **bf),
            q=torch.zeros(B, d.HNp, **bf) if d.rot != "alibi" else None,
            a=torch.zeros(d.H * B, d.D, **f32),
            lna=torch.zeros(d.H * B, d.D, **bf),
            xy=torch.zeros(B, d.HN, **bf),
            part=torch.zeros(S * B, d.D, **f32),
            pos=torch.zeros(1, device=dev, dtype=torch.int32),
            step=torch.zeros(1, device=dev, dtype=torch.int32),
            table=(torch.zeros(1, d.N, **bf) if d.rot == "rope" else None),
        )
        return buf

    # ---- one step (all launches on the current stream) -------------------------------------------
    def _step(self, buf, W, rho: List[torch.Tensor], settings, seed: int, pos_host: Optional[int],
              last: Optional[List[torch.Tensor]] = None):
        """`last` (ALiBi models): per layer, the step up to which every state row is current - the decay is then
        applied lazily, only to the rows a step touches (see `_catch_up`)."""
        ops = native.ops
        d, S = buf["d"], buf["S"]
        B = buf["tok"].shape[0]
        ops.sample_tokens(buf["logits"], buf["tok"], float(settings.temperature), int(settings.top_k or 0),
                          bool(settings.greedy), seed, 0, buf["step"])
        ops.embed_ln_fwd(buf["tok"], W["embed"], buf["cur"])
        per_stream = buf["pos"].numel() > 1        # a pool of streams at different positions (stream_pool.py)
        if d.rot == "rope":
            if per_stream:
                buf["table"].copy_(G.rope_table_rows(buf["pos"], d.freqs))     # one table row per stream
            else:
                ops.rope_table_step(buf["pos"], d.freqs, buf["table"])
        cur, nxt = buf["cur"], buf["nxt"]
        for l in range(d.L):
            if d.rot == "rope":
                G.gemm(cur, W["encoder"], M=B, N=d.HN, K=d.D, epi=G.EPI_RELU, flags=G.F_ROPE | G.F_TABLE,
                       in0=buf["table"], out0=buf["x"], out1=buf["q"], theta=d.theta, T=buf["table"].shape[0],
                       n_per_head=d.N, freqs=d.freqs,       # row m reads table row m % T
                       tma_epilogue=not per_stream)         # a few rows: the per-thread epilogue, as for T = 1
                q = buf["q"]
            elif d.rot == "pope" and (per_stream or self.pope_graph):
                # the position(s) come from device memory: the encoder GEMM stops at the ReLU and the rotation
                # q = softplus(x) * (cos, sin)(2 pi frac(pos f)) is a few elementwise ops on [streams, H*N]
                G.gemm(cur, W["encoder"], M=B, N=d.HN, K=d.D, epi=G.EPI_RELU, out0=buf["x"], theta=d.theta)
                ph = G.rot_phases(buf["pos"], d.freqs)                       # [streams, N], or [1, N] shared
                mag = torch.nn.functional.softplus(buf["x"].float()).view(B, d.H, d.N)
                qv = buf["q"].view(B, d.H, 2, d.N)                           # per head: [real N | imaginary N]
                qv[:, :, 0] = mag * ph.cos()[:, None]
                qv[:, :, 1] = mag * ph.sin()[:, None]
                q = buf["q"]
            elif d.rot == "pope":
                G.gemm(cur, W["encoder"], M=B, N=d.N, K=d.D, nz=(d.H, 1), b_off=(d.N, 0, 0, 0), c_off=(0, 0, d.N, 0),
                       o1_off=(d.Np, 0, d.N), epi=G.EPI_RELU, flags=G.F_POPE, out0=buf["x"], out1=buf["q"],
                       theta=d.theta, T=1, pos0=int(pos_host), n_per_head=d.N, freqs=d.freqs)
                q = buf["q"]
            else:
                G.gemm(cur, W["encoder"], M=B, N=d.HN, K=d.D, epi=G.EPI_RELU, out0=buf["x"], theta=d.theta)
                q = buf["x"]
            # `a` is zero here: cleared at allocation and again by every pass that reads it
            if last is not None:
                ops.decode_state_update(q, cur, rho[l], buf["a"], d.slopes, last[l], buf["step"])
            else:
                ops.decode_state_update(q, cur, rho[l], buf["a"], d.slopes)
            ops.layernorm_f32_clear(buf["a"], buf["lna"])
            G.gemm(buf["lna"], W["encoder_v"], M=B, N=d.N, K=d.D, nz=(d.H, 1), a_off=(B, 0, 0, 0),
                   b_off=(d.N, 0, 0, 0), c_off=(0, 0, d.N, 0), epi=G.EPI_RELU_GATE, flags=G.F_NO_OUT0, in0=buf["x"],
                   out1=buf["xy"], theta=d.theta)
            ks = d.HN // S
            G.gemm(buf["xy"], W["decoder"], M=B, N=d.D, K=ks, b_mn=True, nz=(S, 1), a_off=(0, 0, ks, 0),
                   b_off=(0, 0, ks, 0), c_off=(B, 0, 0, 0), flags=G.F_OUT_F32, out0=buf["part"])
            ops.block_out_parts(cur, buf["part"], nxt)         # sum of the split-K partial tiles + layer tail
            cur, nxt = nxt, cur
        if d.V % 8 == 0:
            G.gemm(cur, W["lm_head"], M=B, N=d.V, K=d.D, b_mn=True, flags=G.F_OUT_F32, out0=buf["logits"])
        else:
            # the TMA descriptor of the head needs 16-byte rows (V % 8 == 0 in bf16); character
            # vocabularies rarely have that, and the head is a [B, D] x [D, V] product: library matmul
            torch.matmul(cur.float(), W["lm_head"].float(), out=buf["logits"])
        if per_stream:
            buf["pos"].add_(1)
        else:
            ops.bump_counter(buf["pos"], 1)
        ops.bump_counter(buf["step"], 1)

    @staticmethod
    def _catch_up(rho, last, step, slopes) -> None:
        """Lazy decay: bring every state row up to date before the state leaves the engine,
        rho[b,h,n] *= gamma_h^(step - last[b,h,n])."""
        H = slopes.numel()
        for r, t in zip(rho, last):
            lag = (step.view(1, 1, 1) - t).float()
            r.mul_(torch.exp(-slopes.float().view(1, H, 1) * lag).unsqueeze(-1))
            t.copy_(step.view(1, 1, 1).expand_as(t))

    # ---- public ------------------------------------------------------------------------------------
    @torch.no_grad()
    def generate(self, toks: torch.Tensor, settings, generator=None,
                 on_token: Optional[Callable[[torch.Tensor], None]] = None) -> torch.Tensor:
        from . import generation as GEN
        state, last = GEN.prefill_state(self.model, toks, toks.device)
        new = self.continue_from(state, last, settings, int(settings.max_new_tokens), on_token)
        return torch.cat([toks, new], dim=1)

    @torch.no_grad()
    def continue_from(self, state, last, settings, n: int, on_token: Optional[Callable[[torch.Tensor], None]] = None,
                      step0: int = 0) -> torch.Tensor:
        """Decode `n` tokens per stream from a recurrent state and the logits of the last token seen
        (what `prefill_state` or an earlier call left). Returns the new tokens [B, n]; `state` is
        advanced and `self.last_logits` holds the logits after the last new token. `step0` is the
        number of tokens this stream of calls has sampled so far: the random stream of the device
        sampler continues from there instead of repeating."""
        model = self.model
        dev = last.device
        B = last.shape[0]
        c = model.config
        seed = int(settings.seed if settings.seed is not None else torch.initial_seed() & 0x7FFFFFFF) & 0xFFFFFFFF
        key = (B, str(dev), float(settings.temperature), int(settings.top_k or 0), bool(settings.greedy), seed)
        ctx = self._cache.get(key)
        if ctx is None:
            buf = self._alloc(B, dev)
            rho = [torch.zeros(B, c.n_head, c.state_latent, c.n_embd, device=dev) for _ in range(c.n_layer)]
            # ALiBi: lazy decay (rows whose query entry is zero are not streamed; the state is brought up to date
            # when it leaves the engine). `lazy_decay=False` on the engine scales every row every step.
            seen = ([torch.zeros(B, c.n_head, c.state_latent, device=dev, dtype=torch.int32) for _ in range(c.n_layer)]
                    if (buf["d"].slopes is not None and self.lazy_decay) else None)
            ctx = dict(buf=buf, rho=rho, graph=None, last=seen)
            self._cache.clear()            # one resident configuration: the state buffers are large
            self._cache[key] = ctx
        buf, rho, seen = ctx["buf"], ctx["rho"], ctx["last"]
        d = buf["d"]
        W = _weights(model)

        def load_state():
            for r, ls in zip(rho, state.layers):
                if ls.rho is None:
                    r.zero_()
                elif ls.rho.data_ptr() != r.data_ptr():      # a continued stream already lives in these buffers
                    r.copy_(ls.rho)
            if last.data_ptr() != buf["logits"].data_ptr():
                buf["logits"].copy_(last.float())
            buf["pos"].fill_(state.position)
            buf["step"].fill_(int(step0))
            buf["a"].zero_()           # (every step leaves it cleared; this covers a step that was interrupted)
            if seen is not None:
                for t in seen:
                    t.fill_(int(step0))    # what comes in is current

        load_state()
        graph_ok = self.use_graph and (d.rot != "pope" or self.pope_graph) and dev.type == "cuda"
        out = []
        n = int(n)
        if graph_ok:
            if ctx["graph"] is None:
                # warm up once on a side stream (lazy initialisation, allocator), rewind, then capture
                s = torch.cuda.Stream()
                s.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(s):
                    self._step(buf, W, rho, settings, seed, None, seen)
                torch.cuda.current_stream().wait_stream(s)
                load_state()
                graph = torch.cuda.CUDAGraph()
                n0 = native.launch_count()
                with torch.cuda.graph(graph):
                    self._step(buf, W, rho, settings, seed, None, seen)
                # kernels of this library inside one replay (what a benchmark reports as its launches per step)
                self.launches_per_step = native.launch_count() - n0
                ctx["graph"], ctx["weights"] = graph, W
                load_state()
            elif any(ctx["weights"][k].data_ptr() != W[k].data_ptr() for k in W):
                # the captured graph reads the weight buffers it was captured with
                for k in W:
                    ctx["weights"][k].copy_(W[k])
            graph = ctx["graph"]
            for _ in range(n):
                graph.replay()
                t = buf["tok"].clone()
                out.append(t.view(-1, 1))
                if on_token is not None:
                    on_token(t)
        else:
            for i in range(n):
                self._step(buf, W, rho, settings, seed, state.position + i, seen)
                t = buf["tok"].clone()
                out.append(t.view(-1, 1))
                if on_token is not None:
                    on_token(t)
        if seen is not None:
            self._catch_up(rho, seen, buf["step"], d.slopes)
        for ls, r in zip(state.layers, rho):
            ls.rho = r
        state.position += n
        self.last_state, self.last_logits = state, buf["logits"]
        return torch.cat(out, dim=1) if out else torch.empty(B, 0, dtype=torch.int64, device=dev)


def attach(model, **kw) -> DecodeEngine:
    """Give `model` a decode engine; `engine.generation.generate_tokens` uses it when eligible."""
    model.decode_engine = DecodeEngine(model, **kw)
    return model.decode_engine

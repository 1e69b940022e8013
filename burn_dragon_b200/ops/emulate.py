"""The kernel path without a GPU: every launch of `ops.fused_bdh` replaced by the fp32 torch statement
of the same contract (`gemm.gemm_reference` for the GEMM + epilogue launches, the functions below for
the row-wise kernels), operating on the very same bf16 / fp32 buffers in place.

This runs the orchestration of the kernel path - operand offsets, batching over (head, batch),
flags, what is saved for the backward pass, the tensor-parallel and context-parallel hooks - on any
device, so that it can be tested on CPU ranks; it says nothing about the CUDA code itself, which the
GPU tests compare against the same statements.

    with emulate.kernel_path():
        loss = model(tokens, targets)          # ops.fused_bdh, launch by launch, in torch ops

Every emulated GEMM launch is also bounds-checked on the host (`gemm.check_extents`: operand and
output windows of the last batch index against the tensor shapes).

`BDH_EMULATE_KERNELS=1` switches it on for a whole process (the multi-rank self tests use that).
The reference has no counterpart: its tests run its one code path on the CPU backend
(tests/model_paths.rs:33-91).
"""
from __future__ import annotations

import os
from contextlib import contextmanager

import torch

from . import gemm as G
from . import reference as R


def _ln_bwd(x: torch.Tensor, dy: torch.Tensor) -> torch.Tensor:
    """Backward of the affine-free LayerNorm (eps 1e-5, biased variance) in fp32."""
    x, dy = x.float(), dy.float()
    mean = x.mean(-1, keepdim=True)
    inv = torch.rsqrt((x - mean).pow(2).mean(-1, keepdim=True) + R.LN_EPS)
    y = (x - mean) * inv
    return (dy - dy.mean(-1, keepdim=True) - y * (dy * y).mean(-1, keepdim=True)) * inv


class TorchOps:
    """`torch.ops.bdh.*` row-wise kernels as in-place torch functions with the same argument lists."""

    count = 0

    @staticmethod
    def layernorm_fwd(x, y):
        y.copy_(R.layer_norm(x.float()))

    @staticmethod
    def layernorm_bwd(x, dy, dx, accumulate):
        g = _ln_bwd(x, dy)
        dx.copy_(dx.float() + g if accumulate else g)

    @staticmethod
    def embed_ln_fwd(tokens, emb, cur):
        cur.copy_(R.layer_norm(emb.float()[tokens.reshape(-1)]))

    @staticmethod
    def embed_ln_bwd(tokens, emb, dcur, demb):
        t = tokens.reshape(-1)
        demb.index_add_(0, t, _ln_bwd(emb.float()[t], dcur))

    @staticmethod
    def block_out_fwd(cur, mlp, out):
        out.copy_(R.layer_norm(cur.float() + R.layer_norm(mlp.float())))

    @staticmethod
    def layernorm_f32_clear(a, y):
        y.copy_(R.layer_norm(a.float()))
        a.zero_()

    @staticmethod
    def block_out_parts(cur, part, out):
        mlp = part.float().view(-1, *cur.shape).sum(0)
        out.copy_(R.layer_norm(cur.float() + R.layer_norm(mlp)))

    @staticmethod
    def block_out_bwd(cur, mlp, dout, dcur, dmlp):
        u = cur.float() + R.layer_norm(mlp.float())
        du = _ln_bwd(u, dout)
        dcur.copy_(du)
        dmlp.copy_(_ln_bwd(mlp, du))

    @staticmethod
    def cross_entropy(logits, targets, row_loss, dlogits, grad_scale):
        lp = torch.log_softmax(logits.float(), dim=-1)
        t = targets.reshape(-1)
        row_loss.copy_(-lp.gather(1, t[:, None])[:, 0])
        if dlogits is not None:
            g = lp.exp()
            g[torch.arange(g.shape[0], device=g.device), t] -= 1.0
            dlogits.copy_(g * grad_scale)

    @staticmethod
    def state_scan(seg, start, decay, out16, total, J, H, backward):
        BJ, _, Np, D = seg.shape
        B = BJ // J
        s5, o5 = seg.view(B, J, H, Np, D), out16.view(B, J, H, Np, D)
        g = decay.float().view(1, H, 1, 1) if decay is not None else 1.0
        run = start.float().view(B, H, Np, D).clone() if start is not None else torch.zeros(B, H, Np, D, device=seg.device)
        order = range(J - 1, -1, -1) if backward else range(J)
        for j in order:
            o5[:, j] = run.to(out16.dtype)
            if backward and j == 0:
                break
            run = run * g + s5[:, j]
        if not backward and total is not None:
            total.view(B, H, Np, D).copy_(run)

    @staticmethod
    def pope_rotate(x, freqs, q, H, T, pos0):
        M, HN = x.shape
        N = HN // H
        pos = pos0 + (torch.arange(M, device=x.device) % T)
        ph = G.rot_phases(pos, freqs)                                  # [M, N]
        mag = torch.nn.functional.softplus(x.float()).view(M, H, N)
        qv = q.view(M, H, 2, N)
        qv[:, :, 0] = (mag * ph.cos()[:, None]).to(q.dtype)
        qv[:, :, 1] = (mag * ph.sin()[:, None]).to(q.dtype)

    @staticmethod
    def pope_bwd(dq, x, dxg, freqs, dx, H, T, pos0):
        M, HN = x.shape
        N = HN // H
        pos = pos0 + (torch.arange(M, device=x.device) % T)
        ph = G.rot_phases(pos, freqs)                                  # [M, N]
        d = dq.float().view(M, H, 2, N)
        xf = x.float().view(M, H, N)
        g = (d[:, :, 0] * ph.cos()[:, None] + d[:, :, 1] * ph.sin()[:, None]) * torch.sigmoid(xf)
        g = g + dxg.float().view(M, H, N)
        dx.copy_(torch.where(xf > 0, g, torch.zeros_like(g)).view(M, HN))


    # ---- forward_fast attention (ops/rownorm_attention.py) -----------------------------------------
    @staticmethod
    def _causal(S, T):
        rows = torch.arange(S.shape[0], device=S.device) % T
        return torch.arange(S.shape[1], device=S.device)[None, :] < rows[:, None]        # column s < t

    @staticmethod
    def rownorm_fwd(S, rnorm, T):
        m = TorchOps._causal(S, T)
        x = torch.where(m, S.float(), torch.zeros((), device=S.device))
        r = x.abs().sum(-1) + R.ROW_NORM_EPS
        rnorm.copy_(r)
        S.copy_(torch.where(m, x / r[:, None], S.float()))

    @staticmethod
    def rownorm_bwd(grad, normed, rnorm, T):
        m = TorchOps._causal(grad, T)
        g = torch.where(m, grad.float(), torch.zeros((), device=grad.device))
        sn = torch.where(m, normed.float(), torch.zeros((), device=grad.device))
        dot = (g * sn).sum(-1, keepdim=True)
        grad.copy_(torch.where(m, (g - torch.sign(sn) * dot) / rnorm[:, None], grad.float()))

    # ---- decode step (engine/decode_engine.py) ----------------------------------------------------
    @staticmethod
    def sample_tokens(logits, out, temperature, top_k, greedy, seed, step_host, step_dev):
        """Greedy: lowest index among the maxima, as the kernel. Sampling: same distribution
        (temperature, top-k threshold with ties kept), drawn from a torch generator keyed by
        (seed, step) - not the kernel's hash stream, so sampled tokens differ from the GPU's."""
        x = logits.float()
        if greedy:
            out.copy_(torch.argmax(x, dim=-1))
            return
        step = int(step_dev.item()) if step_dev is not None else int(step_host)
        x = R.top_k_filter(x / max(float(temperature), 1e-8), int(top_k) if top_k else None)
        g = torch.Generator(device="cpu").manual_seed((int(seed) * 1000003 + step) & 0x7FFFFFFF)
        p = torch.softmax(x, dim=-1).cpu()
        out.copy_(torch.multinomial(p, 1, generator=g)[:, 0].to(out.device))

    @staticmethod
    def rope_table_step(pos, pair_freqs, table):
        table.copy_(G.rope_table(int(pos.item()), 1, pair_freqs))

    @staticmethod
    def bump_counter(counter, by):
        counter.add_(int(by))

    @staticmethod
    def decode_state_update(q, v, rho, a, slopes, last=None, step_dev=None):
        """a[h*B + b] += q[b, h] . rho[b, h];  rho[b, h] = (rho[b, h] + q[b, h]^T v[b]) * exp(-slope_h).
        With `last` / `step_dev` the decay is lazy: only rows with a non-zero query entry are brought up to date
        (times exp(-slope (step - last))), updated and marked current up to step + 1."""
        B, H, Np, D = rho.shape
        qf = q.float().view(B, H, Np)
        if last is not None:
            step = int(step_dev.reshape(-1)[0])
            live = qf != 0
            lag = (step - last.view(B, H, Np)).float()
            up = torch.where(live, torch.exp(-slopes.float().view(1, H, 1) * lag), torch.ones_like(lag))
            rho.mul_(up.unsqueeze(-1))
            a.view(H, B, D).add_(torch.einsum("bhn,bhnd->hbd", qf, rho))
            new = (rho + qf.unsqueeze(-1) * v.float().view(B, 1, 1, D)) * torch.exp(-slopes.float()).view(1, H, 1, 1)
            rho.copy_(torch.where(live.unsqueeze(-1), new, rho))
            last.view(B, H, Np).copy_(torch.where(live, torch.full_like(last.view(B, H, Np), step + 1), last.view(B, H, Np)))
            return
        a.view(H, B, D).add_(torch.einsum("bhn,bhnd->hbd", qf, rho))
        rho.add_(qf.unsqueeze(-1) * v.float().view(B, 1, 1, D))
        if slopes is not None:
            rho.mul_(torch.exp(-slopes.float()).view(1, H, 1, 1))


def _rotate_by_table(x: torch.Tensor, table: torch.Tensor, T: int, n_per_head: int) -> torch.Tensor:
    """RoPE with (cos, sin) read from the fp16 pair table the kernels use ([T, n_per_head] viewed as
    bf16: element 2i = cos, 2i+1 = sin of pair i): row m uses table row m % T, column n the pair of
    n % n_per_head. The positions are whatever the table was built for."""
    M, N = x.shape
    tab = table.view(torch.float16).float()
    rows = torch.arange(M, device=x.device) % T
    pair = (torch.arange(N, device=x.device) % n_per_head) // 2
    cos, sin = tab[rows][:, 2 * pair], tab[rows][:, 2 * pair + 1]
    pairs = x.reshape(M, -1, 2)
    rotated = torch.stack((-pairs[..., 1], pairs[..., 0]), dim=-1).reshape(M, N)
    return x * cos + rotated * sin


def _gemm(a, b, **kw):
    for k in ("peer_ptrs", "peer_rows", "peer_rank"):      # multi-GPU routing of the output: not emulated
        kw.pop(k, None)
    G.check_extents(a, b, **kw)          # every emulated launch is bounds-checked on the host
    flags = kw.get("flags", 0)
    if kw.get("epi", G.EPI_STORE) == G.EPI_RELU and (flags & G.F_ROPE) and (flags & G.F_TABLE) \
            and tuple(kw.get("nz", (1, 1))) == (1, 1):
        # the rotation comes from the table (which carries the positions), not from pos0
        out1 = kw.pop("out1")
        G.gemm_reference(a, b, **{**kw, "flags": flags & ~(G.F_ROPE | G.F_TABLE), "out1": None})
        x = kw["out0"][:kw["M"], :kw["N"]].float()
        out1[:kw["M"], :kw["N"]] = _rotate_by_table(x, kw["in0"], kw.get("T", 1), kw.get("n_per_head", 1)).to(out1.dtype)
        return
    G.gemm_reference(a, b, **kw)


_state = {"on": False}


def active() -> bool:
    return _state["on"]


def enable(on: bool = True) -> None:
    """Route `ops.fused_bdh` through the torch statements (any device) or back to the kernels."""
    from . import fused_bdh
    if on == _state["on"]:
        return
    from . import native
    if on:
        from . import dual_gemm as DG
        _state["saved"] = (fused_bdh.ops, native.ops, G.gemm, DG.dual)
        fused_bdh.ops = native.ops = TorchOps          # the decode engine reads `native.ops` at call time
        G.gemm = _gemm
        DG.dual = DG.dual_reference
    else:
        from . import dual_gemm as DG
        fused_bdh.ops, native.ops, G.gemm, DG.dual = _state.pop("saved")
    _state["on"] = on


@contextmanager
def kernel_path():
    was = _state["on"]
    enable(True)
    try:
        yield
    finally:
        enable(was)


if os.environ.get("BDH_EMULATE_KERNELS", "0") == "1":
    enable(True)

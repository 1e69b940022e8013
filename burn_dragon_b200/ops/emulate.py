"""The kernel path without a GPU: every launch of `ops.fused_bdh` replaced by the fp32 torch statement
of the same contract (`gemm.gemm_reference` for the GEMM + epilogue launches, the functions below for
the row-wise kernels), operating on the very same bf16 / fp32 buffers in place.

This runs the orchestration of the kernel path - operand offsets, batching over (head, batch),
flags, what is saved for the backward pass, the tensor-parallel and context-parallel hooks - on any
device, so that it can be tested on CPU ranks; it says nothing about the CUDA code itself, which the
GPU tests compare against the same statements.

    with emulate.kernel_path():
        loss = model(tokens, targets)          # ops.fused_bdh, launch by launch, in torch ops

`BDH_EMULATE_KERNELS=1` switches it on for a whole process (the multi-rank self tests use that).
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


def _gemm(a, b, **kw):
    for k in ("peer_ptrs", "peer_rows", "peer_rank"):      # multi-GPU routing of the output: not emulated
        kw.pop(k, None)
    G.gemm_reference(a, b, **kw)


_state = {"on": False}


def active() -> bool:
    return _state["on"]


def enable(on: bool = True) -> None:
    """Route `ops.fused_bdh` through the torch statements (any device) or back to the kernels."""
    from . import fused_bdh
    if on == _state["on"]:
        return
    if on:
        _state["saved"] = (fused_bdh.ops, fused_bdh.G.gemm)
        fused_bdh.ops = TorchOps
        fused_bdh.G.gemm = _gemm
    else:
        fused_bdh.ops, fused_bdh.G.gemm = _state.pop("saved")
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

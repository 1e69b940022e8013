"""Neuron-sharded tensor parallelism for BDH.

Rank r owns neurons [r*N/tp, (r+1)*N/tp) of every head: the matching rows of E, E_v and D (all
stored neuron-major) and, in inference, the matching rows of the recurrent state. Activations of
width D are replicated; everything of neuron width stays local. Four tensors per layer are partial
sums over the neuron shards and have to be reduced across ranks:

    forward   a   = S V           [H*M, D]   (scores are built from the local neuron slice)
              mlp = (x*y) D       [M, D]
    backward  d LN(a) = dy E_v    [H*M, D]
              d cur  = S^T dA + dx E   [M, D]

In the fused mode the GEMM that produces each of them adds its tiles straight into every rank's
replica through the NVSwitch (`multimem.red` in the GEMM epilogue, EPI_F_MC_RED), bracketed by
device-side rank barriers; without multicast the partials are written locally and reduced by the
peer-load all-reduce kernel; `fused=False` is the NCCL baseline. Weight gradients are local to the
shard (no reduction inside a TP group). The reference has no tensor parallelism.
"""
from __future__ import annotations

import copy
from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..engine.optim import FlatAdamW
from ..models.bdh import BDH
from ..ops import gemm as G
from ..ops import native
from ..ops import reference as R


class _Buf:
    def __init__(self, view, mc, sym):
        self.view, self.mc, self.sym = view, mc, sym


class TPComm:
    """Reduction of [rows, D] fp32 partial sums across the TP group."""

    def __init__(self, device, group=None, fused: bool = True):
        self.device, self.group = device, group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.fused = bool(fused and device.type == "cuda" and native.available())
        self.multicast = False
        self._bufs: Dict = {}
        self._flags = None
        if self.fused:
            try:
                from . import symm
                self._symm = symm
                self._flags = symm._Flags.get(device, group if group is not None else dist.group.WORLD)
            except Exception as e:  # noqa: BLE001
                self.fallback_reason = repr(e)
                self.fused = False
        self.flags = G.F_OUT_F32 | G.F_ACCUM

    def _barrier(self, anchor):
        f = self._flags
        f["epoch"] += 1
        native.ops.rank_barrier(anchor, f["buf"].ptrs, self.rank, self.world, f["epoch"])

    def begin(self, key: str, rows: int, cols: int) -> _Buf:
        k = (key, rows, cols)
        b = self._bufs.get(k)
        if b is None:
            n = rows * cols
            if self.fused:
                pad = (-n) % (4 * self.world)
                sym = self._symm.SymmetricBuffer(n + pad, torch.float32, self.device, self.group)
                sym.tensor.zero_()
                sym.barrier()
                b = _Buf(sym.tensor[:n].view(rows, cols), sym.multicast_ptr, sym)
                if sym.multicast_ptr:
                    self.multicast = True
            else:
                b = _Buf(torch.zeros(rows, cols, device=self.device), 0, None)
            self._bufs[k] = b
        b.view.zero_()
        if self.fused and b.mc:
            self.flags = G.F_OUT_F32 | G.F_MC_RED
            self._barrier(b.view)          # every replica is zero before anybody's tiles arrive
        else:
            self.flags = G.F_OUT_F32 | G.F_ACCUM
        return b

    def end(self, b: _Buf) -> torch.Tensor:
        if self.fused and b.mc:
            self._barrier(b.view)          # every rank's tiles have landed in every replica
        elif self.fused:
            f = self._flags
            f["epoch"] += 1
            s = b.sym
            native.ops.allreduce_scale(s.tensor, s.ptrs, f["buf"].ptrs, 0, s.rank, s.world, s.tensor.numel(), 1.0,
                                       f["epoch"], self._symm.COLL_CTAS)
        else:
            dist.all_reduce(b.view, group=self.group)
        return b.view


def shard_rows(w: torch.Tensor, H: int, N: int, rank: int, world: int) -> torch.Tensor:
    """[H*N, D] -> this rank's [H*N/world, D] (neurons [rank*N/world, (rank+1)*N/world) of every head)."""
    Nl = N // world
    return w.view(H, N, -1)[:, rank * Nl:(rank + 1) * Nl].reshape(H * Nl, -1).contiguous()


def unshard_rows(parts, H: int, N: int) -> torch.Tensor:
    world = len(parts)
    Nl = N // world
    return torch.cat([p.view(H, Nl, -1) for p in parts], dim=1).reshape(H * N, -1)


class NeuronTP:
    def __init__(self, model: BDH, lr=1e-3, weight_decay=0.1, beta1=0.9, beta2=0.999, eps=1e-5, fused: bool = True,
                 group=None):
        self.full, self.group = model, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        c = model.config
        H, N = c.n_head, c.latent_per_head
        if N % (64 * self.world):
            raise ValueError("neurons per head must be a multiple of 64 * tp")
        dev = next(model.parameters()).device
        for p in model.parameters():
            dist.broadcast(p.data, src=0, group=group)
        lc = copy.copy(c)
        lc.n_latent_per_head = N // self.world
        self.shard = BDH(lc).to(dev)
        with torch.no_grad():
            self.shard.embed.weight.copy_(model.embed.weight)
            self.shard.lm_head.copy_(model.lm_head)
            for name in ("encoder", "encoder_v", "decoder"):
                getattr(self.shard, name).copy_(shard_rows(getattr(model, name).data, H, N, self.rank, self.world))
        self.shard.recompute = getattr(model, "recompute", False)
        self.comm = TPComm(dev, group, fused)
        self.fused = self.comm.fused
        Nl = N // self.world
        full_freqs = R.build_freqs(N, c.rope_theta, c.rotary_embedding, device=dev)

        def dims_hook(d):
            d.comm = self.comm
            if d.rot == "rope":
                d.freqs_full = full_freqs[self.rank * Nl:(self.rank + 1) * Nl].contiguous()
                d.freqs = d.freqs_full[0::2].contiguous()
            elif d.rot == "pope":
                d.freqs = d.freqs_full = full_freqs[self.rank * Nl:(self.rank + 1) * Nl].contiguous()

        self.shard._dims_hook = dims_hook
        self.opt = FlatAdamW(self.shard, lr, weight_decay, beta1, beta2, eps, shadow_bf16=dev.type == "cuda")
        self.optimizer = self.opt
        self.lr = lr
        self._replicated = [self.shard.embed.weight, self.shard.lm_head]

    def train_step(self, tokens, targets, lr: Optional[float] = None) -> torch.Tensor:
        self.opt.zero_grad()
        loss = self.shard(tokens, targets)
        loss.backward()
        # the replicated tensors see the same gradient on every rank up to summation order; average
        # them so the replicas cannot drift apart
        for p in self._replicated:
            dist.all_reduce(p.grad, group=self.group)
            p.grad.div_(self.world)
        self.opt.step(lr=self.lr if lr is None else lr)
        return loss.detach()

    def gather_state_dict(self) -> Dict[str, torch.Tensor]:
        c = self.full.config
        out = {"embed.weight": self.shard.embed.weight.detach().cpu().clone(),
               "lm_head": self.shard.lm_head.detach().cpu().clone()}
        for name in ("encoder", "encoder_v", "decoder"):
            local = getattr(self.shard, name).detach().contiguous()
            parts = [torch.empty_like(local) for _ in range(self.world)]
            dist.all_gather(parts, local, group=self.group)
            out[name] = unshard_rows(parts, c.n_head, c.latent_per_head).cpu()
        return out

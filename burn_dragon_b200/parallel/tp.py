"""Neuron-sharded tensor parallelism for BDH.

Rank r owns neurons [r*N/tp, (r+1)*N/tp) of every head: the matching rows of E, E_v and D (all
stored neuron-major) and, in inference, the matching rows of the recurrent state. Activations of
width D are replicated; everything of neuron width stays local. Four tensors per layer are partial
sums over the neuron shards and have to be reduced across ranks:

    forward   a   = S V           [H*M, D]   (scores are built from the local neuron slice)
              mlp = (x*y) D       [M, D]
    backward  d LN(a) = dy E_v    [H*M, D]
              d cur  = S^T dA + dx E   [M, D]

In the fused mode the GEMM that produces each of them is also the reduce-scatter: its epilogue
adds every tile into the buffer of the rank that owns the tile's rows (`red.sys` through the peer
mapping, EPI_F_PEER_RED), and a gather kernel broadcasts the finished blocks (`multimem.st`), as
bf16 where the consumer is bf16. `fused="mc_red"` instead adds tiles into every replica at once
with `multimem.red`, `fused="allreduce"` runs the peer-load all-reduce kernel on locally written
partial sums, and `fused=False` is the NCCL baseline. Weight gradients are local to the
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
    """One reduction in flight: `view` is the local fp32 [rows, cols] partial-sum buffer the GEMM writes
    through, `kw` are the extra GEMM arguments (multicast address or peer pointers) for this mode."""

    def __init__(self, view, sym, kw, rows, cols, block_rows=0, out16=None):
        self.view, self.sym, self.kw = view, sym, kw
        self.rows, self.cols, self.block_rows, self.out16 = rows, cols, block_rows, out16


class TPComm:
    """Reduction of [rows, D] fp32 partial sums across the TP group. Modes:

    rs         the producing GEMM's epilogue adds each tile into the buffer of the rank that owns
               its rows (reduce-scatter over peer mappings, overlapped with the GEMM tile by tile);
               a gather kernel then sends every owner's finished block to all ranks, as bf16 when
               the consumer wants bf16. Per GPU this moves (w-1)/w of the tensor in and at most as
               much out - the all-reduce minimum - at any group size.
    mc_red     the epilogue adds each tile into every rank's replica with one `multimem.red`
               through the switch. Every GPU receives w copies of the tensor: only for w = 2.
    allreduce  partial sums are written locally and reduced by the peer-load all-reduce kernel.
    nccl       partial sums are written locally and reduced by NCCL (the baseline).
    """

    def __init__(self, device, group=None, fused=True):
        self.device, self.group = device, group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        mode = fused if isinstance(fused, str) else ("rs" if fused else "nccl")
        if not (device.type == "cuda" and native.available()):
            mode = "nccl"
        self.multicast = False
        self._bufs: Dict = {}
        self._flags = None
        if mode != "nccl":
            try:
                from . import symm
                self._symm = symm
                self._flags = symm._Flags.get(device, group if group is not None else dist.group.WORLD)
            except Exception as e:  # noqa: BLE001
                self.fallback_reason = repr(e)
                mode = "nccl"
        self.mode = mode
        self.fused = mode != "nccl"
        self.flags = G.F_OUT_F32 | G.F_ACCUM

    def _epoch(self) -> int:
        self._flags["epoch"] += 1
        return self._flags["epoch"]

    def _barrier(self, anchor):
        native.ops.rank_barrier(anchor, self._flags["buf"].ptrs, self.rank, self.world, self._epoch())

    def _make(self, key, rows, cols) -> _Buf:
        n = rows * cols
        if not self.fused:
            return _Buf(torch.zeros(rows, cols, device=self.device), None, {}, rows, cols)
        # owner blocks of whole rows, an even number of them, so that a block is a multiple of 8 floats
        block_rows = -(-rows // self.world)
        block_rows += block_rows % 2
        total = max(n, block_rows * cols * self.world)
        total += (-total) % (8 * self.world)
        sym = self._symm.SymmetricBuffer(total, torch.float32, self.device, self.group)
        sym.tensor.zero_()
        out16 = None
        if self.mode == "rs":
            out16 = self._symm.SymmetricBuffer(total, torch.bfloat16, self.device, self.group)
        sym.barrier()
        if sym.multicast_ptr:
            self.multicast = True
        mode = self.mode
        if mode == "mc_red" and not sym.multicast_ptr:
            mode = "allreduce"
        kw = {}
        if mode == "mc_red":
            kw = dict(mc_out=sym.multicast_ptr)
        elif mode == "rs":
            kw = dict(peer_ptrs=sym.ptrs, peer_rows=block_rows)
        b = _Buf(sym.tensor[:n].view(rows, cols), sym, kw, rows, cols, block_rows, out16)
        b.mode = mode
        return b

    def begin(self, key: str, rows: int, cols: int) -> _Buf:
        k = (key, rows, cols)
        b = self._bufs.get(k)
        if b is None:
            b = self._bufs[k] = self._make(key, rows, cols)
        mode = getattr(b, "mode", "nccl")
        if mode == "rs":
            # only the owned block receives sums; it must be zero on every rank before any tile arrives
            lo = min(self.rank * b.block_rows, rows)
            hi = min(lo + b.block_rows, rows)
            if hi > lo:
                b.view[lo:hi].zero_()
            self._barrier(b.view)
            self.flags = G.F_OUT_F32 | G.F_PEER_RED
        elif mode == "mc_red":
            b.view.zero_()
            self._barrier(b.view)          # every replica is zero before anybody's tiles arrive
            self.flags = G.F_OUT_F32 | G.F_MC_RED
        else:
            b.view.zero_()
            self.flags = G.F_OUT_F32 | G.F_ACCUM
        return b

    def end(self, b: _Buf, bf16: bool = False) -> torch.Tensor:
        """The reduced tensor: fp32 (a view of the reduction buffer, valid until the next `begin` with
        the same key and shape) or, with `bf16`, a fresh bf16 tensor."""
        mode = getattr(b, "mode", "nccl")
        if mode == "rs":
            s, f = b.sym, self._flags
            o = b.out16
            native.ops.gather_blocks(s.tensor, s.ptrs, f["buf"].ptrs, s.multicast_ptr,
                                     o.ptrs if bf16 else [], o.multicast_ptr if bf16 else 0, s.rank, s.world,
                                     s.tensor.numel(), b.block_rows * b.cols, self._epoch(), self._symm.COLL_CTAS)
            if bf16:
                # the gather buffer is reused by the next reduction with this key: hand out a copy
                return o.tensor[:b.rows * b.cols].view(b.rows, b.cols).clone()
            return b.view
        if mode == "mc_red":
            self._barrier(b.view)          # every rank's tiles have landed in every replica
        elif mode == "allreduce":
            s = b.sym
            native.ops.allreduce_scale(s.tensor, s.ptrs, self._flags["buf"].ptrs, s.multicast_ptr, s.rank, s.world,
                                       s.tensor.numel(), 1.0, self._epoch(), self._symm.COLL_CTAS)
        else:
            dist.all_reduce(b.view, group=self.group)
        return b.view.to(torch.bfloat16) if bf16 else b.view


def shard_rows(w: torch.Tensor, H: int, N: int, rank: int, world: int) -> torch.Tensor:
    """[H*N, D] -> this rank's [H*N/world, D] (neurons [rank*N/world, (rank+1)*N/world) of every head)."""
    Nl = N // world
    return w.view(H, N, -1)[:, rank * Nl:(rank + 1) * Nl].reshape(H * Nl, -1).contiguous()


def unshard_rows(parts, H: int, N: int) -> torch.Tensor:
    world = len(parts)
    Nl = N // world
    return torch.cat([p.view(H, Nl, -1) for p in parts], dim=1).reshape(H * N, -1)


class NeuronTP:
    def __init__(self, model: BDH, lr=1e-3, weight_decay=0.1, beta1=0.9, beta2=0.999, eps=1e-5, fused=True,
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

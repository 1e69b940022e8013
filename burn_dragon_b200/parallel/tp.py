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
stores every tile through the peer mapping of the rank that owns the tile's rows (EPI_F_PEER_RS),
and a gather kernel adds up each owner's slots and broadcasts the finished blocks (`multimem.st`),
as bf16 where the consumer is bf16. `fused="mc_red"` instead adds tiles into every replica at once
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
from ..utils import profiling as prof


class _Buf:
    """One reduction in flight: `view` is the fp32 [rows, cols] tensor handed to the GEMM as out0 (the
    local partial-sum buffer, or - reduce-scatter mode - only the carrier of the leading dimension),
    `kw` are the extra GEMM arguments of the mode (multicast address or peer pointers)."""

    def __init__(self, mode, view, sym, kw, rows, cols, block_rows=0):
        self.mode, self.view, self.sym, self.kw = mode, view, sym, kw
        self.rows, self.cols, self.block_rows = rows, cols, block_rows
        self.out = {}       # dtype -> symmetric output buffer of the gather (reduce-scatter mode)


class TPComm:
    """Reduction of [rows, D] fp32 partial sums across the TP group. Modes:

    rs         the producing GEMM is also the reduce-scatter: its epilogue stores each tile through
               the peer mapping of the rank that owns the tile's rows, into the slot this rank has
               in the owner's buffer, tile by tile while the GEMM runs. A gather kernel then adds up
               each owner's slots and sends the finished block to all ranks, as bf16 when the
               consumer wants bf16. Per GPU this moves (w-1)/w of the tensor in fp32 and (w-1)/w of
               it in the output type, with no atomics, no zero-fill and a fixed summation order.
               Needs a single producing launch per reduction; buffers that several launches add
               into (`launches > 1`) use `allreduce`.
    mc_red     the epilogue adds each tile into every rank's replica with one `multimem.red`
               through the switch. Every GPU receives w copies of the tensor: only sensible for w = 2.
    allreduce  partial sums are accumulated locally and reduced by the all-reduce kernel
               (`multimem.ld_reduce` + `multimem.st`, or peer loads and stores).
    nccl       partial sums are accumulated locally and reduced by NCCL (the baseline).
    """

    def __init__(self, device, group=None, fused=True):
        self.device, self.group = device, group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        mode = fused if isinstance(fused, str) else ("rs" if fused else "nccl")
        wanted = mode != "nccl"
        if not (device.type == "cuda" and native.available()):
            mode = "nccl"
        self.multicast = False
        self._bufs: Dict = {}
        self._flags = None
        self.fallback_reason = None
        if mode != "nccl":
            try:
                from . import symm
                self._symm = symm
                self._flags = symm._Flags.get(device, group if group is not None else dist.group.WORLD)
            except Exception as e:  # noqa: BLE001
                self.fallback_reason = repr(e)
                mode = "nccl"
        if wanted:
            # the mode is a collective decision: either every rank reduces inside its GEMM epilogues or none does
            from . import dist_utils
            if not dist_utils.all_agree(mode != "nccl", group, device if device.type == "cuda" else None):
                self.fallback_reason = self.fallback_reason or "a peer rank could not set up symmetric memory"
                mode = "nccl"
                if self.rank == 0 and device.type == "cuda":
                    print(f"TPComm: fused reductions unavailable, using NCCL ({self.fallback_reason})", flush=True)
        self.mode = mode
        self.fused = mode != "nccl"
        self.flags = G.F_OUT_F32 | G.F_ACCUM

    def _epoch(self) -> int:
        self._flags["epoch"] += 1
        return self._flags["epoch"]

    def _barrier(self, anchor):
        native.ops.rank_barrier(anchor, self._flags["buf"].ptrs, self.rank, self.world, self._epoch())

    def _make(self, rows, cols, launches) -> _Buf:
        n = rows * cols
        mode = self.mode
        if mode == "rs" and launches > 1:
            mode = "allreduce"
        if mode == "nccl":
            return _Buf(mode, torch.zeros(rows, cols, device=self.device), None, {}, rows, cols)
        # owner blocks of whole rows, an even number of them, so that a block is a multiple of 8 floats
        block_rows = -(-rows // self.world)
        block_rows += block_rows % 2
        total = block_rows * cols * self.world
        total += (-total) % (8 * self.world)
        sym = self._symm.SymmetricBuffer(total, torch.float32, self.device, self.group)
        sym.tensor.zero_()
        sym.barrier()
        if sym.multicast_ptr:
            self.multicast = True
        if mode == "mc_red" and not sym.multicast_ptr:
            mode = "allreduce"
        kw = {}
        if mode == "mc_red":
            kw = dict(mc_out=sym.multicast_ptr)
        elif mode == "rs":
            kw = dict(peer_ptrs=sym.ptrs, peer_rows=block_rows, peer_rank=self.rank)
        return _Buf(mode, sym.tensor[:n].view(rows, cols), sym, kw, rows, cols, block_rows)

    def begin(self, key: str, rows: int, cols: int, launches: int = 1) -> _Buf:
        k = (key, rows, cols, launches > 1)
        b = self._bufs.get(k)
        if b is None:
            b = self._bufs[k] = self._make(rows, cols, launches)
        if b.mode == "rs":
            # nothing to prepare: every slot is overwritten, and the previous gather's closing barrier
            # has already ordered this step's stores after the owners' reads
            self.flags = G.F_OUT_F32 | G.F_PEER_RS
        elif b.mode == "mc_red":
            b.view.zero_()
            self._barrier(b.view)          # every replica is zero before anybody's tiles arrive
            self.flags = G.F_OUT_F32 | G.F_MC_RED
        else:
            b.view.zero_()
            self.flags = G.F_OUT_F32 | G.F_ACCUM
        return b

    def end(self, b: _Buf, bf16: bool = False) -> torch.Tensor:
        """The reduced tensor: fp32 (a view of a reduction buffer, valid until the next `begin` with
        the same key and shape) or, with `bf16`, a fresh bf16 tensor."""
        with prof.phase("comm.tp_reduce"):       # the half of the reduction that is a launch of its own
            return self._end(b, bf16)

    def _end(self, b: _Buf, bf16: bool) -> torch.Tensor:
        if b.mode == "rs":
            dt = torch.bfloat16 if bf16 else torch.float32
            o = b.out.get(dt)
            if o is None:
                o = b.out[dt] = self._symm.SymmetricBuffer(b.sym.tensor.numel(), dt, self.device, self.group)
                o.barrier()
            s = b.sym
            native.ops.gather_blocks(s.tensor, s.ptrs, self._flags["buf"].ptrs, o.ptrs, o.multicast_ptr, bf16,
                                     s.rank, s.world, b.block_rows * b.cols, self._epoch(), self._symm.COLL_CTAS)
            res = o.tensor[:b.rows * b.cols].view(b.rows, b.cols)
            # the gather buffer is reused by the next reduction with this key: hand out a copy
            return res.clone() if bf16 else res
        if b.mode == "mc_red":
            self._barrier(b.view)          # every rank's tiles have landed in every replica
        elif b.mode == "allreduce":
            s = b.sym
            native.ops.allreduce_scale(s.tensor, s.ptrs, self._flags["buf"].ptrs, s.multicast_ptr, s.rank, s.world,
                                       s.tensor.numel(), 1.0, self._epoch(), self._symm.COLL_CTAS)
        else:
            dist.all_reduce(b.view, group=self.group)
        return b.view.to(torch.bfloat16) if bf16 else b.view


class _CopyToShards(torch.autograd.Function):
    """Replicated tensor entering a neuron-sharded product: identity forward, sum of the ranks'
    partial gradients backward."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        with prof.phase("comm.tp_reduce"):
            dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromShards(torch.autograd.Function):
    """Partial sums over the neuron shards: summed forward, identity backward."""

    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous().clone()
        with prof.phase("comm.tp_reduce"):
            dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class TorchTP:
    """The two collectives of neuron sharding for the torch path of the model (any device, any
    backend): what the kernel path fuses into GEMM epilogues, stated with `all_reduce`."""

    def __init__(self, group=None):
        self.group = group

    def copy(self, x):
        return _CopyToShards.apply(x, self.group)

    def reduce(self, x):
        return _ReduceFromShards.apply(x, self.group)


def shard_rows(w: torch.Tensor, H: int, N: int, rank: int, world: int) -> torch.Tensor:
    """[H*N, D] -> this rank's [H*N/world, D] (neurons [rank*N/world, (rank+1)*N/world) of every head)."""
    Nl = N // world
    return w.view(H, N, -1)[:, rank * Nl:(rank + 1) * Nl].reshape(H * Nl, -1).contiguous()


def unshard_rows(parts, H: int, N: int) -> torch.Tensor:
    world = len(parts)
    Nl = N // world
    return torch.cat([p.view(H, Nl, -1) for p in parts], dim=1).reshape(H * N, -1)


class _TPOptimizerFacade:
    """The shard's optimizer as the trainer and the checkpoint code see it: steps go to the local
    FlatAdamW, state goes in and out in the unsharded layout (one full-size tensor per parameter,
    the same record a single-device run writes), so a run can resume under another group size."""

    def __init__(self, owner: "NeuronTP"):
        self.owner = owner
        self.inner = owner.opt

    def __getattr__(self, name):
        return getattr(self.inner, name)

    def _full(self, buf) -> Dict[str, torch.Tensor]:
        o, f = self.owner, self.inner.flat
        c = o.full.config
        out = {}
        for i, n in enumerate(f.names):
            local = f.view(buf, i).detach().contiguous()
            if n in ("encoder", "encoder_v", "decoder"):
                parts = [torch.empty_like(local) for _ in range(o.world)]
                dist.all_gather(parts, local, group=o.group)
                out[n] = unshard_rows(parts, c.n_head, c.latent_per_head).cpu()
            else:
                out[n] = local.cpu().clone()
        return out

    def logical_state_dict(self) -> Dict:
        """Collective: every rank of the group calls it."""
        return dict(step=self.inner.step_count, m=self._full(self.inner.m), v=self._full(self.inner.v))

    def load_logical_state_dict(self, sd: Dict) -> None:
        o, f = self.owner, self.inner.flat
        c = o.full.config
        for buf, key in ((self.inner.m, "m"), (self.inner.v, "v")):
            for i, n in enumerate(f.names):
                t = sd[key][n]
                if n in ("encoder", "encoder_v", "decoder"):
                    t = shard_rows(t, c.n_head, c.latent_per_head, o.rank, o.world)
                f.view(buf, i).copy_(t.to(buf.device))
        self.inner.step_count = int(sd["step"])


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
        # the torch path of the shard (CPU ranks, shapes the kernels do not take): same sharding, with
        # this rank's slice of the rotary frequencies and all_reduce where the partial sums meet
        self.shard._tp = TorchTP(group)
        if c.rotary_embedding in ("rope", "pope"):
            self.shard.freqs.data = full_freqs[self.rank * Nl:(self.rank + 1) * Nl].clone()
        self.opt = FlatAdamW(self.shard, lr, weight_decay, beta1, beta2, eps, shadow_bf16=dev.type == "cuda")
        self.optimizer = _TPOptimizerFacade(self)
        self.eval_model = self.shard        # evaluating the shard under its hooks gives the full model's loss
        self.fast_train = False             # set by the trainer: train on the row-normalised forward
        self.grad_clip = None               # set by the trainer: clip the global norm of the gradient
        self.last_grad_norm = None
        self.lr = lr
        self._replicated = [self.shard.embed.weight, self.shard.lm_head]

    def train_step(self, tokens, targets, lr: Optional[float] = None, micro=(0, 1)) -> torch.Tensor:
        """`micro = (i, n)`: micro-batch i of n of an accumulated step (one update after the last one)."""
        i, n_micro = micro
        if i == 0:
            self.opt.zero_grad()
        loss = self.shard.forward_fast(tokens, targets) if self.fast_train else self.shard(tokens, targets)
        loss.backward()
        if i + 1 < n_micro:
            return loss.detach()
        # the replicated tensors see the same gradient on every rank up to summation order; average
        # them so the replicas cannot drift apart
        with prof.phase("comm.replicated_grads"):
            for p in self._replicated:
                dist.all_reduce(p.grad, group=self.group)
                p.grad.div_(self.world)
        scale = 1.0 / n_micro
        if self.grad_clip:
            # global norm: the sharded tensors partition their gradients over the ranks, the replicated
            # ones are whole (and equal) on every rank
            rep = {id(p) for p in self._replicated}
            sq_shard = sum((p.grad.float() ** 2).sum() for p in self.shard.parameters() if id(p) not in rep and p.grad is not None)
            sq_rep = sum((p.grad.float() ** 2).sum() for p in self._replicated)
            with prof.phase("comm.grad_norm"):
                dist.all_reduce(sq_shard, group=self.group)
            self.last_grad_norm = (sq_shard + sq_rep).sqrt() * scale
            scale = scale * float(torch.clamp(self.grad_clip / (self.last_grad_norm + 1e-6), max=1.0))
        self.opt.step(lr=self.lr if lr is None else lr, grad_scale=scale)
        return loss.detach()

    @torch.no_grad()
    def sync_from_model(self) -> None:
        """Re-shard after the full model's weights were replaced (checkpoint load)."""
        c = self.full.config
        self.shard.embed.weight.copy_(self.full.embed.weight)
        self.shard.lm_head.copy_(self.full.lm_head)
        for name in ("encoder", "encoder_v", "decoder"):
            getattr(self.shard, name).copy_(shard_rows(getattr(self.full, name).data, c.n_head, c.latent_per_head,
                                                       self.rank, self.world))
        self.opt.flat.refresh_shadow()

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

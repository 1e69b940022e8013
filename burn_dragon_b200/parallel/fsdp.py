"""Fully sharded data parallelism for the BDH stack.

`ShardedState` (the fused path, `FSDP(fused=True)` on GPUs): every rank keeps 1/world of the rows of the
three [H*N, D] weights - fp32 master, both Adam moments AND the fp32 gradient - plus one bf16 working copy
of all weights in symmetric memory, which is what the GEMMs read. No rank holds a full fp32 weight or a
full fp32 gradient:

  * every weight-gradient GEMM of every layer adds its tiles straight into the owner's gradient slice from
    its epilogue (`red.add` over NVLink through the owner's peer mapping: GEMM flags PEER_RS | ATOMIC), so the
    reduce-scatter is spread over the whole backward pass and overlaps it tile by tile;
  * one kernel per step (`csrc/collectives.cu: shard_adamw_ag`) waits for all ranks, applies AdamW to the
    local slices, stores the refreshed bf16 rows into every rank's working copy (the all-gather) and clears
    the gradient slice;
  * the two small replicated tensors (embedding, LM head: vocab x D) are all-reduced and updated on every rank.

The NCCL-only baseline (`fused=False`, and every CPU run) keeps full local gradients and does
`reduce_scatter_tensor` + AdamW on the shard + `all_gather`.

Persistent bytes per parameter and rank: 2 (bf16 working copy) + 16 / world, against 2 + 16 on one GPU.

The reference is single-device (src/bin/train.rs:395); nothing here has a counterpart there.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..engine.optim import FlatParams
from ..ops import native
from ..utils import profiling as prof


class _ShardedOptimizerFacade:
    """What checkpointing needs from an optimizer: logical (unsharded) state in, logical state out."""

    def __init__(self, owner):
        self.owner = owner

    @property
    def step_count(self):
        return self.owner.step_count

    def logical_state_dict(self) -> Dict:
        """Collective: every rank calls it. One full-size tensor per parameter and moment - the record a
        single-device run writes - so the run can resume under any strategy or group size."""
        o, f = self.owner, self.owner.flat
        out = dict(step=o.step_count, m={}, v={})
        for key, shard in (("m", o.m), ("v", o.v)):
            full = o._gather(shard)
            for i, n in enumerate(f.names):
                out[key][n] = f.view(full, i).detach().cpu().clone()
        return out

    def load_logical_state_dict(self, sd: Dict) -> None:
        o, f = self.owner, self.owner.flat
        o.step_count = int(sd["step"])
        if o.sharded is not None:
            o.sharded.step_count = o.step_count      # the fused kernel's bias correction counts steps itself
        for key, shard in (("m", o.m), ("v", o.v)):
            full = torch.zeros(o.numel, dtype=torch.float32, device=shard.device)
            for i, n in enumerate(f.names):
                f.view(full, i).copy_(sd[key][n].to(shard.device))
            shard.copy_(full[o.lo:o.hi])


class _ShardedStateFacade:
    """Checkpoint interface of the fully sharded state (logical tensors in, logical tensors out)."""

    def __init__(self, owner):
        self.owner = owner

    @property
    def step_count(self):
        return self.owner.step_count

    def logical_state_dict(self) -> Dict:
        mom = self.owner.state.gather_moments()
        return dict(step=self.owner.step_count, m=mom["m"], v=mom["v"])

    def load_logical_state_dict(self, sd: Dict) -> None:
        self.owner.step_count = self.owner.state.step_count = int(sd["step"])
        self.owner.state.load_moments(sd)


SHARDED = ("encoder", "encoder_v", "decoder")      # [H*N, D] each: sharded by rows
REPLICATED = ("embed.weight", "lm_head")            # vocab x D each: kept whole on every rank


class GradSink:
    """Destination of the sharded parameters' weight gradients during the fused backward pass
    (`ops.fused_bdh` asks it where each weight-gradient GEMM writes)."""

    def __init__(self, rows: int, cols: int, world: int, rank: int):
        self.rows, self.cols, self.world, self.rank = rows, cols, world, rank
        self.rows_per_rank = rows // world
        self.acc = None          # symmetric fp32 [3, rows_per_rank, cols]: this rank's gradient slices
        self.ptrs = None         # per parameter: every rank's address of that parameter's slice
        self.local_full = None   # emulated path: full local gradients, reduce-scattered at the end of the step

    # data parallelism with replicated optimizer state sets this: the layers accumulate locally (as without a
    # sink) and only the LAST weight-gradient launch of a backward pass - layer 0, whose epilogue first takes up
    # the local sum - sends tiles to the owners: one gradient's worth of NVLink traffic per step instead of one
    # per layer. Fully sharded data parallelism keeps no local full-size gradient, so every launch sends.
    last_layer_only = False

    def launch(self, name: str, base_flags: int, final: bool = True, local=None):
        """-> (out0, flags, extra keyword arguments) of the GEMM that adds into `name`'s gradient. `final`:
        this is the last layer of the backward pass; `local`: the local fp32 accumulation of the layers before."""
        from ..ops import gemm as G
        if self.last_layer_only and self.ptrs is not None:
            if not final:
                return local, base_flags, {}
            return local, (base_flags & ~G.F_ACCUM) | G.F_OUT_F32 | G.F_ATOMIC | G.F_PEER_RS | G.F_ACCUM, dict(
                peer_ptrs=self.ptrs[name], peer_rows=self.rows_per_rank, peer_rank=self.rank)
        if self.ptrs is not None:
            # out0 = this rank's own slice: it gives the kernel the row pitch of every owner's block
            return self.acc[SHARDED.index(name)], (base_flags & ~G.F_ACCUM) | G.F_OUT_F32 | G.F_ATOMIC | G.F_PEER_RS, dict(
                peer_ptrs=self.ptrs[name], peer_rows=self.rows_per_rank, peer_rank=self.rank)
        return self.local_full[name], base_flags, {}


class ShardedState:
    """Row-sharded fp32 state (master, moments, gradient) of the three big weights, the bf16 working copy of
    everything, and the replicated small tensors."""

    def __init__(self, model, group, lr, weight_decay, beta1, beta2, eps, emulate: bool = False):
        from ..ops import native
        self.model, self.group = model, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.lr, self.weight_decay, self.beta1, self.beta2, self.eps = lr, weight_decay, beta1, beta2, eps
        self.emulate = emulate
        params = dict(model.named_parameters())
        if set(params) != set(SHARDED) | set(REPLICATED):
            raise ValueError("fully sharded mode knows the BDH parameter set only")
        big = [params[n] for n in SHARDED]
        R, D = big[0].shape
        if any(tuple(p.shape) != (R, D) for p in big) or R % (128 * self.world):
            raise ValueError(f"cannot shard [{R}, {D}] weights by rows of 128 over {self.world} ranks")
        dev = big[0].device
        self.R, self.D, self.rpr = R, D, R // self.world
        for p in params.values():
            dist.broadcast(p.data, src=0, group=group)
        # ---- bf16 working copy of every weight: [embed | lm_head | pad | encoder | encoder_v | decoder] ----
        small_n = sum(params[n].numel() for n in REPLICATED)
        self.small_n = small_n
        self.big_off = (small_n + 63) // 64 * 64
        total = self.big_off + 3 * R * D
        if emulate:
            self.shadow_buf = None
            self.shadow = torch.zeros(total, dtype=torch.bfloat16, device=dev)
        else:
            from . import symm
            self.shadow_buf = symm.SymmetricBuffer(total, torch.bfloat16, dev, group)
            self.shadow = self.shadow_buf.tensor
        # ---- replicated small tensors: fp32 master, gradient, moments (whole) ----
        self.small_master = torch.cat([params[n].data.reshape(-1).float() for n in REPLICATED])
        self.small_grad = torch.zeros_like(self.small_master)
        self.small_m, self.small_v = torch.zeros_like(self.small_master), torch.zeros_like(self.small_master)
        # ---- sharded rows: fp32 master slice and moments, [3, rpr, D] ----
        lo, hi = self.rank * self.rpr, (self.rank + 1) * self.rpr
        self.master = torch.stack([p.data[lo:hi].float() for p in big]).contiguous()
        self.m, self.v = torch.zeros_like(self.master), torch.zeros_like(self.master)
        self.sink = GradSink(R, D, self.world, self.rank)
        if emulate:
            self.acc = torch.zeros_like(self.master)
            self.sink.local_full = {n: torch.zeros(R, D, dtype=torch.float32, device=dev) for n in SHARDED}
        else:
            from . import symm
            self.acc_buf = symm.SymmetricBuffer(3 * self.rpr * D, torch.float32, dev, group)
            self.acc = self.acc_buf.tensor.view(3, self.rpr, D)
            self.acc.zero_()
            self.sink.acc = self.acc
            self.sink.ptrs = {n: [p + 4 * i * self.rpr * D for p in self.acc_buf.ptrs] for i, n in enumerate(SHARDED)}
            self.flags = symm._Flags.get(dev, self.acc_buf.group)
        # ---- the module's parameters: the small ones are fp32 views of the replicated master, the big ones
        # bf16 views of the working copy (no rank holds them in fp32) ----
        self.shadow[:small_n].copy_(self.small_master)
        off = 0
        self.views = {}
        for n in REPLICATED:
            p = params[n]
            k = p.numel()
            p.data = self.small_master[off:off + k].view_as(p)
            p.grad = self.small_grad[off:off + k].view_as(p)
            self.views[n] = self.shadow[off:off + k].view(p.shape)
            off += k
        for i, n in enumerate(SHARDED):
            p = params[n]
            view = self.shadow[self.big_off + i * R * D:self.big_off + (i + 1) * R * D].view(R, D)
            view.copy_(p.data)
            p.data = view
            p.grad = None
            self.views[n] = view
        model._bf16_shadow = dict(embed=self.views["embed.weight"], encoder=self.views["encoder"],
                                  encoder_v=self.views["encoder_v"], decoder=self.views["decoder"],
                                  lm_head=self.views["lm_head"])
        model._grad_sink = self.sink
        self.step_count = 0
        if not emulate:
            torch.cuda.synchronize()
        dist.barrier(group=group)

    # ---- bytes -------------------------------------------------------------------------------------
    def persistent_bytes(self) -> dict:
        """What this rank holds between steps, by kind."""
        b = lambda t: t.numel() * t.element_size()
        return dict(working_copy_bf16=b(self.shadow), master_fp32=b(self.master) + b(self.small_master),
                    moments_fp32=2 * (b(self.m) + b(self.small_m)), gradient_fp32=b(self.acc) + b(self.small_grad),
                    unsharded_fp32_equivalent=16 * (3 * self.R * self.D + self.small_n))

    # ---- step ----------------------------------------------------------------------------------------
    def zero_small_grad(self) -> None:
        self.small_grad.zero_()

    @torch.no_grad()
    def step(self, lr: float, n_micro: int, grad_clip=None):
        """Reduce what is left to reduce, update, refresh every rank's working copy. Returns the gradient
        norm when clipping (else None)."""
        from ..ops import native
        self.step_count += 1
        world = self.world
        with prof.phase("comm.replicated_grads"):
            dist.all_reduce(self.small_grad, group=self.group)
        if self.emulate:
            # the emulated sink collected full local gradients: reduce-scatter them now
            for i, n in enumerate(SHARDED):
                full = self.sink.local_full[n]
                dist.all_reduce(full, group=self.group)
                self.acc[i].add_(full[self.rank * self.rpr:(self.rank + 1) * self.rpr])
                full.zero_()
        scale = 1.0 / (world * n_micro)
        norm = None
        if grad_clip:
            if not self.emulate:
                # every rank's additions have to be in before the slice is read
                self.flags["epoch"] += 1
                native.ops.rank_barrier(self.acc, self.flags["buf"].ptrs, self.rank, world, self.flags["epoch"])
            sq = (self.acc.float() ** 2).sum()
            with prof.phase("comm.grad_norm"):
                dist.all_reduce(sq, group=self.group)               # the slices partition the gradient
            norm = (sq + (self.small_grad ** 2).sum()).sqrt() * scale
            scale = scale * float(torch.clamp(grad_clip / (norm + 1e-6), max=1.0))
        # replicated tensors: plain AdamW on every rank
        self._adamw(self.small_master, self.small_grad, self.small_m, self.small_v, self.shadow[:self.small_n], lr, scale)
        if self.emulate:
            flat_acc = self.acc.view(-1)
            self._adamw(self.master.view(-1), flat_acc, self.m.view(-1), self.v.view(-1), None, lr, scale)
            flat_acc.zero_()
            parts = [torch.empty_like(self.master) for _ in range(world)]
            dist.all_gather(parts, self.master, group=self.group)
            for i, n in enumerate(SHARDED):
                self.views[n].copy_(torch.cat([p[i] for p in parts]))
            return norm
        n_loc = self.rpr * self.D
        seg_lo = [0, n_loc, 2 * n_loc, 3 * n_loc]
        seg_dst = [self.big_off + i * self.R * self.D + self.rank * n_loc for i in range(3)]
        self.flags["epoch"] += 1
        with prof.phase("comm.shard_adamw_ag"):      # one kernel: barrier, AdamW on the slices, all-gather by stores
            native.ops.shard_adamw_ag(self.flags["buf"].ptrs, self.shadow_buf.ptrs, self.rank, world, self.acc,
                                      self.master, self.m, self.v, seg_lo, seg_dst, float(lr), self.beta1, self.beta2,
                                      self.eps, self.weight_decay, self.step_count, float(scale), self.flags["epoch"],
                                      _coll_ctas())
        return norm

    def _adamw(self, master, grad, m, v, shadow, lr, scale) -> None:
        from ..ops import native
        if master.is_cuda and native.available() and shadow is not None:
            native.ops.adamw(master, grad, m, v, shadow, lr, self.beta1, self.beta2, self.eps, self.weight_decay,
                             self.step_count, scale)
            return
        g = grad * scale
        m.mul_(self.beta1).add_(g, alpha=1 - self.beta1)
        v.mul_(self.beta2).addcmul_(g, g, value=1 - self.beta2)
        bc1, bc2 = 1 - self.beta1 ** self.step_count, 1 - self.beta2 ** self.step_count
        master.mul_(1 - lr * self.weight_decay)
        master.addcdiv_(m / bc1, (v / bc2).sqrt_().add_(self.eps), value=-lr)
        if shadow is not None:
            shadow.copy_(master)

    # ---- logical (unsharded) views: collective, every rank calls them -------------------------------------------
    def _gather_rows(self, local: torch.Tensor) -> Dict[str, torch.Tensor]:
        parts = [torch.empty_like(local) for _ in range(self.world)]
        dist.all_gather(parts, local.contiguous(), group=self.group)
        return {n: torch.cat([p[i] for p in parts]).cpu() for i, n in enumerate(SHARDED)}

    def _small(self, flat: torch.Tensor) -> Dict[str, torch.Tensor]:
        out, off = {}, 0
        for n in REPLICATED:
            shape = self.views[n].shape
            k = self.views[n].numel()
            out[n] = flat[off:off + k].view(shape).detach().cpu().clone()
            off += k
        return out

    def gather_weights(self) -> Dict[str, torch.Tensor]:
        return {**self._small(self.small_master), **self._gather_rows(self.master)}

    def gather_moments(self) -> Dict[str, Dict[str, torch.Tensor]]:
        return dict(m={**self._small(self.small_m), **self._gather_rows(self.m)},
                    v={**self._small(self.small_v), **self._gather_rows(self.v)})

    @torch.no_grad()
    def load_weights(self, sd: Dict[str, torch.Tensor]) -> None:
        """fp32 weights in the unsharded layout -> this rank's slices and the working copy."""
        dev = self.master.device
        lo, hi = self.rank * self.rpr, (self.rank + 1) * self.rpr
        off = 0
        for n in REPLICATED:
            k = self.views[n].numel()
            self.small_master[off:off + k].copy_(sd[n].reshape(-1).to(dev))
            off += k
        self.shadow[:self.small_n].copy_(self.small_master)
        for i, n in enumerate(SHARDED):
            self.master[i].copy_(sd[n][lo:hi].to(dev))
            self.views[n].copy_(sd[n].to(dev))

    @torch.no_grad()
    def load_moments(self, sd: Dict) -> None:
        dev = self.master.device
        lo, hi = self.rank * self.rpr, (self.rank + 1) * self.rpr
        for key, small, big in (("m", self.small_m, self.m), ("v", self.small_v, self.v)):
            off = 0
            for n in REPLICATED:
                k = self.views[n].numel()
                small[off:off + k].copy_(sd[key][n].reshape(-1).to(dev))
                off += k
            for i, n in enumerate(SHARDED):
                big[i].copy_(sd[key][n][lo:hi].to(dev))


def _coll_ctas() -> int:
    from . import symm
    return symm.COLL_CTAS


class FSDP:
    def __init__(self, model, lr=1e-3, weight_decay=0.1, beta1=0.9, beta2=0.999, eps=1e-5, fused: bool = True,
                 group=None):
        from ..ops import emulate
        self.model, self.group = model, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.lr, self.weight_decay, self.beta1, self.beta2, self.eps = lr, weight_decay, beta1, beta2, eps
        dev = next(model.parameters()).device
        self.step_count = 0
        self.fast_train = False             # set by the trainer: train on the row-normalised forward
        self.grad_clip = None               # set by the trainer: clip the global norm of the averaged gradient
        self.last_grad_norm = None
        self.fallback_reason = None
        self.state = None
        want_fused = bool(fused)
        # the fused path: fully sharded state with the reduce-scatter done by the weight-gradient epilogues; on CPU
        # ranks the same host logic runs over the emulated kernel path (gradients reduce-scattered by the library)
        can_try = want_fused and ((dev.type == "cuda" and native.available()) or (dev.type == "cpu" and emulate.active()))
        if can_try:
            try:
                self.state = ShardedState(model, group, lr, weight_decay, beta1, beta2, eps, emulate=dev.type != "cuda")
            except Exception as e:  # noqa: BLE001 - recorded; the NCCL path is used instead
                self.fallback_reason = repr(e)
        if want_fused and self.world > 1:
            # the mode is a collective decision: either every rank runs the in-kernel collectives or none does
            from . import dist_utils
            ok = dist_utils.all_agree(self.state is not None, group, dev)
            if not ok:
                self.fallback_reason = self.fallback_reason or "a peer rank could not set up the sharded state"
                if self.state is not None:
                    raise RuntimeError("FSDP: this rank built the sharded state but a peer could not; "
                                       f"restart with fused=False ({self.fallback_reason})")
                if self.rank == 0 and dev.type == "cuda":
                    print(f"FSDP: fused NVLink collectives unavailable, using NCCL ({self.fallback_reason})", flush=True)
        self.fused = self.state is not None
        if self.fused:
            self.optimizer = _ShardedStateFacade(self)
            return
        self.flat = FlatParams(model, shadow_bf16=True, align=64)
        dist.broadcast(self.flat.master, src=0, group=group)
        n = self.flat.numel
        self.pad = (-n) % (4 * self.world)
        self.numel = n + self.pad
        per = self.numel // self.world
        self.lo, self.hi = per * self.rank, (self.numel if self.rank == self.world - 1 else per * (self.rank + 1))
        self.sharded = None
        if not self.fused:
            full = torch.zeros(self.numel, dtype=torch.float32, device=dev)
            full[:n].copy_(self.flat.master)
            self.master = full[self.lo:self.hi].clone()
            self.m, self.v = torch.zeros_like(self.master), torch.zeros_like(self.master)
            self._grad_pad = torch.zeros(self.numel, dtype=torch.float32, device=dev)
            self._shard_grad = torch.zeros(self.hi - self.lo, dtype=torch.float32, device=dev)
            self.flat.refresh_shadow()
        self.optimizer = _ShardedOptimizerFacade(self)

    # ---- step -----------------------------------------------------------------------------------
    def train_step(self, tokens, targets, lr: Optional[float] = None, micro=(0, 1)) -> torch.Tensor:
        """`micro = (i, n)`: micro-batch i of n of an accumulated step. Gradients add up locally in the
        flat buffer; the reduction and the update happen once, after the last one, scaled by 1/n."""
        i, n_micro = micro
        if self.state is not None:
            if i == 0:
                self.state.zero_small_grad()
            loss = self.model.forward_fast(tokens, targets) if self.fast_train else self.model(tokens, targets)
            loss.backward()           # the big weights' gradients leave through the sink during this call
            if i + 1 < n_micro:
                return loss.detach()
            self.step_count += 1
            self.last_grad_norm = self.state.step(self.lr if lr is None else lr, n_micro, self.grad_clip)
            return loss.detach()
        if i == 0:
            self.flat.zero_grad()
        loss = self.model.forward_fast(tokens, targets) if self.fast_train else self.model(tokens, targets)
        loss.backward()
        if i + 1 < n_micro:
            return loss.detach()
        self.step_count += 1
        lr = self.lr if lr is None else lr
        # NCCL baseline: reduce-scatter, local AdamW on the shard, all-gather of fp32 then cast
        n = self.flat.numel
        self._grad_pad[:n].copy_(self.flat.grad)
        with prof.phase("comm.reduce_scatter"):
            if (self.numel % self.world) == 0 and dist.get_backend(self.group) == "nccl":
                dist.reduce_scatter_tensor(self._shard_grad, self._grad_pad, group=self.group)
            else:
                dist.all_reduce(self._grad_pad, group=self.group)
                self._shard_grad.copy_(self._grad_pad[self.lo:self.hi])
        g = self._shard_grad / (self.world * n_micro)
        if self.grad_clip:
            sq = (g * g).sum()
            with prof.phase("comm.grad_norm"):
                dist.all_reduce(sq, group=self.group)          # the shards partition the gradient
            self.last_grad_norm = sq.sqrt()
            g = g * torch.clamp(self.grad_clip / (self.last_grad_norm + 1e-6), max=1.0)
        self.m.mul_(self.beta1).add_(g, alpha=1 - self.beta1)
        self.v.mul_(self.beta2).addcmul_(g, g, value=1 - self.beta2)
        bc1, bc2 = 1 - self.beta1 ** self.step_count, 1 - self.beta2 ** self.step_count
        self.master.mul_(1 - lr * self.weight_decay)
        self.master.addcdiv_(self.m / bc1, (self.v / bc2).sqrt_().add_(self.eps), value=-lr)
        with prof.phase("comm.all_gather"):
            full = self._gather(self.master)
        self.flat.master.copy_(full[:n])
        self.flat.refresh_shadow()
        return loss.detach()

    # ---- logical (unsharded) views --------------------------------------------------------------------
    def _gather(self, shard: torch.Tensor) -> torch.Tensor:
        # the padded length is a multiple of the world size, so every rank's slice has the same length
        parts = [torch.empty_like(shard) for _ in range(self.world)]
        dist.all_gather(parts, shard.contiguous(), group=self.group)
        return torch.cat(parts)

    def sync_params(self) -> None:
        """Bring the module's fp32 parameters up to date with the sharded master weights."""
        if self.state is not None:
            return                      # the module reads the bf16 working copy, which every step refreshes
        full = self._gather(self.master)
        self.flat.master.copy_(full[:self.flat.numel])

    @torch.no_grad()
    def sync_from_model(self) -> None:
        """Re-shard after the module's weights were replaced (checkpoint load): the parameters are
        views of the flat fp32 buffer, this rank's master slice and the bf16 copy follow it."""
        if self.state is not None:
            return                      # weights reach the sharded state through `load_weights`
        n = self.flat.numel
        full = torch.zeros(self.numel, dtype=torch.float32, device=self.flat.master.device)
        full[:n].copy_(self.flat.master)
        self.master.copy_(full[self.lo:self.hi])
        self.flat.refresh_shadow()

    def load_weights(self, sd: Dict[str, torch.Tensor]) -> bool:
        """Checkpoint load: fp32 weights in the unsharded layout. Returns False when the module's own
        `load_state_dict` should be used instead (the NCCL path keeps full fp32 parameters)."""
        if self.state is None:
            return False
        self.state.load_weights(sd)
        return True

    def gather_state_dict(self) -> Dict[str, torch.Tensor]:
        if self.state is not None:
            return self.state.gather_weights()
        self.sync_params()
        return {k: v.detach().cpu().clone() for k, v in self.model.state_dict().items()}

"""Sharded data parallelism (ZeRO / FSDP style) for the BDH stack.

Every rank computes full local gradients into a symmetric fp32 buffer. One kernel per step then
(`csrc/collectives.cu: rs_adamw_ag`) reduce-scatters the gradients over NVLink (peer loads or
multimem.ld_reduce), applies AdamW to the 1/world slice of fp32 master weights and moments this
rank owns, and writes the refreshed bf16 parameters into every rank's symmetric parameter buffer -
so gradients, master weights and both moments are sharded, and the only replicated thing is the
bf16 working copy the GEMMs read. The NCCL-only baseline (`fused=False`) does the same with
`reduce_scatter_tensor` + the local AdamW kernel + `all_gather_into_tensor`.

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


class FSDP:
    def __init__(self, model, lr=1e-3, weight_decay=0.1, beta1=0.9, beta2=0.999, eps=1e-5, fused: bool = True,
                 group=None):
        self.model, self.group = model, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.lr, self.weight_decay, self.beta1, self.beta2, self.eps = lr, weight_decay, beta1, beta2, eps
        self.flat = FlatParams(model, shadow_bf16=True, align=64)
        dist.broadcast(self.flat.master, src=0, group=group)
        self.step_count = 0
        n = self.flat.numel
        self.pad = (-n) % (4 * self.world)
        self.numel = n + self.pad
        per = self.numel // self.world
        self.lo, self.hi = per * self.rank, (self.numel if self.rank == self.world - 1 else per * (self.rank + 1))
        dev = self.flat.master.device
        self.fused = bool(fused and dev.type == "cuda" and native.available())
        self.sharded = None
        self.fallback_reason = None
        want_fused = bool(fused)
        if self.fused:
            try:
                from . import symm
                self.sharded = symm.ShardedAdamW(self.flat.master, group, lr, weight_decay, beta1, beta2, eps)
            except Exception as e:  # noqa: BLE001 - recorded; the NCCL path is used instead
                self.fallback_reason = repr(e)
        if want_fused and self.world > 1:
            # the mode is a collective decision: either every rank runs the in-kernel collectives or none does
            from . import dist_utils
            self.fused = dist_utils.all_agree(self.sharded is not None, group, dev)
            if not self.fused:
                self.fallback_reason = self.fallback_reason or "a peer rank could not set up symmetric memory"
                self.sharded = None
                if self.rank == 0 and dev.type == "cuda":
                    print(f"FSDP: fused NVLink collectives unavailable, using NCCL ({self.fallback_reason})", flush=True)
        if self.fused:
            # gradients and the bf16 working copy now live in symmetric memory
            self.flat.grad = self.sharded.grad[:n]
            self.flat.shadow = self.sharded.shadow[:n]
            self.flat.zero_grad()
            self.flat.register_shadow()
            self.master, self.m, self.v = self.sharded.master, self.sharded.m, self.sharded.v
        if not self.fused:
            full = torch.zeros(self.numel, dtype=torch.float32, device=dev)
            full[:n].copy_(self.flat.master)
            self.master = full[self.lo:self.hi].clone()
            self.m, self.v = torch.zeros_like(self.master), torch.zeros_like(self.master)
            self._grad_pad = torch.zeros(self.numel, dtype=torch.float32, device=dev)
            self._shard_grad = torch.zeros(self.hi - self.lo, dtype=torch.float32, device=dev)
            self.flat.refresh_shadow()
        self.optimizer = _ShardedOptimizerFacade(self)
        self.fast_train = False             # set by the trainer: train on the row-normalised forward
        self.grad_clip = None               # set by the trainer: clip the global norm of the averaged gradient
        self.last_grad_norm = None

    # ---- step -----------------------------------------------------------------------------------
    def train_step(self, tokens, targets, lr: Optional[float] = None, micro=(0, 1)) -> torch.Tensor:
        """`micro = (i, n)`: micro-batch i of n of an accumulated step. Gradients add up locally in the
        flat buffer; the reduction and the update happen once, after the last one, scaled by 1/n."""
        i, n_micro = micro
        if i == 0:
            self.flat.zero_grad()
        loss = self.model.forward_fast(tokens, targets) if self.fast_train else self.model(tokens, targets)
        loss.backward()
        if i + 1 < n_micro:
            return loss.detach()
        self.step_count += 1
        lr = self.lr if lr is None else lr
        clip = 1.0
        if self.fused:
            extra = 1.0
            if self.grad_clip:
                # the norm of the averaged gradient is needed BEFORE the fused kernel reduces it: sum the
                # gradients with one library all-reduce; the kernel then adds up world identical copies,
                # which the extra 1/world below takes out again
                with prof.phase("comm.grad_norm"):
                    dist.all_reduce(self.flat.grad, group=self.group)
                self.last_grad_norm = self.flat.grad.norm() / (self.world * n_micro)
                clip = float(torch.clamp(self.grad_clip / (self.last_grad_norm + 1e-6), max=1.0))
                extra = 1.0 / self.world
            with prof.phase("comm.rs_adamw_ag"):       # one kernel: reduce-scatter + AdamW + all-gather
                self.sharded.step(lr, grad_scale=clip * extra / n_micro)
            return loss.detach()
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
        full = self._gather(self.master)
        self.flat.master.copy_(full[:self.flat.numel])

    @torch.no_grad()
    def sync_from_model(self) -> None:
        """Re-shard after the module's weights were replaced (checkpoint load): the parameters are
        views of the flat fp32 buffer, this rank's master slice and the bf16 copy follow it."""
        n = self.flat.numel
        full = torch.zeros(self.numel, dtype=torch.float32, device=self.flat.master.device)
        full[:n].copy_(self.flat.master)
        self.master.copy_(full[self.lo:self.hi])
        self.flat.refresh_shadow()

    def gather_state_dict(self) -> Dict[str, torch.Tensor]:
        self.sync_params()
        return {k: v.detach().cpu().clone() for k, v in self.model.state_dict().items()}

"""Flat-buffer AdamW with an fp32 master copy and a bf16 working copy, and the LR schedules.

All parameters of a module are re-pointed at views of one contiguous fp32 buffer; gradients live
in a second flat fp32 buffer (so data-parallel reduction is a single collective over one pointer),
and one kernel launch updates master weights, both moments and the bf16 shadow the kernels read.
AdamW semantics are the decoupled form the reference trains with (src/bin/train.rs:259-264 sets
only the weight decay; betas 0.9 / 0.999 and eps 1e-5 are the defaults here).

Schedules restate the reference's resolution rules (src/bin/train.rs:421-506):
constant | cosine{min_lr,num_iters} | linear{final_lr,num_iters} | exponential{gamma} |
step{gamma,step_size} | noam{warmup_steps,model_size}; `initial_lr` defaults to the optimizer's
learning rate, `num_iters` to the total number of steps.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from ..ops import native


class FlatParams:
    """Owns flat master / grad (/ bf16 shadow) buffers and re-points a module's parameters at them."""

    def __init__(self, module: torch.nn.Module, shadow_bf16: bool = True, align: int = 64):
        self.module = module
        params = [(n, p) for n, p in module.named_parameters() if p.requires_grad]
        self.names = [n for n, _ in params]
        self.params = [p for _, p in params]
        dev = self.params[0].device
        self.offsets: List[int] = []
        total = 0
        for p in self.params:
            self.offsets.append(total)
            total += (p.numel() + align - 1) // align * align
        self.numel = total
        self.master = torch.zeros(total, dtype=torch.float32, device=dev)
        self.grad = torch.zeros(total, dtype=torch.float32, device=dev)
        self.shadow = torch.zeros(total, dtype=torch.bfloat16, device=dev) if shadow_bf16 else None
        for p, off in zip(self.params, self.offsets):
            view = self.master[off:off + p.numel()].view_as(p)
            view.copy_(p.data)
            p.data = view
            p.grad = self.grad[off:off + p.numel()].view_as(p)
        module._flat_params = self
        self.refresh_shadow()

    def view(self, buf: torch.Tensor, i: int) -> torch.Tensor:
        p = self.params[i]
        return buf[self.offsets[i]:self.offsets[i] + p.numel()].view_as(p)

    def refresh_shadow(self) -> None:
        if self.shadow is None:
            return
        self.shadow.copy_(self.master)
        self.register_shadow()

    def register_shadow(self) -> None:
        """Expose the bf16 copies to a model that knows how to use them (`_bf16_shadow`)."""
        if self.shadow is None:
            return
        by_name = {n: self.view(self.shadow, i) for i, n in enumerate(self.names)}
        if all(k in by_name for k in ("embed.weight", "encoder", "encoder_v", "decoder", "lm_head")):
            self.module._bf16_shadow = dict(embed=by_name["embed.weight"], encoder=by_name["encoder"],
                                            encoder_v=by_name["encoder_v"], decoder=by_name["decoder"],
                                            lm_head=by_name["lm_head"])

    def zero_grad(self) -> None:
        self.grad.zero_()
        for i, p in enumerate(self.params):
            if p.grad is None or p.grad.data_ptr() != self.view(self.grad, i).data_ptr():
                p.grad = self.view(self.grad, i)


class FlatAdamW:
    def __init__(self, module: torch.nn.Module, lr: float = 1e-3, weight_decay: float = 0.1, beta1: float = 0.9,
                 beta2: float = 0.999, eps: float = 1e-5, shadow_bf16: bool = True,
                 flat: Optional[FlatParams] = None):
        self.flat = flat if flat is not None else FlatParams(module, shadow_bf16)
        self.lr, self.weight_decay, self.beta1, self.beta2, self.eps = lr, weight_decay, beta1, beta2, eps
        self.m = torch.zeros_like(self.flat.master)
        self.v = torch.zeros_like(self.flat.master)
        self.step_count = 0

    def zero_grad(self) -> None:
        self.flat.zero_grad()

    @torch.no_grad()
    def step(self, lr: Optional[float] = None, grad_scale: float = 1.0) -> None:
        lr = self.lr if lr is None else lr
        self.step_count += 1
        f = self.flat
        if f.master.is_cuda and native.available():
            native.ops.adamw(f.master, f.grad, self.m, self.v, f.shadow, lr, self.beta1, self.beta2, self.eps,
                                self.weight_decay, self.step_count, grad_scale)
            return
        g = f.grad * grad_scale
        self.m.mul_(self.beta1).add_(g, alpha=1 - self.beta1)
        self.v.mul_(self.beta2).addcmul_(g, g, value=1 - self.beta2)
        bc1 = 1 - self.beta1 ** self.step_count
        bc2 = 1 - self.beta2 ** self.step_count
        f.master.mul_(1 - lr * self.weight_decay)
        f.master.addcdiv_(self.m / bc1, (self.v / bc2).sqrt_().add_(self.eps), value=-lr)
        if f.shadow is not None:
            f.shadow.copy_(f.master)

    def state_dict(self) -> Dict:
        return dict(m=self.m, v=self.v, step=self.step_count, lr=self.lr)

    def load_state_dict(self, sd: Dict) -> None:
        self.m.copy_(sd["m"])
        self.v.copy_(sd["v"])
        self.step_count = int(sd["step"])


class LRSchedule:
    """lr(step) for step = 0, 1, ... (the value used by optimizer step number step+1)."""

    def __init__(self, cfg, base_lr: float, total_steps: int, model_size: int = 256):
        self.kind = cfg.type if cfg is not None else "constant"
        self.cfg = cfg
        self.init = (cfg.initial_lr if cfg is not None and cfg.initial_lr is not None else base_lr)
        self.total = max(1, total_steps)
        self.model_size = model_size

    def __call__(self, step: int) -> float:
        c, k, lr0 = self.cfg, self.kind, self.init
        if k == "constant":
            return lr0
        if k == "cosine":
            n = max(1, c.num_iters or self.total)
            lo = c.min_lr or 0.0
            t = min(step, n) / n
            return lo + 0.5 * (lr0 - lo) * (1 + math.cos(math.pi * t))
        if k == "linear":
            n = max(1, c.num_iters or self.total)
            t = min(step, n) / n
            return lr0 + (c.final_lr - lr0) * t
        if k == "exponential":
            return lr0 * (c.gamma ** step)
        if k == "step":
            size = max(1, c.step_size or self.total)
            return lr0 * ((c.gamma if c.gamma is not None else 0.1) ** (step // size))
        if k == "noam":
            warm = max(1, c.warmup_steps or max(1, self.total // 10))
            size = c.model_size or self.model_size
            s = step + 1
            return lr0 * (size ** -0.5) * min(s ** -0.5, s * warm ** -1.5)
        raise ValueError(f"unknown schedule {k}")

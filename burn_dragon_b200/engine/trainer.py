"""Training engine: one object that owns model, optimizer, parallel wrapper and the step function.

`Trainer.train_step(tokens, targets)` is the public per-step call (what `train` and `bench.py` use):
zero grads -> loss -> backward -> gradient reduction -> AdamW with the scheduled LR. It mirrors the
reference's TrainStep (src/bin/train.rs:134-146) plus what burn-train's Learner does around it
(optimizer step, LR scheduler step, src/bin/train.rs:380-419).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..parallel import dist_utils
from ..parallel.ddp import DataParallel
from ..utils import profiling as prof
from .optim import FlatAdamW, LRSchedule


class Trainer:
    def __init__(self, model: torch.nn.Module, lr: float = 1e-3, weight_decay: float = 0.1, beta1: float = 0.9,
                 beta2: float = 0.999, eps: float = 1e-5, schedule: Optional[LRSchedule] = None,
                 parallel: str = "single", fused_collectives: bool = True, fast_train: bool = False,
                 grad_clip: Optional[float] = None, wrapper=None, grad_accum: int = 1):
        self.model = model
        self.fast_train = fast_train
        self.grad_clip = grad_clip
        self.schedule = schedule
        self.parallel = parallel
        self.step_index = 0
        # micro-batches per optimizer step: gradients of `grad_accum` calls are summed in the flat
        # gradient buffer, reduced across ranks once and applied with scale 1/grad_accum
        self.grad_accum = max(1, int(grad_accum))
        self._micro = 0
        if wrapper is not None:
            if fast_train and not hasattr(model, "forward_fast"):
                raise ValueError("fast_train needs a model with a `forward_fast` path")
            wrapper.fast_train = bool(fast_train)
            wrapper.grad_clip = grad_clip
        self.track_grad_norm = False      # set by the metrics logger on the steps it logs
        self.last_grad_norm = None
        self.wrapper = wrapper
        if wrapper is not None:
            # FSDP / TP wrappers own parameter storage, gradient reduction and the optimizer
            self.opt = wrapper.optimizer
            self.dp = None
        else:
            shadow = next(model.parameters()).is_cuda
            self.opt = FlatAdamW(model, lr, weight_decay, beta1, beta2, eps, shadow_bf16=shadow)
            self.dp = DataParallel(self.opt.flat, mode="fused" if fused_collectives else "nccl") \
                if parallel == "ddp" and dist_utils.world_size() > 1 else None
            if self.dp is not None:
                self.dp.broadcast_parameters()
        self.base_lr = lr
        # a kernel whose bounded wait ran out returns early and leaves its work undone: watch the status
        # word (one 4-byte async copy per step, no synchronisation) and stop the rank when it is set
        from ..parallel.watchdog import StatusMonitor
        self.status = StatusMonitor()
        self.status.enabled = next(model.parameters()).is_cuda

    def current_lr(self) -> float:
        return self.schedule(self.step_index) if self.schedule is not None else self.base_lr

    def loss_fn(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        if self.fast_train and hasattr(self.model, "forward_fast"):
            return self.model.forward_fast(tokens, targets)
        return self.model(tokens, targets)

    def train_step(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """One optimizer step. Returns the (local) loss as a 0-d device tensor; no host sync."""
        if self.wrapper is not None:
            with prof.phase("step"):
                loss = self.wrapper.train_step(tokens, targets, self.current_lr(), micro=(self._micro, self.grad_accum))
            self._micro = (self._micro + 1) % self.grad_accum
            if self._micro == 0:
                self.step_index += 1
                self.last_grad_norm = self.wrapper.last_grad_norm      # (only measured when clipping)
                self.status.poll()
            return loss
        with prof.phase("step"):
            if self._micro == 0:
                self.opt.zero_grad()
            with prof.phase("forward"):
                loss = self.loss_fn(tokens, targets)
            with prof.phase("backward"):
                loss.backward()
            self._micro += 1
            if self._micro < self.grad_accum:
                return loss.detach()           # more micro-batches to come: no reduction, no update
            self._micro = 0
            with prof.phase("grad_reduce"):
                scale = (self.dp.reduce_gradients() if self.dp is not None else 1.0) / self.grad_accum
            if self.grad_clip or self.track_grad_norm:
                # norm of the averaged gradient, kept on the device (read it with `.item()` when logging)
                self.last_grad_norm = self.opt.flat.grad.norm() * scale
            if self.grad_clip:
                scale = scale * float(torch.clamp(self.grad_clip / (self.last_grad_norm + 1e-6), max=1.0))
            with prof.phase("optimizer"):
                self.opt.step(lr=self.current_lr(), grad_scale=scale)
        self.step_index += 1
        self.status.poll()
        return loss.detach()

    @torch.no_grad()
    def eval_step(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        # a tensor-parallel wrapper evaluates its shard (the full module's weights are stale while it trains)
        m = getattr(self.wrapper, "eval_model", None) or self.model
        was = m.training
        m.eval()
        try:
            if self.fast_train and hasattr(m, "forward_fast"):
                return m.forward_fast(tokens, targets).detach()
            return m(tokens, targets).detach()
        finally:
            m.train(was)

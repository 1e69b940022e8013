"""Context (sequence) parallelism for BDH: rank r holds tokens [r*T, (r+1)*T) of every sequence.

Linear attention makes this a state hand-off rather than a ring of key/value blocks: inside a layer
every rank computes its local causal part and the state its segment would add,

    rho_loc^r = sum_s g^(T-s) q_s^T v_s                                   [B, H, N', D]

the ranks exchange these (one all-gather per layer), and rank r continues from the state all
earlier tokens left behind,

    rho_in^r = g^(rT) rho_0 + sum_{r' < r} g^((r-1-r') T) rho_loc^{r'},    a_t += g^t q_t . rho_in^r

so the result equals the single-device forward over the concatenated sequence. For training the
same hand-off is an autograd function (`scan_grad`: the gradient of every later rank's starting
state flows back to the earlier ranks' segment states), so `loss()` + `reduce_gradients()` give the
loss and gradients of whole sequences that no single rank holds (on the kernel path the hand-off and
its reverse are explicit steps of the layer's forward and backward pass). After the call
every rank holds the state of the whole sequence, so decoding can continue on any of them. The
message is the state itself (33 MB fp32 per layer for the base model), so this pays when the
per-rank segment is much longer than the state is wide. The reference has no sequence parallelism
(its long-context mechanism is the recurrence alone, src/model/state.rs:5-16).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist


class _ExclusiveStateScan(torch.autograd.Function):
    """Differentiable state hand-off. Forward: all-gather the segment states and return what this rank
    starts from, sum_{r' < r} g^((r-1-r') T) rho_loc^{r'}. Backward: the gradient of every later
    rank's starting state flows back to this rank's segment state with the same decay weights
    (one all-gather of the incoming gradients)."""

    @staticmethod
    def forward(ctx, rho_loc, g_T, rank, world, group):
        parts = [torch.empty_like(rho_loc) for _ in range(world)]
        dist.all_gather(parts, rho_loc.contiguous(), group=group)
        run = torch.zeros_like(rho_loc)
        out = run
        for r in range(world):
            if r == rank:
                out = run
            run = run * g_T + parts[r]
        ctx.g_T, ctx.rank, ctx.world, ctx.group = g_T, rank, world, group
        return out.clone()

    @staticmethod
    def backward(ctx, grad_in):
        grads = [torch.empty_like(grad_in) for _ in range(ctx.world)]
        dist.all_gather(grads, grad_in.contiguous(), group=ctx.group)
        # rho_in^r contains g^((r-1-rank) T) rho_loc^rank for every r > rank
        acc = torch.zeros_like(grad_in)
        w = 1.0
        for r in range(ctx.rank + 1, ctx.world):
            acc = acc + grads[r] * w
            w = w * ctx.g_T
        return acc, None, None, None, None


class ContextParallel:
    def __init__(self, model, group=None):
        self.model, self.group = model, group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)

    # ---- collective used inside every layer --------------------------------------------------------
    def scan(self, rho_loc: torch.Tensor, rho0: Optional[torch.Tensor], g_T) -> Tuple[Optional[torch.Tensor], torch.Tensor]:
        """rho_loc [B, H, N', D]: this rank's segment state; rho0: state before the whole sequence (same
        on every rank) or None; g_T: per-head decay over one segment, broadcastable to rho ([1, H, 1, 1])
        or 1.0. Returns (state this rank starts from - None if it is exactly zero -, state after the
        whole sequence)."""
        parts = [torch.empty_like(rho_loc) for _ in range(self.world)]
        dist.all_gather(parts, rho_loc.contiguous(), group=self.group)
        run = rho0.to(rho_loc.dtype) if rho0 is not None else None
        rho_in = None
        for r in range(self.world):
            if r == self.rank:
                rho_in = run
            run = parts[r] if run is None else run * g_T + parts[r]
        return rho_in, run

    def scan_backward(self, d_start: torch.Tensor, g_T) -> torch.Tensor:
        """Backward of `scan` for the kernel path (which writes its own backward pass): d_start is the
        gradient of the state this rank started from; returns the gradient of this rank's own segment
        state, sum over the later ranks r' of g_T^(r' - 1 - rank) d_start^{r'} (one all-gather)."""
        grads = [torch.empty_like(d_start) for _ in range(self.world)]
        dist.all_gather(grads, d_start.contiguous(), group=self.group)
        acc = torch.zeros_like(d_start)
        w = 1.0
        for r in range(self.rank + 1, self.world):
            acc = acc + grads[r] * w
            w = w * g_T
        return acc

    def scan_grad(self, rho_loc: torch.Tensor, g_T) -> torch.Tensor:
        """Differentiable `scan` for training (no state before the sequence): the state this rank
        starts from, as a function of every earlier rank's segment state."""
        return _ExclusiveStateScan.apply(rho_loc, g_T, self.rank, self.world, self.group)

    def loss(self, tokens_local: torch.Tensor, targets_local: torch.Tensor) -> torch.Tensor:
        """Training loss of this rank's segment of sequences that are split over the ranks (rank r
        holds tokens [r*T, (r+1)*T) of every sequence). The gradients of later segments reach earlier
        ranks through the state hand-off; call `reduce_gradients()` after `backward()`. The mean over
        the ranks' losses is the loss of the whole sequences. Runs on the kernels where they cover the
        model (the hand-off and its reverse are then part of the kernel path's own forward and backward
        pass, `ops/fused_bdh.py::_scan_forward/_scan_backward`), else on the torch path."""
        from ..ops import fused_bdh
        from ..ops import reference as R
        model = self.model
        start = self.rank * tokens_local.shape[1]
        model._cp = self
        try:
            if getattr(self, "use_kernels", True) and fused_bdh.can_run(model, tokens_local, None):
                model._train_pos0 = start
                try:
                    return fused_bdh.loss(model, tokens_local, targets_local)
                finally:
                    model._train_pos0 = 0
            logits = model._forward_torch(tokens_local, None, "parallel", start=start)
        finally:
            model._cp = None
        return R.cross_entropy_mean(logits, targets_local)

    def reduce_gradients(self) -> None:
        """Average the parameter gradients over the group (every rank then holds the gradient of the
        whole-sequence mean loss)."""
        for p in self.model.parameters():
            if p.grad is not None:
                dist.all_reduce(p.grad, group=self.group)
                p.grad.div_(self.world)

    # ---- public ------------------------------------------------------------------------------------
    @torch.no_grad()
    def forward_with_state(self, tokens_local: torch.Tensor, state, mode: str = "auto") -> torch.Tensor:
        """Logits [B, T, V] of this rank's segment; `state` (same on every rank) is advanced over the
        whole sequence of world * T tokens."""
        T = tokens_local.shape[1]
        p0 = state.position
        model = self.model
        model._cp = self
        try:
            state.position = p0 + self.rank * T
            logits = model.forward_with_state(tokens_local, state, mode)
        finally:
            model._cp = None
        state.position = p0 + self.world * T
        return logits

    @torch.no_grad()
    def prefill_any(self, tokens_full: torch.Tensor):
        """`prefill` for a prompt of any length: the largest prefix that splits evenly over the ranks
        runs context-parallel, the few tokens left over run replicated on every rank. Returns
        (state, logits of the last prompt token [B, V]), the same on every rank."""
        P = tokens_full.shape[1]
        even = (P // self.world) * self.world
        if even == 0:
            state = self.model.init_state()
            return state, self.model.forward_with_state(tokens_full, state)[:, -1]
        state, last = self.prefill(tokens_full[:, :even])
        if even < P:
            last = self.model.forward_with_state(tokens_full[:, even:].contiguous(), state)[:, -1]
        return state, last

    @torch.no_grad()
    def prefill(self, tokens_full: torch.Tensor):
        """Split a [B, P] prompt (P divisible by the group size) over the ranks, run it, and return
        (state after the prompt, logits of the last prompt token [B, V]) on every rank."""
        P = tokens_full.shape[1]
        if P % self.world:
            raise ValueError("prompt length must be a multiple of the context-parallel group size")
        T = P // self.world
        state = self.model.init_state()
        logits = self.forward_with_state(tokens_full[:, self.rank * T:(self.rank + 1) * T].contiguous(), state)
        last = logits[:, -1].contiguous()
        dist.broadcast(last, src=dist.get_global_rank(self.group, self.world - 1) if self.group is not None
                       else self.world - 1, group=self.group)
        return state, last

"""Continuous batching for cached decoding: a fixed pool of stream slots that requests join and leave
between decode steps.

Every stream of a BDH model is a constant-size recurrent state, so a slot is just one row of the
per-layer state tensors `[slots, H, N', D]`, one row of logits and one position. A request is
prefilled on its own (any prompt length), its state is copied into a free slot, and from then on
every `step()` advances all slots at once with the decode engine's step - one batched launch
sequence (one CUDA-graph replay on a GPU) whatever mixture of positions the slots are at: the RoPE
table carries one row per stream. Slots that nobody uses run along on a zero state; their tokens
are ignored. Sampling settings belong to the pool (they are baked into the captured step).

For PoPE (whose GEMM epilogue takes one scalar position) the pooled step ends the encoder GEMM at
the ReLU and applies the rotation per stream with elementwise ops on the [slots, H*N] activations.
The reference decodes one stream, one token at a time, with host-side sampling
(src/generation.rs:106-129).
"""
from __future__ import annotations

from typing import List

import torch

from ..ops.fused_bdh import _weights
from . import generation as GEN
from .decode_engine import DecodeEngine


def state_bytes_per_stream(config) -> int:
    """fp32 recurrent state of one stream: L layers x H heads x N' x D."""
    return 4 * config.n_layer * config.n_head * config.state_latent * config.n_embd


def max_slots(model, device, fraction: float = 0.8) -> int:
    """How many streams fit in `fraction` of the free device memory (the state dominates: 33.5 MB per
    layer for the base model, 537 MB per layer for the large PoPE one)."""
    device = torch.device(device)
    if device.type != "cuda":
        return 1 << 30
    free, _ = torch.cuda.mem_get_info(device)
    return int(fraction * free // max(1, state_bytes_per_stream(model.config)))


class StreamPool:
    def __init__(self, model, slots: int, settings: GEN.GenerationSettings, device=None, use_graph: bool = True):
        c = model.config
        self.model = model
        self.device = torch.device(device) if device is not None else next(model.parameters()).device
        fit = max_slots(model, self.device)
        if int(slots) > fit:
            raise ValueError(f"{slots} stream slots need {slots * state_bytes_per_stream(c) / 2**30:.1f} GiB of recurrent "
                             f"state; {fit} fit in the free memory of {self.device}")
        self.slots = int(slots)
        self.settings = settings
        self.seed = int(settings.seed if settings.seed is not None else 0) & 0xFFFFFFFF
        self.engine = DecodeEngine(model, use_graph=use_graph)
        probe = torch.zeros(1, 1, dtype=torch.int64, device=self.device)
        probe_settings = GEN.GenerationSettings(1, settings.temperature, settings.top_k, greedy=settings.greedy)
        if not self.engine.can_run(probe, probe_settings):
            raise ValueError("this model / device is not eligible for the decode engine")
        self.buf = self.engine._alloc(self.slots, self.device)
        d = self.buf["d"]
        # one position per slot (the engine's step sees `pos.numel() > 1` and builds a table row per stream)
        self.buf["pos"] = torch.zeros(self.slots, device=self.device, dtype=torch.int32)
        if d.rot == "rope":
            self.buf["table"] = torch.zeros(self.slots, d.N, device=self.device, dtype=torch.bfloat16)
        self.rho = [torch.zeros(self.slots, c.n_head, c.state_latent, c.n_embd, device=self.device)
                    for _ in range(c.n_layer)]
        # ALiBi models: lazy decay (per state row, the step up to which it is current; engine/decode_engine.py).
        # Slot states only ever enter the pool (`add`) or are cleared (`release`), so nothing has to be caught up.
        self.seen = ([torch.zeros(self.slots, c.n_head, c.state_latent, device=self.device, dtype=torch.int32)
                      for _ in range(c.n_layer)] if (d.slopes is not None and self.engine.lazy_decay) else None)
        self.active: List[bool] = [False] * self.slots
        self.steps = 0
        self.graph = None
        self.W = _weights(model)          # bf16 working copies, fixed for the life of the pool (`refresh_weights`)
        self.warm_up()

    # ---- slots -------------------------------------------------------------------------------------
    def free_slots(self) -> int:
        return self.active.count(False)

    @torch.no_grad()
    def add(self, prompt_ids) -> int:
        """Prefill one prompt (any length) and seat it in a free slot. Returns the slot index; its
        first token comes out of the next `step()`."""
        try:
            slot = self.active.index(False)
        except ValueError:
            raise RuntimeError("no free stream slot") from None
        state, last = GEN.prefill_state(self.model, prompt_ids, self.device)
        for r, l in zip(self.rho, state.layers):
            if l.rho is None:
                r[slot].zero_()
            else:
                r[slot].copy_(l.rho[0])
        self.buf["logits"][slot].copy_(last[0].float())
        self.buf["pos"][slot] = int(state.position)
        if self.seen is not None:
            for t in self.seen:
                t[slot].fill_(self.steps)        # the prefilled state is current as of the pool's step counter
        self.active[slot] = True
        return slot

    def release(self, slot: int) -> None:
        """Free a slot. Its state is cleared so that the idle row stays numerically quiet."""
        self.active[slot] = False
        for r in self.rho:
            r[slot].zero_()
        self.buf["logits"][slot].zero_()
        self.buf["pos"][slot] = 0

    # ---- decoding ------------------------------------------------------------------------------------
    def _capture(self) -> None:
        """Capture the step once, on an empty pool (the warm-up run advances state and counters, so
        everything is zeroed again afterwards)."""
        W = self.W
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self.engine._step(self.buf, W, self.rho, self.settings, self.seed, None, self.seen)
        torch.cuda.current_stream().wait_stream(s)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.engine._step(self.buf, W, self.rho, self.settings, self.seed, None, self.seen)
        self.graph = graph
        for r in self.rho:
            r.zero_()
        for t in (self.seen or []):
            t.zero_()
        for k in ("logits", "pos", "step"):
            self.buf[k].zero_()

    @torch.no_grad()
    def step(self) -> torch.Tensor:
        """One decode step for every slot: sample each stream's next token from its current logits and
        advance its state by that token. Returns the tokens [slots] (entries of free slots are
        meaningless)."""
        if self.graph is not None:
            self.graph.replay()
        else:
            self.engine._step(self.buf, self.W, self.rho, self.settings, self.seed, None, self.seen)
        self.steps += 1
        return self.buf["tok"].clone()

    def warm_up(self) -> None:
        """Capture the step (GPU; a no-op elsewhere). Called at construction, while the pool is empty."""
        if self.engine.use_graph and self.device.type == "cuda" and self.graph is None:
            self._capture()

    @torch.no_grad()
    def refresh_weights(self) -> None:
        """Copy the model's current weights into the buffers the (captured) step reads."""
        for k, w in _weights(self.model).items():
            if w.data_ptr() != self.W[k].data_ptr():
                self.W[k].copy_(w)


class _Handle:
    """One request seated in the pool: text pieces arrive on `queue`, `None` marks the end."""

    def __init__(self, slot: int, remaining: int, printer, eos_id):
        import queue
        self.slot, self.remaining, self.printer, self.eos_id = slot, remaining, printer, eos_id
        self.queue: "queue.Queue" = queue.Queue()
        self.tokens = 0


class PoolScheduler:
    """Runs the pool from one background thread: requests (`submit`) are seated between steps, every
    step's tokens are handed to their requests as text, finished streams free their slot at once.
    `gpu_lock` is shared with anything else that uses the device (the server's exclusive path)."""

    def __init__(self, pool: StreamPool, tokenizer, gpu_lock=None):
        import threading
        self.pool, self.tokenizer = pool, tokenizer
        self.gpu_lock = gpu_lock if gpu_lock is not None else threading.Lock()
        self.cv = threading.Condition()
        self.handles: dict = {}
        self.stopping = False
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def submit(self, prompt_ids: List[int], max_tokens: int, timeout: float = 300.0) -> _Handle:
        """Blocks until a slot is free, prefills the prompt, seats it. Returns the request's handle."""
        import time
        deadline = time.time() + timeout
        with self.cv:
            while self.pool.free_slots() == 0:
                left = deadline - time.time()
                if left <= 0 or self.stopping:
                    raise TimeoutError("no stream slot became free")
                self.cv.wait(left)
            with self.gpu_lock:
                slot = self.pool.add(torch.tensor([list(prompt_ids)], dtype=torch.int64, device=self.pool.device))
            pieces: List[str] = []
            h = _Handle(slot, int(max_tokens), GEN.StreamPrinter(self.tokenizer, write=pieces.append),
                        getattr(self.tokenizer, "eos_id", None))
            h.pieces = pieces
            self.handles[slot] = h
            self.cv.notify_all()
        return h

    def _finish(self, h: _Handle) -> None:
        with self.gpu_lock:
            self.pool.release(h.slot)
        del self.handles[h.slot]
        h.queue.put(None)
        self.cv.notify_all()          # (called with the condition held) a slot is free again

    def _run(self) -> None:
        while True:
            with self.cv:
                while not self.handles and not self.stopping:
                    self.cv.wait()
                if self.stopping:
                    for h in list(self.handles.values()):
                        h.queue.put(None)
                    return
                for h in [h for h in self.handles.values() if h.remaining <= 0]:
                    self._finish(h)              # a request for zero tokens, or a client that went away
                seated = list(self.handles.values())
            if not seated:
                continue
            # the step runs outside the condition's lock, so that new requests can queue up for the
            # device lock meanwhile; a stream seated after this point joins from the next step on
            with self.gpu_lock:
                toks = self.pool.step().tolist()
            with self.cv:
                for h in seated:
                    t = toks[h.slot]
                    h.remaining -= 1
                    if h.eos_id is not None and t == h.eos_id:
                        h.remaining = 0
                    else:
                        h.tokens += 1
                        h.printer.push(t)
                        if h.pieces:
                            h.queue.put("".join(h.pieces))
                            h.pieces.clear()
                    if h.remaining <= 0:
                        self._finish(h)
                self.cv.notify_all()              # a slot may have become free

    def stop(self) -> None:
        with self.cv:
            self.stopping = True
            self.cv.notify_all()
        self.thread.join(timeout=5)


def _selftest() -> int:
    """`python -m burn_dragon_b200.engine.stream_pool`: on the current device, streams with prompts of
    different lengths join and leave a pool; each one's greedy tokens must equal what it produces
    alone on the decode engine. Prints PASS / FAIL lines; exit code 0 only when everything matched."""
    from ..models.bdh import BDH, BDHConfig
    from ..ops import native
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    ok = True
    for rot in ("rope", "alibi", "pope"):
        torch.manual_seed(0)
        m = BDH(BDHConfig(n_layer=2, n_embd=64, n_head=2, n_latent_per_head=128, vocab_size=256, dropout=0.0,
                          rotary_embedding=rot)).to(dev).eval()
        with torch.no_grad():
            m.encoder.mul_(4.0); m.encoder_v.mul_(4.0); m.decoder.mul_(4.0)
        g = torch.Generator().manual_seed(3)
        prompts = [torch.randint(0, 256, (1, n), generator=g).to(dev) for n in (64, 128, 192)]
        eng = DecodeEngine(m)
        alone = [eng.generate(p, GEN.GenerationSettings(8, greedy=True))[0, p.shape[1]:].tolist() for p in prompts]
        for slots in (4, 64):
            pool = StreamPool(m, slots, GEN.GenerationSettings(None, greedy=True), dev)
            got = {0: [], 1: [], 2: []}
            a = pool.add(prompts[0])
            for _ in range(3):
                got[0].append(int(pool.step()[a]))
            b = pool.add(prompts[1])
            for _ in range(5):
                t = pool.step()
                got[0].append(int(t[a])); got[1].append(int(t[b]))
            pool.release(a)
            c = pool.add(prompts[2])
            for _ in range(8):
                t = pool.step()
                got[1].append(int(t[b])); got[2].append(int(t[c]))
            same = got[0] == alone[0] and got[1][:8] == alone[1] and got[2] == alone[2]
            status = native.status_code() if dev.type == "cuda" else 0
            print(f"{'PASS' if same and status == 0 else 'FAIL'} stream_pool {rot} slots={slots} graph={pool.graph is not None} "
                  f"status={status}", flush=True)
            ok = ok and same and status == 0
    return 0 if ok else 1


if __name__ == "__main__":
    import sys
    sys.exit(_selftest())

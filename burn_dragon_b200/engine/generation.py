"""Generation runtime: prefill, cached decode, sampling, context strategies, streaming text.

API follows the reference (src/generation.rs:13-260): `prefill_state`, `sample_next_token`,
`generate_tokens` (with a per-token callback), `generate_text`, `resolve_context_strategy`. What is
different: every function takes a batch of independent streams `[B, P]` (the reference is batch 1),
sampling runs on the device (the reference copies the logits to the host for every token) and is
seedable, and there is a greedy mode. The prefill is one parallel pass that also produces the
recurrent state; the reference runs its per-timestep loop for the prompt too.
"""
from __future__ import annotations

import codecs
import sys
from dataclasses import dataclass
from typing import Callable, List, Optional

import torch



@dataclass(frozen=True)
class ContextStrategy:
    kind: str = "infinite"       # "infinite" | "sliding"
    window: int = 0


@dataclass
class GenerationSettings:
    max_new_tokens: Optional[int] = None
    temperature: float = 1.0
    top_k: Optional[int] = None
    strategy: ContextStrategy = ContextStrategy()
    greedy: bool = False
    seed: Optional[int] = None
    eos_id: Optional[int] = None      # stop a stream at EOS (the reference's wasm loop does, its CLI does not)


def resolve_context_strategy(cfg, default_window: int) -> ContextStrategy:
    """window 0 means "the training block size" (src/generation.rs:245-260)."""
    if cfg is None or cfg.type == "infinite":
        return ContextStrategy("infinite", 0)
    win = cfg.window if cfg.window else max(1, default_window)
    return ContextStrategy("sliding", int(win))


def normalize_max_tokens(v: Optional[int]) -> Optional[int]:
    return int(v) if v is not None and v >= 0 else None


def _as_batch(prompt_tokens, device) -> torch.Tensor:
    t = torch.as_tensor(prompt_tokens, dtype=torch.long, device=device)
    if t.dim() == 1:
        t = t.unsqueeze(0)
    if t.shape[1] == 0:
        raise ValueError("prompt must contain at least one token")
    return t


PREFILL_SEGMENT = 4096


@torch.no_grad()
def prefill_state(model, prompt_tokens, device=None, segment: Optional[int] = None):
    """Run the prompt, return (state, last_logits [B, V]) (src/generation.rs:74-104). Prompts longer
    than `segment` tokens (default PREFILL_SEGMENT) are run segment by segment with the recurrent
    state carried across, so score memory is O(segment^2) whatever the prompt length; the result is
    the same function of the prompt."""
    device = device if device is not None else next(model.parameters()).device
    toks = _as_batch(prompt_tokens, device)
    state = model.init_state()
    seg = int(segment or PREFILL_SEGMENT)
    P = toks.shape[1]
    logits = None
    for lo in range(0, max(P, 1), seg):
        part = toks[:, lo:lo + seg]
        logits = model.forward_with_state(part, state)
        if logits.shape[1] != part.shape[1]:
            raise RuntimeError(f"prefill produced mismatched length: expected {part.shape[1]}, got {logits.shape[1]}")
    state.viz = None
    return state, logits[:, -1]


def _sample(last_logits, settings: GenerationSettings, generator):
    from ..ops import sampling
    return sampling.sample(last_logits, settings.temperature, settings.top_k, settings.greedy, generator)


@torch.no_grad()
def sample_next_token(model, state, last_logits, temperature=1.0, top_k=None, greedy=False, generator=None):
    """Draw the next token of every stream from `last_logits`, advance the model by that token and
    return (next [B], logits [B, V]) (src/generation.rs:106-129)."""
    s = GenerationSettings(temperature=temperature, top_k=top_k, greedy=greedy)
    nxt = _sample(last_logits, s, generator)
    logits = model.forward_with_state(nxt.view(-1, 1), state)
    return nxt, logits[:, -1]


@torch.no_grad()
def generate_tokens(model, prompt_tokens, device=None, settings: Optional[GenerationSettings] = None,
                    on_token: Optional[Callable[[torch.Tensor], None]] = None) -> torch.Tensor:
    """Prompt + generated tokens, [B, P + n] (src/generation.rs:158-203). `on_token` receives the
    [B] tensor of new tokens after every step. With `max_new_tokens=None` generation only ends when
    every stream has produced EOS (if `eos_id` is set) - otherwise pass a limit."""
    settings = settings or GenerationSettings()
    device = device if device is not None else next(model.parameters()).device
    toks = _as_batch(prompt_tokens, device)
    if settings.max_new_tokens is None and settings.eos_id is None:
        raise ValueError("generate_tokens needs max_new_tokens or eos_id to terminate")
    gen = None
    if settings.seed is not None:
        gen = torch.Generator(device=device).manual_seed(settings.seed)
    engine = getattr(model, "decode_engine", None)
    if engine is not None and engine.can_run(toks, settings):
        return engine.generate(toks, settings, gen, on_token)
    state, last = prefill_state(model, toks, device)
    win = settings.strategy.window if settings.strategy.kind == "sliding" else 0
    if win and state.position > win:
        state.trim(win)
    out = [toks]
    done = torch.zeros(toks.shape[0], dtype=torch.bool, device=device)
    n = 0
    while settings.max_new_tokens is None or n < settings.max_new_tokens:
        nxt = _sample(last, settings, gen)
        if settings.eos_id is not None:
            nxt = torch.where(done, torch.full_like(nxt, settings.eos_id), nxt)
            done |= nxt == settings.eos_id
        out.append(nxt.view(-1, 1))
        n += 1
        if on_token is not None:
            on_token(nxt)
        if settings.eos_id is not None and bool(done.all()):
            break
        last = model.forward_with_state(nxt.view(-1, 1), state)[:, -1]
        if win and state.position > win:
            state.trim(win)
    return torch.cat(out, dim=1)


def generate_text(model, tokenizer, training, generation, device=None) -> str:
    """Encode the configured prompt, generate, decode everything (src/generation.rs:205-236)."""
    strategy = resolve_context_strategy(generation.context_strategy, training.block_size)
    ids = tokenizer.encode(generation.prompt, False, False)
    if strategy.kind == "sliding" and len(ids) > strategy.window:
        ids = ids[-strategy.window:]
    settings = GenerationSettings(normalize_max_tokens(generation.max_tokens), generation.temperature,
                                  generation.top_k, strategy, getattr(generation, "greedy", False),
                                  getattr(generation, "seed", None))
    if settings.max_new_tokens is None:
        settings.eos_id = tokenizer.eos_id
        if settings.eos_id is None:
            raise ValueError("generation.max_tokens is required when the tokenizer has no EOS token")
    toks = generate_tokens(model, ids, device, settings)
    return tokenizer.decode([int(t) for t in toks[0].tolist() if t >= 0])


class StreamPrinter:
    """Incremental, UTF-8-safe text output for a token stream (the reference's streaming loop,
    src/bin/infer.rs:254-273): bytes are buffered until they form complete characters."""

    def __init__(self, tokenizer, write: Callable[[str], None] = None):
        self.tok = tokenizer
        self.write = write or (lambda s: (sys.stdout.write(s), sys.stdout.flush()))
        self.ids: List[int] = []
        self.emitted = 0
        self._dec = codecs.getincrementaldecoder("utf-8")(errors="replace")

    def push(self, token_id: int) -> str:
        from ..data.tokenizer import ByteTokenizer
        self.ids.append(int(token_id))
        if isinstance(self.tok, ByteTokenizer):
            t = int(token_id)
            piece = self._dec.decode(bytes([t])) if 0 <= t < 256 else ""
        else:
            text = self.tok.decode(self.ids)
            piece = text[self.emitted:]
            self.emitted = len(text)
        if piece:
            self.write(piece)
        return piece

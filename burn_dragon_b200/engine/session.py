"""In-process inference sessions: the programmatic interface the reference exposes to its web page,
as a plain Python API (no browser, no window).

    sess = load_model(model_bytes, vocab_json, config_json)      # src/web.rs:86-207 `loadModel`
    sess.start_stream("ROMEO:", max_tokens=200, temperature=0.8, top_k=40)   # :212-264, prefill
    while not sess.done:
        piece = sess.next_chunk()                                  # :267-333, sample until printable

`load_model` accepts what the page fetches: a Burn record (f32, or the f16 file `quantize` writes:
the reference tries one then the other, src/web.rs:173-187), the character vocabulary JSON and the
run's `config.json` (`{run_name, block_size, overrides}`); without a config the model dimensions are
read off the tensor shapes. On a GPU the model gets the batched decode engine, and a session may
serve several prompts at once (`start_stream([...])`): every stream has its own recurrent state.
"""
from __future__ import annotations

import json
from typing import Dict, List, Optional, Sequence, Union

import torch

from ..data.tokenizer import ByteTokenizer, CharVocab
from ..models.bdh import BDH, BDHConfig
from . import burn_record as BR
from . import generation as GEN


def model_from_record(rec: "BR.BurnRecord", overrides: Optional[Dict] = None) -> BDH:
    """BDH whose shape is taken from the record and whose remaining hyper-parameters come from the
    run's model overrides (layer count, positional mode, ...)."""
    dims = BR.infer_dims(rec)
    ov = dict(overrides or {})
    kw = dict(vocab_size=dims["vocab_size"], n_embd=dims["n_embd"], n_head=dims["n_head"],
              n_latent_per_head=dims["n_latent_per_head"], dropout=0.0)
    for k in ("n_layer", "rotary_embedding", "relu_threshold", "rope_theta"):
        if ov.get(k) is not None:
            kw[k] = ov[k]
    mult = ov.get("mlp_internal_dim_multiplier")
    if mult is not None and int(mult) * dims["n_embd"] // dims["n_head"] != dims["n_latent_per_head"]:
        raise ValueError("config.json does not match the checkpoint: mlp_internal_dim_multiplier * n_embd / n_head "
                         f"= {int(mult) * dims['n_embd'] // dims['n_head']}, tensors have {dims['n_latent_per_head']}")
    model = BDH(BDHConfig(**kw)).eval()
    model.load_state_dict(BR.to_state_dict(rec))
    return model


class InferenceSession:
    def __init__(self, model: BDH, tokenizer, device=None, block_size: Optional[int] = None):
        self.device = torch.device(device) if device is not None else next(model.parameters()).device
        self.model = model.to(self.device).eval()
        self.tokenizer = tokenizer
        self.block_size = block_size
        if self.device.type == "cuda":
            from . import decode_engine
            decode_engine.attach(self.model)
        self._reset()

    def _reset(self):
        self.state = None
        self.logits = None
        self.settings: Optional[GEN.GenerationSettings] = None
        self.generated = 0
        self.finished: Optional[torch.Tensor] = None
        self.printers: List[GEN.StreamPrinter] = []
        self.pending: List[List[str]] = []
        self.generator = None
        self._pool = None

    # ---- stream control --------------------------------------------------------------------------
    @property
    def done(self) -> bool:
        return self.finished is None or bool(self.finished.all())

    @torch.no_grad()
    def start_stream(self, prompt: Union[str, Sequence[str]], max_tokens: Optional[int] = 256, temperature: float = 1.0,
                     top_k: Optional[int] = None, greedy: bool = False, seed: Optional[int] = None,
                     context_window: Optional[int] = None) -> None:
        """Prefill. `prompt` is one string or a list of strings (one stream each; prompts of different
        token counts need a model / device the decode engine takes, and are decoded by a stream pool).
        `context_window` keeps only the last tokens of the prompt (the sliding context strategy,
        src/generation.rs:214-218)."""
        self._reset()
        prompts = [prompt] if isinstance(prompt, str) else list(prompt)
        ids = [self.tokenizer.encode(p) for p in prompts]
        if context_window:
            ids = [i[-int(context_window):] for i in ids]
        if not ids or any(len(i) == 0 for i in ids):
            raise ValueError("prompt must contain at least one token")
        eos = getattr(self.tokenizer, "eos_id", None)
        if len({len(i) for i in ids}) != 1:
            return self._start_pooled(ids, max_tokens, temperature, top_k, greedy, seed, eos)
        toks = torch.tensor(ids, dtype=torch.int64, device=self.device)
        self.settings = GEN.GenerationSettings(GEN.normalize_max_tokens(max_tokens), temperature, top_k, greedy=greedy,
                                               seed=seed, eos_id=eos)
        if self.settings.max_new_tokens is None and eos is None:
            raise ValueError("max_tokens is required when the tokenizer has no EOS token")
        if seed is not None:
            self.generator = torch.Generator(device=self.device).manual_seed(int(seed))
        self.state, self.logits = GEN.prefill_state(self.model, toks, self.device)
        self.finished = torch.zeros(len(ids), dtype=torch.bool, device=self.device)
        self.pending = [[] for _ in ids]
        self.printers = [GEN.StreamPrinter(self.tokenizer, write=self.pending[i].append) for i in range(len(ids))]

    def _start_pooled(self, ids, max_tokens, temperature, top_k, greedy, seed, eos) -> None:
        """Prompts of different lengths: every stream is prefilled on its own and seated in a stream
        pool (engine/stream_pool.py) whose step carries one position per stream."""
        from .stream_pool import StreamPool
        n = GEN.normalize_max_tokens(max_tokens)
        if n is None:
            raise ValueError("max_tokens is required for prompts of different lengths")
        self.settings = GEN.GenerationSettings(n, temperature, top_k, greedy=greedy, seed=seed, eos_id=eos)
        try:
            self._pool = StreamPool(self.model, len(ids), self.settings, self.device)
        except ValueError as e:
            raise ValueError("prompts of one session call must have the same number of tokens on this model / "
                             f"device ({e})") from None
        for i in ids:
            self._pool.add(torch.tensor([i], dtype=torch.int64, device=self.device))
        self.logits = self._pool.buf["logits"]
        self.state = True              # (no single ModelState: the pool owns one state row per stream)
        self.finished = torch.zeros(len(ids), dtype=torch.bool, device=self.device)
        self.pending = [[] for _ in ids]
        self.printers = [GEN.StreamPrinter(self.tokenizer, write=self.pending[i].append) for i in range(len(ids))]

    # ---- state snapshots ---------------------------------------------------------------------------
    def snapshot(self) -> Dict:
        """Copy of everything a stream is: the recurrent state (constant size, whatever the length of
        the text so far), the logits of the last token and the counters. Restoring it later continues
        from this point - e.g. prefill a long shared prefix once and branch many completions off it."""
        if self.state is None:
            raise RuntimeError("call start_stream first")
        if self._pool is not None:
            raise RuntimeError("snapshots are per stream: start the prompts of different lengths one by one")
        return dict(position=self.state.position,
                    rho=[None if l.rho is None else l.rho.detach().clone() for l in self.state.layers],
                    logits=self.logits.detach().clone(), generated=self.generated, finished=self.finished.clone(),
                    settings=self.settings)

    def restore(self, snap: Dict, max_tokens: Optional[int] = None, seed: Optional[int] = None) -> None:
        """Continue from a snapshot (of this session or of another session of the same model).
        `max_tokens` / `seed` replace the snapshot's limit and sampling seed."""
        import dataclasses
        self._reset()
        self.state = self.model.init_state()
        self.state.position = int(snap["position"])
        for l, r in zip(self.state.layers, snap["rho"]):
            l.rho = None if r is None else r.to(self.device).clone()
        self.logits = snap["logits"].to(self.device).clone()
        self.generated = 0 if max_tokens is not None else int(snap["generated"])
        s = snap["settings"]
        self.settings = dataclasses.replace(s, max_new_tokens=s.max_new_tokens if max_tokens is None else int(max_tokens),
                                            seed=s.seed if seed is None else int(seed))
        if self.settings.seed is not None:
            self.generator = torch.Generator(device=self.device).manual_seed(int(self.settings.seed))
        n = self.logits.shape[0]
        self.finished = snap["finished"].to(self.device).clone() if max_tokens is None else \
            torch.zeros(n, dtype=torch.bool, device=self.device)
        self.pending = [[] for _ in range(n)]
        self.printers = [GEN.StreamPrinter(self.tokenizer, write=self.pending[i].append) for i in range(n)]

    def _take(self, tokens: List[int]) -> None:
        """One new token per stream: EOS ends a stream, anything else goes to its printer."""
        eos = self.settings.eos_id
        for i, t in enumerate(tokens):
            if bool(self.finished[i]):
                continue
            if eos is not None and t == eos:
                self.finished[i] = True
            else:
                self.printers[i].push(t)

    @torch.no_grad()
    def next_chunk(self, max_tokens: int = 4) -> Union[str, List[str]]:
        """Sample up to `max_tokens` tokens per stream, stopping early once every live stream has
        produced printable text (a multi-byte character may need several byte tokens). Returns the
        new text: a string for a single-stream session, else one string per stream. A stream ends at
        EOS or at the session's token limit; `done` turns true when all have ended."""
        if self.finished is None:
            raise RuntimeError("call start_stream first")
        s = self.settings
        eng = getattr(self.model, "decode_engine", None)
        if self._pool is not None:
            for _ in range(max(1, int(max_tokens))):
                if self.done or self.generated >= s.max_new_tokens:
                    self.finished.fill_(True)
                    break
                self._take(self._pool.step().tolist())
                self.generated += 1
        elif eng is not None and s.max_new_tokens is not None and eng.can_run(self.logits, s):
            # GPU: the whole chunk is decoded on the device (sampling included) by replaying the
            # captured decode step; only the chunk's token ids come back to the host
            n = min(max(1, int(max_tokens)), s.max_new_tokens - self.generated)
            if self.done or n <= 0:
                self.finished.fill_(True)
            else:
                new = eng.continue_from(self.state, self.logits, s, n, step0=self.generated)
                self.logits = eng.last_logits
                self.generated += n
                for column in new.t().tolist():
                    self._take(column)
                if self.generated >= s.max_new_tokens:
                    self.finished.fill_(True)
        else:
            for _ in range(max(1, int(max_tokens))):
                if self.done or (s.max_new_tokens is not None and self.generated >= s.max_new_tokens):
                    self.finished.fill_(True)
                    break
                nxt, self.logits = GEN.sample_next_token(self.model, self.state, self.logits, s.temperature, s.top_k,
                                                         s.greedy, self.generator)
                self.generated += 1
                self._take(nxt.tolist())
                if all(self.pending[i] or bool(self.finished[i]) for i in range(len(self.pending))):
                    break
        out = ["".join(p) for p in self.pending]
        for p in self.pending:
            p.clear()
        return out[0] if len(out) == 1 else out


def load_model(model_bytes: bytes, vocab_json: Optional[str] = None, config_json: Optional[str] = None,
               device=None) -> InferenceSession:
    """Build a session from the three artefacts of a trained run. `vocab_json` None selects the byte
    tokenizer (its vocabulary needs no file)."""
    rec = BR.parse(bytes(model_bytes))
    cfg = json.loads(config_json) if config_json else {}
    model = model_from_record(rec, cfg.get("overrides"))
    if vocab_json is not None:
        tok = CharVocab.from_json_str(vocab_json)
    else:
        tok = ByteTokenizer(add_special_tokens=model.config.vocab_size > 256)
    if len(tok) != model.config.vocab_size:
        raise ValueError(f"vocabulary has {len(tok)} entries, the checkpoint was trained with {model.config.vocab_size}")
    if device is None:
        device = "cuda" if torch.cuda.is_available() else "cpu"
    return InferenceSession(model, tok, device, cfg.get("block_size"))

"""Token-sequence datasets and the random-window batch loader.

Behaviour follows the reference data layer (src/dataset/mod.rs:14-118, factory.rs:10-214,
shakespeare.rs:42-110, huggingface.rs:36-581, scheduler.rs:14-279):

* a dataset is one long token array plus `train_len` (the training split is the prefix);
* `sample_batch` draws `batch_size` uniformly random windows of `block_size + 1` tokens from the
  split; targets are the inputs shifted by one;
* `steps_per_epoch = ceil(span / (block_size * batch_size))`, at least 1;
* the validation split falls back to the training span when what is left after it is not longer
  than one window;
* `RandomDataLoader` yields `steps_per_epoch` batches per pass with an optional global cap on the
  number of batches across passes.

Differences on purpose: sampling is seeded (the reference uses an unseeded thread RNG), batches
are assembled by the C++ window gatherer into pinned host memory when it is built (numpy
otherwise), downloads are refused with a clear error when the file is not cached and there is no
network, and a `synthetic` source provides uniform random bytes for benchmarks.
`ResidentDataLoader` is the device-side variant of the loader: the corpus lives on the training
device and the windows are drawn and gathered there.
"""
from __future__ import annotations

import csv
import dataclasses
import json
import os
import urllib.request
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Iterable, Iterator, List, Optional, Tuple

import numpy as np
import torch

from . import tokenizer as T

TRAIN, VAL = "train", "val"
SHAKESPEARE_URL = "https://raw.githubusercontent.com/karpathy/char-rnn/master/data/tinyshakespeare/input.txt"
DEFAULT_RECORD_DELIMITER = "\n"


@dataclass
class SequenceBatch:
    inputs: torch.Tensor   # [B, T] int64
    targets: torch.Tensor  # [B, T] int64


class TokenSequenceDataset:
    """One token array + split bookkeeping (src/dataset/scheduler.rs:14-70)."""

    def __init__(self, tokens: np.ndarray, train_len: int, block_size: int, batch_size: int,
                 train_split_ratio: float, tokenizer: T.Tokenizer, seed: int = 0):
        self.tokens = np.ascontiguousarray(tokens, dtype=np.int64)
        self.train_len = int(train_len)
        self.block_size = int(block_size)
        self.batch_size = int(batch_size)
        self.train_split_ratio = float(min(max(train_split_ratio, 0.0), 1.0))
        self.tokenizer = tokenizer
        self.rng = np.random.default_rng(seed)

    def split_offset_and_span(self, split: str) -> Tuple[int, int]:
        if split == TRAIN:
            return 0, self.train_len
        remaining = max(0, len(self.tokens) - self.train_len)
        if remaining <= self.block_size + 1:
            return 0, self.train_len
        return self.train_len, remaining

    def steps_per_epoch(self, split: str) -> int:
        _, span = self.split_offset_and_span(split)
        per_step = self.block_size * self.batch_size
        if per_step == 0:
            return 1
        return max(1, -(-span // per_step))

    def sample_starts(self, split: str) -> np.ndarray:
        offset, span = self.split_offset_and_span(split)
        max_start = max(0, span - (self.block_size + 1))
        if max_start == 0:
            return np.full(self.batch_size, offset, dtype=np.int64)
        return offset + self.rng.integers(0, max_start + 1, size=self.batch_size, dtype=np.int64)

    def sample_batch(self, split: str = TRAIN, device=None, pin: bool = False) -> SequenceBatch:
        """B random windows; targets are inputs shifted by one (src/dataset/scheduler.rs:72-110)."""
        starts = self.sample_starts(split)
        win = gather_windows(self.tokens, starts, self.block_size + 1, pin=pin)
        if device is not None:
            win = win.to(device, non_blocking=True)
        return SequenceBatch(win[:, :-1], win[:, 1:])

    def decode(self, ids: Iterable[int]) -> str:
        return self.tokenizer.decode([int(i) for i in ids if int(i) >= 0])


def gather_windows(tokens: np.ndarray, starts: np.ndarray, width: int, pin: bool = False) -> torch.Tensor:
    """[len(starts), width] int64 tensor of token windows. Uses the native gatherer when built."""
    out = torch.empty(len(starts), width, dtype=torch.int64, pin_memory=bool(pin and torch.cuda.is_available()))
    from ..utils import hostlib
    if hostlib.available():
        hostlib.gather_windows(tokens, starts, width, out)
    else:
        idx = starts[:, None] + np.arange(width)[None, :]
        out.copy_(torch.from_numpy(tokens[idx]))
    return out


class RandomDataLoader:
    """`steps_per_epoch` random batches per pass, optional global cap over all passes
    (src/dataset/scheduler.rs:125-279)."""

    def __init__(self, dataset: TokenSequenceDataset, split: str, device=None, steps_per_epoch: int = 1,
                 total_steps: Optional[int] = None, pin: bool = True, stream: Optional[Tuple[int, int]] = None):
        """`stream = (seed, data_rank)` makes the draws counter-based: batch number i of this loader is
        drawn from `default_rng([seed, data_rank, i])`, so a rank's sequence of batches depends only on
        its own key and on how many batches it has drawn. A checkpoint then needs the count alone and
        every rank of a resumed job continues its OWN sequence (restoring one rank's generator state on
        all ranks would make them draw identical windows). Without `stream` the dataset's shared
        generator is used and its state is what gets checkpointed (single-process runs)."""
        self.dataset, self.split, self.device, self.pin = dataset, split, device, pin
        self.steps_per_epoch = max(1, int(steps_per_epoch))
        self.total_steps = total_steps if total_steps and total_steps > 0 else None
        self.consumed = 0
        self.stream = (int(stream[0]), int(stream[1])) if stream is not None else None
        self.draws = 0

    def _next_rng(self) -> None:
        if self.stream is not None:
            self.dataset.rng = np.random.default_rng([self.stream[0], self.stream[1], self.draws])
        self.draws += 1

    def num_items(self) -> int:
        return self.steps_per_epoch * self.dataset.batch_size

    def __len__(self) -> int:
        if self.total_steps is not None:
            return max(0, min(self.total_steps - self.consumed, self.steps_per_epoch))
        return self.steps_per_epoch

    def __iter__(self) -> Iterator[SequenceBatch]:
        steps = len(self)
        for _ in range(steps):
            if self.total_steps is not None:
                if self.consumed >= self.total_steps:
                    return
                self.consumed += 1
            self._next_rng()
            yield self.dataset.sample_batch(self.split, self.device, self.pin)

    def state_dict(self) -> Dict:
        sd = dict(consumed=self.consumed, draws=self.draws)
        if self.stream is None:
            sd["rng"] = self.dataset.rng.bit_generator.state
        return sd

    def load_state_dict(self, sd: Dict) -> None:
        self.consumed = int(sd["consumed"])
        self.draws = int(sd.get("draws", self.consumed))
        # a generator state in the file belongs to the rank that wrote it: only a loader without a
        # per-rank stream key (single process) takes it over
        if "rng" in sd and self.stream is None:
            self.dataset.rng.bit_generator.state = sd["rng"]


# ------------------------------------------------------------------------------------------------
# sources
# ------------------------------------------------------------------------------------------------
class ResidentDataLoader(RandomDataLoader):
    """The same batches-per-pass contract with the token array RESIDENT on the training device: window
    starts are drawn and the windows gathered there, so a step costs no host work and no host-to-device
    copy (`[dataset] device_resident = true`). A corpus of n tokens takes 4 n bytes of device memory
    (2 n for vocabularies up to 32768). The draws come from a torch generator on that device, so the
    sequence of batches differs from the host loader's for the same seed; it is reproducible and
    its state is checkpointed like the host loader's."""

    def __init__(self, dataset: TokenSequenceDataset, split: str, device, steps_per_epoch: int = 1,
                 total_steps: Optional[int] = None, seed: int = 0):
        super().__init__(dataset, split, device, steps_per_epoch, total_steps, pin=False)
        self.seed = int(seed)
        device = torch.device(device if device is not None else "cpu")
        offset, span = dataset.split_offset_and_span(split)
        small = int(dataset.tokens.max(initial=0)) < 32768
        self.tokens = torch.from_numpy(np.ascontiguousarray(dataset.tokens[offset:offset + span])).to(
            torch.int16 if small else torch.int32).to(device)
        self.width = dataset.block_size + 1
        self.max_start = max(0, span - self.width)
        self.generator = torch.Generator(device=device).manual_seed(int(seed))
        self._arange = torch.arange(self.width, device=device)

    def sample_batch(self) -> SequenceBatch:
        B = self.dataset.batch_size
        # counter-based like the host loader: batch i comes from a generator seeded with (seed, i), where
        # `seed` already differs per data-parallel rank, so the count is all a checkpoint has to carry
        self.generator.manual_seed((self.seed * 0x9E3779B1 + self.draws * 0x85EBCA77 + 0x632BE5AB) & 0x7FFFFFFFFFFFFFFF)
        self.draws += 1
        starts = torch.randint(0, self.max_start + 1, (B,), generator=self.generator, device=self.tokens.device)
        win = self.tokens[starts[:, None] + self._arange[None, :]].long()
        return SequenceBatch(win[:, :-1], win[:, 1:])

    def __iter__(self) -> Iterator[SequenceBatch]:
        for _ in range(len(self)):
            if self.total_steps is not None:
                if self.consumed >= self.total_steps:
                    return
                self.consumed += 1
            yield self.sample_batch()

    def state_dict(self) -> Dict:
        return dict(consumed=self.consumed, draws=self.draws)

    def load_state_dict(self, sd: Dict) -> None:
        self.consumed = int(sd["consumed"])
        self.draws = int(sd.get("draws", self.consumed))


def _clamp_train_len(n_tokens: int, ratio: float, block_size: int) -> int:
    ratio = min(max(ratio, 0.0), 1.0)
    t = int(np.float32(n_tokens) * np.float32(ratio))
    return min(max(t, block_size + 1), n_tokens - 1)


def _fetch(url: str, dest: Path, what: str) -> None:
    if os.environ.get("BDH_OFFLINE", "0") == "1":
        raise FileNotFoundError(f"{what} is not cached at {dest} and BDH_OFFLINE=1 forbids downloading it")
    try:
        headers = {}
        tok = os.environ.get("HF_TOKEN")
        if tok and "huggingface.co" in url:
            headers["Authorization"] = f"Bearer {tok}"
        req = urllib.request.Request(url, headers=headers)
        with urllib.request.urlopen(req, timeout=30) as r:
            data = r.read()
    except Exception as e:  # noqa: BLE001
        raise FileNotFoundError(f"{what} is not cached at {dest} and could not be downloaded from {url}: {e}") from e
    dest.parent.mkdir(parents=True, exist_ok=True)
    dest.write_bytes(data)


def shakespeare_dataset(cache_dir, block_size, batch_size, train_split_ratio, tok_cfg, url=None, seed=0):
    """tinyshakespeare, downloaded once into `cache_dir/tinyshakespeare.txt` (shakespeare.rs:42-110)."""
    cache = Path(cache_dir)
    cache.mkdir(parents=True, exist_ok=True)
    path = cache / "tinyshakespeare.txt"
    if not path.exists():
        _fetch(url or SHAKESPEARE_URL, path, "tinyshakespeare")
    text = path.read_text()
    tok = T.load_or_fit(tok_cfg, cache, [text])
    T.validate_corpus(tok_cfg, tok, text)
    tokens = tok.encode_array(text)
    if len(tokens) <= block_size + 1:
        raise ValueError("encoded dataset smaller than block size")
    return TokenSequenceDataset(tokens, _clamp_train_len(len(tokens), train_split_ratio, block_size), block_size,
                                batch_size, train_split_ratio, tok, seed)


def synthetic_dataset(n_tokens, block_size, batch_size, vocab=256, seed=0, train_split_ratio=0.9):
    """Uniform random tokens in [0, vocab): what the throughput benchmarks train on."""
    rng = np.random.default_rng(seed)
    tokens = rng.integers(0, vocab, size=max(int(n_tokens), block_size + 2), dtype=np.int64)
    tok = T.ByteTokenizer(add_special_tokens=False)
    return TokenSequenceDataset(tokens, _clamp_train_len(len(tokens), train_split_ratio, block_size), block_size,
                                batch_size, train_split_ratio, tok, seed)


# ---- hugging face ---------------------------------------------------------------------------------
@dataclass
class HFSpec:
    repo_id: str
    revision: Optional[str]
    format: str
    train_files: List[str]
    validation_files: List[str]
    text_fields: List[str]
    field_separator: str
    template: Optional[str]
    max_records: Optional[int]


def hf_preset(kind: str, revision=None, max_records=None) -> HFSpec:
    """Canned sources of the reference (src/dataset/factory.rs:129-214)."""
    if kind == "deep_math":
        return HFSpec("zwhe99/DeepMath-103K", revision, "parquet",
                      [f"data/train-{i:05d}-of-00010.parquet" for i in range(10)], [],
                      ["question", "final_answer"], "\n\n", "Question:\n{question}\n\nAnswer:\n{final_answer}",
                      max_records)
    if kind == "tiny_chat":
        return HFSpec("starhopp3r/TinyChat", revision, "text", ["tinychat.txt"], [], ["text"], "\n\n", None,
                      max_records)
    if kind == "webscale_rl":
        return HFSpec("Salesforce/Webscale-RL", revision, "parquet", [f"data/part-{i}.parquet" for i in range(12)],
                      [], ["pretrain_text", "question", "answer", "domain", "persona"], "\n\n",
                      "Context:\n{pretrain_text}\n\nDomain: {domain}\nPersona: {persona}\n\nQuestion: "
                      "{question}\nAnswer: {answer}", max_records)
    if kind == "poetry_foundation":
        return HFSpec("suayptalha/Poetry-Foundation-Poems", revision, "csv", ["PoetryFoundationData.csv"], [],
                      ["Title", "Poem"], "\n\n\n", "{Title}\n\n\n{Poem}\n\n\n\n\n\n", max_records)
    raise ValueError(f"unknown dataset preset {kind}")


def render_template(template: str, fields: Dict[str, str]) -> str:
    """`{field}` substitution; unknown / empty / unclosed placeholders are errors; the result ends
    with a newline (src/dataset/huggingface.rs:536-581)."""
    out, i, n = [], 0, len(template)
    while i < n:
        ch = template[i]
        if ch == "{":
            j = template.find("}", i + 1)
            if j < 0:
                raise ValueError("unclosed template placeholder")
            key = template[i + 1:j].strip()
            if not key:
                raise ValueError("empty template placeholder {}")
            if key not in fields:
                raise ValueError(f"unknown template placeholder {{{key}}}")
            out.append(fields[key])
            i = j + 1
        else:
            out.append(ch)
            i += 1
    s = "".join(out)
    return s if s.endswith("\n") else s + "\n"


def render_record(spec: HFSpec, fields: Dict[str, str]) -> Optional[str]:
    if not fields:
        return None
    if spec.template:
        return render_template(spec.template, fields)
    ordered = []
    for f in spec.text_fields:
        if f not in fields:
            raise ValueError(f"template field `{f}` missing from record")
        ordered.append(fields[f])
    joined = ordered[0] if len(ordered) == 1 else (spec.field_separator or DEFAULT_RECORD_DELIMITER).join(ordered)
    return joined if joined.endswith("\n") else joined + "\n"


def _as_text(v) -> str:
    return v if isinstance(v, str) else json.dumps(v)


def collect_records(path: Path, spec: HFSpec, records: List[str]) -> None:
    lim = spec.max_records

    def full():
        return lim is not None and len(records) >= lim

    if spec.format == "jsonl":
        with open(path) as f:
            for line in f:
                if full():
                    break
                if not line.strip():
                    continue
                obj = json.loads(line)
                fields = {}
                for k in spec.text_fields:
                    if k not in obj:
                        raise ValueError(f"missing `{k}` in dataset record")
                    fields[k] = _as_text(obj[k])
                r = render_record(spec, fields)
                if r is not None:
                    records.append(r)
    elif spec.format == "text":
        name = spec.text_fields[0] if spec.text_fields else "text"
        with open(path) as f:
            for line in f:
                if full():
                    break
                line = line.rstrip("\n").rstrip("\r")
                if not line.strip():
                    continue
                r = render_record(spec, {name: line})
                if r is not None:
                    records.append(r)
    elif spec.format == "csv":
        with open(path, newline="") as f:
            reader = csv.reader(f)
            headers = next(reader)
            idx = {}
            for k in spec.text_fields:
                if k not in headers:
                    raise ValueError(f"missing field `{k}` in csv file {path}")
                idx[k] = headers.index(k)
            for row in reader:
                if full():
                    break
                if not row:
                    continue
                r = render_record(spec, {k: (row[i] if i < len(row) else "") for k, i in idx.items()})
                if r is not None:
                    records.append(r)
    elif spec.format == "parquet":
        import pyarrow.parquet as pq
        table = pq.read_table(path, columns=spec.text_fields)
        cols = {k: table.column(k).to_pylist() for k in spec.text_fields}
        for i in range(table.num_rows):
            if full():
                break
            fields = {k: ("" if cols[k][i] is None else _as_text(cols[k][i])) for k in spec.text_fields}
            r = render_record(spec, fields)
            if r is not None:
                records.append(r)
    else:
        raise ValueError(f"unknown record format {spec.format}")


def _hf_file(cache: Path, spec: HFSpec, name: str) -> Path:
    local = cache / "huggingface" / spec.repo_id.replace("/", "--") / (spec.revision or "main") / name
    if not local.exists():
        url = f"https://huggingface.co/datasets/{spec.repo_id}/resolve/{spec.revision or 'main'}/{name}"
        _fetch(url, local, f"{spec.repo_id}:{name}")
    return local


def _token_cache_path(cache: Path, spec: HFSpec, tok_cfg, files: List[Path]) -> Path:
    """Name of the encoded-corpus cache for this (dataset spec, tokenizer, source files) combination:
    any change of a source file's size or time stamp, of the record template or of the tokenizer
    settings gives another name, so a stale cache is never read."""
    import hashlib
    h = hashlib.sha1()
    h.update(repr((spec.repo_id, spec.revision, spec.format, spec.train_files, spec.validation_files,
                   spec.text_fields, spec.field_separator, spec.template, spec.max_records)).encode())
    h.update(repr(sorted(dataclasses.asdict(tok_cfg).items()) if dataclasses.is_dataclass(tok_cfg)
                  else repr(tok_cfg)).encode())
    vp = T.storage_path(tok_cfg, cache)
    for f in files + ([vp] if vp is not None else []):
        st = f.stat() if f.exists() else None
        h.update(repr((str(f.name), None if st is None else (st.st_size, st.st_mtime_ns))).encode())
    return cache / f"tokens-{h.hexdigest()[:16]}.npz"


def huggingface_dataset(cache_dir, block_size, batch_size, train_split_ratio, tok_cfg, spec: HFSpec, seed=0):
    """Records from a Hugging Face dataset repo, concatenated (src/dataset/huggingface.rs:36-191).
    The encoded corpus is cached beside the downloaded files (the reference re-reads and re-encodes
    every shard on every start); a later run with the same files and tokenizer maps it from disk."""
    if not spec.text_fields:
        raise ValueError("huggingface dataset requires at least one text field")
    cache = Path(cache_dir)
    cache.mkdir(parents=True, exist_ok=True)
    vocab_file = T.storage_path(tok_cfg, cache)
    local = [cache / "huggingface" / spec.repo_id.replace("/", "--") / (spec.revision or "main") / n
             for n in list(spec.train_files) + list(spec.validation_files)]
    if all(f.exists() for f in local) and (vocab_file is None or vocab_file.exists()):
        cached = _token_cache_path(cache, spec, tok_cfg, local)
        if cached.exists():
            with np.load(cached) as z:
                tokens, train_len = z["tokens"], int(z["train_len"])
            tok = T.load_or_fit(tok_cfg, cache, [])
            if len(tokens) > block_size + 1:
                train_len = min(max(train_len, block_size + 1), len(tokens) - 1)
                return TokenSequenceDataset(tokens, train_len, block_size, batch_size, train_split_ratio, tok, seed)
    train_records: List[str] = []
    for name in spec.train_files:
        if spec.max_records is not None and len(train_records) >= spec.max_records:
            break
        collect_records(_hf_file(cache, spec, name), spec, train_records)
    val_records: List[str] = []
    for name in spec.validation_files:
        collect_records(_hf_file(cache, spec, name), spec, val_records)
    if not train_records and not val_records:
        raise ValueError("huggingface dataset contains no records")
    tok = T.load_or_fit(tok_cfg, cache, train_records + val_records)
    for r in train_records + val_records:
        T.validate_corpus(tok_cfg, tok, r)
    parts, train_len, val_count = [], 0, 0
    for r in train_records:
        e = tok.encode_array(r)
        if len(e) < 2:
            continue
        train_len += len(e)
        parts.append(e)
    for r in val_records:
        e = tok.encode_array(r)
        if len(e) < 2:
            continue
        val_count += len(e)
        parts.append(e)
    tokens = np.concatenate(parts) if parts else np.zeros(0, dtype=np.int64)
    if len(tokens) <= block_size + 1:
        raise ValueError("encoded huggingface dataset smaller than block size")
    if val_count == 0:
        train_len = _clamp_train_len(len(tokens), train_split_ratio, block_size)
    elif train_len <= block_size:
        train_len = min(block_size + 1, len(tokens) - 1)
    if all(f.exists() for f in local):
        try:        # best effort: a read-only cache directory only costs the next start its speed-up
            np.savez(_token_cache_path(cache, spec, tok_cfg, local), tokens=tokens, train_len=np.int64(train_len))
        except OSError:
            pass
    return TokenSequenceDataset(tokens, train_len, block_size, batch_size, train_split_ratio, tok, seed)


def build_dataset(cfg, training) -> TokenSequenceDataset:
    """Dispatch on `[dataset].type` (src/dataset/factory.rs:10-127)."""
    bs, bt = training.block_size, training.batch_size
    seed = getattr(training, "seed", 0)
    if cfg.type == "shakespeare":
        return shakespeare_dataset(cfg.cache_dir, bs, bt, cfg.train_split_ratio, cfg.tokenizer, cfg.url, seed)
    if cfg.type == "synthetic":
        return synthetic_dataset(cfg.synthetic_tokens, bs, bt, 256, cfg.seed, cfg.train_split_ratio)
    if cfg.type == "hugging_face":
        spec = HFSpec(cfg.repo_id, cfg.revision, cfg.format, cfg.train_files, cfg.validation_files, cfg.text_fields,
                      cfg.field_separator, cfg.template, cfg.max_records)
    else:
        spec = hf_preset(cfg.type, cfg.revision, cfg.max_records)
    return huggingface_dataset(cfg.cache_dir, bs, bt, cfg.train_split_ratio, cfg.tokenizer, spec, seed)

"""Byte and character tokenizers.

Behaviour follows the reference (src/tokenizer/mod.rs:18-175, byte.rs:15-72, char_vocab.rs:12-239):

* ByteTokenizer: ids 0..255 are raw bytes; with `add_special_tokens` BOS=256, EOS=257, PAD=258
  are appended (vocab 259). Decoding drops PAD/BOS, stops at EOS and is lossy UTF-8.
* CharVocab: insertion-ordered set of characters, always starting with PAD U+0000, BOS U+0001,
  EOS U+0002 and (optionally) UNK U+0003. Unknown characters map to UNK, or raise if the vocabulary
  has none; UNK decodes as '?'. Stored as JSON {chars, bos, eos, pad, unk}.

Bulk encode/decode of long corpora go through numpy lookup tables rather than per-character
Python loops.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Iterable, List, Optional, Sequence

import numpy as np

PAD_CHAR, BOS_CHAR, EOS_CHAR, UNK_CHAR = "\u0000", "\u0001", "\u0002", "\u0003"


class Tokenizer:
    """Interface (src/tokenizer/mod.rs:18-28)."""

    def encode(self, text: str, add_bos: bool = False, add_eos: bool = False) -> List[int]:
        raise NotImplementedError

    def decode(self, ids: Sequence[int]) -> str:
        raise NotImplementedError

    def __len__(self) -> int:
        raise NotImplementedError

    bos_id: Optional[int] = None
    eos_id: Optional[int] = None
    pad_id: Optional[int] = None
    unk_id: Optional[int] = None

    def encode_array(self, text: str) -> np.ndarray:
        return np.asarray(self.encode(text), dtype=np.int64)


class ByteTokenizer(Tokenizer):
    def __init__(self, add_special_tokens: bool = True):
        self.add_special_tokens = add_special_tokens
        self.vocab_size = 256
        if add_special_tokens:
            self.bos_id, self.eos_id, self.pad_id = 256, 257, 258
            self.vocab_size = 259

    def encode(self, text, add_bos=False, add_eos=False):
        ids = list(text.encode("utf-8"))
        if add_bos and self.bos_id is not None:
            ids.insert(0, self.bos_id)
        if add_eos and self.eos_id is not None:
            ids.append(self.eos_id)
        return ids

    def encode_array(self, text):
        return np.frombuffer(text.encode("utf-8"), dtype=np.uint8).astype(np.int64)

    def decode(self, ids):
        out = bytearray()
        for i in ids:
            i = int(i)
            if i == self.pad_id or i == self.bos_id:
                continue
            if i == self.eos_id and self.eos_id is not None:
                break
            if 0 <= i < 256:
                out.append(i)
        return out.decode("utf-8", errors="replace")

    def __len__(self):
        return self.vocab_size

    def __eq__(self, other):
        return isinstance(other, ByteTokenizer) and other.add_special_tokens == self.add_special_tokens


class CharVocab(Tokenizer):
    def __init__(self, chars: Sequence[str], include_unknown: bool):
        if not chars:
            raise ValueError("vocabulary cannot be empty")
        self.id2ch = list(chars)
        self.ch2id = {}
        for i, ch in enumerate(self.id2ch):
            if ch in self.ch2id:
                raise ValueError(f"duplicate character {ch!r}")
            self.ch2id[ch] = i
        for name, ch in (("BOS", BOS_CHAR), ("EOS", EOS_CHAR), ("PAD", PAD_CHAR)):
            if ch not in self.ch2id:
                raise ValueError(f"missing {name} character in vocabulary")
        self.bos_id, self.eos_id, self.pad_id = self.ch2id[BOS_CHAR], self.ch2id[EOS_CHAR], self.ch2id[PAD_CHAR]
        self.unk_id = self.ch2id.get(UNK_CHAR) if include_unknown else None

    @staticmethod
    def fit(texts: Iterable[str], include_unknown: bool = True) -> "CharVocab":
        chars = [PAD_CHAR, BOS_CHAR, EOS_CHAR] + ([UNK_CHAR] if include_unknown else [])
        seen = set(chars)
        for text in texts:
            # first-occurrence order, as an insertion-ordered set would give
            for ch in dict.fromkeys(text):
                if ch not in seen:
                    seen.add(ch)
                    chars.append(ch)
        return CharVocab(chars, include_unknown)

    # ---- JSON record ----
    def to_record(self) -> dict:
        return dict(chars=self.id2ch, bos=self.bos_id, eos=self.eos_id, pad=self.pad_id, unk=self.unk_id)

    @staticmethod
    def from_record(rec: dict) -> "CharVocab":
        v = CharVocab(rec["chars"], rec.get("unk") is not None)
        v.bos_id, v.eos_id, v.pad_id, v.unk_id = rec["bos"], rec["eos"], rec["pad"], rec.get("unk")
        return v

    def save(self, path) -> None:
        p = Path(path)
        p.parent.mkdir(parents=True, exist_ok=True)
        p.write_text(json.dumps(self.to_record(), indent=2, ensure_ascii=True))

    @staticmethod
    def load(path) -> "CharVocab":
        return CharVocab.from_json_str(Path(path).read_text())

    @staticmethod
    def from_json_str(data: str) -> "CharVocab":
        return CharVocab.from_record(json.loads(data))

    # ---- encode / decode ----
    def contains(self, ch: str) -> bool:
        return ch in self.ch2id

    def _lookup(self, ch: str) -> int:
        i = self.ch2id.get(ch)
        if i is None:
            if self.unk_id is None:
                raise KeyError(f"character {ch!r} missing from vocabulary and no <unk> token configured")
            return self.unk_id
        return i

    def encode(self, text, add_bos=False, add_eos=False):
        ids = [self._lookup(ch) for ch in text]
        if add_bos:
            ids.insert(0, self.bos_id)
        if add_eos:
            ids.append(self.eos_id)
        return ids

    def _table(self) -> np.ndarray:
        t = getattr(self, "_cp_table", None)
        if t is None:
            t = np.full(max(ord(c) for c in self.id2ch) + 1, -1, dtype=np.int32)
            for ch, i in self.ch2id.items():
                t[ord(ch)] = i
            self._cp_table = t
        return t

    def encode_array(self, text):
        from ..utils import hostlib
        if hostlib.available():
            # native scan of the UTF-8 bytes (the whole-corpus path of the dataset builders)
            try:
                return hostlib.encode_utf8_chars(text.encode("utf-8", "surrogatepass"), self._table(), self.unk_id)
            except KeyError as e:
                raise KeyError(f"character {e.args[0]!r} missing from vocabulary and no <unk> token configured") from None
        cps = np.frombuffer(text.encode("utf-32-le"), dtype=np.uint32)
        if cps.size == 0:
            return np.zeros(0, dtype=np.int64)
        table = np.full(int(max(cps.max(), max(ord(c) for c in self.id2ch))) + 1,
                        -1 if self.unk_id is None else self.unk_id, dtype=np.int64)
        for ch, i in self.ch2id.items():
            table[ord(ch)] = i
        out = table[cps]
        if self.unk_id is None and (out < 0).any():
            bad = chr(int(cps[np.argmax(out < 0)]))
            raise KeyError(f"character {bad!r} missing from vocabulary and no <unk> token configured")
        return out

    def decode(self, ids):
        out = []
        for i in ids:
            i = int(i)
            if not 0 <= i < len(self.id2ch):
                raise IndexError(f"token id {i} out of range")
            if i == self.pad_id or i == self.bos_id:
                continue
            if i == self.eos_id:
                break
            out.append("?" if i == self.unk_id else self.id2ch[i])
        return "".join(out)

    def __len__(self):
        return len(self.id2ch)

    def __eq__(self, other):
        return isinstance(other, CharVocab) and self.to_record() == other.to_record()


# ---- TokenizerConfig helpers (src/tokenizer/mod.rs:92-175) ----------------------------------------
def storage_path(cfg, cache_dir) -> Optional[Path]:
    if cfg.type != "char":
        return None
    if cfg.vocab_path:
        p = Path(cfg.vocab_path)
        return p if p.is_absolute() else Path(cache_dir) / p
    return Path(cache_dir) / "vocab.json"


def load_tokenizer(cfg, path=None) -> Tokenizer:
    if cfg.type == "char":
        return CharVocab.load(path)
    return ByteTokenizer(cfg.add_special_tokens)


def fit_tokenizer(cfg, texts: Iterable[str]) -> Tokenizer:
    if cfg.type == "char":
        return CharVocab.fit(texts, cfg.include_unknown)
    return ByteTokenizer(cfg.add_special_tokens)


def save_tokenizer(cfg, tok: Tokenizer, path) -> None:
    if cfg.type == "char":
        if not isinstance(tok, CharVocab):
            raise TypeError("expected char tokenizer")
        tok.save(path)


def validate_corpus(cfg, tok: Tokenizer, text: str) -> None:
    if cfg.type == "char" and not cfg.include_unknown:
        for ch in set(text):
            if not tok.contains(ch):
                raise ValueError(f"vocabulary missing character {ch!r} found in dataset")


def load_or_fit(cfg, cache_dir, texts: Iterable[str]) -> Tokenizer:
    """Load the stored vocabulary if there is one, else fit on `texts` and store it."""
    path = storage_path(cfg, cache_dir)
    if path is not None and path.exists():
        return load_tokenizer(cfg, path)
    tok = fit_tokenizer(cfg, texts)
    if path is not None:
        save_tokenizer(cfg, tok, path)
    return tok

"""Reader / writer for the reference's checkpoint files (`model-N.bin`, Burn `BinFileRecorder`).

File = bincode 2 (varint integers) of BurnRecord{metadata, item}:

    metadata : 5 strings  float ("f32" | "f16"), int ("i32"), format (recorder type name),
               version ("0.19.1"), settings ("FullPrecisionSettings" | "HalfPrecisionSettings")
    item     : the BDH module record in field order (reference: src/model/bdh.rs:19-34)
        5 constant placeholders (n_layer, n_embd, n_head, multiplier, vocab_size)   -> 5 x 0x00
        kernel config                                                               -> 0 bytes
        embed.weight  : param
        dropout       : 1 placeholder byte
        attention     : 5 placeholder bytes
        encoder, encoder_v, decoder, lm_head : params
    param    : String id (13 chars) . Vec<u8> raw little-endian data . Vec<usize> shape . dtype enum

Hyper-parameters are not in the file; they come from the side-car `config.json`, the vocabulary from
`vocab.json` (reference: src/bin/train.rs:691-718, src/tokenizer/char_vocab.rs:232-239).

Layout conversion: the reference stores encoder / encoder_v as [H, D, N] and decoder as [H*N, D];
this framework keeps all three neuron-major [H*N, D].
"""
from __future__ import annotations

import json
import random
import string
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Optional, Tuple

import numpy as np
import torch

from ..utils import hostlib

FULL = ("f32", "i32", "burn_core::record::file::BinFileRecorder<burn_core::record::settings::FullPrecisionSettings>",
        "0.19.1", "FullPrecisionSettings")
HALF = ("f16", "i32", "burn_core::record::file::BinFileRecorder<burn_core::record::settings::HalfPrecisionSettings>",
        "0.19.1", "HalfPrecisionSettings")
# Variant index of burn-tensor 0.19.1's `DType` enum, which is declared in the order
# F64, F32, Flex32, F16, BF16, ...: F32 = 1 is what the reference's shipped f32 record carries, so
# F16 is variant 3 (2 is Flex32, a 4-byte type). No reference-written f16 file exists to pin this.
DTYPE_F32 = 1
DTYPE_F16 = 3
DTYPE_F16_LEGACY = 2   # written for f16 by earlier versions of this library; accepted on read only
PARAM_ORDER = ("embed.weight", "encoder", "encoder_v", "decoder", "lm_head")


# ---- bincode primitives -----------------------------------------------------------------------------
def read_varint(buf: bytes, pos: int) -> Tuple[int, int]:
    b = buf[pos]
    if b < 251:
        return b, pos + 1
    n = {251: 2, 252: 4, 253: 8}.get(b)
    if n is None:
        raise ValueError(f"unsupported varint tag {b} at {pos}")
    return int.from_bytes(buf[pos + 1:pos + 1 + n], "little"), pos + 1 + n


def write_varint(v: int) -> bytes:
    if v < 251:
        return bytes([v])
    if v <= 0xFFFF:
        return b"\xfb" + v.to_bytes(2, "little")
    if v <= 0xFFFFFFFF:
        return b"\xfc" + v.to_bytes(4, "little")
    return b"\xfd" + v.to_bytes(8, "little")


def read_string(buf: bytes, pos: int) -> Tuple[str, int]:
    n, pos = read_varint(buf, pos)
    return buf[pos:pos + n].decode("utf-8"), pos + n


def write_string(s: str) -> bytes:
    b = s.encode("utf-8")
    return write_varint(len(b)) + b


@dataclass
class ParamRecord:
    id: str
    data: np.ndarray      # shaped, float32 or float16
    dtype_tag: int


@dataclass
class BurnRecord:
    metadata: Tuple[str, str, str, str, str]
    params: Dict[str, ParamRecord]      # keyed by PARAM_ORDER names

    @property
    def half(self) -> bool:
        return self.metadata[0] == "f16"


def _read_param(buf: bytes, pos: int, np_dtype) -> Tuple[ParamRecord, int]:
    if hostlib.available():
        nxt, pid, off, ln, shape, tag = hostlib.scan_param(buf, pos)
    else:
        pid, p = read_string(buf, pos)
        ln, p = read_varint(buf, p)
        off = p
        p += ln
        nd, p = read_varint(buf, p)
        shape = []
        for _ in range(nd):
            d, p = read_varint(buf, p)
            shape.append(d)
        tag, nxt = read_varint(buf, p)
    arr = np.frombuffer(buf, dtype=np_dtype, count=ln // np.dtype(np_dtype).itemsize, offset=off).reshape(shape)
    return ParamRecord(pid, arr, tag), nxt


def _write_param(p: ParamRecord) -> bytes:
    raw = np.ascontiguousarray(p.data).tobytes()
    out = [write_string(p.id), write_varint(len(raw)), raw, write_varint(p.data.ndim)]
    out += [write_varint(int(d)) for d in p.data.shape]
    out.append(write_varint(p.dtype_tag))
    return b"".join(out)


def parse(buf: bytes) -> BurnRecord:
    pos = 0
    meta = []
    for _ in range(5):
        s, pos = read_string(buf, pos)
        meta.append(s)
    np_dtype = np.float16 if meta[0] == "f16" else np.float32
    if buf[pos:pos + 5] != b"\x00" * 5:
        raise ValueError("unexpected module header (expected five constant placeholders)")
    pos += 5
    params = {}
    params["embed.weight"], pos = _read_param(buf, pos, np_dtype)
    if buf[pos:pos + 6] != b"\x00" * 6:
        raise ValueError("unexpected dropout/attention placeholders")
    pos += 6
    for name in PARAM_ORDER[1:]:
        params[name], pos = _read_param(buf, pos, np_dtype)
    if pos != len(buf):
        raise ValueError(f"{len(buf) - pos} trailing bytes after the last parameter")
    # the per-tensor dtype tag has to agree with the float type the metadata names
    ok_tags = (DTYPE_F16, DTYPE_F16_LEGACY) if meta[0] == "f16" else (DTYPE_F32,)
    for name, p in params.items():
        if p.dtype_tag not in ok_tags:
            raise ValueError(f"{name}: dtype tag {p.dtype_tag} does not match a `{meta[0]}` record "
                             f"(expected {ok_tags[0]})")
        if p.dtype_tag == DTYPE_F16_LEGACY:
            p.dtype_tag = DTYPE_F16
    return BurnRecord(tuple(meta), params)


def serialize(rec: BurnRecord) -> bytes:
    out = [write_string(s) for s in rec.metadata]
    out.append(b"\x00" * 5)
    out.append(_write_param(rec.params["embed.weight"]))
    out.append(b"\x00" * 6)
    for name in PARAM_ORDER[1:]:
        out.append(_write_param(rec.params[name]))
    return b"".join(out)


def load(path) -> BurnRecord:
    return parse(Path(path).read_bytes())


def save(rec: BurnRecord, path) -> None:
    p = Path(path)
    p.parent.mkdir(parents=True, exist_ok=True)
    p.write_bytes(serialize(rec))


def new_param_id(rng: Optional[random.Random] = None) -> str:
    """13 lowercase alphanumerics, the shape of the ids the reference writes."""
    r = rng or random
    return "".join(r.choice(string.ascii_lowercase + string.digits) for _ in range(13))


# ---- model <-> record -----------------------------------------------------------------------------
def infer_dims(rec: BurnRecord) -> Dict[str, int]:
    """Model dimensions implied by the tensor shapes of a record."""
    V, D = rec.params["embed.weight"].data.shape
    H, D2, N = rec.params["encoder"].data.shape
    assert D == D2
    return dict(vocab_size=int(V), n_embd=int(D), n_head=int(H), n_latent_per_head=int(N))


def to_state_dict(rec: BurnRecord) -> Dict[str, torch.Tensor]:
    """Reference layout -> this framework's parameter layout (fp32)."""
    p = {k: torch.from_numpy(np.array(v.data, dtype=np.float32)) for k, v in rec.params.items()}
    H, D, N = p["encoder"].shape
    return {
        "embed.weight": p["embed.weight"],
        "encoder": p["encoder"].permute(0, 2, 1).reshape(H * N, D).contiguous(),
        "encoder_v": p["encoder_v"].permute(0, 2, 1).reshape(H * N, D).contiguous(),
        "decoder": p["decoder"].contiguous(),
        "lm_head": p["lm_head"].contiguous(),
    }


def from_model(model, half: bool = False, ids: Optional[Dict[str, str]] = None) -> BurnRecord:
    """This framework's BDH -> a record in the reference's layout (f32, or f16 when `half`)."""
    c = model.config
    H, N, D = c.n_head, c.latent_per_head, c.n_embd
    sd = {k: v.detach().float().cpu() for k, v in model.state_dict().items()}
    tensors = {
        "embed.weight": sd["embed.weight"],
        "encoder": sd["encoder"].view(H, N, D).permute(0, 2, 1).contiguous(),
        "encoder_v": sd["encoder_v"].view(H, N, D).permute(0, 2, 1).contiguous(),
        "decoder": sd["decoder"],
        "lm_head": sd["lm_head"],
    }
    params = {}
    for name in PARAM_ORDER:
        a = tensors[name].numpy()
        if half:
            a = hostlib.f32_to_f16(a) if hostlib.available() else a.astype(np.float16)
        params[name] = ParamRecord((ids or {}).get(name) or new_param_id(), a, DTYPE_F16 if half else DTYPE_F32)
    return BurnRecord(HALF if half else FULL, params)


def load_into(model, path) -> None:
    """Load a reference checkpoint (f32 or f16) into a BDH whose config matches its shapes."""
    rec = load(path)
    sd = to_state_dict(rec)
    own = model.state_dict()
    for k, v in sd.items():
        if tuple(own[k].shape) != tuple(v.shape):
            raise ValueError(f"{k}: checkpoint shape {tuple(v.shape)} != model shape {tuple(own[k].shape)}")
    model.load_state_dict(sd, strict=True)
    flat = getattr(model, "_flat_params", None)
    if flat is not None:
        flat.refresh_shadow()


def quantize_file(src, dst=None) -> Path:
    """f32 record -> f16 record next to it, named `<stem>-f16.bin` (src/bin/quantize.rs:36-86)."""
    src = Path(src)
    rec = load(src)
    params = {}
    for k, p in rec.params.items():
        a = np.asarray(p.data, dtype=np.float32)
        a16 = hostlib.f32_to_f16(a) if hostlib.available() else a.astype(np.float16)
        params[k] = ParamRecord(p.id, a16, DTYPE_F16)
    out = Path(dst) if dst else src.with_name(src.stem + "-f16.bin")
    save(BurnRecord(HALF, params), out)
    return out


def read_run_config(path) -> Dict:
    """`runs/<name>/config.json` = {run_name, block_size, overrides} (src/bin/train.rs:691-718)."""
    return json.loads(Path(path).read_text())

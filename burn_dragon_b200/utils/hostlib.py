"""ctypes front end of the host-side native library (`_host.so`): window gathering for the data
loader, bincode varints and parameter scanning for the Burn record codec, fp32->fp16 conversion.
Built by `burn_dragon_b200.build`; every caller has a numpy fallback, so a missing library only
costs speed."""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import numpy as np

_LIB = None
_PATH = Path(__file__).resolve().parent.parent / "_host.so"


def _load():
    global _LIB
    if _LIB is None and _PATH.exists():
        try:
            lib = ctypes.CDLL(str(_PATH))
            lib.bdh_gather_windows.restype = ctypes.c_int
            lib.bdh_record_scan_param.restype = ctypes.c_int64
            lib.bdh_varint_read.restype = ctypes.c_int
            lib.bdh_varint_write.restype = ctypes.c_int
            lib.bdh_encode_utf8_chars.restype = ctypes.c_int64
            lib.bdh_sim_flag_barrier.restype = ctypes.c_int
            lib.bdh_oracle_forward.restype = ctypes.c_int
            _LIB = lib
        except OSError:
            _LIB = False
    return _LIB or None


def available() -> bool:
    return _load() is not None


def gather_windows(tokens: np.ndarray, starts: np.ndarray, width: int, out) -> None:
    """out (torch int64 [rows, width], contiguous host tensor) <- token windows."""
    lib = _load()
    starts = np.ascontiguousarray(starts, dtype=np.int64)
    rc = lib.bdh_gather_windows(ctypes.c_void_p(tokens.ctypes.data), ctypes.c_int64(len(tokens)),
                                ctypes.c_void_p(starts.ctypes.data), ctypes.c_int64(len(starts)),
                                ctypes.c_int64(width), ctypes.c_void_p(out.data_ptr()),
                                ctypes.c_int(min(8, os.cpu_count() or 1)))
    if rc != 0:
        raise IndexError("window start out of range")


def scan_param(buf: bytes, pos: int):
    """Parse one serialized parameter at `pos`. Returns (next_pos, id, data_off, data_len, shape, dtype)."""
    lib = _load()
    out = (ctypes.c_int64 * 13)()
    nxt = lib.bdh_record_scan_param(ctypes.c_char_p(buf), ctypes.c_int64(len(buf)), ctypes.c_int64(pos), out)
    if nxt < 0:
        raise ValueError("malformed parameter record")
    pid = buf[out[0]:out[0] + out[1]].decode("utf-8")
    shape = [int(out[5 + i]) for i in range(int(out[4]))]
    return int(nxt), pid, int(out[2]), int(out[3]), shape, int(out[12])


def f32_to_f16(a: np.ndarray) -> np.ndarray:
    lib = _load()
    a = np.ascontiguousarray(a, dtype=np.float32)
    out = np.empty(a.shape, dtype=np.uint16)
    lib.bdh_f32_to_f16(ctypes.c_void_p(a.ctypes.data), ctypes.c_void_p(out.ctypes.data), ctypes.c_int64(a.size))
    return out.view(np.float16)


def encode_utf8_chars(data: bytes, table: np.ndarray, unk_id) -> np.ndarray:
    """Character ids of UTF-8 `data` through `table` (int32, code point -> id or -1). Raises KeyError
    with the first character that is not in the vocabulary when `unk_id` is None."""
    lib = _load()
    table = np.ascontiguousarray(table, dtype=np.int32)
    out = np.empty(len(data), dtype=np.int64)
    bad = ctypes.c_int64(0)
    n = lib.bdh_encode_utf8_chars(ctypes.c_char_p(data), ctypes.c_int64(len(data)), ctypes.c_void_p(table.ctypes.data),
                                  ctypes.c_int64(table.size), ctypes.c_int32(-1 if unk_id is None else int(unk_id)),
                                  ctypes.c_void_p(out.ctypes.data), ctypes.byref(bad))
    if n < 0:
        raise KeyError(chr(bad.value))
    return out[:n]


def simulate_flag_barrier(world: int, ctas: int, calls: int, first_epoch: int = 0, seed: int = 0,
                          spin_limit: int = 50_000_000) -> int:
    """Run the cross-rank flag barrier protocol on real threads (one per rank and CTA) with random
    yields; 0 = every ordering check held, 1 = a stale or early payload was seen, 2 = a wait ran out."""
    lib = _load()
    return int(lib.bdh_sim_flag_barrier(ctypes.c_int(world), ctypes.c_int(ctas), ctypes.c_int(calls),
                                        ctypes.c_uint32(first_epoch & 0xFFFFFFFF), ctypes.c_uint64(seed),
                                        ctypes.c_int64(spin_limit)))


def oracle_forward(model, tokens, pos0: int = 0, want_state: bool = False):
    """Logits [T, V] of one token sequence through the plain C++ restatement of the canonical
    (recurrent) BDH forward (csrc/host/oracle.cpp: fp32 weights, double accumulators). With
    `want_state` also returns the last layer's final state [H, N', D] (float64)."""
    import torch
    lib = _load()
    c = model.config
    kind = {"alibi": 0, "rope": 1, "pope": 2}[c.rotary_embedding]
    f32 = lambda t: np.ascontiguousarray(t.detach().cpu().to(torch.float32).numpy())
    w = [f32(model.embed.weight), f32(model.encoder), f32(model.encoder_v), f32(model.decoder), f32(model.lm_head)]
    freqs, slopes = f32(model.freqs), f32(model.slopes)
    toks = np.ascontiguousarray(np.asarray(tokens, dtype=np.int64).reshape(-1))
    T, H, N, D, V = len(toks), c.n_head, c.latent_per_head, c.n_embd, c.vocab_size
    logits = np.empty((T, V), dtype=np.float32)
    Np = 2 * N if kind == 2 else N
    rho = np.empty((H, Np, D), dtype=np.float64) if want_state else None
    ptr = lambda a: ctypes.c_void_p(a.ctypes.data)
    rc = lib.bdh_oracle_forward(ptr(w[0]), ptr(w[1]), ptr(w[2]), ptr(w[3]), ptr(w[4]), ptr(freqs), ptr(slopes), ptr(toks),
                                ctypes.c_int(T), ctypes.c_int(c.n_layer), ctypes.c_int(D), ctypes.c_int(H),
                                ctypes.c_int(N), ctypes.c_int(V), ctypes.c_int(kind),
                                ctypes.c_float(float(c.relu_threshold)), ctypes.c_int(pos0), ptr(logits),
                                ptr(rho) if want_state else ctypes.c_void_p(0))
    if rc != 0:
        raise ValueError("oracle_forward: bad argument")
    return (logits, rho) if want_state else logits

"""Image files for the headless visualiser: linear float RGB -> 8-bit sRGB, and a dependency-free
PNG writer (the reference shows these images in a window, src/viz/bevy_app.rs:155-242; here they
are device buffers that can be written to disk)."""
from __future__ import annotations

import struct
import zlib

import numpy as np


def linear_to_srgb8(rgb: np.ndarray) -> np.ndarray:
    """[..., 3] linear floats -> uint8 sRGB (inverse of `encoder.srgb_to_linear`)."""
    v = np.clip(np.asarray(rgb, dtype=np.float32), 0.0, 1.0)
    out = np.where(v <= 0.0031308, v * 12.92, 1.055 * np.power(v, 1.0 / 2.4) - 0.055)
    return np.clip(np.rint(out * 255.0), 0, 255).astype(np.uint8)


def _chunk(tag: bytes, data: bytes) -> bytes:
    return struct.pack(">I", len(data)) + tag + data + struct.pack(">I", zlib.crc32(tag + data) & 0xFFFFFFFF)


def write_png(path, rgb8: np.ndarray) -> None:
    """rgb8: uint8 [height, width, 3] -> 8-bit truecolour PNG, no interlace, filter type 0."""
    a = np.ascontiguousarray(rgb8, dtype=np.uint8)
    if a.ndim != 3 or a.shape[2] != 3:
        raise ValueError("expected an [height, width, 3] uint8 array")
    h, w, _ = a.shape
    rows = np.concatenate([np.zeros((h, 1), dtype=np.uint8), a.reshape(h, w * 3)], axis=1)
    png = (b"\x89PNG\r\n\x1a\n" + _chunk(b"IHDR", struct.pack(">IIBBBBB", w, h, 8, 2, 0, 0, 0)) +
           _chunk(b"IDAT", zlib.compress(rows.tobytes(), 6)) + _chunk(b"IEND", b""))
    with open(path, "wb") as f:
        f.write(png)


def read_png_rgb8(path) -> np.ndarray:
    """Reader for the files `write_png` makes (filter 0 rows only)."""
    buf = open(path, "rb").read()
    if buf[:8] != b"\x89PNG\r\n\x1a\n":
        raise ValueError("not a PNG file")
    pos, w, h, data = 8, 0, 0, b""
    while pos < len(buf):
        n, tag = struct.unpack(">I4s", buf[pos:pos + 8])
        body = buf[pos + 8:pos + 8 + n]
        if tag == b"IHDR":
            w, h = struct.unpack(">II", body[:8])
        elif tag == b"IDAT":
            data += body
        pos += 12 + n
    rows = np.frombuffer(zlib.decompress(data), dtype=np.uint8).reshape(h, 1 + 3 * w)
    if rows[:, 0].any():
        raise ValueError("only filter type 0 is supported")
    return rows[:, 1:].reshape(h, w, 3).copy()

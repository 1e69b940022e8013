"""Activation -> image encoder (src/viz/encoder.rs:18-298, frame.rs:4-57, palette.rs).

Four images `[units_height, history, 4]` (fp32 RGBA, linear colour): x ("writes"), y ("activity"),
x*y ("interaction") and the per-neuron state energy rho ("memory"). Each decoded token fills
column `token_index % history`; visible layers are stacked with a 20-row gap, newest layers last.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from ..ops import native

LAYER_GAP = 20
VIZ_MAX_RES = 8192
SOFT_CLIP, ACTIVE_EPS, INTENSITY_GAMMA = 0.35, 1e-3, 1.15

COLOR_ACTIVITY = ((0.059, 0.165, 0.208), (0.176, 0.902, 1.000))
COLOR_WRITES = ((0.176, 0.106, 0.027), (1.000, 0.620, 0.173))
COLOR_INTERACTION = ((0.063, 0.192, 0.118), (0.235, 0.961, 0.604))
COLOR_MEMORY = ((0.176, 0.067, 0.153), (1.000, 0.365, 0.839))
COLOR_SEPARATOR = (0.255, 0.282, 0.325)


def srgb_to_linear(v: float) -> float:
    return v / 12.92 if v <= 0.04045 else ((v + 0.055) / 1.055) ** 2.4


def _lin(c: Sequence[float]) -> List[float]:
    return [srgb_to_linear(x) for x in c]


def clamp_history(history: int) -> int:
    return min(max(history, 1), VIZ_MAX_RES)


def clamp_layers(layers: int, latent_total: int) -> int:
    layers, latent_total = max(layers, 1), max(latent_total, 1)
    step = max(latent_total + LAYER_GAP, 1)
    return min(layers, max((VIZ_MAX_RES + LAYER_GAP) // step, 1))


def units_height(layers: int, latent_total: int) -> int:
    layers, latent_total = max(layers, 1), max(latent_total, 1)
    return max(latent_total * layers + LAYER_GAP * (layers - 1), 1)


@dataclass
class VizConfig:
    history: int = 256
    layer_focus: int = 0
    stride_tokens: int = 1
    gain_x: float = 1.0
    gain_xy: float = 1.0


@dataclass
class VizFrame:
    units_x: torch.Tensor
    units_y: torch.Tensor
    units_xy: torch.Tensor
    units_rho: torch.Tensor
    cursor: int
    token_index: int


def encode_units_reference(values: torch.Tensor, gain: float, low, high, sep, units_per_head: int) -> torch.Tensor:
    """[units] -> [units, 4] column, plain torch (the definition the kernel is tested against)."""
    v = values.float().clamp_min(0.0)
    sc = v * gain
    inten = ((sc / (sc + SOFT_CLIP)) * (v / (v + ACTIVE_EPS * 4.0))).pow(INTENSITY_GAMMA).unsqueeze(-1)
    lo = torch.tensor(low, device=v.device)
    hi = torch.tensor(high, device=v.device)
    rgb = (lo + (hi - lo) * inten) * inten
    if units_per_head > 0:
        idx = torch.arange(v.numel(), device=v.device)
        is_sep = ((idx > 0) & (idx % units_per_head == 0)).unsqueeze(-1)
        rgb = torch.where(is_sep, torch.maximum(rgb, torch.tensor(sep, device=v.device)), rgb)
    return torch.cat((rgb, torch.ones_like(inten)), dim=-1)


class VizEncoder:
    def __init__(self, config: VizConfig, model_config=None, device=None, layers: Optional[int] = None,
                 heads: Optional[int] = None, latent_per_head: Optional[int] = None):
        if model_config is not None:
            layers, heads, latent_per_head = model_config.n_layer, model_config.n_head, model_config.latent_per_head
        self.config = VizConfig(**{**config.__dict__, "history": clamp_history(config.history)})
        self.heads, self.latent_per_head = heads, latent_per_head
        self.latent_total = max(heads * latent_per_head, 1)
        self.layers_visible = clamp_layers(max(layers, 1), self.latent_total)
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        h = units_height(self.layers_visible, self.latent_total)
        shape = (h, self.config.history, 4)
        self.units_x = torch.zeros(shape, device=self.device)
        self.units_y = torch.zeros(shape, device=self.device)
        self.units_xy = torch.zeros(shape, device=self.device)
        self.units_rho = torch.zeros(shape, device=self.device)
        self.token_index = 0
        self._sep = _lin(COLOR_SEPARATOR)

    def should_capture(self, token_index: Optional[int] = None) -> bool:
        t = self.token_index if token_index is None else token_index
        return t % max(self.config.stride_tokens, 1) == 0

    def _write(self, image, values, gain, colors, row0, cursor):
        lo, hi = _lin(colors[0]), _lin(colors[1])
        v = values.reshape(-1).float().contiguous()
        if image.is_cuda and native.available():
            native.ops.viz_encode_units(v, image, cursor, row0, float(gain), lo, hi, self._sep, self.latent_per_head)
        else:
            image[row0:row0 + v.numel(), cursor] = encode_units_reference(v, gain, lo, hi, self._sep,
                                                                          self.latent_per_head)

    def step(self, layers: Sequence[Optional[dict]], token_index: Optional[int] = None, stream: int = 0) -> VizFrame:
        """`layers`: per-layer dicts with x_last / y_last / xy_last / rho_last of shape [B, H, N] (what
        `ModelState.take_viz()` returns); stream `stream` of the batch is drawn."""
        t = self.token_index if token_index is None else token_index
        cursor = t % max(self.config.history, 1)
        avail = max(len(layers), 1)
        count = max(min(self.layers_visible, avail), 1)
        start = avail - count
        zeros = torch.zeros(self.heads, self.latent_per_head, device=self.device)
        for i in range(count):
            off = i * (self.latent_total + LAYER_GAP)
            if i > 0:
                for img in (self.units_x, self.units_y, self.units_xy, self.units_rho):
                    img[off - LAYER_GAP:off, cursor] = 0
            st = layers[start + i] if start + i < len(layers) else None

            def pick(name):
                if st is None or st.get(name) is None:
                    return zeros
                v = st[name]
                return v[stream] if v.dim() == 3 else v
            self._write(self.units_x, pick("x_last"), self.config.gain_x, COLOR_WRITES, off, cursor)
            self._write(self.units_y, pick("y_last"), self.config.gain_xy, COLOR_ACTIVITY, off, cursor)
            self._write(self.units_xy, pick("xy_last"), self.config.gain_xy, COLOR_INTERACTION, off, cursor)
            self._write(self.units_rho, pick("rho_last"), self.config.gain_xy, COLOR_MEMORY, off, cursor)
        self.token_index = t + 1
        return VizFrame(self.units_x, self.units_y, self.units_xy, self.units_rho, cursor, t)

    def panel_grid(self, gap: int = 8) -> torch.Tensor:
        """The four images as one 2x2 grid (x | y over x*y | rho), the arrangement of the reference's
        window (src/viz/bevy_app.rs:538-641), linear RGBA float [2h + gap, 2w + gap, 4]."""
        h, w, _ = self.units_x.shape
        grid = torch.zeros(2 * h + gap, 2 * w + gap, 4, device=self.units_x.device)
        grid[..., 3] = 1.0
        grid[:h, :w] = self.units_x
        grid[:h, w + gap:] = self.units_y
        grid[h + gap:, :w] = self.units_xy
        grid[h + gap:, w + gap:] = self.units_rho
        return grid

    def save(self, path) -> None:
        """Write the four images to an .npz file; `.png` writes the 2x2 panel grid as 8-bit sRGB
        (the headless stand-in for the reference's window), `.ppm` the x image alone."""
        import numpy as np
        path = str(path)
        imgs = dict(x=self.units_x, y=self.units_y, xy=self.units_xy, rho=self.units_rho)
        if path.endswith(".png"):
            from .image import linear_to_srgb8, write_png
            write_png(path, linear_to_srgb8(self.panel_grid()[..., :3].cpu().numpy()))
            return
        if path.endswith(".ppm"):
            a = (self.units_x[..., :3].clamp(0, 1).pow(1 / 2.2) * 255).byte().cpu().numpy()
            with open(path, "wb") as f:
                f.write(f"P6 {a.shape[1]} {a.shape[0]} 255\n".encode())
                f.write(a.tobytes())
            return
        np.savez_compressed(path, **{k: v.cpu().numpy() for k, v in imgs.items()})

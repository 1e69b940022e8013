"""Headless activation visualiser: activations -> RGBA ring-buffer images on the device.

The reference renders these images in a Bevy window that shares a wgpu device with the model
(src/viz/bevy_app.rs, src/viz/mod.rs); a graphics stack is not available here, so the images stay
device buffers and can be written to `.npz` / `.ppm` files. The arithmetic is the reference's
(src/viz/encoder.rs, frame.rs, palette.rs, transport.rs).
"""
from .encoder import VizConfig, VizEncoder, VizFrame, clamp_history, clamp_layers, units_height  # noqa: F401
from .transport import channel  # noqa: F401

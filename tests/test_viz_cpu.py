import torch

from burn_dragon_b200.models.bdh import BDH, BDHConfig
from burn_dragon_b200.viz import VizConfig, VizEncoder, channel, clamp_history, clamp_layers, units_height
from burn_dragon_b200.viz.encoder import LAYER_GAP


def test_frame_helpers():
    assert clamp_history(0) == 1 and clamp_history(10 ** 6) == 8192
    assert units_height(2, 8) == 2 * 8 + LAYER_GAP
    assert clamp_layers(100, 4000) == 2 and clamp_layers(3, 8) == 3


def test_state_capture_shapes_and_encoder_output():
    torch.manual_seed(0)
    cfg = BDHConfig(n_layer=2, n_embd=16, n_head=2, mlp_internal_dim_multiplier=1, vocab_size=32, dropout=0.0)
    m = BDH(cfg).eval()
    m.capture_viz = True
    st = m.init_state()
    m.forward_with_state(torch.randint(0, 32, (1, 5)), st, mode="recurrent")
    layers = st.take_viz()
    assert st.viz is None and len(layers) == 2
    assert layers[0]["x_last"].shape == (1, 2, 8) and layers[0]["rho_last"].shape == (1, 2, 8)
    enc = VizEncoder(VizConfig(history=4), cfg)
    fr = enc.step(layers, token_index=6)
    assert fr.units_x.shape == (units_height(2, 16), 4, 4) and fr.cursor == 2 and fr.token_index == 6
    col = fr.units_y[:, 2]
    assert torch.all(col[:16, 3] == 1) and torch.all(fr.units_y[:, 0] == 0)
    assert torch.all(col[16:16 + LAYER_GAP] == 0)                 # gap rows between layers stay dark
    assert enc.should_capture(4) and not VizEncoder(VizConfig(stride_tokens=3), cfg).should_capture(4)


def test_separator_and_intensity_monotone():
    enc = VizEncoder(VizConfig(history=2), layers=1, heads=2, latent_per_head=4)
    vals = torch.tensor([[0.0, 0.1, 1.0, 10.0], [0.0, 0.0, 0.0, 0.0]])
    fr = enc.step([dict(x_last=vals, y_last=vals, xy_last=vals, rho_last=vals)], 0)
    x = fr.units_x[:, 0]
    assert x[0, :3].sum() == 0 and x[1, 0] < x[2, 0] < x[3, 0]
    assert x[4, :3].sum() > 0                                     # head boundary row carries the separator


def test_mailbox_keeps_latest():
    tx, rx = channel()
    tx.try_send(1)
    tx.try_send(2)
    assert rx.drain_latest() == 2 and rx.drain_latest() is None


def test_panel_grid_png_roundtrip(tmp_path):
    import numpy as np
    import torch
    from burn_dragon_b200.viz.encoder import VizConfig, VizEncoder, srgb_to_linear
    from burn_dragon_b200.viz.image import linear_to_srgb8, read_png_rgb8
    enc = VizEncoder(VizConfig(history=8), layers=2, heads=2, latent_per_head=4)
    torch.manual_seed(0)
    for t in range(5):
        enc.step([dict(x_last=torch.rand(1, 2, 4), y_last=torch.rand(1, 2, 4), xy_last=torch.rand(1, 2, 4),
                       rho_last=torch.rand(1, 2, 4)) for _ in range(2)])
    h, w, _ = enc.units_x.shape
    grid = enc.panel_grid(gap=3)
    assert tuple(grid.shape) == (2 * h + 3, 2 * w + 3, 4)
    assert torch.equal(grid[:h, :w], enc.units_x) and torch.equal(grid[h + 3:, w + 3:], enc.units_rho)
    enc.save(tmp_path / "panels.png")
    img = read_png_rgb8(tmp_path / "panels.png")
    assert img.shape == (2 * h + 8, 2 * w + 8, 3)
    assert np.array_equal(img[:h, :w], linear_to_srgb8(enc.units_x[..., :3].numpy()))
    # sRGB transfer is the inverse of the encoder's linearisation
    for v in (0.0, 0.02, 0.5, 1.0):
        assert abs(int(linear_to_srgb8(np.array([[srgb_to_linear(v)] * 3]))[0, 0]) - round(v * 255)) <= 1

"""Mamba-2 / Mamba-3 oracles: the chunked SSD form equals the literal recurrence, and the models'
cached state makes split and whole sequences agree."""
import pytest
import torch

from burn_dragon_b200.models.mamba import MambaConfig, MambaLM
from burn_dragon_b200.ops import ssd as SSD


@pytest.mark.parametrize("T,chunk", [(37, 8), (64, 64), (130, 64)])
def test_ssd_chunked_equals_sequential(T, chunk):
    torch.manual_seed(0)
    B, H, P, N = 2, 3, 4, 6
    xw = torch.randn(B, T, H, P, dtype=torch.float64)
    loga = -torch.rand(B, T, H, dtype=torch.float64)
    Bm, Cm = torch.randn(B, T, N, dtype=torch.float64), torch.randn(B, T, N, dtype=torch.float64)
    h0 = torch.randn(B, H, N, P, dtype=torch.float64)
    y1, h1 = SSD.ssd_sequential(xw, loga, Bm, Cm, h0)
    y2, h2 = SSD.ssd_chunked(xw, loga, Bm, Cm, h0, chunk)
    assert torch.allclose(y1, y2, atol=1e-10) and torch.allclose(h1, h2, atol=1e-10)
    ys, h = [], h0.clone()
    for t in range(T):
        y, h = SSD.ssd_step(xw[:, t], loga[:, t], Bm[:, t], Cm[:, t], h)
        ys.append(y)
    assert torch.allclose(torch.stack(ys, 1), y1, atol=1e-10)


def _lm(version, r=1):
    torch.manual_seed(0)
    return MambaLM(MambaConfig(version=version, n_layer=2, d_model=16, d_state=8, headdim=8, expand=2, chunk_size=8,
                               mimo_rank=r, vocab_size=32)).double().eval()


@pytest.mark.parametrize("version,r", [(2, 1), (3, 1), (3, 2)])
def test_state_split_equals_full_and_decode(version, r):
    m = _lm(version, r)
    tok = torch.randint(0, 32, (2, 21))
    with torch.no_grad():
        full = m(tok)
        st = m.init_state()
        a = m.forward_with_state(tok[:, :9], st)
        b = m.forward_with_state(tok[:, 9:20], st)
        c = m.forward_with_state(tok[:, 20:], st)          # single-token decode step
    assert st.position == 21
    assert torch.allclose(torch.cat([a, b, c], 1), full, atol=1e-8)


@pytest.mark.parametrize("version", [2, 3])
def test_training_reduces_loss_and_generate(version):
    torch.manual_seed(0)
    m = MambaLM(MambaConfig(version=version, n_layer=1, d_model=16, d_state=8, headdim=8, chunk_size=8, vocab_size=32))
    opt = torch.optim.AdamW(m.parameters(), lr=1e-2)
    tok = torch.randint(0, 32, (4, 17))
    first = None
    for _ in range(8):
        loss = m(tok[:, :-1], tok[:, 1:])
        first = first if first is not None else loss.item()
        opt.zero_grad(); loss.backward(); opt.step()
    assert loss.item() < first
    out = m.eval().generate(tok[:, :5], 4, greedy=True)
    assert out.shape == (4, 9)


def test_factory_builds_mamba_from_preset():
    from burn_dragon_b200 import config as C
    from burn_dragon_b200.models.factory import build_model
    cfg = C.load_preset("mamba2")
    m = build_model(cfg, vocab_size=64)
    assert m.config.version == 2 and m.config.d_state == 128 and m.config.n_heads == 8
    assert build_model(C.load_preset("mamba3"), 64).config.version == 3

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


def test_written_out_ssd_backward_equals_autograd():
    """`ssd_backward_sequential` (the scan's dual form, the oracle for a backward kernel) against
    autograd of the literal recurrence and of the chunked form, float64."""
    import torch
    from burn_dragon_b200.ops import ssd as S
    torch.manual_seed(3)
    B, T, H, P, N = 2, 70, 3, 8, 16
    dt = torch.float64
    xw = torch.randn(B, T, H, P, dtype=dt, requires_grad=True)
    loga = (-torch.rand(B, T, H, dtype=dt) * 0.3).requires_grad_()
    Bm = torch.randn(B, T, N, dtype=dt, requires_grad=True)
    Cm = torch.randn(B, T, N, dtype=dt, requires_grad=True)
    dy = torch.randn(B, T, H, P, dtype=dt)
    with torch.no_grad():
        got = S.ssd_backward_sequential(xw, loga, Bm, Cm, dy)
    for fn in (S.ssd_sequential, lambda *a: S.ssd_chunked(*a, chunk=16)):
        want = torch.autograd.grad(fn(xw, loga, Bm, Cm)[0], (xw, loga, Bm, Cm), dy)
        for g, w, name in zip(got, want, ("xw", "loga", "B", "C")):
            assert (g - w).abs().max().item() < 1e-9 * max(1.0, w.abs().max().item()), name


def test_dual_form_autograd_function_equals_autograd_of_the_chunked_form():
    """`ssd_dual`: forward by the regular dispatch, backward written out (d xw through the reversed
    dual scan, d B / d C from chunk states) - same gradients as differentiating the chunked form,
    for a length that is not a multiple of the chunk."""
    import torch
    from burn_dragon_b200.ops import ssd as S
    torch.manual_seed(4)
    B, T, H, P, N = 2, 150, 3, 8, 16
    dt = torch.float64
    mk = lambda *s: torch.randn(*s, dtype=dt)
    xw, Bm, Cm = mk(B, T, H, P).requires_grad_(), mk(B, T, N).requires_grad_(), mk(B, T, N).requires_grad_()
    loga = (-torch.rand(B, T, H, dtype=dt) * 0.3).requires_grad_()
    dy = mk(B, T, H, P)
    y, hT = S.ssd_dual(xw, loga, Bm, Cm, chunk=64)
    y_ref, h_ref = S.ssd_chunked(xw, loga, Bm, Cm, None, 64)
    assert torch.allclose(y, y_ref, atol=1e-10) and torch.allclose(hT, h_ref, atol=1e-10) and not hT.requires_grad
    got = torch.autograd.grad(y, (xw, loga, Bm, Cm), dy)
    want = torch.autograd.grad(y_ref, (xw, loga, Bm, Cm), dy)
    for g, w, name in zip(got, want, ("xw", "loga", "B", "C")):
        assert (g - w).abs().max().item() < 1e-9 * max(1.0, w.abs().max().item()), name


@pytest.mark.parametrize("version", [2, 3])
def test_mamba_gradients_with_the_dual_form_scan(version, monkeypatch):
    """`BDH_SSD_DUAL=1` (here: the module switch it sets): a Mamba training step through the written-out
    backward gives the loss and the parameter gradients of the autograd path."""
    from burn_dragon_b200.ops import ssd as S
    torch.manual_seed(0)
    m = MambaLM(MambaConfig(version=version, n_layer=2, d_model=16, d_state=8, headdim=8, chunk_size=8, vocab_size=32))
    tok = torch.randint(0, 32, (3, 21))
    loss = m(tok[:, :-1], tok[:, 1:])
    loss.backward()
    want = {n: p.grad.clone() for n, p in m.named_parameters() if p.grad is not None}
    m.zero_grad()
    monkeypatch.setattr(S, "_DUAL", "1")
    calls = []
    real = S.ssd_dual
    monkeypatch.setattr(S, "ssd_dual", lambda *a, **k: (calls.append(1), real(*a, **k))[1])
    loss2 = m(tok[:, :-1], tok[:, 1:])
    loss2.backward()
    assert calls and abs(loss2.item() - loss.item()) < 1e-5
    for n, p in m.named_parameters():
        if n in want:
            assert torch.allclose(p.grad, want[n], atol=2e-5, rtol=1e-3), n

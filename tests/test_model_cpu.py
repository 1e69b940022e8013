"""CPU tier: the three forms of the canonical attention agree, model paths run and train."""
import pytest
import torch

from burn_dragon_b200.models.bdh import BDH, BDHConfig, build_model_config
from burn_dragon_b200.ops import reference as R


def _cfg(rot, **kw):
    base = dict(n_layer=2, n_embd=32, n_head=2, mlp_internal_dim_multiplier=4, vocab_size=32, dropout=0.0,
                rotary_embedding=rot)
    base.update(kw)
    return BDHConfig(**base)


@pytest.mark.parametrize("rot", ["alibi", "rope", "pope"])
def test_recurrent_parallel_chunked_agree(rot):
    torch.manual_seed(0)
    B, H, T, N, D = 2, 2, 37, 16, 8
    x = torch.relu(torch.randn(B, H, T, N, dtype=torch.float64))
    v = torch.randn(B, 1, T, D, dtype=torch.float64)
    freqs = R.build_freqs(N, 65536.0, rot).double()
    q = R.rotate(x, rot, freqs, 3)
    slopes = R.alibi_slopes(H).double() if rot == "alibi" else None
    decay = torch.exp(-slopes) if slopes is not None else None
    rho0 = torch.randn(B, H, q.shape[-1], D, dtype=torch.float64)
    a_r, rho_r = R.linear_attention_recurrent(q, v, decay, rho0)
    a_p, rho_p = R.linear_attention_parallel(q, v, slopes, rho0)
    a_c, rho_c = R.linear_attention_chunked(q, v, slopes, rho0, chunk=8)
    for a, rho in ((a_p, rho_p), (a_c, rho_c)):
        assert torch.allclose(a, a_r, atol=1e-9, rtol=1e-9)
        assert torch.allclose(rho, rho_r, atol=1e-9, rtol=1e-9)


@pytest.mark.parametrize("rot", ["alibi", "rope", "pope"])
def test_model_paths_shapes_and_backward(rot):
    # mirrors the reference's model smoke test: both forward functions, state position, backward
    m = BDH(_cfg(rot))
    tok = torch.randint(0, 32, (2, 4))
    lf = m.forward_fast(tok)
    st = m.init_state()
    ls = m.forward_with_state(tok, st, mode="recurrent")
    assert lf.shape == ls.shape == (2, 4, 32)
    assert st.position == 4
    lf.sum().backward()
    m.zero_grad()
    m(tok, mode="recurrent").sum().backward()
    assert all(p.grad is not None for p in m.parameters())


def test_state_split_equals_full():
    m = BDH(_cfg("rope")).double()
    tok = torch.randint(0, 32, (2, 12))
    st = m.init_state()
    a = m.forward_with_state(tok[:, :5], st, mode="recurrent")
    b = m.forward_with_state(tok[:, 5:], st, mode="parallel")
    full = m(tok, mode="chunked")
    assert torch.allclose(torch.cat([a, b], 1), full, atol=1e-9)


def test_alibi_decay_is_exp_of_minus_slope():
    m = BDH(_cfg("alibi"))
    assert torch.allclose(m.slopes, torch.tensor([1.0, 2 ** -0.5]))
    # two-token forward: the second token's attention is q1.q0 * exp(-m_h) * v0
    x = torch.relu(torch.randn(1, 2, 2, 4))
    v = torch.randn(1, 1, 2, 3)
    a, _ = R.linear_attention_recurrent(x, v, torch.exp(-m.slopes), None)
    want = (x[:, :, 1] * x[:, :, 0]).sum(-1, keepdim=True) * torch.exp(-m.slopes).view(1, 2, 1) * v[:, :, 0]
    assert torch.allclose(a[:, :, 1], want, atol=1e-6)
    assert torch.all(a[:, :, 0] == 0)


def test_training_step_reduces_loss():
    torch.manual_seed(0)
    m = BDH(_cfg("alibi", n_layer=1))
    opt = torch.optim.AdamW(m.parameters(), lr=1e-2, weight_decay=0.1)
    tok = torch.randint(0, 32, (4, 16))
    first = None
    for _ in range(5):
        loss = m(tok[:, :-1], tok[:, 1:])
        assert torch.isfinite(loss)
        first = first if first is not None else loss.item()
        opt.zero_grad(); loss.backward(); opt.step()
    assert loss.item() < first


def test_generate_batch_streams_independent():
    m = BDH(_cfg("rope")).eval()
    p = torch.randint(0, 32, (3, 5))
    out = m.generate(p, 6, greedy=True)
    assert out.shape == (3, 11)
    single = m.generate(p[1:2], 6, greedy=True)
    assert torch.equal(out[1:2], single)


def test_build_model_config_overrides():
    from burn_dragon_b200.config import ModelOverrides
    cfg = build_model_config(ModelOverrides(n_layer=3, n_embd=64, n_head=4, rotary_embedding="pope"), 128, 50)
    assert (cfg.n_layer, cfg.n_embd, cfg.latent_per_head, cfg.vocab_size, cfg.block_size) == (3, 64, 64, 50, 128)
    assert cfg.state_latent == 128


def test_gradient_accumulation_equals_one_large_batch():
    import torch
    from burn_dragon_b200.engine.trainer import Trainer
    from burn_dragon_b200.models.bdh import BDH, BDHConfig

    def make():
        torch.manual_seed(0)
        return BDH(BDHConfig(n_layer=2, n_embd=32, n_head=2, n_latent_per_head=16, vocab_size=64, dropout=0.0))

    tok = torch.randint(0, 64, (4, 17), generator=torch.Generator().manual_seed(1))
    a, b = make(), make()
    ta, tb = Trainer(a, lr=1e-2), Trainer(b, lr=1e-2, grad_accum=2)
    for _ in range(2):
        ta.train_step(tok[:, :-1], tok[:, 1:])
        tb.train_step(tok[:2, :-1], tok[:2, 1:])
        assert tb.step_index == ta.step_index - 1
        tb.train_step(tok[2:, :-1], tok[2:, 1:])
        assert tb.step_index == ta.step_index
    for (n, p), (_, q) in zip(a.named_parameters(), b.named_parameters()):
        assert torch.allclose(p, q, rtol=1e-4, atol=1e-6), n


def test_cpp_oracle_equals_torch_recurrent_path():
    """The plain C++ restatement of the forward pass (no torch, no shared code) against the torch
    recurrent path: logits and the final state, every positional mode."""
    import numpy as np
    import pytest
    import torch
    from burn_dragon_b200.models.bdh import BDH, BDHConfig
    from burn_dragon_b200.utils import hostlib
    assert hostlib.available()
    for rot in ("alibi", "rope", "pope"):
        torch.manual_seed(1)
        m = BDH(BDHConfig(n_layer=3, n_embd=24, n_head=2, n_latent_per_head=10, vocab_size=50, dropout=0.0,
                          rotary_embedding=rot, relu_threshold=0.01)).eval()
        with torch.no_grad():
            for p in (m.encoder, m.encoder_v, m.decoder):
                p.mul_(8.0)
        toks = torch.randint(0, 50, (1, 21))
        st = m.init_state()
        with torch.no_grad():
            want = m.forward_with_state(toks, st, mode="recurrent")[0].numpy()
        got, rho = hostlib.oracle_forward(m, toks[0].tolist(), want_state=True)
        assert np.allclose(got, want, rtol=2e-4, atol=2e-5), (rot, np.abs(got - want).max())
        assert np.allclose(rho, st.layers[-1].rho[0].numpy(), rtol=2e-4, atol=2e-5), rot
    with pytest.raises(ValueError):
        hostlib.oracle_forward(m, [0, 99])


def test_phase_timers_fall_back_to_the_host_clock():
    """`utils.profiling` without a CUDA device: phases are timed with the host clock; `comm_ms` adds up
    the collectives that are launches of their own."""
    import time
    from burn_dragon_b200.utils import profiling as prof
    assert not prof.timers_on()
    with prof.phase("ignored"):
        pass
    assert prof.report() == {}
    prof.enable(timers=True)
    try:
        for _ in range(2):
            with prof.phase("step"):
                with prof.phase("comm.tp_reduce"):
                    time.sleep(0.01)
                with prof.phase("grad_reduce"):
                    time.sleep(0.005)
        rep = prof.report()
    finally:
        prof.enable(timers=False)
    assert rep["step"]["calls"] == 2 and rep["comm.tp_reduce"]["calls"] == 2
    assert 25.0 <= prof.comm_ms(rep) <= rep["step"]["ms"] + 1e-6
    assert prof.report() == {}

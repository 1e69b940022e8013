import torch

from burn_dragon_b200.config import ContextStrategyConfig, GenerationConfig, TrainingHyperparameters
from burn_dragon_b200.data.tokenizer import ByteTokenizer, CharVocab
from burn_dragon_b200.engine import generation as GEN
from burn_dragon_b200.models.bdh import BDH, BDHConfig
from burn_dragon_b200.ops import reference as R


def _model():
    torch.manual_seed(0)
    return BDH(BDHConfig(n_layer=2, n_embd=32, n_head=2, vocab_size=259, dropout=0.0, rotary_embedding="rope")).eval()


def test_top_k_keeps_ties_and_masks_rest():
    logits = torch.tensor([[1.0, 3.0, 3.0, 2.0, 0.0]])
    f = R.top_k_filter(logits, 2)
    assert torch.isinf(f[0, [0, 3, 4]]).all() and (f[0, [1, 2]] == 3.0).all()
    f1 = R.top_k_filter(logits, 1)       # ties at the threshold survive
    assert (f1[0, [1, 2]] == 3.0).all()
    assert torch.equal(R.top_k_filter(logits, 0), logits) and torch.equal(R.top_k_filter(logits, 5), logits)


def test_sampling_distribution_and_seed():
    logits = torch.log(torch.tensor([[0.7, 0.2, 0.1]])).repeat(20000, 1)
    g = torch.Generator().manual_seed(1)
    s = R.sample_logits(logits, generator=g)
    freq = torch.bincount(s, minlength=3).float() / len(s)
    assert torch.allclose(freq, torch.tensor([0.7, 0.2, 0.1]), atol=0.02)
    g2 = torch.Generator().manual_seed(1)
    assert torch.equal(s, R.sample_logits(logits, generator=g2))
    assert (R.sample_logits(logits, greedy=True) == 0).all()
    # degenerate rows fall back to uniform instead of failing
    bad = torch.full((4, 5), float("-inf"))
    assert R.sample_logits(bad).shape == (4,)


def test_generate_tokens_matches_manual_loop_and_callback():
    m = _model()
    prompt = torch.randint(0, 256, (2, 7))
    seen = []
    out = GEN.generate_tokens(m, prompt, settings=GEN.GenerationSettings(max_new_tokens=5, greedy=True),
                              on_token=lambda t: seen.append(t.clone()))
    assert out.shape == (2, 12) and len(seen) == 5
    state, last = GEN.prefill_state(m, prompt)
    toks = []
    for _ in range(5):
        nxt, last = GEN.sample_next_token(m, state, last, greedy=True)
        toks.append(nxt)
    assert torch.equal(out[:, 7:], torch.stack(toks, 1))
    assert state.position == 12


def test_generate_text_sliding_truncates_prompt_and_eos_stop():
    m = _model()
    tok = ByteTokenizer(True)
    tr = TrainingHyperparameters(block_size=4)
    g = GenerationConfig(prompt="hello world", max_tokens=3, context_strategy=ContextStrategyConfig("sliding", 0),
                         greedy=True)
    text = GEN.generate_text(m, tok, tr, g)
    assert text.startswith("orld")                 # window 0 -> block size 4 -> last 4 prompt bytes
    s = GEN.resolve_context_strategy(ContextStrategyConfig("sliding", 9), 4)
    assert (s.kind, s.window) == ("sliding", 9)
    assert GEN.normalize_max_tokens(-1) is None and GEN.normalize_max_tokens(5) == 5


def test_stream_printer_utf8_safe():
    tok = ByteTokenizer(False)
    got = []
    sp = GEN.StreamPrinter(tok, got.append)
    for b in "hé✓".encode():
        sp.push(b)
    assert "".join(got) == "hé✓"
    cv = CharVocab.fit(["abc"])
    got2 = []
    sp2 = GEN.StreamPrinter(cv, got2.append)
    for i in cv.encode("cab"):
        sp2.push(i)
    assert "".join(got2) == "cab"


def test_segmented_prefill_equals_one_shot():
    """A prompt run in segments with the state carried across gives the same last logits and state."""
    import torch
    from burn_dragon_b200.engine import generation as GEN
    from burn_dragon_b200.models.bdh import BDH, BDHConfig
    for rot in ("alibi", "rope", "pope"):
        torch.manual_seed(0)
        m = BDH(BDHConfig(n_layer=2, n_embd=32, n_head=2, n_latent_per_head=16, vocab_size=64, dropout=0.0,
                          rotary_embedding=rot)).eval()
        toks = torch.randint(0, 64, (2, 50))
        with torch.no_grad():
            s1, l1 = GEN.prefill_state(m, toks)
            s2, l2 = GEN.prefill_state(m, toks, segment=16)
        assert s1.position == s2.position == 50
        assert torch.allclose(l1, l2, rtol=1e-4, atol=1e-5), rot
        for a, b in zip(s1.layers, s2.layers):
            assert torch.allclose(a.rho, b.rho, rtol=1e-4, atol=1e-5), rot

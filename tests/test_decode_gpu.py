"""Decode kernels: recurrent state update, batched sampler, graph-captured decode engine."""
import pytest
import torch

from burn_dragon_b200.engine import decode_engine as DE
from burn_dragon_b200.engine import generation as GEN
from burn_dragon_b200.models.bdh import BDH, BDHConfig
from burn_dragon_b200.ops import native, sampling
from burn_dragon_b200.ops import reference as R

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("decay", [False, True])
@pytest.mark.parametrize("D", [64, 256, 512])
def test_state_update_matches_recurrence(decay, D):
    B, H, Np = 3, 2, 320
    g = torch.Generator(device="cuda").manual_seed(0)
    q = torch.relu(torch.randn(B, H * Np, device="cuda", generator=g) - 0.5).to(torch.bfloat16)
    v = torch.randn(B, D, device="cuda", generator=g).to(torch.bfloat16)
    rho = torch.randn(B, H, Np, D, device="cuda", generator=g)
    slopes = torch.tensor([0.3, 0.7], device="cuda") if decay else None
    qf = q.float().view(B, H, 1, Np)
    a_ref, rho_ref = R.linear_attention_recurrent(qf, v.float().view(B, 1, 1, D),
                                                  torch.exp(-slopes) if decay else None, rho.clone())
    a = torch.zeros(H * B, D, device="cuda")
    native.ops.decode_state_update(q, v, rho, a, slopes)
    torch.cuda.synchronize()
    assert _rel(a.view(H, B, D).transpose(0, 1), a_ref[:, :, 0]) < 1e-5
    assert _rel(rho, rho_ref) < 1e-6


def test_sampler_greedy_topk_and_distribution():
    probs = torch.tensor([0.5, 0.25, 0.15, 0.1, 0.0, 0.0, 0.0, 0.0], device="cuda")
    logits = torch.log(probs + 1e-30).repeat(40000, 1).contiguous()
    s = sampling.sample(logits, seed=123)
    freq = torch.bincount(s, minlength=8).float() / len(s)
    assert torch.allclose(freq, probs, atol=0.015), freq
    assert (sampling.sample(logits, greedy=True) == 0).all()
    s2 = sampling.sample(logits, top_k=2, seed=5)
    assert set(s2.unique().tolist()) <= {0, 1}
    f2 = torch.bincount(s2, minlength=8).float() / len(s2)
    assert abs(f2[0].item() - 2 / 3) < 0.02
    hot = sampling.sample(logits / 1.0, temperature=0.05, seed=9)      # low temperature ~ arg-max
    assert (hot == 0).float().mean() > 0.99
    tied = torch.zeros(1000, 16, device="cuda")
    tied[:, 3] = tied[:, 7] = 5.0
    s3 = sampling.sample(tied, top_k=1, seed=1)                        # ties at the threshold survive
    assert set(s3.unique().tolist()) == {3, 7}
    bad = torch.full((64, 256), float("-inf"), device="cuda")
    s4 = sampling.sample(bad, seed=2)
    assert int(s4.min()) >= 0 and int(s4.max()) < 256


def _model(rot, vocab=256):
    torch.manual_seed(0)
    m = BDH(BDHConfig(n_layer=2, n_embd=64, n_head=2, n_latent_per_head=256, vocab_size=vocab, dropout=0.0,
                      rotary_embedding=rot)).cuda().eval()
    with torch.no_grad():
        m.encoder.mul_(4.0); m.encoder_v.mul_(4.0); m.decoder.mul_(4.0)
        for p in m.parameters():
            p.copy_(p.to(torch.bfloat16).float())
    return m


@pytest.mark.parametrize("rot", ["alibi", "rope", "pope"])
@pytest.mark.parametrize("graph", [True, False])
def test_engine_matches_fp32_recurrence_teacher_forced(rot, graph):
    m = _model(rot)
    eng = DE.attach(m, use_graph=graph)
    B, P, n = 4, 64, 12
    prompt = torch.randint(0, 256, (B, P), device="cuda")
    settings = GEN.GenerationSettings(max_new_tokens=n, temperature=1.0, top_k=40, seed=11)
    native.clear_status()
    out = GEN.generate_tokens(m, prompt, settings=settings)
    assert native.status_code() == 0
    assert out.shape == (B, P + n) and torch.equal(out[:, :P], prompt)
    # feed the same tokens through the literal fp32 recurrence and compare state and next-token logits
    m.use_native = False
    st = m.init_state()
    with torch.no_grad():
        ref_logits = m.forward_with_state(out, st, mode="recurrent")[:, -1]
    assert eng.last_state.position == st.position == P + n
    assert _rel(eng.last_logits, ref_logits) < 0.08
    for a, b in zip(eng.last_state.layers, st.layers):
        assert _rel(a.rho, b.rho) < 0.05


def test_engine_with_a_character_vocabulary_of_69_symbols():
    """The LM head of a character-level model has a width that is no multiple of 8 (69 here), which
    a TMA row pitch cannot express: the captured step then takes the head product from a library
    matmul into the same logits buffer, and the sampler sees exactly V columns."""
    V = 69
    m = _model("rope", vocab=V)
    eng = DE.attach(m)
    B, P, n = 3, 48, 16
    prompt = torch.randint(0, V, (B, P), device="cuda")
    native.clear_status()
    out = GEN.generate_tokens(m, prompt, settings=GEN.GenerationSettings(max_new_tokens=n, temperature=1.0, seed=5))
    assert native.status_code() == 0
    assert out.shape == (B, P + n) and int(out.max()) < V and int(out.min()) >= 0
    m.use_native = False
    st = m.init_state()
    with torch.no_grad():
        ref_logits = m.forward_with_state(out, st, mode="recurrent")[:, -1]
    assert eng.last_logits.shape[-1] == V
    assert _rel(eng.last_logits, ref_logits) < 0.08


def test_engine_greedy_is_deterministic_and_streams_independent():
    m = _model("rope")
    DE.attach(m)
    prompt = torch.randint(0, 256, (3, 64), device="cuda")
    s = GEN.GenerationSettings(max_new_tokens=8, greedy=True)
    a = GEN.generate_tokens(m, prompt, settings=s)
    b = GEN.generate_tokens(m, prompt, settings=s)
    assert torch.equal(a, b)
    single = GEN.generate_tokens(m, prompt[1:2], settings=s)
    assert torch.equal(single, a[1:2])


@pytest.mark.parametrize("rot", ["rope", "alibi"])
def test_chunked_continuation_equals_one_call(rot):
    """`continue_from` in chunks (the streaming-session path) produces the tokens of one `generate`
    call: greedy, and sampled with a fixed seed (the sampler's random stream continues across chunks)."""
    torch.manual_seed(0)
    m = BDH(BDHConfig(n_layer=2, n_embd=64, n_head=2, n_latent_per_head=128, vocab_size=256, dropout=0.0,
                      rotary_embedding=rot)).cuda().eval()
    eng = DE.attach(m)
    toks = torch.randint(0, 256, (3, 64), device="cuda")
    for s in (GEN.GenerationSettings(12, greedy=True), GEN.GenerationSettings(12, 1.0, 40, seed=7)):
        whole = eng.generate(toks, s)[:, 64:]
        state, last = GEN.prefill_state(m, toks, toks.device)
        parts, done = [], 0
        for n in (5, 4, 3):
            parts.append(eng.continue_from(state, last, s, n, step0=done))
            last, done = eng.last_logits, done + n
        assert state.position == 64 + 12
        assert torch.equal(torch.cat(parts, dim=1), whole), s


def test_session_streams_on_the_decode_engine():
    import json
    from burn_dragon_b200.data.tokenizer import CharVocab
    from burn_dragon_b200.engine import burn_record as BR
    from burn_dragon_b200.engine import session as S
    torch.manual_seed(0)
    vocab = CharVocab.fit(["hello world, this is a tiny corpus of text."], include_unknown=True)
    V = (len(vocab) + 7) // 8 * 8
    chars = vocab.id2ch + [chr(0x2500 + i) for i in range(V - len(vocab))]       # pad the vocabulary to a multiple of 8
    vocab = CharVocab(chars, True)
    m = BDH(BDHConfig(n_layer=2, n_embd=64, n_head=2, mlp_internal_dim_multiplier=4, vocab_size=len(vocab),
                      dropout=0.0, rotary_embedding="rope")).eval()
    blob = BR.serialize(BR.from_model(m))
    cfg = json.dumps(dict(run_name="t", block_size=64, overrides=dict(n_layer=2, n_embd=64, n_head=2,
                                                                      mlp_internal_dim_multiplier=4,
                                                                      rotary_embedding="rope")))
    sess = S.load_model(blob, json.dumps(vocab.to_record()), cfg, device="cuda")
    prompt = "hello world, this is a tiny corpus of text. hello world, this is"      # 64 characters
    assert len(prompt) == 64
    n0 = native.launch_count()
    sess.start_stream(prompt, max_tokens=10, greedy=True)
    text = ""
    while not sess.done:
        text += sess.next_chunk(max_tokens=4)
    assert native.launch_count() > n0 and sess.generated == 10
    ids = torch.tensor([vocab.encode(prompt)], device="cuda")
    want = GEN.generate_tokens(sess.model, ids, "cuda", GEN.GenerationSettings(10, greedy=True))[0, 64:].tolist()
    if vocab.eos_id in want:
        want = want[:want.index(vocab.eos_id)]
    assert text == vocab.decode(want)


def test_stream_pool_on_the_device_in_a_child_process():
    """Continuous batching on the GPU (graph-captured step, per-stream rotary table): streams that join
    and leave a pool produce the tokens they produce alone. Runs in a child process with its own CUDA
    context."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-m", "burn_dragon_b200.engine.stream_pool"], capture_output=True, text=True,
                       timeout=300, cwd=root, env=dict(os.environ, PYTHONPATH=root))
    assert r.returncode == 0 and r.stdout.count("PASS stream_pool") == 6, r.stdout[-1500:] + r.stderr[-1500:]


def test_pope_step_with_device_position_is_captured_and_matches_recurrence():
    """`DecodeEngine(pope_graph=True)`: the PoPE step reads its position from device memory, is captured
    in a CUDA graph, and follows the literal fp32 recurrence like the step with the fused rotation."""
    m = _model("pope")
    eng = DE.attach(m, pope_graph=True)
    B, P, n = 4, 64, 12
    prompt = torch.randint(0, 256, (B, P), device="cuda")
    settings = GEN.GenerationSettings(max_new_tokens=n, temperature=1.0, top_k=40, seed=11)
    native.clear_status()
    out = GEN.generate_tokens(m, prompt, settings=settings)
    assert native.status_code() == 0
    assert next(iter(eng._cache.values()))["graph"] is not None
    m.use_native = False
    st = m.init_state()
    with torch.no_grad():
        ref_logits = m.forward_with_state(out, st, mode="recurrent")[:, -1]
    assert eng.last_state.position == st.position == P + n
    assert _rel(eng.last_logits, ref_logits) < 0.08
    for a, b in zip(eng.last_state.layers, st.layers):
        assert _rel(a.rho, b.rho) < 0.05


@pytest.mark.parametrize("D", [64, 256, 512])
def test_decode_row_kernels_match_their_definitions(D):
    """`layernorm_f32_clear` (LayerNorm of fp32 rows that are cleared in the same pass) and `block_out_parts`
    (sum of split-K partial tiles + layer tail) against the torch statement."""
    from burn_dragon_b200.ops import reference as R
    torch.manual_seed(0)
    rows, parts = 37, 4
    a = torch.randn(rows, D, device="cuda") * 3 + 0.5
    want = R.layer_norm(a)
    y = torch.empty(rows, D, device="cuda", dtype=torch.bfloat16)
    native.ops.layernorm_f32_clear(a, y)
    assert float(a.abs().max()) == 0.0
    assert (y.float() - want).abs().max().item() < 3e-2
    cur = torch.randn(rows, D, device="cuda").bfloat16()
    part = torch.randn(parts * rows, D, device="cuda")
    out = torch.empty_like(cur)
    native.ops.block_out_parts(cur, part, out)
    want = R.layer_norm(cur.float() + R.layer_norm(part.view(parts, rows, D).sum(0)))
    assert (out.float() - want).abs().max().item() < 3e-2


@pytest.mark.parametrize("D", [64, 256])
def test_lazy_decay_equals_decaying_every_row_every_step(D):
    """ALiBi decay applied lazily (rows with a zero query entry are skipped and caught up with
    gamma^(steps missed) when next touched) against the kernel that scales every row every step: same
    attention outputs at every step and, after the final catch-up, the same state."""
    from burn_dragon_b200.engine.decode_engine import DecodeEngine
    B, H, Np, steps = 3, 2, 320, 7
    g = torch.Generator(device="cuda").manual_seed(0)
    slopes = torch.tensor([0.3, 0.05], device="cuda")
    rho_d = torch.randn(B, H, Np, D, device="cuda", generator=g)
    rho_l = rho_d.clone()
    seen = torch.full((B, H, Np), 4, device="cuda", dtype=torch.int32)
    step = torch.full((1,), 4, device="cuda", dtype=torch.int32)
    for _ in range(steps):
        q = torch.relu(torch.randn(B, H * Np, device="cuda", generator=g) - 0.8).to(torch.bfloat16)   # ~20 % live
        v = torch.randn(B, D, device="cuda", generator=g).to(torch.bfloat16)
        a_d, a_l = torch.zeros(H * B, D, device="cuda"), torch.zeros(H * B, D, device="cuda")
        native.ops.decode_state_update(q, v, rho_d, a_d, slopes)
        native.ops.decode_state_update(q, v, rho_l, a_l, slopes, seen, step)
        step += 1
        assert _rel(a_l, a_d) < 1e-5
    assert _rel(rho_l, rho_d) > 1e-3            # untouched rows are still behind ...
    DecodeEngine._catch_up([rho_l], [seen], step, slopes)
    assert _rel(rho_l, rho_d) < 1e-5            # ... until the state leaves the engine
    assert int(seen.min()) == int(seen.max()) == int(step)

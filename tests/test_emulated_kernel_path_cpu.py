"""The kernel path's orchestration on CPU: `ops.fused_bdh` with every launch replaced by the fp32
statement of the same contract (`ops.emulate`), against the torch definition of the model."""
import pytest
import torch

from burn_dragon_b200.models.bdh import BDH, BDHConfig
from burn_dragon_b200.ops import emulate, fused_bdh


def _model(rot, dropout=0.0):
    torch.manual_seed(0)
    m = BDH(BDHConfig(n_layer=2, n_embd=64, n_head=2, n_latent_per_head=128, vocab_size=256, dropout=dropout,
                      rotary_embedding=rot))
    with torch.no_grad():
        m.encoder.mul_(4.0); m.encoder_v.mul_(4.0); m.decoder.mul_(4.0)
        for p in m.parameters():
            p.copy_(p.to(torch.bfloat16).float())
    return m


def _rel(a, b):
    a, b = a.float().flatten(), b.float().flatten()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def _cos(a, b):
    a, b = a.float().flatten(), b.float().flatten()
    return (torch.dot(a, b) / (a.norm() * b.norm() + 1e-20)).item()


@pytest.mark.parametrize("rot", ["alibi", "rope", "pope"])
def test_loss_and_gradients(rot):
    m = _model(rot)
    tok, tgt = torch.randint(0, 256, (2, 128)), torch.randint(0, 256, (2, 128))
    assert not fused_bdh.can_run(m, tok, None)            # no GPU, no emulation: the torch path would run
    with emulate.kernel_path():
        assert fused_bdh.can_run(m, tok, None)
        loss_k = m(tok, tgt)
        loss_k.backward()
    gk = {n: p.grad.clone() for n, p in m.named_parameters()}
    m.zero_grad()
    loss_t = m(tok, tgt, mode="parallel")
    loss_t.backward()
    assert abs(loss_k.item() - loss_t.item()) < 2e-2
    for n, p in m.named_parameters():
        assert _cos(gk[n], p.grad) > 0.99 and _rel(gk[n], p.grad) < 0.12, (n, _cos(gk[n], p.grad), _rel(gk[n], p.grad))


@pytest.mark.parametrize("rot", ["alibi", "rope", "pope"])
def test_prefill_state_and_continuation(rot):
    m = _model(rot).eval()
    tok = torch.randint(0, 256, (1, 256))
    with torch.no_grad():
        st_t = m.init_state()
        want = m.forward_with_state(tok, st_t, mode="recurrent")
        with emulate.kernel_path():
            st_a = m.init_state()
            whole = m.forward_with_state(tok, st_a)
            st_b = m.init_state()
            parts = torch.cat([m.forward_with_state(tok[:, :128], st_b), m.forward_with_state(tok[:, 128:], st_b)], 1)
    assert st_a.position == st_b.position == 256
    assert _rel(whole, want) < 0.05 and _rel(parts, want) < 0.05
    assert _rel(st_a.layers[-1].rho, st_t.layers[-1].rho) < 0.05
    assert _rel(st_b.layers[-1].rho, st_t.layers[-1].rho) < 0.05


def test_recompute_modes_and_dropout():
    m = _model("rope")
    tok, tgt = torch.randint(0, 256, (2, 64)), torch.randint(0, 256, (2, 64))
    with emulate.kernel_path():
        m(tok, tgt).backward()
        g0 = {n: p.grad.clone() for n, p in m.named_parameters()}
        for mode, layers in ((True, 2), (1, 1)):
            m.zero_grad()
            m.recompute = mode
            m(tok, tgt).backward()
            assert m._recomputed_layers == layers
            for n, p in m.named_parameters():
                assert torch.allclose(g0[n], p.grad, rtol=1e-4, atol=1e-6), (mode, n)
        # dropout: a recomputed layer draws the same mask as its first forward
        d = _model("alibi", dropout=0.3).train()
        d.recompute = False
        d(tok, tgt).backward()
        g_saved = {n: p.grad.clone() for n, p in d.named_parameters()}
        calls = d._drop_calls
        d.zero_grad()
        d.recompute = True
        d._drop_calls = calls - 1          # same call counter, hence the same mask seeds
        d(tok, tgt).backward()
        for n, p in d.named_parameters():
            assert torch.allclose(g_saved[n], p.grad, rtol=1e-4, atol=1e-6), n


# ---- the decode engine's step, launch by launch ---------------------------------------------------
def _decode_model(rot):
    torch.manual_seed(0)
    m = BDH(BDHConfig(n_layer=2, n_embd=64, n_head=2, n_latent_per_head=128, vocab_size=256, dropout=0.0,
                      rotary_embedding=rot)).eval()
    with torch.no_grad():
        m.encoder.mul_(4.0); m.encoder_v.mul_(4.0); m.decoder.mul_(4.0)
        for p in m.parameters():
            p.copy_(p.to(torch.bfloat16).float())
    return m


@pytest.mark.parametrize("rot", ["alibi", "rope", "pope"])
def test_decode_engine_step_teacher_forced(rot):
    from burn_dragon_b200.engine import decode_engine as DE
    from burn_dragon_b200.engine import generation as GEN
    m = _decode_model(rot)
    prompt = torch.randint(0, 256, (3, 64))
    with emulate.kernel_path():
        eng = DE.attach(m)
        assert eng.can_run(prompt, GEN.GenerationSettings(10, greedy=True))
        out = GEN.generate_tokens(m, prompt, settings=GEN.GenerationSettings(10, 1.0, 40, seed=5))
        assert out.shape == (3, 74) and torch.equal(out[:, :64], prompt)
        last_logits, last_state = eng.last_logits.clone(), eng.last_state
    st = m.init_state()
    with torch.no_grad():
        ref = m.forward_with_state(out, st, mode="recurrent")[:, -1]
    assert last_state.position == st.position == 74
    assert _rel(last_logits, ref) < 0.08
    for a, b in zip(last_state.layers, st.layers):
        assert _rel(a.rho, b.rho) < 0.05


def test_decode_engine_chunks_streams_and_sessions():
    from burn_dragon_b200.data.tokenizer import ByteTokenizer
    from burn_dragon_b200.engine import decode_engine as DE
    from burn_dragon_b200.engine import generation as GEN
    from burn_dragon_b200.engine import session as S
    m = _decode_model("rope")
    toks = torch.randint(0, 256, (3, 64))
    s = GEN.GenerationSettings(12, greedy=True)
    with emulate.kernel_path():
        eng = DE.attach(m)
        whole = eng.generate(toks, s)[:, 64:]
        assert torch.equal(eng.generate(toks[1:2], s)[:, 64:], whole[1:2])      # streams are independent
        state, last = GEN.prefill_state(m, toks, toks.device)
        parts, done = [], 0
        for n in (5, 4, 3):
            parts.append(eng.continue_from(state, last, s, n, step0=done))
            last, done = eng.last_logits, done + n
        assert torch.equal(torch.cat(parts, dim=1), whole) and state.position == 76
        # a streaming session takes the engine route when it is eligible
        sess = S.InferenceSession(m, ByteTokenizer(False), "cpu")
        m.decode_engine = eng
        prompt = "the quick brown fox jumps over the lazy dog, twice over the dog!"      # 64 bytes
        assert len(prompt) == 64
        sess.start_stream(prompt, max_tokens=6, greedy=True)
        before = eng.last_state
        text = ""
        while not sess.done:
            text += sess.next_chunk(max_tokens=4)
        assert sess.generated == 6 and eng.last_state is not before          # the engine decoded the chunks
        ids = torch.tensor([list(prompt.encode())])
        want = GEN.generate_tokens(m, ids, settings=s.__class__(6, greedy=True))[0, 64:].tolist()
    assert text == bytes(want).decode("utf-8", errors="replace")


def test_decode_engine_with_a_vocabulary_that_is_not_a_multiple_of_8():
    """Character vocabularies (the shipped checkpoint has 69 tokens) decode on the engine: only the
    LM head leaves the GEMM kernel."""
    from burn_dragon_b200.engine import decode_engine as DE
    from burn_dragon_b200.engine import generation as GEN
    torch.manual_seed(0)
    m = BDH(BDHConfig(n_layer=2, n_embd=64, n_head=2, n_latent_per_head=128, vocab_size=69, dropout=0.0,
                      rotary_embedding="alibi")).eval()
    with torch.no_grad():
        m.encoder.mul_(4.0); m.encoder_v.mul_(4.0); m.decoder.mul_(4.0)
    prompt = torch.randint(0, 69, (2, 64))
    s = GEN.GenerationSettings(8, greedy=True)
    with emulate.kernel_path():
        eng = DE.attach(m)
        assert eng.can_run(prompt, s)
        out = GEN.generate_tokens(m, prompt, settings=s)
        logits = eng.last_logits.clone()
    st = m.init_state()
    with torch.no_grad():
        ref = m.forward_with_state(out, st, mode="recurrent")[:, -1]
    assert out.shape == (2, 72) and int(out.max()) < 69
    assert _rel(logits, ref) < 0.08


@pytest.mark.parametrize("rot", ["rope", "alibi", "pope"])
def test_stream_pool_joins_and_leaves_between_steps(rot):
    """Continuous batching: streams with prompts of different lengths join a pool at different times;
    each one's greedy tokens equal what it produces alone."""
    from burn_dragon_b200.engine import decode_engine as DE
    from burn_dragon_b200.engine import generation as GEN
    from burn_dragon_b200.engine.stream_pool import StreamPool
    m = _decode_model(rot)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 256, (1, n), generator=g) for n in (64, 128, 64)]
    s = GEN.GenerationSettings(64, greedy=True)
    with emulate.kernel_path():
        eng = DE.attach(m)
        alone = [eng.generate(p, GEN.GenerationSettings(8, greedy=True))[0, p.shape[1]:].tolist() for p in prompts]
        pool = StreamPool(m, slots=4, settings=s, device="cpu")
        got = {0: [], 1: [], 2: []}
        a = pool.add(prompts[0])
        for _ in range(3):                               # stream 0 runs alone for three steps
            got[0].append(int(pool.step()[a]))
        b = pool.add(prompts[1])                         # a longer prompt joins: positions now differ
        for _ in range(5):
            t = pool.step()
            got[0].append(int(t[a])); got[1].append(int(t[b]))
        pool.release(a)                                  # stream 0 is done; its slot is reused
        c = pool.add(prompts[2])
        assert c == a and pool.free_slots() == 2
        for _ in range(8):
            t = pool.step()
            got[1].append(int(t[b])); got[2].append(int(t[c]))
    assert got[0] == alone[0]
    assert got[1][:8] == alone[1]
    assert got[2] == alone[2]


def test_http_server_continuous_batching():
    """Concurrent requests with prompts of different lengths share the pooled decode step; each gets
    the text it gets when served alone."""
    import json
    import threading
    import urllib.request
    from burn_dragon_b200.data.tokenizer import ByteTokenizer
    from burn_dragon_b200.engine import generation as GEN
    from burn_dragon_b200.engine import server as SV
    from burn_dragon_b200.engine import session as S
    m = _decode_model("rope")
    prompts = ["the quick brown fox ", "jumps over the lazy dog and keeps running far away ", "hello"]
    with emulate.kernel_path():
        sess = S.InferenceSession(m, ByteTokenizer(False), "cpu")
        srv = SV.make_server(sess, "127.0.0.1", 0, pool_slots=2, pool_settings=GEN.GenerationSettings(None, greedy=True))
        port = srv.server_address[1]
        threading.Thread(target=srv.serve_forever, daemon=True).start()
        try:
            def post(body):
                req = urllib.request.Request(f"http://127.0.0.1:{port}/generate", data=json.dumps(body).encode(),
                                             headers={"Content-Type": "application/json"})
                return urllib.request.urlopen(req, timeout=120).read().decode()

            alone = [json.loads(post(dict(prompt=p, max_tokens=10, greedy=True, seed=1)))["text"] for p in prompts]
            results = [None] * 3

            def worker(i):
                if i == 1:      # one of them streams
                    lines = [json.loads(l) for l in post(dict(prompt=prompts[i], max_tokens=10, greedy=True,
                                                              stream=True)).splitlines() if l.strip()]
                    results[i] = "".join(l.get("text", "") for l in lines)
                else:
                    results[i] = json.loads(post(dict(prompt=prompts[i], max_tokens=10, greedy=True)))["text"]

            threads = [threading.Thread(target=worker, args=(i,)) for i in range(3)]     # 3 requests, 2 slots
            for t in threads:
                t.start()
            for t in threads:
                t.join(timeout=180)
            assert results == alone
            metrics = urllib.request.urlopen(f"http://127.0.0.1:{port}/metrics", timeout=30).read().decode()
            assert "bdh_requests_total 6" in metrics
        finally:
            srv.scheduler.stop()
            srv.shutdown()
            srv.server_close()


@pytest.mark.parametrize("alibi", [True, False])
def test_rownorm_attention_op(alibi):
    """The `forward_fast` attention as its launch sequence (scores with additive bias, row kernels,
    value product, the four backward products) against the torch statement."""
    from burn_dragon_b200.ops import reference as R
    from burn_dragon_b200.ops import rownorm_attention as RA
    torch.manual_seed(3)
    B, H, T, N, D = 2, 3, 256, 128, 64
    q = (torch.randn(B, H, T, N) * 0.3).relu().requires_grad_(True)
    v = torch.randn(B, 1, T, D).requires_grad_(True)
    slopes = torch.tensor([0.5, 0.25, 0.125]) if alibi else None
    g = torch.randn(B, H, T, D)
    with emulate.kernel_path():
        assert RA.can_run(q, v)
        a = RA.attention_rownorm(q, v, slopes)
        a.backward(g)
    dq, dv = q.grad.clone(), v.grad.clone()
    qr = q.detach().to(torch.bfloat16).float().requires_grad_(True)
    vr = v.detach().to(torch.bfloat16).float().requires_grad_(True)
    ar = R.attention_rownorm(qr, vr, slopes)
    ar.backward(g)
    assert _rel(a, ar) < 2e-2 and _rel(dv, vr.grad) < 3e-2 and _rel(dq, qr.grad) < 3e-2


@pytest.mark.parametrize("rot", ["alibi", "rope", "pope"])
def test_forward_fast_on_the_kernel_path(rot):
    """`forward_fast` (bias + row normalisation) as a kernel-path launch sequence, forward and backward,
    against its torch definition."""
    m = _model(rot)
    tok, tgt = torch.randint(0, 256, (2, 128)), torch.randint(0, 256, (2, 128))
    with emulate.kernel_path():
        logits_k = m.forward_fast(tok).float()
        loss_k = m.forward_fast(tok, tgt)
        loss_k.backward()
    gk = {n: p.grad.clone() for n, p in m.named_parameters()}
    m.zero_grad()
    logits_t = m.forward_fast(tok)
    loss_t = m.forward_fast(tok, tgt)
    loss_t.backward()
    assert _rel(logits_k, logits_t) < 0.05
    assert abs(loss_k.item() - loss_t.item()) < 2e-2
    for n, p in m.named_parameters():
        assert _cos(gk[n], p.grad) > 0.99 and _rel(gk[n], p.grad) < 0.15, (n, _cos(gk[n], p.grad), _rel(gk[n], p.grad))
    # With ALiBi it is a different function from the canonical one (additive bias instead of decay).
    # Without it the two coincide: a positive per-row scale of the scores cancels in the LayerNorm
    # that follows the attention.
    with torch.no_grad():
        diff = _rel(logits_t, m(tok, mode="parallel"))
    assert diff > 1e-2 if rot == "alibi" else diff < 1e-3


def test_session_with_prompts_of_different_lengths():
    from burn_dragon_b200.data.tokenizer import ByteTokenizer
    from burn_dragon_b200.engine import session as S
    m = _decode_model("rope")
    prompts = ["short prompt", "a prompt that is quite a bit longer than the other one"]
    with emulate.kernel_path():
        sess = S.InferenceSession(m, ByteTokenizer(False), "cpu")
        sess.start_stream(prompts, max_tokens=7, greedy=True)
        both = ["", ""]
        while not sess.done:
            a, b = sess.next_chunk(3)
            both[0] += a; both[1] += b
        assert sess.generated == 7
        alone = []
        for p in prompts:
            sess.start_stream(p, max_tokens=7, greedy=True)
            t = ""
            while not sess.done:
                t += sess.next_chunk(3)
            alone.append(t)
    assert both == alone
    # without an eligible engine (plain CPU) the equal-length rule stays
    plain = S.InferenceSession(m, ByteTokenizer(False), "cpu")
    with pytest.raises(ValueError):
        plain.start_stream(prompts, max_tokens=3)


def test_stream_pool_self_test_entry_runs():
    """`python -m burn_dragon_b200.engine.stream_pool` (the device self test the GPU tier starts as a
    child process), here on the emulated path."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-m", "burn_dragon_b200.engine.stream_pool"], capture_output=True, text=True,
                       timeout=600, cwd=root, env=dict(os.environ, PYTHONPATH=root, BDH_EMULATE_KERNELS="1"))
    assert r.returncode == 0 and r.stdout.count("PASS stream_pool") == 6, r.stdout[-1500:] + r.stderr[-1500:]


def test_pope_decode_step_with_the_position_in_device_memory():
    """`DecodeEngine(pope_graph=True)`: the PoPE step that reads its position from a device word (the
    graph-capturable form) produces the tokens and logits of the step with the fused rotation epilogue."""
    from burn_dragon_b200.engine import decode_engine as DE
    from burn_dragon_b200.engine import generation as GEN
    m = _decode_model("pope")
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, 256, (2, 64), generator=g)
    s = GEN.GenerationSettings(12, greedy=True)
    with emulate.kernel_path():
        fused = DE.DecodeEngine(m, pope_graph=False)
        want = fused.generate(prompt, s)
        want_logits = fused.last_logits.clone()
        eng = DE.DecodeEngine(m, pope_graph=True)
        got = eng.generate(prompt, s)
        # a second call continues from the state and the position the first one left
        more = eng.continue_from(eng.last_state, eng.last_logits, s, 4, step0=12)
        more_ref = fused.continue_from(fused.last_state, fused.last_logits, s, 4, step0=12)
    assert torch.equal(got, want) and _rel(eng.last_logits, fused.last_logits) < 0.02
    assert torch.equal(more, more_ref)
    assert want_logits.shape == (2, 256)


@pytest.mark.parametrize("rot", ["alibi", "rope"])
def test_latent_block_pattern_runs_on_the_kernel_path(rot):
    """A sparse latent `BlockPattern1d` no longer leaves the kernels: the inactive neuron blocks are dropped from
    every operand. Loss, gradients (zero on inactive rows) and the prefill state equal the torch path's."""
    from burn_dragon_b200.ops import emulate, fused_bdh
    from burn_dragon_b200.ops.block_sparse import BlockPattern1d, BlockPattern2d, BlockSparseConfig
    torch.manual_seed(0)
    m = BDH(BDHConfig(n_layer=2, n_embd=64, n_head=2, n_latent_per_head=256, vocab_size=256, dropout=0.0,
                      rotary_embedding=rot))
    m.config.block_sparse = BlockSparseConfig(BlockPattern1d.from_blocks(64, [0, 3]), BlockPattern2d.dense(128))
    tok, tgt = torch.randint(0, 256, (2, 128)), torch.randint(0, 256, (2, 128))
    m.use_native = False
    ref = m(tok, tgt, mode="parallel")
    ref.backward()
    want = {n: p.grad.clone() for n, p in m.named_parameters()}
    st_ref = m.init_state()
    with torch.no_grad():
        lg_ref = m.forward_with_state(tok, st_ref, mode="parallel")
    m.zero_grad()
    m.use_native = True
    with emulate.kernel_path():
        assert fused_bdh.can_run(m, tok, None)
        got = m(tok, tgt)
        got.backward()
        st = m.init_state()
        with torch.no_grad():
            lg = m.forward_with_state(tok, st)
    assert abs(got.item() - ref.item()) < 2e-2
    for n, p in m.named_parameters():
        assert ((p.grad - want[n]).norm() / (want[n].norm() + 1e-12)).item() < 0.1, n
    inactive = m.encoder.grad.view(2, 256, 64)[:, 64:192]
    assert float(inactive.abs().max()) == 0.0
    assert ((lg - lg_ref).norm() / lg_ref.norm()).item() < 0.05
    for a, b in zip(st.layers, st_ref.layers):
        assert a.rho.shape == b.rho.shape and ((a.rho - b.rho).norm() / (b.rho.norm() + 1e-12)).item() < 0.05


def test_time_block_pattern_in_the_row_normalised_mode_on_the_kernel_path():
    """`forward_fast` with a sparse `BlockPattern2d`: the block-pair mask is applied to the scores on the kernel path
    (forward and backward) and equals the torch statement (src/kernel/linear_attention.rs:54-112)."""
    from burn_dragon_b200.ops import emulate, fused_bdh
    from burn_dragon_b200.ops.block_sparse import BlockPattern1d, BlockPattern2d, BlockSparseConfig
    torch.manual_seed(0)
    m = BDH(BDHConfig(n_layer=1, n_embd=64, n_head=2, n_latent_per_head=128, vocab_size=256, dropout=0.0,
                      rotary_embedding="alibi"))
    m.config.block_sparse = BlockSparseConfig(BlockPattern1d.dense(64),
                                              BlockPattern2d.from_pairs(32, [(0, 0), (1, 1), (2, 0), (2, 2), (3, 1), (3, 3)]))
    tok, tgt = torch.randint(0, 256, (2, 128)), torch.randint(0, 256, (2, 128))
    m.use_native = False
    ref = m.forward_fast(tok, tgt)
    ref.backward()
    want = {n: p.grad.clone() for n, p in m.named_parameters()}
    m.zero_grad()
    m.use_native = True
    with emulate.kernel_path():
        got = m.forward_fast(tok, tgt)
        got.backward()
    assert abs(got.item() - ref.item()) < 2e-2
    for n, p in m.named_parameters():
        assert ((p.grad - want[n]).norm() / (want[n].norm() + 1e-12)).item() < 0.1, n


@pytest.mark.parametrize("rot", ["alibi", "rope", "pope"])
def test_chunk_state_attention_equals_the_quadratic_form(rot):
    """Attention over segments of C tokens with the state handed on between them (and its gradient handed
    back) is the same function as one quadratic form over the whole sequence: loss and every gradient of
    the chunked kernel path against the unchunked kernel path and the torch definition."""
    m = _model(rot)
    tok, tgt = torch.randint(0, 256, (2, 256)), torch.randint(0, 256, (2, 256))
    with emulate.kernel_path():
        m.attention_chunk = 64                 # four segments per sequence
        d = fused_bdh._Dims(m, 2, 256)
        assert d.J == 4 and d.handoff
        loss_c = m(tok, tgt)
        loss_c.backward()
        gc = {n: p.grad.clone() for n, p in m.named_parameters()}
        m.zero_grad()
        m.attention_chunk = 256                # one segment: the quadratic form
        loss_q = m(tok, tgt)
        loss_q.backward()
        gq = {n: p.grad.clone() for n, p in m.named_parameters()}
        m.zero_grad()
    m.attention_chunk = None
    loss_t = m(tok, tgt, mode="parallel")
    loss_t.backward()
    assert abs(loss_c.item() - loss_q.item()) < 5e-3 and abs(loss_c.item() - loss_t.item()) < 2e-2
    for n, p in m.named_parameters():
        assert _rel(gc[n], gq[n]) < 0.05, (n, _rel(gc[n], gq[n]))
        assert _cos(gc[n], p.grad) > 0.99 and _rel(gc[n], p.grad) < 0.12, (n, _cos(gc[n], p.grad), _rel(gc[n], p.grad))


@pytest.mark.parametrize("rot", ["alibi", "rope", "pope"])
def test_chunked_prefill_equals_the_recurrence(rot):
    """recurrent == chunked: logits and final state of a prefill that runs as segments with a carried state,
    started from a non-empty state, against the token-by-token recurrence."""
    m = _model(rot).eval()
    tok = torch.randint(0, 256, (2, 64 + 256))
    with torch.no_grad():
        st_t = m.init_state()
        want = m.forward_with_state(tok, st_t, mode="recurrent")
        with emulate.kernel_path():
            m.attention_chunk = 64
            st = m.init_state()
            first = m.forward_with_state(tok[:, :64], st)             # leaves a state behind
            rest = m.forward_with_state(tok[:, 64:], st)              # four segments continuing from it
        m.attention_chunk = None
    got = torch.cat([first, rest], 1)
    assert _rel(got, want) < 0.05
    assert st.position == st_t.position
    for a, b in zip(st.layers, st_t.layers):
        assert _rel(a.rho, b.rho) < 0.05


def test_pope_layers_that_drop_their_rotated_query_give_the_same_gradients():
    """A PoPE layer may keep x only and write q = softplus(x) (cos, sin) again in its backward pass
    (`model.drop_rotated`): same loss, gradients equal up to the bf16 rounding of x."""
    m = _model("pope")
    tok, tgt = torch.randint(0, 256, (2, 128)), torch.randint(0, 256, (2, 128))
    with emulate.kernel_path():
        l0 = m(tok, tgt)
        l0.backward()
        g0 = {n: p.grad.clone() for n, p in m.named_parameters()}
        m.zero_grad()
        m.drop_rotated = 1
        m.recompute = 1
        l1 = m(tok, tgt)
        l1.backward()
    assert (m._recomputed_layers, m._dropped_q_layers) == (1, 1)
    assert l0.item() == l1.item()
    for n, p in m.named_parameters():
        assert _rel(p.grad, g0[n]) < 5e-3, (n, _rel(p.grad, g0[n]))


def test_memory_plan_picks_the_cheapest_mix_that_fits(monkeypatch):
    """`memory_plan` with a faked device memory: the large PoPE configuration (8 sequences of 2048 tokens) on a
    180 GB device keeps every layer and lets a few rebuild their query; with less memory it starts to recompute
    layers; RoPE models and explicit settings are left alone."""
    import types
    cfg = BDHConfig(n_layer=8, n_embd=512, n_head=8, n_latent_per_head=16384, vocab_size=256, dropout=0.0,
                    rotary_embedding="pope")
    m = types.SimpleNamespace(config=cfg, training=True, encoder=torch.zeros(1), freqs=torch.zeros(16384), slopes=None,
                              recompute="auto")
    d = fused_bdh._Dims(m, 8, 2048)
    per, work = fused_bdh.layer_activation_bytes(d), fused_bdh.backward_working_bytes(d)
    assert 17e9 < per < 19e9 and 20e9 < work < 25e9

    def with_free(gb):
        monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
        monkeypatch.setattr(torch.cuda, "mem_get_info", lambda: (int(gb * 1e9), int(192e9)))
        monkeypatch.setattr(torch.cuda, "memory_reserved", lambda: 0)
        monkeypatch.setattr(torch.cuda, "memory_allocated", lambda: 0)
        return fused_bdh.memory_plan(m, d)

    r, k = with_free(188)
    assert r == 0 and 3 <= k <= 6                      # nothing recomputed, some layers rebuild q
    r2, k2 = with_free(90)
    assert r2 > 0 and r2 + k2 <= 8                     # less memory: some layers are recomputed as well
    assert r2 * 5.4 + k2 <= fused_bdh.recompute_count(m, d) * 5.4 + 1e-9      # never worse than recompute alone
    m.drop_rotated = 0
    assert with_free(188) == (fused_bdh.recompute_count(m, d), 0)
    m.drop_rotated = None
    m.recompute = 3
    assert with_free(188) == (3, 0)                    # an explicit recompute count is taken as given


def test_time_block_pattern_skips_whole_tiles():
    """A banded `BlockPattern2d` over 1024 tokens leaves most 128 x 256 score tiles without an active entry:
    those tiles are not computed (tile predicate of the causal walker); result and gradients still equal the
    torch statement."""
    from burn_dragon_b200.ops.block_sparse import BlockPattern1d, BlockPattern2d, BlockSparseConfig
    torch.manual_seed(0)
    m = BDH(BDHConfig(n_layer=1, n_embd=64, n_head=2, n_latent_per_head=64, vocab_size=256, dropout=0.0,
                      rotary_embedding="alibi"))
    nb = 8                                                   # blocks of 128 tokens; keep the diagonal and one below
    pairs = [(r, c) for r in range(nb) for c in range(nb) if 0 <= r - c <= 1]
    m.config.block_sparse = BlockSparseConfig(BlockPattern1d.dense(64), BlockPattern2d.from_pairs(128, pairs))
    tok, tgt = torch.randint(0, 256, (1, 1024)), torch.randint(0, 256, (1, 1024))
    m.use_native = False
    ref = m.forward_fast(tok, tgt)
    ref.backward()
    want = {n: p.grad.clone() for n, p in m.named_parameters()}
    m.zero_grad()
    m.use_native = True
    with emulate.kernel_path():
        d = fused_bdh._Dims(m, 1, 1024, fast=True)
        skip = d.tile_skip
        assert skip.shape == (8, 4) and int(skip.sum()) >= 16       # at least half of the 32 tiles are skipped
        assert int(skip[7, 0]) == 1 and int(skip[7, 3]) == 0 and int(skip[0, 0]) == 0
        got = m.forward_fast(tok, tgt)
        got.backward()
    assert abs(got.item() - ref.item()) < 2e-2
    for n, p in m.named_parameters():
        assert ((p.grad - want[n]).norm() / (want[n].norm() + 1e-12)).item() < 0.1, n

"""Headless inference sessions (the reference's web-page interface as a Python API)."""
import json
import os
from pathlib import Path

import pytest
import torch

from burn_dragon_b200.data.tokenizer import CharVocab
from burn_dragon_b200.engine import burn_record as BR
from burn_dragon_b200.engine import generation as GEN
from burn_dragon_b200.engine import session as S
from burn_dragon_b200.models.bdh import BDH, BDHConfig

_REF = Path(os.environ.get("BDH_REFERENCE_DIR", Path(__file__).resolve().parents[2] / "reference"))
ASSET = _REF / "www" / "assets" / "model" / "tiny_shakespeare"


def _artefacts(rot="rope", half=False):
    torch.manual_seed(0)
    vocab = CharVocab.fit(["hello world, this is a tiny corpus."], include_unknown=True)
    m = BDH(BDHConfig(n_layer=2, n_embd=32, n_head=2, mlp_internal_dim_multiplier=2, vocab_size=len(vocab),
                      dropout=0.0, rotary_embedding=rot)).eval()
    blob = BR.serialize(BR.from_model(m, half=half))
    cfg = json.dumps(dict(run_name="t", block_size=32, overrides=dict(
        n_layer=2, n_embd=32, n_head=2, mlp_internal_dim_multiplier=2, rotary_embedding=rot)))
    return m, vocab, blob, json.dumps(vocab.to_record()), cfg


@pytest.mark.parametrize("half", [False, True])
def test_session_greedy_equals_generate_tokens(half):
    m, vocab, blob, vjson, cjson = _artefacts(half=half)
    sess = S.load_model(blob, vjson, cjson, device="cpu")
    assert sess.block_size == 32 and sess.model.config.n_layer == 2
    sess.start_stream("hello", max_tokens=12, greedy=True)
    text = ""
    chunks = 0
    while not sess.done:
        text += sess.next_chunk(max_tokens=4)
        chunks += 1
    assert chunks >= 3
    ids = torch.tensor([vocab.encode("hello")])
    want = GEN.generate_tokens(sess.model, ids, "cpu", GEN.GenerationSettings(12, greedy=True))[0, 5:].tolist()
    eos = vocab.eos_id
    if eos in want:
        want = want[:want.index(eos)]
    assert text == vocab.decode(want)


def test_session_serves_several_streams_and_respects_limits():
    m, vocab, blob, vjson, cjson = _artefacts("alibi")
    sess = S.load_model(blob, vjson, cjson, device="cpu")
    sess.start_stream(["hello", "world"], max_tokens=6, temperature=1.0, top_k=5, seed=3)
    out = ["", ""]
    while not sess.done:
        a, b = sess.next_chunk(max_tokens=2)
        out[0] += a
        out[1] += b
    assert sess.generated <= 6
    # same seed, same text
    sess.start_stream(["hello", "world"], max_tokens=6, temperature=1.0, top_k=5, seed=3)
    again = ["", ""]
    while not sess.done:
        a, b = sess.next_chunk(max_tokens=2)
        again[0] += a
        again[1] += b
    assert again == out
    with pytest.raises(ValueError):
        sess.start_stream(["hello", "hi"], max_tokens=2)


def test_load_model_rejects_mismatched_artefacts():
    m, vocab, blob, vjson, cjson = _artefacts()
    other = CharVocab.fit(["abc"], include_unknown=True)
    with pytest.raises(ValueError):
        S.load_model(blob, json.dumps(other.to_record()), cjson, device="cpu")
    bad = json.loads(cjson)
    bad["overrides"]["mlp_internal_dim_multiplier"] = 8
    with pytest.raises(ValueError):
        S.load_model(blob, vjson, json.dumps(bad), device="cpu")


@pytest.mark.skipif(not (ASSET / "model.bin").exists(), reason="reference checkpoint not mounted")
def test_shipped_checkpoint_streams_text():
    sess = S.load_model((ASSET / "model.bin").read_bytes(), (ASSET / "vocab.json").read_text(),
                        (ASSET / "config.json").read_text(), device="cpu")
    assert sess.model.config.n_layer == 4 and sess.model.config.rotary_embedding == "alibi"
    sess.start_stream("First Citizen:\n", max_tokens=24, greedy=True)
    text = ""
    while not sess.done:
        text += sess.next_chunk()
    assert len(text) > 0 and all(ch in sess.tokenizer.ch2id or ch == "?" for ch in text)


def test_http_server_generate_and_stream():
    """The HTTP front end returns what the session API returns: whole text, and the same text in chunks."""
    import threading
    import urllib.request
    from burn_dragon_b200.engine import server as SV
    m, vocab, blob, vjson, cjson = _artefacts("alibi")
    sess = S.load_model(blob, vjson, cjson, device="cpu")
    srv = SV.make_server(sess, "127.0.0.1", 0)
    port = srv.server_address[1]
    th = threading.Thread(target=srv.serve_forever, daemon=True)
    th.start()
    try:
        base = f"http://127.0.0.1:{port}"
        health = json.loads(urllib.request.urlopen(base + "/health", timeout=30).read())
        assert health["status"] == "ok" and health["model"]["n_layer"] == 2
        page = urllib.request.urlopen(base + "/", timeout=30)
        html = page.read().decode()
        assert page.headers["Content-Type"].startswith("text/html") and '"/generate"' in html and "/health" in html

        def post(body):
            req = urllib.request.Request(base + "/generate", data=json.dumps(body).encode(),
                                         headers={"Content-Type": "application/json"})
            return urllib.request.urlopen(req, timeout=60)

        whole = json.loads(post(dict(prompt="hello", max_tokens=10, greedy=True)).read())
        lines = [json.loads(l) for l in post(dict(prompt="hello", max_tokens=10, greedy=True, stream=True,
                                                  chunk_tokens=3)).read().decode().splitlines() if l.strip()]
        assert lines[-1]["done"] is True and lines[-1]["tokens"] == whole["tokens"] <= 10
        assert "".join(l["text"] for l in lines[:-1]) == whole["text"]
        ref = S.load_model(blob, vjson, cjson, device="cpu")
        ref.start_stream("hello", max_tokens=10, greedy=True)
        text = ""
        while not ref.done:
            text += ref.next_chunk()
        assert whole["text"] == text
        two = json.loads(post(dict(prompt=["hello", "world"], max_tokens=4, greedy=True)).read())
        assert isinstance(two["text"], list) and len(two["text"]) == 2
        import urllib.error
        with pytest.raises(urllib.error.HTTPError) as err:
            post(dict(prompt=["hello", "hi"], max_tokens=4))
        assert err.value.code == 400
        metrics = urllib.request.urlopen(base + "/metrics", timeout=30).read().decode()
        vals = {l.split()[0]: float(l.split()[1]) for l in metrics.splitlines() if l and not l.startswith("#")}
        assert vals["bdh_requests_total"] == 4 and vals["bdh_request_errors_total"] == 1
        assert vals["bdh_generated_tokens_total"] == 2 * whole["tokens"] + 2 * 4
        assert vals["bdh_generate_busy_seconds_total"] > 0
    finally:
        srv.shutdown()
        srv.server_close()


def test_snapshot_restore_branches_from_a_shared_prefix():
    m, vocab, blob, vjson, cjson = _artefacts("rope")
    sess = S.load_model(blob, vjson, cjson, device="cpu")
    sess.start_stream("hello world", max_tokens=8, greedy=True)
    snap = sess.snapshot()
    first = ""
    while not sess.done:
        first += sess.next_chunk()
    # branch 1: same continuation from the snapshot
    sess.restore(snap)
    again = ""
    while not sess.done:
        again += sess.next_chunk()
    assert again == first
    # branch 2: a fresh token limit from the same prefix state, in another session of the same model
    other = S.load_model(blob, vjson, cjson, device="cpu")
    other.restore(snap, max_tokens=3)
    short = ""
    while not other.done:
        short += other.next_chunk()
    assert other.generated == 3 and first.startswith(short)

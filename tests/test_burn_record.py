"""Burn record codec against the one golden artefact of the reference: the shipped web checkpoint."""
import os
from pathlib import Path

import numpy as np
import pytest
import torch

from burn_dragon_b200.data.tokenizer import CharVocab
from burn_dragon_b200.engine import burn_record as BR
from burn_dragon_b200.models.bdh import BDH, BDHConfig

# the reference checkout sits beside this repository (or where BDH_REFERENCE_DIR points)
_REF = Path(os.environ.get("BDH_REFERENCE_DIR", Path(__file__).resolve().parents[2] / "reference"))
ASSET = _REF / "www" / "assets" / "model" / "tiny_shakespeare"
needs_asset = pytest.mark.skipif(not (ASSET / "model.bin").exists(), reason="reference checkpoint not mounted")

SNIPPET = ("First Citizen:\nBefore we proceed any further, hear me speak.\n\nAll:\nSpeak, speak.\n\n"
           "First Citizen:\nYou are all resolved rather to die than to famish?\n\nAll:\nResolved. resolved.\n")


@needs_asset
def test_byte_exact_reencode():
    raw = (ASSET / "model.bin").read_bytes()
    rec = BR.parse(raw)
    assert rec.metadata == BR.FULL
    assert [tuple(rec.params[k].data.shape) for k in BR.PARAM_ORDER] == \
        [(69, 128), (4, 128, 128), (4, 128, 128), (512, 128), (128, 69)]
    assert all(len(p.id) == 13 and p.dtype_tag == BR.DTYPE_F32 for p in rec.params.values())
    assert BR.serialize(rec) == raw


def _load_model():
    rec = BR.load(ASSET / "model.bin")
    rc = BR.read_run_config(ASSET / "config.json")["overrides"]
    dims = BR.infer_dims(rec)
    cfg = BDHConfig(n_layer=rc["n_layer"], n_embd=rc["n_embd"], n_head=rc["n_head"],
                    mlp_internal_dim_multiplier=rc["mlp_internal_dim_multiplier"], vocab_size=dims["vocab_size"],
                    dropout=0.0, rotary_embedding=rc["rotary_embedding"])
    assert cfg.latent_per_head == dims["n_latent_per_head"]
    m = BDH(cfg).eval()
    m.load_state_dict(BR.to_state_dict(rec))
    return m


@needs_asset
def test_golden_cross_entropy_recurrent_path():
    """The shipped weights through the canonical (recurrent) path score ~1.1 nats/char on Shakespeare
    text; the row-normalised parallel path is a different function and scores far worse."""
    m = _load_model()
    vocab = CharVocab.from_json_str((ASSET / "vocab.json").read_text())
    ids = torch.tensor([vocab.encode(SNIPPET)])
    with torch.no_grad():
        ce_rec = m(ids[:, :-1], ids[:, 1:], mode="recurrent").item()
        ce_par = m(ids[:, :-1], ids[:, 1:], mode="parallel").item()
        ce_fast = m.forward_fast(ids[:, :-1], ids[:, 1:]).item()
    assert abs(ce_rec - ce_par) < 1e-4
    assert ce_rec < 1.6, ce_rec
    assert ce_fast > ce_rec + 1.0


@needs_asset
def test_model_roundtrip_through_record(tmp_path):
    m = _load_model()
    rec = BR.from_model(m)
    BR.save(rec, tmp_path / "model-1.bin")
    m2 = BDH(m.config)
    BR.load_into(m2, tmp_path / "model-1.bin")
    for (k, a), (_, b) in zip(m.state_dict().items(), m2.state_dict().items()):
        assert torch.equal(a, b), k
    # the exported tensors are byte-identical to the reference's own file
    ref = BR.load(ASSET / "model.bin")
    for k in BR.PARAM_ORDER:
        assert np.array_equal(rec.params[k].data, ref.params[k].data), k


@needs_asset
def test_quantize_f16(tmp_path):
    src = tmp_path / "model-3.bin"
    src.write_bytes((ASSET / "model.bin").read_bytes())
    out = BR.quantize_file(src)
    assert out.name == "model-3-f16.bin"
    rec = BR.load(out)
    assert rec.half and rec.metadata[4] == "HalfPrecisionSettings"
    full = BR.load(src)
    for k in BR.PARAM_ORDER:
        assert rec.params[k].data.dtype == np.float16
        assert np.allclose(rec.params[k].data.astype(np.float32), full.params[k].data, atol=2e-3, rtol=1e-3)
    m = BDH(BDHConfig(n_layer=4, n_embd=128, n_head=4, vocab_size=69, dropout=0.0))
    BR.load_into(m, out)
    # f16 tensors carry variant 3 of burn-tensor's DType (F64, F32, Flex32, F16, ...)
    assert all(p.dtype_tag == BR.DTYPE_F16 == 3 for p in rec.params.values())
    # a tag that contradicts the metadata is rejected; the tag earlier versions wrote is still read
    raw = bytearray(out.read_bytes())
    assert raw[-1] == 3
    raw[-1] = BR.DTYPE_F16_LEGACY
    assert BR.parse(bytes(raw)).params["lm_head"].dtype_tag == BR.DTYPE_F16
    raw[-1] = BR.DTYPE_F32
    with pytest.raises(ValueError, match="dtype tag"):
        BR.parse(bytes(raw))


def test_varint_roundtrip():
    for v in (0, 1, 250, 251, 65535, 65536, 2 ** 32 - 1, 2 ** 32, 2 ** 40):
        b = BR.write_varint(v)
        got, pos = BR.read_varint(b, 0)
        assert got == v and pos == len(b)


def test_varint_and_string_roundtrip_property():
    """bincode varints and length-prefixed strings: decode(encode(x)) == x over the whole u64 range."""
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=300, deadline=None)
    @given(st.integers(min_value=0, max_value=2 ** 64 - 1))
    def ints(v):
        enc = BR.write_varint(v)
        got, pos = BR.read_varint(enc + b"\xff", 0)
        assert got == v and pos == len(enc)
        assert len(enc) == (1 if v < 251 else 3 if v < 2 ** 16 else 5 if v < 2 ** 32 else 9)

    @settings(max_examples=100, deadline=None)
    @given(st.text(max_size=40))
    def strings(s):
        enc = BR.write_string(s)
        got, pos = BR.read_string(enc, 0)
        assert got == s and pos == len(enc)

    ints()
    strings()


def test_char_vocab_roundtrip_property():
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=100, deadline=None)
    @given(st.text(alphabet=st.characters(blacklist_categories=("Cs",), min_codepoint=4), min_size=1, max_size=60))
    def roundtrip(text):
        v = CharVocab.fit([text], include_unknown=True)
        ids = v.encode(text)
        assert v.decode(ids) == text
        assert v.encode_array(text).tolist() == ids

    roundtrip()


@needs_asset
def test_infer_cli_runs_the_shipped_model_directory(capsys):
    """`infer --checkpoint <exported model directory>` (model.bin + vocab.json + config.json side by side)."""
    from burn_dragon_b200 import cli
    rc = cli.main(["infer", "--checkpoint", str(ASSET), "--prompt", "ROMEO:", "--max-tokens", "24", "--greedy",
                   "--device", "cpu"])
    out = capsys.readouterr().out
    assert rc == 0 and "ROMEO:" in out
    tail = out.split("ROMEO:", 1)[1]
    assert len(tail.strip()) >= 10


@needs_asset
def test_eval_cli_scores_shakespeare_text(tmp_path, capsys):
    """`eval` on the shipped checkpoint: a Shakespeare snippet scores about 1.1-1.6 nats per character,
    and the windowed evaluation (state carried across windows) equals one long call."""
    import json
    from burn_dragon_b200 import cli
    text = tmp_path / "t.txt"
    text.write_text(SNIPPET)
    outs = []
    for window in (32, 4096):
        assert cli.main(["eval", "--checkpoint", str(ASSET), "--text", str(text), "--device", "cpu",
                         "--window", str(window)]) == 0
        outs.append(json.loads(capsys.readouterr().out.strip().splitlines()[-1]))
    assert outs[0]["tokens"] == outs[1]["tokens"] == len(SNIPPET) - 1
    assert 0.5 < outs[1]["nats_per_token"] < 1.8
    assert abs(outs[0]["nats_per_token"] - outs[1]["nats_per_token"]) < 1e-3


@needs_asset
def test_cpp_oracle_scores_the_shipped_checkpoint():
    """Shipped weights through the C++ oracle: same cross-entropy as the torch recurrent path on the
    first 150 characters of the corpus (about 1.1 nats per character)."""
    import torch.nn.functional as F
    from burn_dragon_b200.utils import hostlib
    m = _load_model()
    vocab = CharVocab.from_json_str((ASSET / "vocab.json").read_text())
    ids = vocab.encode(SNIPPET[:150])
    logits = torch.from_numpy(hostlib.oracle_forward(m, ids[:-1]))
    ce_cpp = F.cross_entropy(logits, torch.tensor(ids[1:])).item()
    with torch.no_grad():
        ce_torch = m(torch.tensor([ids[:-1]]), torch.tensor([ids[1:]]), mode="recurrent").item()
    assert abs(ce_cpp - ce_torch) < 1e-4
    assert abs(ce_cpp - 1.1055) < 0.02, ce_cpp

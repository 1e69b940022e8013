"""Config merge rules, tokenizers, datasets and the loader (CPU tier)."""
import json

import numpy as np
import pytest
import torch

from burn_dragon_b200 import config as C
from burn_dragon_b200.data import dataset as D
from burn_dragon_b200.data import tokenizer as T

BASE = """
[dataset]
cache_dir = "data"
type = "shakespeare"
[dataset.tokenizer]
type = "char"
vocab_path = "vocab.json"
[training]
block_size = 8
batch_size = 2
max_iters = 10
log_frequency = 5
[optimizer]
learning_rate = 0.001
weight_decay = 0.1
[optimizer.lr_schedule]
type = "cosine"
min_lr = 0.0001
num_iters = 100
[generation]
prompt = "hi"
[model]
n_layer = 2
"""


def _write(tmp_path, name, text):
    p = tmp_path / name
    p.write_text(text)
    return p


def test_layered_merge_order_and_deep_merge(tmp_path):
    a = _write(tmp_path, "a.toml", BASE)
    b = _write(tmp_path, "b.toml", "[training]\nbatch_size = 7\n[model]\nn_embd = 64\n")
    c = _write(tmp_path, "c.toml", "[training]\nbatch_size = 9\n")
    cfg = C.load_training_config([a, b, c])
    assert cfg.training.batch_size == 9 and cfg.training.block_size == 8
    assert cfg.model.n_layer == 2 and cfg.model.n_embd == 64
    assert cfg.optimizer.lr_schedule.type == "cosine" and cfg.optimizer.lr_schedule.min_lr == 0.0001


def test_type_change_clears_table(tmp_path):
    a = _write(tmp_path, "a.toml", BASE)
    b = _write(tmp_path, "b.toml", '[optimizer.lr_schedule]\ntype = "linear"\nfinal_lr = 0.0002\n')
    s = C.load_training_config([a, b]).optimizer.lr_schedule
    assert s.type == "linear" and s.final_lr == 0.0002 and s.min_lr is None and s.num_iters is None
    same = _write(tmp_path, "c.toml", '[optimizer.lr_schedule]\ntype = "cosine"\nnum_iters = 5\n')
    s2 = C.load_training_config([a, same]).optimizer.lr_schedule
    assert s2.min_lr == 0.0001 and s2.num_iters == 5           # same tag: merged, not cleared


def test_hf_config_and_errors(tmp_path):
    a = _write(tmp_path, "a.toml", BASE)
    hf = _write(tmp_path, "hf.toml", '[dataset]\ncache_dir = "hfdata"\ntype = "hugging_face"\nrepo_id = "x/y"\nformat = "parquet"\n'
                'train_files = ["a.parquet"]\ntext_fields = ["q", "a"]\ntemplate = "{q} {a}"\nmax_records = 3\n')
    d = C.load_training_config([a, hf]).dataset
    # a changed `type` tag clears the base [dataset] table, tokenizer sub-table included
    assert (d.type, d.repo_id, d.format, d.max_records, d.cache_dir) == ("hugging_face", "x/y", "parquet", 3, "hfdata")
    assert d.tokenizer.vocab_path is None
    with pytest.raises(C.ConfigError):
        C.load_training_config([a, _write(tmp_path, "bad.toml", "[training]\nbogus = 1\n")])
    with pytest.raises(C.ConfigError):
        C.load_training_config([])
    with pytest.raises(C.ConfigError):
        C.load_training_config([_write(tmp_path, "m.toml", "[dataset]\ncache_dir='x'\n")])


def test_presets_load():
    cfg = C.load_preset("tiny")
    assert (cfg.model.n_layer, cfg.model.n_embd, cfg.training.batch_size) == (4, 128, 64)
    assert cfg.model.rotary_embedding == "alibi" and cfg.training.epochs == 30
    big = C.load_preset("b200_base")
    assert big.training.epochs is None and big.model.n_latent_per_head == 8192


def test_schedules():
    from burn_dragon_b200.engine.optim import LRSchedule
    cos = LRSchedule(C.LearningRateScheduleConfig("cosine", None, 0.1, 10), 1.0, 100)
    assert cos(0) == 1.0 and abs(cos(10) - 0.1) < 1e-9 and cos(50) == cos(10)
    lin = LRSchedule(C.LearningRateScheduleConfig("linear", final_lr=0.0), 1.0, 4)
    assert [round(lin(i), 2) for i in range(5)] == [1.0, 0.75, 0.5, 0.25, 0.0]
    st = LRSchedule(C.LearningRateScheduleConfig("step", gamma=0.5, step_size=2), 1.0, 10)
    assert [st(i) for i in (0, 1, 2, 4)] == [1.0, 1.0, 0.5, 0.25]
    ex = LRSchedule(C.LearningRateScheduleConfig("exponential", gamma=0.9), 2.0, 10)
    assert abs(ex(2) - 2.0 * 0.81) < 1e-12
    noam = LRSchedule(C.LearningRateScheduleConfig("noam", warmup_steps=4, model_size=64), 1.0, 100)
    assert noam(0) < noam(3) and noam(3) >= noam(20)


def test_byte_tokenizer():
    t = T.ByteTokenizer(True)
    assert len(t) == 259 and (t.bos_id, t.eos_id, t.pad_id) == (256, 257, 258)
    ids = t.encode("hé", add_bos=True, add_eos=True)
    assert ids[0] == 256 and ids[-1] == 257 and t.decode(ids) == "hé"
    assert t.decode([104, 257, 105]) == "h"            # stops at EOS
    assert t.decode([258, 104, 300]) == "h"            # PAD skipped, out-of-range ignored
    assert len(T.ByteTokenizer(False)) == 256 and T.ByteTokenizer(False).encode("a", True, True) == [97]


def test_char_vocab_roundtrip_and_unk(tmp_path):
    v = T.CharVocab.fit(["hello", "world"], include_unknown=True)
    assert v.id2ch[:4] == ["\x00", "\x01", "\x02", "\x03"] and v.id2ch[4:] == list("helowrd")
    ids = v.encode("hold!", add_bos=True, add_eos=True)
    assert ids[0] == v.bos_id and ids[-1] == v.eos_id and ids[-2] == v.unk_id
    assert v.decode(ids) == "hold?"
    v.save(tmp_path / "v.json")
    v2 = T.CharVocab.load(tmp_path / "v.json")
    assert v2 == v and json.loads((tmp_path / "v.json").read_text())["unk"] == 3
    strict = T.CharVocab.fit(["ab"], include_unknown=False)
    with pytest.raises(KeyError):
        strict.encode("abc")
    assert np.array_equal(v.encode_array("hello"), np.array(v.encode("hello")))


def _corpus(tmp_path, n=4000):
    d = tmp_path / "cache"
    d.mkdir()
    rng = np.random.default_rng(0)
    (d / "tinyshakespeare.txt").write_text("".join(rng.choice(list("abcdefg \n"), n)))
    return d


def test_shakespeare_dataset_batches(tmp_path):
    d = _corpus(tmp_path)
    ds = D.shakespeare_dataset(d, 16, 4, 0.9, C.TokenizerConfig("char", True, True, "vocab.json"))
    assert (d / "vocab.json").exists() and ds.train_len == int(np.float32(4000) * np.float32(0.9))
    b = ds.sample_batch(D.TRAIN)
    assert b.inputs.shape == b.targets.shape == (4, 16) and b.inputs.dtype == torch.int64
    assert torch.equal(b.inputs[:, 1:], b.targets[:, :-1])
    assert ds.steps_per_epoch(D.TRAIN) == -(-ds.train_len // 64)
    off, span = ds.split_offset_and_span(D.VAL)
    assert off == ds.train_len and span == 4000 - ds.train_len
    bv = ds.sample_batch(D.VAL)
    assert int(bv.inputs.min()) >= 0
    byte_ds = D.shakespeare_dataset(d, 16, 4, 0.9, C.TokenizerConfig("byte", True, True, None))
    assert len(byte_ds.tokenizer) >= 256


def test_loader_step_cap_and_state(tmp_path):
    ds = D.synthetic_dataset(5000, 8, 2, seed=1)
    ld = D.RandomDataLoader(ds, D.TRAIN, None, steps_per_epoch=4, total_steps=6, pin=False)
    assert len(list(ld)) == 4 and len(list(ld)) == 2 and len(list(ld)) == 0
    ld2 = D.RandomDataLoader(D.synthetic_dataset(5000, 8, 2, seed=1), D.TRAIN, None, 4, None, pin=False)
    first = [b.inputs.clone() for b in ld2]
    sd = ld2.state_dict()
    nxt = [b.inputs.clone() for b in ld2]
    ld2.load_state_dict(sd)
    again = [b.inputs.clone() for b in ld2]
    assert all(torch.equal(a, b) for a, b in zip(nxt, again)) and not torch.equal(first[0], nxt[0])


def test_hf_records_jsonl_csv_text_template(tmp_path):
    spec = D.HFSpec("x/y", None, "jsonl", [], [], ["q", "a"], " | ", None, None)
    p = tmp_path / "t.jsonl"
    p.write_text('{"q": "one", "a": 1}\n\n{"q": "two", "a": "2"}\n')
    recs = []
    D.collect_records(p, spec, recs)
    assert recs == ["one | 1\n", "two | 2\n"]
    spec_t = D.HFSpec("x/y", None, "csv", [], [], ["Title", "Poem"], "\n", "{Title}: { Poem }", 1)
    c = tmp_path / "t.csv"
    c.write_text('Title,Poem,Other\nA,"x, y",z\nB,w,z\n')
    recs = []
    D.collect_records(c, spec_t, recs)
    assert recs == ["A: x, y\n"]
    with pytest.raises(ValueError):
        D.render_template("{nope}", {"a": "b"})
    with pytest.raises(ValueError):
        D.render_template("{a", {"a": "b"})
    txt = tmp_path / "t.txt"
    txt.write_text("line one\n\nline two\n")
    recs = []
    D.collect_records(txt, D.HFSpec("x/y", None, "text", [], [], ["text"], "\n", None, None), recs)
    assert recs == ["line one\n", "line two\n"]
    assert D.hf_preset("deep_math").train_files[9] == "data/train-00009-of-00010.parquet"


def test_hf_dataset_offline_from_cache(tmp_path, monkeypatch):
    monkeypatch.setenv("BDH_OFFLINE", "1")
    spec = D.HFSpec("me/ds", None, "text", ["a.txt"], [], ["text"], "\n", None, None)
    with pytest.raises(FileNotFoundError):
        D.huggingface_dataset(tmp_path, 8, 2, 0.9, C.TokenizerConfig("byte", True, False, None), spec)
    f = tmp_path / "huggingface" / "me--ds" / "main" / "a.txt"
    f.parent.mkdir(parents=True)
    f.write_text("\n".join("sample text number %d" % i for i in range(50)))
    ds = D.huggingface_dataset(tmp_path, 8, 2, 0.9, C.TokenizerConfig("byte", True, False, None), spec)
    assert len(ds.tokens) > 500 and ds.sample_batch().inputs.shape == (2, 8)
    # the encoded corpus is cached; a second start reads it instead of the shards, and a changed
    # shard gets a fresh encoding
    caches = list(tmp_path.glob("tokens-*.npz"))
    assert len(caches) == 1
    monkeypatch.setattr(D, "collect_records", lambda *a, **k: (_ for _ in ()).throw(AssertionError("cache not used")))
    again = D.huggingface_dataset(tmp_path, 8, 2, 0.9, C.TokenizerConfig("byte", True, False, None), spec)
    assert np.array_equal(again.tokens, ds.tokens) and again.train_len == ds.train_len
    monkeypatch.undo()
    monkeypatch.setenv("BDH_OFFLINE", "1")
    f.write_text("\n".join("other text %d" % i for i in range(80)))
    fresh = D.huggingface_dataset(tmp_path, 8, 2, 0.9, C.TokenizerConfig("byte", True, False, None), spec)
    assert len(fresh.tokens) != len(ds.tokens) and len(list(tmp_path.glob("tokens-*.npz"))) == 2


def test_char_vocab_native_encode_matches_python():
    from burn_dragon_b200.data.tokenizer import CharVocab
    from burn_dragon_b200.utils import hostlib
    text = "héllo wörld — ∑ 🙂 abc\nline two"
    v = CharVocab.fit([text], include_unknown=True)
    assert hostlib.available()
    for s in (text, "", "zzz 🙂 qq", "abc"):
        assert v.encode_array(s).tolist() == v.encode(s)
    strict = CharVocab.fit(["abc"], include_unknown=False)
    import pytest
    with pytest.raises(KeyError):
        strict.encode_array("abd")


def test_profiling_hooks_without_cuda_and_metrics_fields(tmp_path):
    import json
    import torch
    from burn_dragon_b200.engine.trainer import Trainer
    from burn_dragon_b200.models.bdh import BDH, BDHConfig
    from burn_dragon_b200.utils import profiling as prof
    prof.enable(nvtx=True, timers=True)
    try:
        m = BDH(BDHConfig(n_layer=1, n_embd=32, n_head=2, n_latent_per_head=16, vocab_size=64, dropout=0.0))
        tr = Trainer(m, lr=1e-3)
        tr.track_grad_norm = m.measure_sparsity = True
        tok = torch.randint(0, 64, (2, 17))
        tr.train_step(tok[:, :-1], tok[:, 1:])
        assert float(tr.last_grad_norm) > 0
        assert 0.0 < float(m.last_sparsity["xy"]) <= float(m.last_sparsity["x"]) <= 1.0
        rep = prof.report()
        # (without a CUDA device NVTX is skipped and the timers use the host clock)
        assert {"step", "forward", "backward", "optimizer"} <= set(rep) and rep["step"]["ms"] >= rep["forward"]["ms"] > 0
    finally:
        prof.enable(nvtx=False, timers=False)


def test_device_resident_loader_contract_and_resume():
    """`ResidentDataLoader`: batches are gathered on the device from a resident token array; same
    contract as the host loader (shape, shifted targets, split bounds, global step cap), reproducible,
    and its generator state survives a checkpoint."""
    import numpy as np
    import torch
    from burn_dragon_b200.data import dataset as D
    ds = D.synthetic_dataset(5000, block_size=16, batch_size=4, vocab=256, seed=1)
    # make the two splits distinguishable: validation tokens are >= 128
    off, span = ds.split_offset_and_span(D.VAL)
    ds.tokens[:off] %= 128
    ds.tokens[off:] = 128 + ds.tokens[off:] % 128
    tr = D.ResidentDataLoader(ds, D.TRAIN, "cpu", steps_per_epoch=3, total_steps=5, seed=7)
    va = D.ResidentDataLoader(ds, D.VAL, "cpu", steps_per_epoch=2, seed=7)
    assert tr.tokens.dtype == torch.int16 and tr.tokens.numel() == off
    first = list(tr)
    assert len(first) == 3 and all(b.inputs.shape == (4, 16) and b.inputs.dtype == torch.int64 for b in first)
    for b in first:
        assert torch.equal(b.inputs[:, 1:], b.targets[:, :-1]) and int(b.inputs.max()) < 128 and int(b.targets.max()) < 128
        # every window is a contiguous slice of the corpus
        for row_in, row_t in zip(b.inputs, b.targets):
            w = torch.cat([row_in, row_t[-1:]]).numpy()
            starts = np.flatnonzero(ds.tokens[:off - 16] == w[0])
            assert any(np.array_equal(ds.tokens[s:s + 17], w) for s in starts)
    assert all(int(b.inputs.min()) >= 128 for b in va)
    sd = tr.state_dict()
    rest = list(tr)
    assert len(rest) == 2 and tr.consumed == 5 and list(tr) == []          # the global cap
    again = D.ResidentDataLoader(ds, D.TRAIN, "cpu", steps_per_epoch=3, total_steps=5, seed=7)
    again.load_state_dict(sd)
    resumed = list(again)
    assert len(resumed) == 2 and all(torch.equal(a.inputs, b.inputs) for a, b in zip(rest, resumed))
    # another rank (its own seed) that restores the state rank 0 wrote continues ITS sequence, not rank 0's
    other = D.ResidentDataLoader(ds, D.TRAIN, "cpu", steps_per_epoch=3, total_steps=5, seed=8)
    uninterrupted = [b.inputs for b in other] + [b.inputs for b in other]
    other2 = D.ResidentDataLoader(ds, D.TRAIN, "cpu", steps_per_epoch=3, total_steps=5, seed=8)
    other2.load_state_dict(sd)
    resumed2 = [b.inputs for b in other2]
    assert all(torch.equal(a, b) for a, b in zip(uninterrupted[3:], resumed2))
    assert not any(torch.equal(a, b.inputs) for a, b in zip(resumed2, resumed))
    same = D.ResidentDataLoader(ds, D.TRAIN, "cpu", steps_per_epoch=3, total_steps=5, seed=7)
    assert all(torch.equal(a.inputs, b.inputs) for a, b in zip(first, same))


def test_host_loader_resume_keeps_per_rank_streams():
    """Every rank of a data-parallel job restores the loader state that rank 0 wrote. With the
    per-rank stream key the ranks keep drawing different windows after the resume, and each rank's
    batches equal those of its uninterrupted run."""
    import torch
    from burn_dragon_b200.data import dataset as D

    def loader(rank):
        ds = D.synthetic_dataset(20000, block_size=16, batch_size=4, vocab=256, seed=1)
        return D.RandomDataLoader(ds, D.TRAIN, None, steps_per_epoch=3, total_steps=9, pin=False, stream=(1337, rank))

    full = {}
    for r in (0, 1):
        ld = loader(r)
        full[r] = [b.inputs.clone() for b in ld] + [b.inputs.clone() for b in ld] + [b.inputs.clone() for b in ld]
        assert len(full[r]) == 9
    assert not any(torch.equal(a, b) for a, b in zip(full[0], full[1]))
    # rank 0 writes the state after 3 batches; both ranks restore it
    l0 = loader(0)
    list(l0)
    sd = l0.state_dict()
    assert "rng" not in sd and sd["draws"] == 3
    for r in (0, 1):
        ld = loader(r)
        ld.load_state_dict(sd)
        resumed = [b.inputs for b in ld]
        assert len(resumed) == 3 and all(torch.equal(a, b) for a, b in zip(resumed, full[r][3:6])), r

"""Run directories, checkpoints and bit-exact resume (CPU tier)."""
import json

import torch

from burn_dragon_b200 import config as C
from burn_dragon_b200.data import dataset as D
from burn_dragon_b200.engine import checkpoint as CK
from burn_dragon_b200.engine.trainer import Trainer
from burn_dragon_b200.models.bdh import BDH, BDHConfig


def _setup(seed=0):
    torch.manual_seed(seed)
    m = BDH(BDHConfig(n_layer=2, n_embd=32, n_head=2, vocab_size=256, dropout=0.0, rotary_embedding="rope"))
    tr = Trainer(m, lr=1e-2)
    ds = D.synthetic_dataset(4000, 16, 4, seed=3)
    ld = D.RandomDataLoader(ds, D.TRAIN, None, 100, None, pin=False)
    return m, tr, ld


def _steps(tr, ld, n):
    it = iter(ld)
    return [float(tr.train_step(*(lambda b: (b.inputs, b.targets))(next(it)))) for _ in range(n)]


def test_run_dir_layout(tmp_path):
    cfg = C.load_preset("tiny")
    run_dir, name = CK.create_run_dir(tmp_path / "runs")
    assert "-" in name and not run_dir.exists()
    CK.write_latest_run(tmp_path / "runs", name)
    p = CK.write_run_config(cfg, run_dir, name)
    data = json.loads(p.read_text())
    assert data["run_name"] == name and data["block_size"] == 512 and data["overrides"]["n_embd"] == 128
    assert (tmp_path / "runs" / "latest").read_text() == name
    assert CK.resolve_run_dir(None, tmp_path / "runs") == run_dir


def test_resume_is_bit_exact(tmp_path):
    m, tr, ld = _setup()
    _steps(tr, ld, 3)
    CK.save_checkpoint(tmp_path / "run", 1, m, tr, ld)
    cont = _steps(tr, ld, 3)
    m2, tr2, ld2 = _setup(seed=99)                       # different init: everything must come from disk
    mp, sp, ep = CK.resolve_checkpoint(str(tmp_path / "run"))
    assert ep == 1 and mp.name == "model-1.bin" and sp.name == "state-1.pt"
    CK.load_checkpoint(m2, mp, sp, tr2, ld2)
    assert tr2.step_index == 3 and tr2.opt.step_count == 3
    assert _steps(tr2, ld2, 3) == cont
    for a, b in zip(m.parameters(), m2.parameters()):
        assert torch.equal(a, b)


def test_latest_epoch_and_explicit_file(tmp_path):
    m, tr, ld = _setup()
    for e in (1, 2, 10):
        CK.save_checkpoint(tmp_path / "r", e, m, tr, ld)
    assert CK.find_latest_epoch(tmp_path / "r" / "checkpoint") == 10
    mp, sp, ep = CK.resolve_checkpoint(str(tmp_path / "r"), epoch=2)
    assert ep == 2
    mp2, sp2, ep2 = CK.resolve_checkpoint(str(mp))
    assert mp2 == mp and sp2 is None and ep2 == 2


def test_export_then_infer_from_the_exported_directory(tmp_path, capsys):
    """train -> export (f16) -> infer from the exported directory."""
    from burn_dragon_b200 import cli
    cfg = tmp_path / "t.toml"
    cfg.write_text("[training]\nbatch_size = 2\nblock_size = 16\nlog_frequency = 1\n"
                   "[model]\nn_layer = 1\nn_embd = 32\nn_head = 2\ndropout = 0.0\n")
    runs = tmp_path / "runs"
    assert cli.main(["train", "-c", str(cfg), "--synthetic", "--device", "cpu", "--max-iters", "2", "--runs", str(runs)]) == 0
    out = tmp_path / "exported"
    assert cli.main(["export", "--runs", str(runs), "--output", str(out), "--f16"]) == 0
    assert (out / "model.bin").exists() and (out / "config.json").exists()
    capsys.readouterr()
    assert cli.main(["infer", "--checkpoint", str(out), "--prompt", "ab", "--max-tokens", "5", "--greedy",
                     "--device", "cpu"]) == 0
    cap = capsys.readouterr()
    assert "loaded" in cap.err and cap.out.startswith("ab")


def test_train_then_infer_a_non_bdh_model_through_the_cli(tmp_path, capsys):
    """Model families without a Burn record (weights live in state-N.pt): byte-trained run, then infer."""
    import os
    from burn_dragon_b200 import cli
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    over = tmp_path / "o.toml"
    over.write_text("[training]\nbatch_size = 2\nblock_size = 64\nlog_frequency = 1\n")
    runs = tmp_path / "runs"
    preset = os.path.join(root, "config", "mamba2.toml")
    assert cli.main(["train", "-c", preset, "-c", str(over), "--synthetic", "--device", "cpu", "--max-iters", "2",
                     "--runs", str(runs)]) == 0
    capsys.readouterr()
    assert cli.main(["infer", "--runs", str(runs), "-c", preset, "--prompt", "ab", "--max-tokens", "6", "--greedy",
                     "--device", "cpu"]) == 0
    assert capsys.readouterr().out.startswith("ab")


def test_train_and_resume_with_the_device_resident_loader(tmp_path, capsys):
    """`[dataset] device_resident = true`: batches gathered on the device; a resumed run continues the
    loader's generator (and a run saved with the host loader can be continued with the resident one)."""
    from burn_dragon_b200 import cli
    over = tmp_path / "o.toml"
    over.write_text("[training]\nbatch_size = 2\nblock_size = 32\nlog_frequency = 1\n\n[dataset]\ndevice_resident = true\n\n"
                    "[model]\nn_layer = 1\nn_embd = 32\nn_head = 2\n")
    host = tmp_path / "h.toml"
    host.write_text(over.read_text().replace("device_resident = true", "device_resident = false"))
    runs = tmp_path / "runs"
    base = ["--synthetic", "--device", "cpu", "--runs", str(runs)]
    assert cli.main(["train", "-c", str(over), "--max-iters", "3"] + base) == 0
    assert "[valid       3]" in capsys.readouterr().out
    assert cli.main(["train", "-c", str(over), "--max-iters", "5", "--resume", "latest"] + base) == 0
    out = capsys.readouterr().out
    assert "step 3" in out and "[valid       5]" in out
    assert cli.main(["train", "-c", str(host), "--max-iters", "6", "--resume", "latest"] + base) == 0
    assert "[valid       6]" in capsys.readouterr().out
    assert cli.main(["train", "-c", str(over), "--max-iters", "7", "--resume", "latest"] + base) == 0
    assert "[valid       7]" in capsys.readouterr().out

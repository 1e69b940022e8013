"""Host-side logic of the parallel layer on gloo CPU ranks (world size 2)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_job(cmd, env, timeout):
    """Run a launcher command in its own session; if it does not finish in time, end that session's
    process group (the launcher and the ranks it started - nothing else) and fail."""
    import signal
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env, cwd=ROOT,
                            start_new_session=True)
    try:
        so, se = proc.communicate(timeout=timeout)
    except subprocess.TimeoutExpired:
        os.killpg(proc.pid, signal.SIGKILL)
        so, se = proc.communicate()
        raise AssertionError(f"job did not finish in {timeout} s:\n" + (so + se)[-4000:])
    return subprocess.CompletedProcess(cmd, proc.returncode, so, se)


def run_ranks(case, n=2, cpu=True, env=None, timeout=300):
    port = 29600 + (os.getpid() + hash(case)) % 300
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "ranks", "selftest.py"),
           "--case", case] + (["--cpu"] if cpu else [])
    e = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="2")
    e.update(env or {})
    r = run_job(cmd, e, timeout)
    assert r.returncode == 0 and f"PASS {case}" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
    return r.stdout


def test_ddp_equals_single_process_gloo():
    out = run_ranks("ddp_nccl")
    assert "mode=nccl" in out


def test_rank_exit_is_detected_on_host():
    run_ranks("rank_exit")


def test_fsdp_host_logic_gloo():
    run_ranks("fsdp")


def test_context_parallel_equals_single_process_gloo():
    run_ranks("cp")


def test_neuron_tensor_parallel_equals_single_process_gloo():
    out = run_ranks("tp")
    assert "rope:nccl" in out and "alibi:nccl" in out and "pope:nccl" in out


def test_checkpoint_resume_under_fsdp_and_tp_gloo():
    out = run_ranks("ckpt")
    assert "fsdp tp" in out


@pytest.mark.parametrize("strategy", ["fsdp", "tp"])
def test_cli_train_and_resume_on_two_ranks(tmp_path, strategy):
    """`train` end to end on two gloo ranks under a sharded wrapper: a run, its checkpoint, a resume."""
    cfg = tmp_path / "par.toml"
    cfg.write_text(f"""
[training]
batch_size = 4
block_size = 32
log_frequency = 2

[model]
n_layer = 2
n_embd = 64
n_head = 2
mlp_internal_dim_multiplier = 4
dropout = 0.0

[parallel]
strategy = "{strategy}"
""")
    runs = tmp_path / "runs"
    base = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
            "127.0.0.1"]
    tail = ["-m", "burn_dragon_b200", "train", "-c", str(cfg), "--synthetic", "--device", "cpu", "--runs", str(runs)]
    e = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="2")
    port = 29300 + (os.getpid() + len(strategy)) % 200
    r = run_job(base + ["--master-port", str(port)] + tail + ["--max-iters", "4"], e, 300)
    assert r.returncode == 0 and "[valid       4]" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
    # logged steps of a multi-rank run carry the exposed-communication columns
    import json
    run = (runs / "latest").read_text().strip()
    recs = [json.loads(l) for l in (runs / run / "metrics.jsonl").read_text().splitlines()]
    train = [x for x in recs if x["split"] == "train"]
    assert train and all(x["comm_ms"] > 0 and 0 < x["comm_share"] < 1 for x in train), recs
    r = run_job(base + ["--master-port", str(port + 1)] + tail + ["--resume", "latest", "--max-iters", "6"], e, 300)
    assert r.returncode == 0 and "step 4" in r.stdout and "[valid       6]" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
    # the checkpoint is layout-free: the same run continues as a single process
    r = run_job([sys.executable] + tail + ["--resume", "latest", "--max-iters", "8"], e, 300)
    assert r.returncode == 0 and "step 6" in r.stdout and "[valid       8]" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


@pytest.mark.parametrize("world,ctas", [(2, 4), (4, 3), (8, 2)])
def test_flag_barrier_protocol_simulation(world, ctas):
    """The arithmetic the collectives kernels use for their cross-rank barrier (slot layout, epoch
    values, wrap-safe comparison), run by real threads with randomised interleavings: no stale or
    early reads, no deadlock - also across the sign bit and the wrap of the 32-bit counter."""
    from burn_dragon_b200.utils import hostlib
    assert hostlib.available()
    for first in (0, 2 ** 30 - 3, 2 ** 31 - 3):        # 2*epoch+phase crosses 2^31 and 2^32
        for seed in range(3):
            assert hostlib.simulate_flag_barrier(world, ctas, 40, first, seed) == 0, (first, seed)


def test_restart_from_checkpoint_after_injected_rank_failure(tmp_path):
    """Failure on the host, recovery from the last checkpoint: rank 1 raises before step 4 (once); the
    launcher restarts the group with the same command line; `--resume auto` continues from the
    checkpoint written at step 2 and the run completes."""
    cfg = tmp_path / "par.toml"
    cfg.write_text("""
[training]
batch_size = 4
block_size = 32
log_frequency = 1
checkpoint_every = 2

[model]
n_layer = 2
n_embd = 64
n_head = 2
mlp_internal_dim_multiplier = 4
dropout = 0.0

[parallel]
strategy = "fsdp"
""")
    runs = tmp_path / "runs"
    port = 29500 + os.getpid() % 90
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--max-restarts=2",
           "--master-addr", "127.0.0.1", "--master-port", str(port), "-m", "burn_dragon_b200", "train", "-c", str(cfg),
           "--synthetic", "--device", "cpu", "--runs", str(runs), "--max-iters", "6", "--resume", "auto"]
    e = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="2",
             BDH_INJECT_FAULT=f"rank=1,step=4,once={tmp_path / 'failed_once'}")
    r = run_job(cmd, e, 300)
    out = r.stdout + r.stderr
    assert r.returncode == 0, out[-4000:]
    assert (tmp_path / "failed_once").exists() and "injected host fault on rank 1 before step 4" in out
    assert "resumed" in r.stdout and "step 2" in r.stdout and "[valid       6]" in r.stdout, out[-4000:]
    run_dirs = [p for p in runs.iterdir() if p.is_dir()]
    assert len(run_dirs) == 1                      # the restart continued the same run
    names = sorted(p.name for p in (run_dirs[0] / "checkpoint").glob("model-*.bin"))
    assert names == ["model-1.bin", "model-2.bin", "model-3.bin"], names


def test_infer_cli_context_parallel_equals_single_process(tmp_path):
    """`infer` under the launcher splits a long prompt over the ranks (context-parallel prefill);
    the greedy continuation equals the single-process one. The prompt length is odd on purpose:
    the left-over token runs replicated."""
    cfg = tmp_path / "t.toml"
    cfg.write_text("[training]\nbatch_size = 2\nblock_size = 16\nlog_frequency = 1\n"
                   "[model]\nn_layer = 2\nn_embd = 32\nn_head = 2\ndropout = 0.0\nrotary_embedding = \"rope\"\n")
    runs = tmp_path / "runs"
    e = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="2")
    r = run_job([sys.executable, "-m", "burn_dragon_b200", "train", "-c", str(cfg), "--synthetic", "--device", "cpu",
                 "--max-iters", "2", "--runs", str(runs)], e, 300)
    assert r.returncode == 0, r.stderr[-2000:]
    prompt = tmp_path / "p.txt"
    prompt.write_text("the quick brown fox jumps over the lazy dog " * 3 + "x")     # 133 bytes
    tail = ["-m", "burn_dragon_b200", "infer", "--runs", str(runs), "-c", str(cfg), "--prompt-file", str(prompt),
            "--max-tokens", "12", "--greedy", "--device", "cpu"]
    one = run_job([sys.executable] + tail, e, 300)
    assert one.returncode == 0, one.stderr[-2000:]
    port = 29250 + os.getpid() % 40
    two = run_job([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
                   "127.0.0.1", "--master-port", str(port)] + tail, e, 300)
    assert two.returncode == 0, two.stdout[-1000:] + two.stderr[-3000:]
    text = one.stdout.strip().splitlines()[-1]
    assert len(text) > 133 and text in two.stdout


@pytest.mark.parametrize("case", ["tp", "cp", "fsdp", "ckpt"])
def test_parallel_wrappers_over_the_emulated_kernel_path(case):
    """The same multi-rank cases with the model on the kernel path's orchestration (every launch
    replaced by its fp32 statement, BDH_EMULATE_KERNELS=1): the tensor-parallel reductions between the
    GEMM launches, the context-parallel state exchange and carry-in, sharded checkpoints."""
    run_ranks(case, env={"BDH_EMULATE_KERNELS": "1"})


@pytest.mark.parametrize("emulated", [False, True])
def test_gradient_accumulation_under_the_wrappers(emulated):
    """Two micro-batches of half the rows and one update equal one step on the whole batch, under
    FSDP and under neuron TP (torch path, and the kernel path's orchestration)."""
    run_ranks("accum", env={"BDH_EMULATE_KERNELS": "1"} if emulated else None)


def test_gradient_clipping_under_the_wrappers():
    """Global-norm clipping under FSDP and neuron TP: same norm and same weights as one process."""
    run_ranks("clip")


@pytest.mark.parametrize("n", [2, 4])
def test_context_parallel_training_gradients(n):
    """Sequences split over the ranks: loss and all parameter gradients equal the single-process ones
    (differentiable state hand-off, every positional mode)."""
    run_ranks("cp_train", n=n)


def test_context_parallel_training_on_the_emulated_kernel_path():
    """The same, with every rank's slice on the kernel path's orchestration: the state hand-off and its
    reverse are steps of the layer's own forward / backward pass there (one or two segments per rank)."""
    run_ranks("cp_train_kernels", n=2, env={"BDH_EMULATE_KERNELS": "1"})


def test_training_loop_aborts_on_a_kernel_status():
    """A bounded wait that ran out makes its kernel return early and sets the status word. The trainer
    polls that word once per step (asynchronously), so the loop must stop with `KernelTimeout` no later
    than one step after the word was set. The status source is faked on the host."""
    import torch
    from burn_dragon_b200.engine.trainer import Trainer
    from burn_dragon_b200.models.bdh import BDH, BDHConfig
    from burn_dragon_b200.parallel.watchdog import KernelTimeout, StatusMonitor

    word = {"value": 0}

    class Done:
        def query(self):
            return True

        def synchronize(self):
            pass

    def read_async(dst):
        dst[0] = word["value"]
        return Done()

    torch.manual_seed(0)
    model = BDH(BDHConfig(n_layer=1, n_embd=32, n_head=2, n_latent_per_head=64, vocab_size=256, dropout=0.0))
    trainer = Trainer(model, lr=1e-3)
    trainer.status = StatusMonitor(read_async)
    tok = torch.randint(0, 256, (2, 17))
    for _ in range(3):
        trainer.train_step(tok[:, :-1], tok[:, 1:])
    word["value"] = 5                      # "peer flag wait timed out", set while step 4 runs
    steps_after = 0
    with pytest.raises(KernelTimeout, match="peer flag"):
        for _ in range(3):
            trainer.train_step(tok[:, :-1], tok[:, 1:])
            steps_after += 1
    assert steps_after <= 1
    # `check()` reports a pending copy at once (what the loop calls where it synchronises anyway)
    mon = StatusMonitor(read_async)
    mon.poll()
    with pytest.raises(KernelTimeout):
        mon.check()

"""Host-side logic of the parallel layer on gloo CPU ranks (world size 2)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_ranks(case, n=2, cpu=True, env=None, timeout=300):
    port = 29600 + (os.getpid() + hash(case)) % 300
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), "-m", "burn_dragon_b200.parallel.selftest",
           "--case", case] + (["--cpu"] if cpu else [])
    e = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="2")
    e.update(env or {})
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=e, cwd=ROOT)
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
    r = subprocess.run(base + ["--master-port", str(port)] + tail + ["--max-iters", "4"], capture_output=True,
                       text=True, timeout=300, env=e, cwd=ROOT)
    assert r.returncode == 0 and "[valid       4]" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
    r = subprocess.run(base + ["--master-port", str(port + 1)] + tail + ["--resume", "latest", "--max-iters", "6"],
                       capture_output=True, text=True, timeout=300, env=e, cwd=ROOT)
    assert r.returncode == 0 and "step 4" in r.stdout and "[valid       6]" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
    # the checkpoint is layout-free: the same run continues as a single process
    r = subprocess.run([sys.executable] + tail + ["--resume", "latest", "--max-iters", "8"], capture_output=True,
                       text=True, timeout=300, env=e, cwd=ROOT)
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

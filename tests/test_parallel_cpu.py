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

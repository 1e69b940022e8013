"""Fused NVLink collectives and data-parallel equality on >= 2 GPUs (child processes, one per GPU)."""
import pytest

from test_parallel_cpu import run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


@pytest.mark.parametrize("no_multimem", ["0", "1"])
def test_symmetric_allreduce(no_multimem):
    run_ranks("allreduce", cpu=False, env={"BDH_NO_MULTIMEM": no_multimem})


def test_sharded_adamw_kernel():
    run_ranks("sharded_adamw", cpu=False)


@pytest.mark.parametrize("case", ["ddp", "ddp_nccl"])
def test_ddp_equals_single_gpu(case):
    out = run_ranks(case, cpu=False)
    assert ("mode=epilogue" if case == "ddp" else "mode=nccl") in out


def test_ddp_with_the_single_allreduce_launch_equals_single_gpu():
    out = run_ranks("ddp", cpu=False, env={"BDH_DDP_EPILOGUE": "0"})
    assert "mode=fused" in out


def test_rank_exit_detected_without_gpu_fault():
    run_ranks("rank_exit", cpu=False, env={"NCCL_NVLS_ENABLE": "0", "BDH_NO_MULTIMEM": "1"})


def test_fsdp_sharded_optimizer_equals_single_gpu():
    out = run_ranks("fsdp", cpu=False)
    assert "fused=True" in out


def test_neuron_tensor_parallel_equals_single_gpu():
    out = run_ranks("tp", cpu=False, timeout=600)
    assert "rope:rs" in out and "pope:nccl" in out


def test_gemm_with_reduction_epilogue_every_mode():
    out = run_ranks("tp_reduce", cpu=False)
    assert "rs" in out


def test_all_gather_inside_the_gemm_kernel():
    run_ranks("ag_gemm", cpu=False)


def test_context_parallel_equals_single_gpu():
    run_ranks("cp", cpu=False)


def test_context_parallel_training_on_the_kernels_equals_single_gpu():
    run_ranks("cp_train_kernels", cpu=False)


def test_checkpoint_resume_under_fsdp_and_tp():
    run_ranks("ckpt", cpu=False)


def test_gradient_accumulation_under_fsdp_and_tp():
    run_ranks("accum", cpu=False)


def test_gradient_clipping_under_fsdp_and_tp():
    run_ranks("clip", cpu=False)

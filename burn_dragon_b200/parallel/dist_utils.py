"""Process-group bootstrap helpers: one process per GPU, rendezvous through the environment. The
reference trains on one device only (`LearningStrategy::SingleDevice`, src/bin/train.rs:395)."""
from __future__ import annotations

import datetime
import os
from typing import Optional

import torch
import torch.distributed as dist


def env_rank() -> int:
    return int(os.environ.get("RANK", "0"))


def env_world() -> int:
    return int(os.environ.get("WORLD_SIZE", "1"))


def env_local_rank() -> int:
    return int(os.environ.get("LOCAL_RANK", "0"))


def init_distributed(backend: Optional[str] = None, timeout_s: float = 600.0) -> bool:
    """Initialise torch.distributed from RANK / WORLD_SIZE / MASTER_* if WORLD_SIZE > 1.
    Returns True when a process group exists after the call."""
    if dist.is_initialized():
        return True
    if env_world() <= 1:
        return False
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    use_cuda = torch.cuda.is_available()
    if backend is None:
        backend = "nccl" if use_cuda else "gloo"
    kw = {}
    if use_cuda:
        torch.cuda.set_device(env_local_rank())
        if backend == "nccl":
            kw["device_id"] = torch.device("cuda", env_local_rank())
    timeout = datetime.timedelta(seconds=timeout_s)
    restart = int(os.environ.get("TORCHELASTIC_RESTART_COUNT", "0") or 0)
    if restart > 0:
        # A launcher that restarts a failed group keeps its key-value store: the addresses the previous
        # incarnation's ranks published are still in it under the same keys, and a new rank would try
        # to connect to a process that no longer exists. Give every incarnation its own key space.
        store, rank_, world_ = next(dist.rendezvous("env://", timeout=timeout))
        store.set_timeout(timeout)
        dist.init_process_group(backend=backend, store=dist.PrefixStore(f"restart{restart}", store), rank=rank_,
                                world_size=world_, timeout=timeout, **kw)
    else:
        dist.init_process_group(backend=backend, timeout=timeout, **kw)
    return True


def world_size() -> int:
    return dist.get_world_size() if dist.is_initialized() else 1


def rank() -> int:
    return dist.get_rank() if dist.is_initialized() else 0


def barrier() -> None:
    if dist.is_initialized():
        dist.barrier()


def max_over_ranks(value: float, device=None) -> float:
    """Max of a host scalar over all ranks (used for device-timed step durations)."""
    if not dist.is_initialized():
        return float(value)
    dev = device if device is not None else ("cuda" if dist.get_backend() == "nccl" else "cpu")
    t = torch.tensor([float(value)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def all_agree(ok: bool, group=None, device=None) -> bool:
    """True only when EVERY rank of the group passes True (an all-reduce MIN of a flag). The parallel
    wrappers use it after trying to set up the in-kernel NVLink collectives: a rank on which the
    set-up failed must not fall back to NCCL alone while its peers launch flag-barrier kernels that
    wait for it - either all ranks run the fused collectives or all run the library ones."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return bool(ok)
    dev = device if device is not None else ("cuda" if dist.get_backend(group) == "nccl" else "cpu")
    t = torch.tensor([1 if ok else 0], dtype=torch.int32, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN, group=group)
    return bool(int(t.item()))

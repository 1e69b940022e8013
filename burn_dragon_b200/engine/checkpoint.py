"""Run directories, checkpoints and resume.

Layout matches the reference (src/bin/train.rs:661-718, src/bin/infer.rs:435-629) so its tools and
ours see the same tree:

    runs/latest                       text file holding the name of the newest run
    runs/<name>/config.json           {run_name, block_size, overrides}
    runs/<name>/checkpoint/model-<epoch>.bin    Burn record (BDH models)
    runs/<name>/checkpoint/state-<epoch>.pt     everything needed to resume (an addition: the
                                                reference cannot resume): optimizer moments and step,
                                                LR-schedule position, loader cursor + RNG, torch RNG,
                                                and the full state dict for non-BDH model kinds

Checkpoints always hold the logical (unsharded) tensors, so a run can be resumed with a different
world size or parallel strategy.
"""
from __future__ import annotations

import dataclasses
import json
import random
import re
import time
from pathlib import Path
from typing import Any, Dict, Optional, Tuple

import torch
import torch.distributed as dist

from . import burn_record as BR

_ADJ = ["amber", "brave", "calm", "clever", "eager", "fuzzy", "gentle", "happy", "jolly", "keen", "lively", "merry",
        "nimble", "proud", "quick", "quirky", "rapid", "shy", "silent", "sunny", "swift", "tidy", "vivid", "witty"]
_NOUN = ["badger", "comet", "dragon", "ember", "falcon", "friends", "garden", "harbor", "hatchling", "island",
         "jungle", "kitten", "lantern", "meadow", "nebula", "otter", "pebble", "quokka", "river", "sparrow",
         "thicket", "umbra", "valley", "willow"]


def create_run_dir(run_root) -> Tuple[Path, str]:
    """A fresh `runs/<adjective-noun>` directory name (not yet created on disk)."""
    root = Path(run_root)
    for _ in range(64):
        name = f"{random.choice(_ADJ)}-{random.choice(_NOUN)}"
        if not (root / name).exists():
            return root / name, name
    name = f"run-{int(time.time())}"
    return root / name, name


def write_latest_run(run_root, run_name: str) -> None:
    root = Path(run_root)
    root.mkdir(parents=True, exist_ok=True)
    (root / "latest").write_text(run_name)


def write_run_config(config, run_dir, run_name: str) -> Path:
    run_dir = Path(run_dir)
    run_dir.mkdir(parents=True, exist_ok=True)
    block = max(1, config.model.block_size or config.training.block_size)
    payload = dict(run_name=run_name, block_size=block, overrides=dataclasses.asdict(config.model))
    p = run_dir / "config.json"
    p.write_text(json.dumps(payload, indent=2))
    return p


def find_latest_epoch(ckpt_dir) -> Optional[int]:
    """Largest N over `model-N.bin` / `state-N.pt` (src/bin/infer.rs:491-511)."""
    best = None
    for p in Path(ckpt_dir).glob("*"):
        m = re.fullmatch(r"(?:model|state)-(\d+)\.(?:bin|pt)", p.name)
        if m:
            best = max(best or 0, int(m.group(1)))
    return best


def resolve_run_dir(spec: Optional[str], run_root="runs") -> Path:
    """None -> runs/<contents of runs/latest>; a run name -> runs/<name>; else a path."""
    root = Path(run_root)
    if spec is None:
        latest = root / "latest"
        if not latest.exists():
            raise FileNotFoundError(f"no checkpoint given and {latest} does not exist")
        return root / latest.read_text().strip()
    p = Path(spec)
    if p.exists():
        return p
    if (root / spec).exists():
        return root / spec
    raise FileNotFoundError(f"run or checkpoint `{spec}` not found")


def resolve_checkpoint(spec: Optional[str], epoch: Optional[int] = None, run_root="runs") -> Tuple[Path, Optional[Path], int]:
    """-> (model file, state file or None, epoch). `spec` may be a model file, a checkpoint
    directory, a run directory, a run name, or None for the latest run (src/bin/infer.rs:435-479)."""
    p = resolve_run_dir(spec, run_root)
    if p.is_file():
        m = re.search(r"-(\d+)(?:-f16)?\.(?:bin|pt)$", p.name)
        return p, None, int(m.group(1)) if m else 0
    ckpt = p / "checkpoint" if (p / "checkpoint").is_dir() else p
    ep = epoch if epoch is not None else find_latest_epoch(ckpt)
    if ep is None and (ckpt / "model.bin").exists():
        # the layout of an exported model (model.bin + vocab.json + config.json side by side), as the
        # reference ships for its web page (www/assets/model/<name>/)
        return ckpt / "model.bin", None, 0
    if ep is None:
        raise FileNotFoundError(f"no checkpoints in {ckpt}")
    model = ckpt / f"model-{ep}.bin"
    state = ckpt / f"state-{ep}.pt"
    if not model.exists() and not state.exists():
        raise FileNotFoundError(f"no checkpoint for epoch {ep} in {ckpt}")
    return model, (state if state.exists() else None), ep


def gather_for_checkpoint(trainer, wrapper=None):
    """The collective half of a checkpoint under a sharded wrapper: EVERY rank calls this, then rank 0
    alone passes the two results to `save_checkpoint`. Returns (weights, optimizer state) in the
    unsharded layout, or (None, None) without a wrapper."""
    if wrapper is None:
        return None, None
    weights = wrapper.gather_state_dict()
    opt = getattr(trainer, "opt", None)
    opt_state = opt.logical_state_dict() if opt is not None and hasattr(opt, "logical_state_dict") else None
    return weights, opt_state


def require_burn_record(model_path, what: str) -> Path:
    """`what` (serve / eval / export) works from a Burn record, i.e. a BDH run; the other model
    families keep their weights in the state file only."""
    p = Path(model_path)
    if not p.exists():
        raise SystemExit(f"{what}: {p} does not exist - this command needs a BDH checkpoint (Burn record); "
                         "Mamba and sparse-graph runs store their weights in state-N.pt and are used through "
                         "`infer`")
    return p


def run_dir_of(model_path) -> Path:
    """The run directory a model file belongs to: the parent of its `checkpoint/` directory, or - for
    an exported model directory - the directory itself. `vocab.json` and `config.json` live there."""
    d = Path(model_path).parent
    return d.parent if d.name == "checkpoint" else d


def save_checkpoint(run_dir, epoch: int, model, trainer=None, loader=None, extra: Optional[Dict[str, Any]] = None,
                    logical_state: Optional[Dict[str, torch.Tensor]] = None,
                    optimizer_state: Optional[Dict[str, Any]] = None) -> Path:
    """Write model-<epoch>.bin (BDH) and state-<epoch>.pt. Under a sharded wrapper `logical_state` and
    `optimizer_state` come from `gather_for_checkpoint` (nothing in here talks to other ranks, so
    calling it on rank 0 alone is safe)."""
    ckpt = Path(run_dir) / "checkpoint"
    ckpt.mkdir(parents=True, exist_ok=True)
    sd = logical_state if logical_state is not None else {k: v.detach().cpu() for k, v in model.state_dict().items()}
    is_bdh = all(k in sd for k in BR.PARAM_ORDER) and len(sd) == len(BR.PARAM_ORDER)
    if is_bdh:
        holder = model
        if logical_state is not None:
            from ..models.bdh import BDH
            holder = BDH(model.config)
            holder.load_state_dict(sd)
        BR.save(BR.from_model(holder), ckpt / f"model-{epoch}.bin")
    state: Dict[str, Any] = dict(epoch=epoch, torch_rng=torch.get_rng_state(), extra=extra or {})
    if not is_bdh:
        state["model"] = sd
    if trainer is not None:
        state["step_index"] = trainer.step_index
        opt = getattr(trainer, "opt", None)
        if optimizer_state is not None:
            state["optimizer"] = optimizer_state
        elif opt is not None and hasattr(opt, "logical_state_dict"):
            if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
                raise RuntimeError("sharded optimizer state must be gathered on every rank first "
                                   "(gather_for_checkpoint)")
            state["optimizer"] = opt.logical_state_dict()
        elif opt is not None:
            f = opt.flat
            state["optimizer"] = dict(step=opt.step_count,
                                      m={n: f.view(opt.m, i).detach().cpu().clone() for i, n in enumerate(f.names)},
                                      v={n: f.view(opt.v, i).detach().cpu().clone() for i, n in enumerate(f.names)})
    if loader is not None:
        state["loader"] = loader.state_dict()
    path = ckpt / f"state-{epoch}.pt"
    torch.save(state, path)
    return path


def load_checkpoint(model, model_path: Path, state_path: Optional[Path], trainer=None, loader=None) -> Dict[str, Any]:
    """Restore weights (+ optimizer / schedule / loader when a state file and the objects are given)."""
    state: Dict[str, Any] = {}
    if state_path is not None and Path(state_path).exists():
        state = torch.load(state_path, map_location="cpu", weights_only=False)
    # a wrapper that keeps no full fp32 parameters (fully sharded data parallelism) takes the weights itself
    take = getattr(getattr(trainer, "wrapper", None), "load_weights", None)
    if "model" in state:
        if not (take and take(state["model"])):
            model.load_state_dict(state["model"])
    elif Path(model_path).exists():
        if not (take and take(BR.to_state_dict(BR.load(model_path)))):
            BR.load_into(model, model_path)
    else:
        raise FileNotFoundError(model_path)
    if trainer is not None and state:
        trainer.step_index = int(state.get("step_index", 0))
        opt, osd = getattr(trainer, "opt", None), state.get("optimizer")
        if opt is not None and osd is not None:
            if hasattr(opt, "load_logical_state_dict"):
                opt.load_logical_state_dict(osd)
            else:
                f = opt.flat
                for i, n in enumerate(f.names):
                    f.view(opt.m, i).copy_(osd["m"][n])
                    f.view(opt.v, i).copy_(osd["v"][n])
                opt.step_count = int(osd["step"])
                # parameters are views of the flat master buffer, so the weights loaded above are
                # already in it; only the bf16 working copy needs refreshing
                f.refresh_shadow()
    if loader is not None and "loader" in state:
        loader.load_state_dict(state["loader"])
    if "torch_rng" in state:
        torch.set_rng_state(state["torch_rng"])
    return state

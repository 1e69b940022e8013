"""Command line entry points: `python -m burn_dragon_b200 <train|infer|eval|serve|export|bench|quantize|build-vocab|ckpt>`.

The flags mirror the reference's binaries (src/bin/train.rs:52-81, src/bin/infer.rs:631-687,
src/bin/quantize.rs): `-c/--config` is repeatable and every file is merged over `config/base.toml`;
`infer` finds the newest run through `runs/latest` and applies its `config.json` when no `-c` is
given. `bench` is an addition (the reference only has criterion benches).
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path
from typing import List, Optional

import torch

from . import config as C


def _load_config(paths: List[str], base: Optional[str] = None) -> C.TrainingConfig:
    base_path = Path(base) if base else C.preset_path("base")
    return C.load_training_config([base_path] + [Path(p) for p in paths])


def _device(name: Optional[str] = None) -> torch.device:
    if name:
        return torch.device(name)
    if torch.cuda.is_available():
        from .parallel import dist_utils
        return torch.device("cuda", dist_utils.env_local_rank())
    return torch.device("cpu")


# ------------------------------------------------------------------------------------------------
# train
# ------------------------------------------------------------------------------------------------
def resolve_train_schedule(training, steps_per_epoch: int):
    """(steps_per_epoch, total_steps, total_epochs, source): `epochs` wins over `max_iters`
    (src/bin/train.rs:508-542)."""
    spe = max(1, steps_per_epoch)
    if training.epochs is not None:
        ep = max(1, training.epochs)
        return spe, max(1, spe * ep), ep, "epochs"
    total = max(1, training.max_iters)
    return spe, total, max(1, -(-total // spe)), "max_iters"


def cmd_build_vocab(cfg: C.TrainingConfig) -> int:
    """Fit / load the tokenizer of the configured dataset and report it (train.rs:585-594)."""
    from .data import dataset as D
    ds = D.build_dataset(cfg.dataset, cfg.training)
    print(f"tokenizer `{cfg.dataset.tokenizer.type}` with {len(ds.tokenizer)} tokens; corpus {len(ds.tokens)} tokens")
    return 0


def cmd_train(args) -> int:
    from .data import dataset as D
    from .engine import checkpoint as CK
    from .engine.metrics import MetricsLogger, theoretical_profile
    from .engine.optim import LRSchedule
    from .engine.trainer import Trainer
    from .models.factory import build_model
    from .parallel import dist_utils
    from .utils import profiling as prof

    cfg = _load_config(args.config, args.base)
    if args.synthetic:
        cfg.dataset.type = "synthetic"
        cfg.dataset.tokenizer = C.TokenizerConfig(type="byte", add_special_tokens=False)
    if args.max_iters is not None:
        cfg.training.max_iters, cfg.training.epochs = args.max_iters, None
    if args.command == "build-vocab":
        return cmd_build_vocab(cfg)
    dist_utils.init_distributed()
    rank, world = dist_utils.rank(), dist_utils.world_size()
    dev = _device(args.device)
    torch.manual_seed(cfg.training.seed)
    ds = D.build_dataset(cfg.dataset, cfg.training)
    # data-parallel ranks draw different windows; the ranks of a tensor-parallel group work on the same batch
    data_rank = 0 if (world > 1 and cfg.parallel.strategy == "tp") else rank
    ds.rng = __import__("numpy").random.default_rng(cfg.training.seed + data_rank)
    model = build_model(cfg, vocab_size=len(ds.tokenizer)).to(dev)
    model.recompute = cfg.training.recompute
    model.attention_chunk = cfg.training.attention_chunk
    if cfg.precision.compute != "bf16":
        model.use_native = False
    spe, total_steps, total_epochs, source = resolve_train_schedule(cfg.training, ds.steps_per_epoch(D.TRAIN))
    if rank == 0:
        print(f"train schedule: steps_per_epoch={spe}, total_steps={total_steps}, epochs={total_epochs}, "
              f"source={source}", flush=True)
    sched = LRSchedule(cfg.optimizer.lr_schedule, cfg.optimizer.learning_rate, total_steps,
                       getattr(getattr(model, "config", None), "n_embd", 256))
    strategy = cfg.parallel.strategy if world > 1 else "single"
    wrapper = None
    if strategy == "tp" and cfg.parallel.tp not in (1, world):
        raise SystemExit(f"[parallel] tp = {cfg.parallel.tp}, but the job has {world} ranks: a tensor-parallel job "
                         "shards over all of its ranks")
    if strategy in ("fsdp", "tp"):
        from .parallel import build_wrapper
        wrapper = build_wrapper(model, cfg, strategy)
    accum = max(1, cfg.training.grad_accum_steps)
    trainer = Trainer(model, cfg.optimizer.learning_rate, cfg.optimizer.weight_decay, cfg.optimizer.beta1,
                      cfg.optimizer.beta2, cfg.optimizer.eps, sched, strategy, cfg.parallel.fused_collectives,
                      cfg.training.fast_train, cfg.training.grad_clip, wrapper, accum)
    if cfg.dataset.device_resident:
        train_loader = D.ResidentDataLoader(ds, D.TRAIN, dev, spe * accum, total_steps * accum,
                                            seed=cfg.training.seed + data_rank)
    else:
        train_loader = D.RandomDataLoader(ds, D.TRAIN, dev, spe * accum, total_steps * accum,   # batches = micro-batches
                                          stream=(cfg.training.seed, data_rank))
    val_spe = ds.steps_per_epoch(D.VAL)
    valid_steps = max(1, min(max(1, total_steps // max(1, cfg.training.log_frequency)), val_spe))
    valid_loader = D.RandomDataLoader(ds, D.VAL, dev, valid_steps, None, stream=(cfg.training.seed + 0x5EED, data_rank))

    run_root = Path(args.runs)
    start_epoch = 0
    resume = args.resume
    if resume == "auto":
        # continue the newest run if it has a checkpoint, else start a new one (what a launcher that
        # restarts failed groups needs: the same command line works for the first start and every restart)
        try:
            CK.resolve_checkpoint(str(CK.resolve_run_dir(None, run_root)))
            resume = "latest"
        except (FileNotFoundError, ValueError):
            resume = None
    if resume:
        run_dir = CK.resolve_run_dir(None if resume == "latest" else resume, run_root)
        run_name = run_dir.name
        mp, sp, start_epoch = CK.resolve_checkpoint(str(run_dir))
        CK.load_checkpoint(model, mp, sp, trainer, train_loader)
        if wrapper is not None:
            wrapper.sync_from_model()
        if rank == 0:
            print(f"resumed {run_name} at epoch {start_epoch}, step {trainer.step_index}", flush=True)
    else:
        # one run directory for the whole job: rank 0 names it
        box = [CK.create_run_dir(run_root) if rank == 0 else None]
        if world > 1:
            torch.distributed.broadcast_object_list(box, src=0)
        run_dir, run_name = Path(box[0][0]), box[0][1]
    if rank == 0:
        run_dir.mkdir(parents=True, exist_ok=True)
        CK.write_latest_run(run_root, run_name)
        CK.write_run_config(cfg, run_dir, run_name)
        tok = ds.tokenizer
        if hasattr(tok, "save"):
            tok.save(run_dir / "vocab.json")
    log = MetricsLogger(run_dir if rank == 0 else None, cfg.training.log_frequency, rank)

    tokens_per_step = cfg.training.batch_size * cfg.training.block_size * (1 if strategy == "tp" else world) * accum
    epoch = start_epoch
    every = cfg.training.checkpoint_every
    from .parallel.watchdog import Heartbeat, HostFaultInjector
    faults = HostFaultInjector(rank)
    # every rank publishes a heartbeat; a peer that left or went silent is noticed on the host before
    # this rank launches a step whose collectives would wait for it
    hb = None
    if world > 1 and cfg.parallel.heartbeat_timeout_s > 0:
        hb = Heartbeat(rank, world, interval_s=min(1.0, cfg.parallel.heartbeat_timeout_s / 4),
                       timeout_s=cfg.parallel.heartbeat_timeout_s)
        hb.start()

    ckpt_index = start_epoch       # number of the newest checkpoint of this run (model-<n>.bin)

    def checkpoint() -> None:
        nonlocal ckpt_index
        ckpt_index += 1
        logical, opt_state = CK.gather_for_checkpoint(trainer, wrapper)      # collective under FSDP / TP
        if rank == 0:
            CK.save_checkpoint(run_dir, ckpt_index, model, trainer, train_loader, logical_state=logical,
                               optimizer_state=opt_state)
        dist_utils.barrier()

    while trainer.step_index < total_steps:
        epoch += 1
        model.train()
        before = trainer.step_index
        timed = False
        for batch in train_loader:
            faults.before_step(trainer.step_index + 1)
            if hb is not None:
                hb.check()
            if trainer._micro == 0:        # the clock of a step starts at its first micro-batch
                t0 = torch.cuda.Event(enable_timing=True) if dev.type == "cuda" else None
                t1 = torch.cuda.Event(enable_timing=True) if dev.type == "cuda" else None
                wall = time.perf_counter()
                if t0 is not None:
                    t0.record()
            lr = trainer.current_lr()
            # the steps that get logged also measure gradient norm and activation sparsity
            logged = (trainer.step_index + 1) % cfg.training.log_frequency == 0 or trainer.step_index + 1 == total_steps
            probe = getattr(wrapper, "eval_model", None) or model
            trainer.track_grad_norm = probe.measure_sparsity = logged
            prev = trainer.step_index
            # logged steps of a multi-rank job also time their phases, for the exposed-communication column
            if trainer._micro == 0:        # (decided at the first micro-batch of an accumulated step)
                timed = logged and world > 1 and not prof.timers_on()
                if timed:
                    prof.enable(timers=True)
            loss = trainer.train_step(batch.inputs, batch.targets)
            step = trainer.step_index
            if step == prev:
                continue               # a micro-batch of an accumulated step: no update yet
            if logged:
                if t1 is not None:
                    t1.record()
                    torch.cuda.synchronize()
                    trainer.status.check()          # the device is idle here: the status copy has landed
                    ms = dist_utils.max_over_ranks(t0.elapsed_time(t1), dev)
                else:
                    ms = (time.perf_counter() - wall) * 1e3
                extra = {}
                if timed:
                    rep = prof.report()
                    prof.enable(timers=False)
                    comm = dist_utils.max_over_ranks(prof.comm_ms(rep), dev)
                    extra.update(comm_ms=comm, comm_share=comm / max(ms, 1e-9))
                if trainer.last_grad_norm is not None:
                    extra["grad_norm"] = float(trainer.last_grad_norm)
                sp = getattr(probe, "last_sparsity", None)
                if sp:
                    extra.update(x_active=float(sp["x"]), xy_active=float(sp["xy"]))
                log.log("train", step, loss=float(loss), lr=lr, step_ms=ms, tokens_per_s=tokens_per_step / ms * 1e3,
                        **extra)
            if every and step % every == 0 and step < total_steps:
                checkpoint()           # periodic checkpoint inside an epoch (`training.checkpoint_every` steps)
        if trainer.step_index == before:
            break           # the loader's global step cap is exhausted
        vloss = [float(trainer.eval_step(b.inputs, b.targets)) for b in valid_loader]
        log.log("valid", trainer.step_index, loss=sum(vloss) / len(vloss), epoch=epoch)
        checkpoint()
        if trainer.step_index >= total_steps:
            break
    trainer.status.check()
    if hb is not None:
        hb.stop(leave=False)
    if rank == 0:
        print(log.summary())
        mc = getattr(model, "config", None)
        if hasattr(mc, "flops_per_token_forward"):
            prof = theoretical_profile(mc, cfg.training.batch_size, cfg.training.block_size)
            print("theoretical profile: " + json.dumps(prof))
        print(f"run directory: {run_dir}")
    return 0


# ------------------------------------------------------------------------------------------------
# infer
# ------------------------------------------------------------------------------------------------
def apply_run_config(cfg: C.TrainingConfig, run_cfg: dict) -> None:
    """Apply `runs/<name>/config.json` over a config (src/bin/infer.rs:534-605)."""
    ov = run_cfg.get("overrides", {})
    for k, v in ov.items():
        if v is not None and hasattr(cfg.model, k):
            setattr(cfg.model, k, v)
    if run_cfg.get("block_size"):
        cfg.training.block_size = int(run_cfg["block_size"])


def cmd_infer(args) -> int:
    from .data import tokenizer as T
    from .engine import checkpoint as CK
    from .engine import generation as GEN
    from .models.factory import build_model

    cfg = _load_config(args.config, args.base)
    model_path, state_path, epoch = CK.resolve_checkpoint(args.checkpoint, args.epoch, args.runs)
    run_dir = CK.run_dir_of(model_path)
    run_cfg_path = run_dir / "config.json"
    if not args.config and run_cfg_path.exists():
        apply_run_config(cfg, json.loads(run_cfg_path.read_text()))
    # generation overrides (src/bin/infer.rs:408-433)
    g = cfg.generation
    if args.prompt is not None:
        g.prompt = args.prompt
    if args.max_tokens is not None:
        g.max_tokens = args.max_tokens
    if args.temperature is not None:
        g.temperature = args.temperature
    if args.top_k is not None:
        g.top_k = args.top_k
    if args.greedy:
        g.greedy = True
    if args.context_mode:
        g.context_strategy = C.ContextStrategyConfig(args.context_mode, args.context_window)
    # tokenizer: the run's vocab.json, else the dataset cache
    vocab = run_dir / "vocab.json"
    byte_vocab = None
    if not vocab.exists():
        # a run without a vocabulary file was trained on bytes: its embedding has 256 (or 259) rows
        V = None
        if model_path.exists() and model_path.suffix == ".bin":
            from .engine import burn_record as BR
            V = BR.infer_dims(BR.load(model_path))["vocab_size"]
        elif state_path is not None:
            weights = torch.load(state_path, map_location="cpu", weights_only=False).get("model", {})
            V = next((int(t.shape[0]) for k, t in weights.items() if "embed" in k and t.dim() == 2), None)
        byte_vocab = V if V in (256, 259) else None
    if byte_vocab is not None:
        tok = T.ByteTokenizer(byte_vocab == 259)
    elif cfg.dataset.tokenizer.type == "char":
        vp = vocab if vocab.exists() else T.storage_path(cfg.dataset.tokenizer, cfg.dataset.cache_dir)
        tok = T.CharVocab.load(vp)
    else:
        tok = T.ByteTokenizer(cfg.dataset.tokenizer.add_special_tokens)
    from .parallel import dist_utils
    world = dist_utils.env_world()
    if world > 1:
        dist_utils.init_distributed()
        if args.streaming or args.viz:
            raise SystemExit("infer under torch.distributed.run (context-parallel prefill) has no --streaming / --viz")
    dev = _device(args.device)
    model = build_model(cfg, vocab_size=len(tok)).to(dev).eval()
    CK.load_checkpoint(model, model_path, state_path)
    if args.fp32:
        model.use_native = False
    print(f"loaded {model_path} (epoch {epoch}) on {dev}", file=sys.stderr)

    if getattr(args, "prompt_file", None):
        g.prompt = Path(args.prompt_file).read_text()
    strategy = GEN.resolve_context_strategy(g.context_strategy, cfg.training.block_size)
    ids = tok.encode(g.prompt, False, False)
    if strategy.kind == "sliding" and len(ids) > strategy.window:
        ids = ids[-strategy.window:]
    max_new = GEN.normalize_max_tokens(g.max_tokens)
    if max_new is None:
        max_new = 256
    settings = GEN.GenerationSettings(max_new, g.temperature, g.top_k, strategy, g.greedy, g.seed)
    viz = None
    if args.viz:
        from .viz.encoder import VizConfig, VizEncoder
        model.capture_viz = True
        model.use_native = False
        viz = VizEncoder(VizConfig(history=args.viz_history), model.config, dev)
    if args.streaming:
        sys.stdout.write(g.prompt)
        sys.stdout.flush()
        printer = GEN.StreamPrinter(tok)
        state, last = GEN.prefill_state(model, ids, dev)
        gen = torch.Generator(device=dev).manual_seed(g.seed) if g.seed is not None and not g.greedy else None
        for _ in range(max_new):
            nxt, last = GEN.sample_next_token(model, state, last, g.temperature, g.top_k, g.greedy, gen)
            printer.push(int(nxt[0]))
            if viz is not None:
                frame = state.take_viz()
                if frame is not None and viz.should_capture():
                    viz.step(frame)
        sys.stdout.write("\n")
        if viz is not None and args.viz_out:
            viz.save(args.viz_out)
    elif world > 1:
        # context parallel: the ranks split the prompt (one segment each, per-layer state exchange),
        # end up with the same state, and decode in lockstep; rank 0 prints
        from .parallel.cp import ContextParallel
        state, last = ContextParallel(model).prefill_any(torch.tensor([ids], dtype=torch.int64, device=dev))
        gen = torch.Generator(device=dev).manual_seed(g.seed if g.seed is not None else 0)
        new = []
        for _ in range(max_new):
            nxt, last = GEN.sample_next_token(model, state, last, g.temperature, g.top_k, g.greedy, gen)
            new.append(int(nxt[0]))
        if dist_utils.rank() == 0:
            print(tok.decode(list(ids) + new))
    else:
        toks = GEN.generate_tokens(model, ids, dev, settings)
        print(tok.decode([int(t) for t in toks[0].tolist()]))
    return 0


def cmd_quantize(args) -> int:
    """f32 checkpoint -> f16 checkpoint next to it (src/bin/quantize.rs:36-86)."""
    from .engine import burn_record as BR
    from .engine import checkpoint as CK
    model_path, _, epoch = CK.resolve_checkpoint(args.checkpoint, args.epoch, args.runs)
    out = BR.quantize_file(model_path, args.output)
    print(f"wrote {out} ({out.stat().st_size} bytes, from epoch {epoch})")
    return 0


def cmd_ckpt(args) -> int:
    """Inspect a checkpoint file: metadata, tensor names, shapes."""
    from .engine import burn_record as BR
    rec = BR.load(args.file)
    print("metadata:", rec.metadata)
    for k, p in rec.params.items():
        print(f"  {k:<14} id={p.id} shape={tuple(p.data.shape)} dtype={p.data.dtype}")
    print("dims:", BR.infer_dims(rec))
    return 0


def cmd_eval(args) -> int:
    """Cross-entropy of a checkpoint on text: a file given with --text (encoded with the run's
    tokenizer, read in windows of the run's block size with the recurrent state carried across
    windows, so the whole file is one long context), reported in nats and bits per token. The
    reference only evaluates inside training (src/bin/train.rs:245-247)."""
    import math
    from .engine import session as S
    from .engine import checkpoint as CK
    from .ops import reference as R
    model_path, _, epoch = CK.resolve_checkpoint(args.checkpoint, args.epoch, args.runs)
    CK.require_burn_record(model_path, "eval")
    run_dir = CK.run_dir_of(model_path)
    vocab, run_cfg = run_dir / "vocab.json", run_dir / "config.json"
    sess = S.load_model(model_path.read_bytes(), vocab.read_text() if vocab.exists() else None,
                        run_cfg.read_text() if run_cfg.exists() else None, args.device)
    model, dev = sess.model, sess.device
    ids = torch.as_tensor(sess.tokenizer.encode_array(Path(args.text).read_text()), dtype=torch.int64, device=dev)
    if args.max_tokens:
        ids = ids[:args.max_tokens + 1]
    if ids.numel() < 2:
        raise SystemExit("need at least two tokens of text")
    window = int(args.window or sess.block_size or 512)
    state = model.init_state()
    total, count = 0.0, 0
    with torch.no_grad():
        for lo in range(0, ids.numel() - 1, window):
            x = ids[lo:lo + window].view(1, -1)
            y = ids[lo + 1:lo + 1 + window].view(1, -1)
            x = x[:, :y.shape[1]]
            logits = model.forward_with_state(x, state)
            total += float(R.cross_entropy_mean(logits.float(), y)) * y.shape[1]
            count += y.shape[1]
    nats = total / count
    print(json.dumps(dict(checkpoint=str(model_path), epoch=epoch, tokens=count, window=window, nats_per_token=nats,
                          bits_per_token=nats / math.log(2), perplexity=math.exp(nats))))
    return 0


def cmd_export(args) -> int:
    """Write a run's newest (or chosen) checkpoint as a self-contained model directory - model.bin,
    vocab.json, config.json side by side - the layout the reference's web page fetches
    (www/assets/model/<name>/, www/index.html:212-260) and that `infer` / `serve` accept."""
    import shutil
    from .engine import burn_record as BR
    from .engine import checkpoint as CK
    model_path, _, epoch = CK.resolve_checkpoint(args.checkpoint, args.epoch, args.runs)
    CK.require_burn_record(model_path, "export")
    run_dir = CK.run_dir_of(model_path)
    out = Path(args.output)
    out.mkdir(parents=True, exist_ok=True)
    if args.f16:
        BR.quantize_file(model_path, out / "model.bin")
    else:
        shutil.copyfile(model_path, out / "model.bin")
    for name in ("vocab.json", "config.json"):
        if (run_dir / name).exists():
            shutil.copyfile(run_dir / name, out / name)
    print(f"exported checkpoint {epoch} of {run_dir} to {out} ({'f16' if args.f16 else 'f32'})")
    return 0


def cmd_serve(args) -> int:
    """Serve a trained run over HTTP (engine/server.py)."""
    from .engine import checkpoint as CK
    from .engine import server, session
    model_path, _, epoch = CK.resolve_checkpoint(args.checkpoint, args.epoch, args.runs)
    CK.require_burn_record(model_path, "serve")
    run_dir = CK.run_dir_of(model_path)
    vocab, run_cfg = run_dir / "vocab.json", run_dir / "config.json"
    sess = session.load_model(model_path.read_bytes(), vocab.read_text() if vocab.exists() else None,
                              run_cfg.read_text() if run_cfg.exists() else None, args.device)
    print(f"serving {model_path} (checkpoint {epoch}) on http://{args.host}:{args.port} [{sess.device}]", flush=True)
    pool_settings = None
    if args.pool_slots > 0:
        from .engine import generation as GEN
        pool_settings = GEN.GenerationSettings(None, args.temperature, args.top_k, greedy=args.greedy, seed=0)
    server.serve(sess, args.host, args.port, pool_slots=args.pool_slots, pool_settings=pool_settings)
    return 0


def cmd_bench(args) -> int:
    from .engine import bench as B
    res = B.run(args.what, args.preset, steps=args.steps, warmup=args.warmup, streams=args.streams,
                prompt=args.prompt_len, new_tokens=args.new_tokens)
    from .parallel import dist_utils
    if dist_utils.rank() == 0:
        print(json.dumps(res))
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="burn_dragon_b200")
    sub = ap.add_subparsers(dest="command", required=True)

    def common(p):
        p.add_argument("-c", "--config", action="append", default=[], help="TOML overlay (repeatable)")
        p.add_argument("--base", default=None, help="base TOML (default: config/base.toml)")
        p.add_argument("--device", default=None)
        p.add_argument("--runs", default="runs", help="run root directory")

    for name in ("train", "build-vocab"):
        p = sub.add_parser(name)
        common(p)
        p.add_argument("--synthetic", action="store_true", help="train on uniform random bytes")
        p.add_argument("--max-iters", type=int, default=None)
        p.add_argument("--resume", default=None, help="run name / path, `latest`, or `auto` (latest if it has a checkpoint, else a new run)")
        p.set_defaults(fn=cmd_train)
    p = sub.add_parser("infer")
    common(p)
    p.add_argument("--checkpoint", default=None)
    p.add_argument("--epoch", type=int, default=None)
    p.add_argument("--prompt", default=None)
    p.add_argument("--prompt-file", default=None, help="read the prompt from a file (long contexts)")
    p.add_argument("--max-tokens", type=int, default=None)
    p.add_argument("--temperature", type=float, default=None)
    p.add_argument("--top-k", type=int, default=None)
    p.add_argument("--greedy", action="store_true")
    p.add_argument("--context-mode", choices=["infinite", "sliding"], default=None)
    p.add_argument("--context-window", type=int, default=None)
    p.add_argument("--streaming", action="store_true")
    p.add_argument("--fp32", action="store_true", help="plain torch fp32 path instead of the bf16 kernels")
    p.add_argument("--viz", action="store_true", help="capture activation images (headless)")
    p.add_argument("--viz-history", type=int, default=256)
    p.add_argument("--viz-out", default=None, help="write the captured images to this file (.npz: four arrays; .png: 2x2 panel grid)")
    p.set_defaults(fn=cmd_infer)
    p = sub.add_parser("quantize")
    common(p)
    p.add_argument("--checkpoint", default=None)
    p.add_argument("--epoch", type=int, default=None)
    p.add_argument("--output", default=None)
    p.set_defaults(fn=cmd_quantize)
    p = sub.add_parser("ckpt")
    p.add_argument("file")
    p.set_defaults(fn=cmd_ckpt)
    p = sub.add_parser("eval", help="cross-entropy of a checkpoint on a text file")
    p.add_argument("--checkpoint", default=None)
    p.add_argument("--epoch", type=int, default=None)
    p.add_argument("--runs", default="runs")
    p.add_argument("--device", default=None)
    p.add_argument("--text", required=True)
    p.add_argument("--window", type=int, default=None, help="tokens per forward call (default: the run's block size)")
    p.add_argument("--max-tokens", type=int, default=None)
    p.set_defaults(fn=cmd_eval)

    p = sub.add_parser("export", help="write model.bin + vocab.json + config.json of a run into one directory")
    p.add_argument("--checkpoint", default=None)
    p.add_argument("--epoch", type=int, default=None)
    p.add_argument("--runs", default="runs")
    p.add_argument("--output", required=True)
    p.add_argument("--f16", action="store_true", help="half-precision record (what `quantize` writes)")
    p.set_defaults(fn=cmd_export)

    p = sub.add_parser("serve", help="HTTP front end for streaming generation from a trained run")
    p.add_argument("--checkpoint", default=None)
    p.add_argument("--epoch", type=int, default=None)
    p.add_argument("--runs", default="runs")
    p.add_argument("--device", default=None)
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--port", type=int, default=8080)
    p.add_argument("--pool-slots", type=int, default=0,
                   help="continuous batching: this many streams share one decode step (0 = one request at a time)")
    p.add_argument("--temperature", type=float, default=1.0, help="sampling settings of the pooled decode step")
    p.add_argument("--top-k", type=int, default=None)
    p.add_argument("--greedy", action="store_true")
    p.set_defaults(fn=cmd_serve)

    p = sub.add_parser("bench")
    p.add_argument("what", choices=["train", "decode", "decode-pool", "reference-shapes", "tiny-cpu"])
    p.add_argument("--preset", default="b200_base")
    p.add_argument("--steps", type=int, default=10)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--streams", type=int, default=64)
    p.add_argument("--prompt-len", type=int, default=1024)
    p.add_argument("--new-tokens", type=int, default=2048)
    p.set_defaults(fn=cmd_bench)
    args = ap.parse_args(argv)
    try:
        return args.fn(args)
    except BaseException as e:  # noqa: BLE001
        # A rank that fails inside a multi-rank job must die at once: the normal interpreter exit would
        # first tear the process group down, which waits for peers that are themselves blocked in a
        # collective waiting for this rank - and the launcher would never learn of the failure.
        import torch.distributed as dist
        if isinstance(e, SystemExit) or not (dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1):
            raise
        import os
        import traceback
        traceback.print_exc()
        sys.stderr.flush()
        sys.stdout.flush()
        os._exit(1)


if __name__ == "__main__":
    sys.exit(main())

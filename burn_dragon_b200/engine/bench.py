"""Benchmarks behind `python -m burn_dragon_b200 bench <what>` (device-timed with CUDA events).

    train             one preset's training step (tokens/s), as `bench.py` does for the base config
    decode            cached decode: `streams` concurrent streams, `prompt` prompt tokens, `new_tokens`
                      generated tokens, greedy and temperature-1.0/top-k-40, for BDH and for Mamba-2
    reference-shapes  the workloads of the reference's criterion benches (bench/train.rs:23-44:
                      (B,T) = (4,64) (8,128) (16,256) (8,512) on the default L6 D256 H4 N256 model;
                      bench/inference.rs:22-41: batch 1, prompt 128/512/1024, 8/16/16 new tokens)
"""
from __future__ import annotations

import time
from typing import Dict

import torch

from .. import config as C
from ..models.bdh import BDH, BDHConfig
from ..models.factory import build_model
from ..ops import native
from . import generation as GEN
from .trainer import Trainer


def _timed(fn, steps: int, warmup: int) -> float:
    """Median-free plain average: ms per call over `steps` calls after `warmup` calls."""
    for _ in range(max(warmup, 0)):
        fn()
    if torch.cuda.is_available():
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    return (time.perf_counter() - t0) * 1e3 / steps


def bench_train(preset: str, steps: int, warmup: int) -> Dict:
    cfg = C.load_preset(preset)
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    torch.manual_seed(cfg.training.seed)
    model = build_model(cfg, vocab_size=cfg.model.vocab_size or 256).to(dev)
    model.recompute = cfg.training.recompute
    tr = Trainer(model, cfg.optimizer.learning_rate, cfg.optimizer.weight_decay)
    B, T = cfg.training.batch_size, cfg.training.block_size
    V = model.config.vocab_size
    batches = [torch.randint(0, V, (B, T + 1), device=dev) for _ in range(4)]
    i = [0]

    def step():
        b = batches[i[0] % 4]
        i[0] += 1
        tr.train_step(b[:, :-1], b[:, 1:])

    n0 = native.launch_count()
    ms = _timed(step, steps, max(3, warmup))
    out = dict(bench="train", preset=preset, batch=B, seq_len=T, ms_per_step=ms, tokens_per_s=B * T / ms * 1e3,
               launches_per_step=(native.launch_count() - n0) / (steps + max(3, warmup)),
               kernel_status=native.status_code())
    mc = model.config
    if hasattr(mc, "flops_per_token_forward"):
        fl = 3 * mc.flops_per_token_forward(T) * B * T
        out.update(step_tflop=fl / 1e12, achieved_tflops=fl / ms / 1e9)
    return out


def bench_decode(preset: str, streams: int, prompt: int, new_tokens: int) -> Dict:
    from . import decode_engine as DE
    from ..parallel import dist_utils
    cfg = C.load_preset(preset)
    # under torch.distributed.run every rank serves its own `streams` streams on its own GPU
    # (decode streams are independent, so the ranks never talk during generation)
    world = dist_utils.env_world()
    if world > 1:
        dist_utils.init_distributed()
        torch.cuda.set_device(dist_utils.env_local_rank())
    dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    torch.manual_seed(0)
    model = build_model(cfg, vocab_size=cfg.model.vocab_size or 256).to(dev).eval()
    V = model.config.vocab_size
    toks = torch.randint(0, V, (streams, prompt), device=dev)
    res = dict(bench="decode", preset=preset, kind=cfg.model.kind, streams=streams, prompt=prompt, new_tokens=new_tokens,
               n_gpus=world, total_streams=streams * world)
    if isinstance(model, BDH) and dev.type == "cuda":
        DE.attach(model)
    for name, s in (("greedy", GEN.GenerationSettings(new_tokens, greedy=True)),
                    ("t1_topk40", GEN.GenerationSettings(new_tokens, 1.0, 40, seed=1))):
        # prefill alone (device-timed), then the whole call; decode time is the difference
        def prefill():
            GEN.prefill_state(model, toks, dev)
        dist_utils.barrier()
        ms_prefill = _timed(prefill, 1, 1)
        ms_total = _timed(lambda: GEN.generate_tokens(model, toks, dev, s), 1, 0)
        if world > 1:       # the job is as slow as its slowest rank
            ms_prefill = dist_utils.max_over_ranks(ms_prefill, dev)
            ms_total = dist_utils.max_over_ranks(ms_total, dev)
        ms_decode = max(ms_total - ms_prefill, 1e-6)
        res[name] = dict(prefill_ms=ms_prefill, prefill_tokens_per_s=world * streams * prompt / ms_prefill * 1e3,
                         decode_ms_per_token=ms_decode / new_tokens,
                         decode_tokens_per_s=world * streams * new_tokens / ms_decode * 1e3)
    res["kernel_status"] = native.status_code()
    return res


def bench_decode_pool(preset: str, streams: int, prompt: int, new_tokens: int) -> Dict:
    """Continuous-batching decode: a pool of `streams` slots, every slot seated with its own prompt
    (lengths prompt, prompt + 64, ... so the streams sit at different positions), then `new_tokens`
    pooled steps, device-timed. Compare with `bench decode` (all streams at one position)."""
    from .stream_pool import StreamPool
    cfg = C.load_preset(preset)
    dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    torch.manual_seed(0)
    model = build_model(cfg, vocab_size=cfg.model.vocab_size or 256).to(dev).eval()
    V = model.config.vocab_size
    res = dict(bench="decode-pool", preset=preset, streams=streams, prompt=prompt, new_tokens=new_tokens)
    for name, s in (("greedy", GEN.GenerationSettings(None, greedy=True)),
                    ("t1_topk40", GEN.GenerationSettings(None, 1.0, 40, seed=1))):
        pool = StreamPool(model, streams, s, dev)
        for i in range(streams):
            pool.add(torch.randint(0, V, (1, prompt + 64 * (i % 4)), device=dev))
        ms = _timed(pool.step, new_tokens, 3)
        res[name] = dict(step_ms=ms, decode_tokens_per_s=streams / ms * 1e3, graph=pool.graph is not None)
        del pool
    res["kernel_status"] = native.status_code()
    return res


def bench_reference_shapes(steps: int, warmup: int) -> Dict:
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    out = dict(bench="reference-shapes", train={}, inference={})
    for name, (B, T) in dict(b4_t64=(4, 64), b8_t128=(8, 128), b16_t256=(16, 256), b16_t512=(8, 512)).items():
        torch.manual_seed(0)
        m = BDH(BDHConfig(dropout=0.0)).to(dev)           # reference default: L6 D256 H4 N256 V256 alibi
        tr = Trainer(m, lr=1e-3, weight_decay=0.1)
        b = torch.randint(0, 256, (B, T + 1), device=dev)
        ms = _timed(lambda: tr.train_step(b[:, :-1], b[:, 1:]), steps, max(3, warmup))
        out["train"][name] = dict(ms_per_step=ms, sequences_per_s=B / ms * 1e3, tokens_per_s=B * T / ms * 1e3)
    m = BDH(BDHConfig(dropout=0.0)).to(dev).eval()
    if dev.type == "cuda":
        from . import decode_engine as DE
        DE.attach(m)
    for P, n in ((128, 8), (512, 16), (1024, 16)):
        toks = torch.randint(0, 256, (1, P), device=dev)
        s = GEN.GenerationSettings(n, 1.0, None, seed=0)
        ms = _timed(lambda: GEN.generate_tokens(m, toks, dev, s), max(1, steps // 2), 1)
        out["inference"][f"prompt{P}_new{n}"] = dict(ms=ms, new_tokens_per_s=n / ms * 1e3)
    return out


def bench_tiny_cpu(steps: int = 5, warmup: int = 2) -> Dict:
    """The CPU reference point: the `tiny` preset's model (config/tiny.toml over config/base.toml),
    fp32, one process, B=4 x T=64 uniform bytes (seed 0): one training step (forward, loss, backward,
    AdamW) and 64 tokens of cached greedy generation, wall-clock on the host. This torch path is also
    the numerical oracle of the kernels; the reference's own CPU backend cannot be built here."""
    import time
    dev = torch.device("cpu")
    torch.manual_seed(0)
    cfg = C.load_preset("tiny")
    m = build_model(cfg, vocab_size=256).to(dev)
    tr = Trainer(m, lr=cfg.optimizer.learning_rate, weight_decay=cfg.optimizer.weight_decay)
    g = torch.Generator().manual_seed(0)
    b = torch.randint(0, 256, (4, 65), generator=g)

    def timed(fn, n, w):
        for _ in range(w):
            fn()
        t0 = time.perf_counter()
        for _ in range(n):
            fn()
        return (time.perf_counter() - t0) / n * 1e3

    ms_train = timed(lambda: tr.train_step(b[:, :-1], b[:, 1:]), steps, warmup)
    m.eval()
    s = GEN.GenerationSettings(64, greedy=True)
    ms_gen = timed(lambda: GEN.generate_tokens(m, b[:1, :64], dev, s), max(1, steps // 2), 1)
    mc = m.config
    # the same forward pass through the plain C++ restatement (one thread, double accumulators)
    from ..utils import hostlib
    ms_cpp = None
    if hostlib.available():
        rows = [b[i, :64].tolist() for i in range(4)]
        ms_cpp = timed(lambda: [hostlib.oracle_forward(m, r) for r in rows], max(1, steps // 2), 1)
    return dict(bench="tiny-cpu", dtype="fp32", threads=torch.get_num_threads(), cpp_oracle_forward_ms=ms_cpp,
                model=dict(n_layer=mc.n_layer, n_embd=mc.n_embd, n_head=mc.n_head, n_latent_per_head=mc.latent_per_head,
                           rotary_embedding=mc.rotary_embedding, dropout=mc.dropout),
                train_ms_per_step=ms_train,
                train_tokens_per_s=4 * 64 / ms_train * 1e3, generate_64_ms=ms_gen,
                decode_tokens_per_s=64 / ms_gen * 1e3, final_loss=float(tr.eval_step(b[:, :-1], b[:, 1:])))


def run(what: str, preset: str = "b200_base", steps: int = 10, warmup: int = 3, streams: int = 64, prompt: int = 1024,
        new_tokens: int = 2048) -> Dict:
    if what == "train":
        return bench_train(preset, steps, warmup)
    if what == "decode":
        return bench_decode(preset, streams, prompt, new_tokens)
    if what == "decode-pool":
        return bench_decode_pool(preset, streams, prompt, new_tokens)
    if what == "reference-shapes":
        return bench_reference_shapes(steps, warmup)
    if what == "tiny-cpu":
        return bench_tiny_cpu(steps, warmup)
    raise ValueError(what)

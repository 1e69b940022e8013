#!/usr/bin/env python
"""Headline benchmark: BDH base training throughput (tokens/s) on N B200s.

Config (the named benchmark config): L=6 shared-weight layers, D=256, 4 heads, N=8192 neurons per
head, byte vocab 256, RoPE causal linear attention, T=512, B=32 per GPU, bf16 compute with fp32
master weights, AdamW lr 1e-3, data-parallel over N GPUs (weak scaling). Tokens are synthetic
uniform random bytes from a per-rank seeded generator; weights are random-init.

  python bench.py --gpus 1 --steps 10 --warmup 3
  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
      --master-port P bench.py --gpus N --steps K --warmup W

Rank 0 prints one JSON line. `value` is device-timed (CUDA events around exactly K steps, barrier +
synchronize on both sides, max over ranks). `e2e` repeats the measurement through the public
Trainer API with a pinned-host -> device copy of every step's batch and a device -> host read of
every step's loss inside the timed region (the host reads step i's loss after it has queued step
i + 1, so the device is not drained between steps).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL = dict(n_layer=6, n_embd=256, n_head=4, n_latent_per_head=8192, vocab_size=256, dropout=0.0,
             rotary_embedding="rope")
SEQ_LEN = 512
BATCH_PER_GPU = 32


def reference_arm(args) -> int:
    """The reference is a Rust crate (Burn 0.19); there is no Rust toolchain or vendored crate set
    in this image and `pip install` of the reference tree has nothing to install, so it cannot run."""
    if int(os.environ.get("RANK", "0")) != 0:
        return 0                  # under the launcher every rank runs this file: one line, from rank 0
    print(json.dumps({"impl": "reference", "unavailable":
                      "reference is a Rust/Burn crate: no cargo/rustc in the image, crates not vendored, "
                      "and it has no setup.py/pyproject.toml for pip to install"}))
    return 0


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            parts = [p.strip() for p in r.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        # median SM clock over the samples of the timed region (the sampler runs only while it is timed)
        med = sm[len(sm) // 2] if sm else None
        return {"sm_mhz": med, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


def decode_arm(args) -> int:
    """Cached recurrent decode of the base model: `--streams` independent streams per GPU (data-parallel over the
    GPUs: every rank serves its own streams, the ranks never talk while decoding), prompt of `--prompt` uniform
    random bytes, `--new-tokens` decoded tokens per stream. `value` = decoded tokens/s of the whole job, device-timed
    over the decode phase (prefill excluded, reported beside it); `e2e` times the public `generate_tokens` call from
    pinned host prompts to host tokens, prefill included."""
    import torch
    from burn_dragon_b200.engine import decode_engine as DE
    from burn_dragon_b200.engine import generation as GEN
    from burn_dragon_b200.models.bdh import BDH, BDHConfig
    from burn_dragon_b200.ops import native
    from burn_dragon_b200.parallel import dist_utils

    world = dist_utils.env_world()
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    dist_utils.init_distributed()
    rank, local = dist_utils.rank(), dist_utils.env_local_rank()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    native.load()
    torch.manual_seed(1337)
    model = BDH(BDHConfig(**MODEL)).to(dev).eval()
    eng = DE.attach(model)
    S, P, N = args.streams, args.prompt, args.new_tokens
    gen = torch.Generator().manual_seed(1000 + rank)
    host_prompt = torch.randint(0, 256, (S, P), generator=gen, dtype=torch.int64).pin_memory()
    settings = (GEN.GenerationSettings(N, greedy=True) if args.sampling == "greedy"
                else GEN.GenerationSettings(N, 1.0, 40, seed=1))
    toks = host_prompt.to(dev)

    def timed(fn):
        torch.cuda.synchronize()
        dist_utils.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = fn()
        e1.record()
        torch.cuda.synchronize()
        dist_utils.barrier()
        return dist_utils.max_over_ranks(e0.elapsed_time(e1), dev), out

    # warm-up: prefill + a short decode (captures the decode step's graph)
    warm = GEN.GenerationSettings(8, greedy=settings.greedy, temperature=settings.temperature, top_k=settings.top_k,
                                  seed=settings.seed)
    for _ in range(max(1, args.warmup // 3)):
        GEN.generate_tokens(model, toks, dev, warm)
    ms_prefill, (state, last) = timed(lambda: GEN.prefill_state(model, toks, dev))
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_decode, new = timed(lambda: eng.continue_from(state, last, settings, N))
    clocks = sampler.stop() if rank == 0 else None

    def e2e():
        t = host_prompt.to(dev, non_blocking=True)
        out = GEN.generate_tokens(model, t, dev, settings)
        return out[:, P:].to("cpu", non_blocking=False)
    ms_e2e, out_host = timed(e2e)
    status = native.status_code()
    if rank == 0:
        total = S * N * world
        print(json.dumps({
            "metric": "BDH cached decode tokens/s (device-timed, max over ranks)",
            "value": total / (ms_decode / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": N, "warmup": 8,
            "ms_per_step": ms_decode / N, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16 weights and activations, fp32 recurrent state",
            "data": "synthetic uniform random bytes, random-init weights",
            "config": {"model": "bdh-base L6 D256 H4 N8192 V256 rope", "streams_per_gpu": S, "prompt_len": P,
                       "new_tokens": N, "sampling": args.sampling, "parallelism": f"dp{world} (independent streams)",
                       "l2": "the recurrent state streamed every step (12.9 GB for 64 streams) is far larger than L2",
                       "prefill_ms": ms_prefill, "prefill_tokens_per_s": S * P * world / (ms_prefill / 1e3)},
            "clocks": clocks,
            "e2e": {"value": total / (ms_e2e / 1e3), "unit": "tokens/s (prefill + decode, host prompt to host tokens)",
                    "h2d_bytes_per_step": S * P * 8 / N, "d2h_bytes_per_step": S * 8},
            "gpu_launches": (eng.launches_per_step or 0) * N,
            "kernel_status": status,
        }))
    if dist_utils.world_size() > 1:
        import torch.distributed as dist
        dist.destroy_process_group()
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--nccl-only", action="store_true", help="NCCL all-reduce instead of the fused NVLink path")
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--seq", type=int, default=None)
    ap.add_argument("--preset", default="base", choices=["base", "large", "tp", "decode"],
                    help="base: BDH base, DDP (the headline config); large: L8 D512 H8 N16384 PoPE T2048 B8/GPU, "
                         "fully sharded (FSDP); tp: L12 D1024 H16 N16384 RoPE T4096 B4, neuron-sharded TP; "
                         "decode: BDH base cached decode, 64 streams per GPU, prompt 1024, 2048 new tokens")
    ap.add_argument("--recompute", default=None,
                    help="large / tp presets: layers whose activations are recomputed in the backward pass "
                         "(an integer, or 'auto' = as few as fit; default: the preset's setting)")
    ap.add_argument("--drop-rotated", type=int, default=None,
                    help="PoPE presets: layers that keep x but not the rotated query q and write q again in their "
                         "backward pass (default: chosen together with --recompute auto)")
    ap.add_argument("--attention-chunk", type=int, default=None,
                    help="tokens per attention segment (states handed on between segments); default: automatic "
                         "(the whole sequence below 4096 tokens, else 1024); --seq length = one quadratic form")
    ap.add_argument("--streams", type=int, default=64, help="decode preset: concurrent streams per GPU")
    ap.add_argument("--prompt", type=int, default=1024, help="decode preset: prompt length")
    ap.add_argument("--new-tokens", type=int, default=2048, help="decode preset: tokens decoded per stream")
    ap.add_argument("--sampling", default="greedy", choices=["greedy", "t1_topk40"], help="decode preset")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.preset == "decode":
        return decode_arm(args)

    import torch
    from burn_dragon_b200.engine.trainer import Trainer
    from burn_dragon_b200.models.bdh import BDH, BDHConfig
    from burn_dragon_b200.ops import native
    from burn_dragon_b200.parallel import dist_utils

    world = dist_utils.env_world()
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if args.gpus > 1 and world == 1:
        raise SystemExit("launch multi-GPU runs with torch.distributed.run (one process per GPU)")
    dist_utils.init_distributed()
    rank, local = dist_utils.rank(), dist_utils.env_local_rank()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    native.load()

    W = max(3, args.warmup)
    K = max(1, args.steps)
    presets = {
        "base": (MODEL, BATCH_PER_GPU, SEQ_LEN, "ddp", False, "bdh-base L6 D256 H4 N8192 V256 rope"),
        "large": (dict(n_layer=8, n_embd=512, n_head=8, n_latent_per_head=16384, vocab_size=256, dropout=0.0,
                       rotary_embedding="pope"), 8, 2048, "fsdp", "auto", "bdh-large L8 D512 H8 N16384 V256 pope"),
        "tp": (dict(n_layer=12, n_embd=1024, n_head=16, n_latent_per_head=16384, vocab_size=256, dropout=0.0,
                    rotary_embedding="rope"), 4, 4096, "tp", "auto", "bdh-tp L12 D1024 H16 N16384 V256 rope"),
    }
    mcfg, B0, T0, strategy, recompute, model_name = presets[args.preset]
    if args.recompute is not None:
        recompute = "auto" if args.recompute == "auto" else int(args.recompute)
    B, T = args.batch or B0, args.seq or T0
    torch.manual_seed(1337)
    model = BDH(BDHConfig(**mcfg)).to(dev)
    model.recompute = recompute
    model.attention_chunk = args.attention_chunk
    model.drop_rotated = args.drop_rotated
    wrapper = None
    if world > 1 and strategy == "fsdp":
        from burn_dragon_b200.parallel.fsdp import FSDP
        wrapper = FSDP(model, lr=1e-3, weight_decay=0.1, fused=not args.nccl_only)
    elif world > 1 and strategy == "tp":
        from burn_dragon_b200.parallel.tp import NeuronTP
        wrapper = NeuronTP(model, lr=1e-3, weight_decay=0.1, fused=not args.nccl_only)
    trainer = Trainer(model, lr=1e-3, weight_decay=0.1, parallel="ddp" if (world > 1 and strategy == "ddp") else "single",
                      fused_collectives=not args.nccl_only, wrapper=wrapper)
    # tensor parallel ranks work on the same batch; data-parallel ranks on different ones
    data_world = 1 if strategy == "tp" else world
    # the collective path that actually runs (not the one that was asked for)
    if world == 1:
        coll_mode, fallback = "none", None
    elif wrapper is not None:
        comm = getattr(wrapper, "comm", None)
        coll_mode = ("fused-nvlink:" + str(getattr(comm, "mode", "wgrad-epilogue red.add + shard_adamw_ag"))) \
            if wrapper.fused else "nccl"
        fallback = getattr(wrapper, "fallback_reason", None) or getattr(comm, "fallback_reason", None)
    else:
        coll_mode = {"fused": "fused-nvlink:allreduce_scale", "nccl": "nccl",
                     "epilogue": "fused-nvlink:wgrad-epilogue red.add + shard_bcast"}.get(trainer.dp.mode, trainer.dp.mode)
        fallback = trainer.dp.fallback_reason
    if world > 1 and not args.nccl_only and not coll_mode.startswith("fused"):
        raise SystemExit(f"bench: the fused NVLink collectives were requested but this run fell back to {coll_mode} "
                         f"({fallback}); pass --nccl-only to measure the library path on purpose")

    # synthetic uniform bytes, per-rank seed; one pinned host buffer per step so e2e copies real data
    gen = torch.Generator().manual_seed(1000 + (0 if strategy == "tp" else rank))
    n_batches = W + K
    host = [torch.randint(0, 256, (B, T + 1), generator=gen, dtype=torch.int64).pin_memory() for _ in range(n_batches)]
    dev_batches = [h.to(dev) for h in host]

    def device_step(i):
        b = dev_batches[i % n_batches]
        return trainer.train_step(b[:, :-1], b[:, 1:])

    # ---------------- device-timed region ----------------
    for i in range(W):
        device_step(i)
    torch.cuda.synchronize()
    dist_utils.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = native.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(K):
        loss = device_step(W + i)
    e1.record()
    torch.cuda.synchronize()
    dist_utils.barrier()
    torch.cuda.synchronize()
    launches = native.launch_count() - launches0
    ms = dist_utils.max_over_ranks(e0.elapsed_time(e1), dev)
    clocks = sampler.stop() if rank == 0 else None
    final_loss = float(loss.item())

    # ---------------- end-to-end region (pinned H2D of inputs + D2H of loss every step) ----------------
    # Every step copies its own inputs from pinned host memory and its loss back to pinned host memory; the host
    # reads the loss of step i once step i + 1 has been queued (a copy-done event per step), the way a training
    # loop that logs every step without draining the device does. Two staging buffers, because the copy for
    # step i + 1 is queued while step i may still be reading its inputs.
    stages = [torch.empty(B, T + 1, dtype=torch.int64, device=dev) for _ in range(2)]
    loss_host = torch.empty(2, dtype=torch.float32).pin_memory()
    done = [torch.cuda.Event(), torch.cuda.Event()]
    losses_read = []

    def e2e_step(i):
        st = stages[i & 1]
        st.copy_(host[i % n_batches], non_blocking=True)
        l = trainer.train_step(st[:, :-1], st[:, 1:])
        loss_host[i & 1:(i & 1) + 1].copy_(l.detach().reshape(1), non_blocking=True)
        done[i & 1].record()

    def read_loss(i):
        done[i & 1].synchronize()
        losses_read.append(float(loss_host[i & 1]))

    for i in range(2):
        e2e_step(i)
    torch.cuda.synchronize()
    dist_utils.barrier()
    torch.cuda.synchronize()
    e0.record()
    for i in range(K):
        e2e_step(W + i)
        if i > 0:
            read_loss(W + i - 1)
    read_loss(W + K - 1)
    e1.record()
    torch.cuda.synchronize()
    dist_utils.barrier()
    assert len(losses_read) == K, "every timed step's loss was read on the host"
    ms_e2e = dist_utils.max_over_ranks(e0.elapsed_time(e1), dev)

    # ---------------- phase split (after both timed regions; three extra steps with phase timers) ----------------
    # device time per step of the collectives that are launches of their own, and of every other phase, max over
    # ranks: what a GEMM epilogue sends is inside the compute phases by design
    from burn_dragon_b200.utils import profiling as prof
    phases = None
    try:
        prof.enable(timers=True)
        prof.report()
        for i in range(3):
            device_step(W + i)
        rep = prof.report()
        prof.enable(timers=False)
        phases = {"comm_ms": dist_utils.max_over_ranks(prof.comm_ms(rep) / 3, dev),
                  "phase_ms": {k: round(dist_utils.max_over_ranks(v["ms"] / 3, dev), 3) for k, v in sorted(rep.items())}}
    except Exception as exc:  # noqa: BLE001 - the split is extra information, never a reason to lose the line
        prof.enable(timers=False)
        phases = {"error": repr(exc)}

    tokens = B * T * data_world * K
    value = tokens / (ms / 1e3)
    e2e_value = tokens / (ms_e2e / 1e3)
    status = native.status_code()
    if rank == 0:
        out = {
            "metric": "BDH train tokens/s (device-timed, max over ranks)",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong" if strategy == "tp" else "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic uniform random bytes, random-init weights",
            "config": {"model": model_name, "global_batch": B * data_world, "seq_len": T,
                       "parallelism": (f"{'dp' if strategy == 'ddp' else strategy}{world}" if world > 1 else "single"),
                       "attention_chunk": args.attention_chunk,
                       "recompute": recompute, "recomputed_layers": getattr(getattr(wrapper, "shard", model), "_recomputed_layers", None),
                       "dropped_q_layers": getattr(getattr(wrapper, "shard", model), "_dropped_q_layers", None),
                       "optimizer": "AdamW lr 1e-3 wd 0.1 (fp32 master, bf16 compute)",
                       "l2": "per-step working set (activations > 20 GB) is far larger than the 126 MB L2",
                       "collectives": coll_mode, "collectives_fallback": fallback,
                       # fully sharded state: what one rank holds between steps (bytes)
                       "persistent_bytes_per_rank": (wrapper.state.persistent_bytes()
                                                     if getattr(wrapper, "state", None) is not None else None)},
            "clocks": clocks, "phases": phases,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": ms_e2e / K,
                    "loss_read": "every step, one step behind (pinned copy + event)", "h2d_bytes_per_step": B * (T + 1) * 8, "d2h_bytes_per_step": 4},
            "gpu_launches": launches,
            "final_loss": final_loss,
            "kernel_status": status,
            "model_flops_per_step": 3 * model.config.flops_per_token_forward(T) * B * T,
        }
        print(json.dumps(out))
    if dist_utils.world_size() > 1:
        import torch.distributed as dist
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())

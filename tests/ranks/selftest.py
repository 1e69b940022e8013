"""Multi-rank self tests, run as `python -m torch.distributed.run --nproc-per-node N
tests/ranks/selftest.py --case <name>` (one process per GPU, or gloo ranks on CPU with `--cpu`). Each case prints `PASS <case>` on rank 0 or raises. The pytest files start these as
child processes.
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch
import torch.distributed as dist

from burn_dragon_b200.parallel import dist_utils


def _bf16_path(dev) -> bool:
    """True when the model runs the bf16 kernel path (on a GPU, or emulated launch by launch on the
    CPU with BDH_EMULATE_KERNELS=1): comparisons against fp32 runs then need bf16 tolerances."""
    from burn_dragon_b200.ops import emulate
    return dev.type == "cuda" or emulate.active()


def _close(a, b, rtol=1e-5, atol=1e-6, what=""):
    if not torch.allclose(a, b, rtol=rtol, atol=atol):
        raise AssertionError(f"{what}: max abs diff {(a - b).abs().max().item()}")


def case_allreduce(dev):
    from burn_dragon_b200.ops import native
    from burn_dragon_b200.parallel import symm
    rank, world = dist.get_rank(), dist.get_world_size()
    for n in (4096, 1 << 20, (1 << 22) + 64 * world):
        torch.manual_seed(100 + rank)
        local = torch.randn(n, device=dev)
        ar = symm.SymmetricAllReduce(local)
        ar.tensor[:n].copy_(local)
        want = local.clone()
        dist.all_reduce(want)
        want /= world
        native.clear_status()
        ar.all_reduce_(scale=1.0 / world)
        torch.cuda.synchronize()
        assert native.status_code() == 0, "peer flag wait timed out"
        _close(ar.tensor[:n], want, 1e-5, 1e-5, f"allreduce n={n}")
        # second call on the same buffer (epoch advances)
        ar.tensor[:n].copy_(local)
        ar.all_reduce_(scale=1.0 / world)
        torch.cuda.synchronize()
        _close(ar.tensor[:n], want, 1e-5, 1e-5, f"allreduce repeat n={n}")
    return f"multicast={'yes' if ar.buf.multicast_ptr else 'no'}"


def case_sharded_adamw(dev):
    from burn_dragon_b200.ops import native
    from burn_dragon_b200.parallel import symm
    rank, world = dist.get_rank(), dist.get_world_size()
    n = 1 << 18
    torch.manual_seed(7)
    master0 = torch.randn(n, device=dev)
    opt = symm.ShardedAdamW(master0, lr=1e-2, weight_decay=0.1)
    ref_w = master0.clone()
    m = torch.zeros(n, device=dev)
    v = torch.zeros(n, device=dev)
    for step in range(1, 4):
        torch.manual_seed(1000 * step + rank)
        g = torch.randn(n, device=dev)
        opt.grad[:n].copy_(g)
        gsum = g.clone()
        dist.all_reduce(gsum)
        gavg = gsum / world
        m.mul_(0.9).add_(gavg, alpha=0.1)
        v.mul_(0.999).addcmul_(gavg, gavg, value=0.001)
        ref_w.mul_(1 - 1e-2 * 0.1).addcdiv_(m / (1 - 0.9 ** step), (v / (1 - 0.999 ** step)).sqrt() + 1e-5, value=-1e-2)
        opt.step()
        torch.cuda.synchronize()
        assert native.status_code() == 0
        _close(opt.master, ref_w[opt.lo:opt.hi], 1e-4, 1e-5, f"master step {step}")
        _close(opt.shadow[:n].float(), ref_w.to(torch.bfloat16).float(), 1e-2, 1e-2, f"shadow step {step}")
    return ""


def _bdh(dev, rot="rope"):
    from burn_dragon_b200.models.bdh import BDH, BDHConfig
    torch.manual_seed(0)
    return BDH(BDHConfig(n_layer=2, n_embd=64, n_head=2, n_latent_per_head=128, vocab_size=256, dropout=0.0,
                         rotary_embedding=rot)).to(dev)


def case_ddp(dev, fused=True):
    """N-rank data parallel training equals one process training on the concatenated batch."""
    from burn_dragon_b200.engine.trainer import Trainer
    rank, world = dist.get_rank(), dist.get_world_size()
    B, T = 2, 64
    g = torch.Generator().manual_seed(5)
    data = torch.randint(0, 256, (world * B, T + 1), generator=g).to(dev)
    mine = data[rank * B:(rank + 1) * B]
    m_dp = _bdh(dev)
    tr = Trainer(m_dp, lr=1e-2, parallel="ddp", fused_collectives=fused)
    if dev.type == "cuda" and fused:
        # (`epilogue`: the reduce-scatter half runs in the weight-gradient epilogues; BDH_DDP_EPILOGUE=0 keeps
        # the single all-reduce launch)
        assert tr.dp.mode in ("fused", "epilogue"), getattr(tr.dp, "fallback_reason", "")
    m_one = _bdh(dev)
    tr1 = Trainer(m_one, lr=1e-2, parallel="single")
    for _ in range(3):
        l_dp = tr.train_step(mine[:, :-1], mine[:, 1:])
        l_one = tr1.train_step(data[:, :-1], data[:, 1:])
    lsum = l_dp.detach().clone().float()
    dist.all_reduce(lsum)
    tol = 2e-2 if _bf16_path(dev) else 1e-5
    assert abs(lsum.item() / world - l_one.item()) < tol * max(1.0, abs(l_one.item())), (lsum.item() / world, l_one.item())
    for (n, a), (_, b) in zip(m_dp.named_parameters(), m_one.named_parameters()):
        rel = ((a - b).norm() / (b.norm() + 1e-12)).item()
        assert rel < (2e-2 if _bf16_path(dev) else 1e-5), (n, rel)
    # every rank holds the same weights
    for p in m_dp.parameters():
        ref = p.detach().clone()
        dist.broadcast(ref, src=0)
        assert torch.equal(ref, p.detach()), "ranks diverged"
    return f"mode={tr.dp.mode}"


def case_rank_exit(dev):
    """A rank that leaves between steps is noticed on the host by the others (heartbeat store),
    before they launch anything that would wait for it."""
    from burn_dragon_b200.parallel.watchdog import Heartbeat
    rank, world = dist.get_rank(), dist.get_world_size()
    hb = Heartbeat(rank, world, interval_s=0.1, timeout_s=1.0)
    hb.start()
    t = torch.ones(4, device=dev)
    dist.all_reduce(t)
    if dev.type == "cuda":
        torch.cuda.synchronize()
    dist.barrier()
    if rank == world - 1:
        hb.stop(leave=True)          # announces the departure; no kernel or collective in flight
        return "left"
    import time
    deadline = time.time() + 10
    while time.time() < deadline and not hb.dead_ranks():
        time.sleep(0.05)
    assert hb.dead_ranks() == [world - 1], hb.dead_ranks()
    hb.stop()
    return "detected"


def case_allreduce_bw(dev):
    """Device-timed all-reduce of the BDH-base gradient buffer (25.3 M fp32 = 101 MB) and of 1 GiB:
    this library's kernel against NCCL, max over ranks, with the NVLink roofline fraction
    (bytes each GPU must send, 2*(W-1)/W * size, over 770 GB/s per direction)."""
    import json
    from burn_dragon_b200.parallel import symm
    rank, world = dist.get_rank(), dist.get_world_size()
    out = {}
    for name, n in (("bdh_base_grads", 25_297_920), ("1GiB", 1 << 28)):
        n = n + (-n) % (4 * world)
        ar = symm.SymmetricAllReduce(torch.empty(n, device=dev))
        ar.tensor.normal_()
        ref = torch.randn(n, device=dev)

        def timed(fn, iters=10):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return dist_utils.max_over_ranks(e0.elapsed_time(e1) / iters, dev)

        ms_f = timed(lambda: ar.all_reduce_(1.0 / world))
        ms_n = timed(lambda: dist.all_reduce(ref))
        sent = 2.0 * (world - 1) / world * n * 4
        out[name] = dict(bytes=n * 4, fused_ms=ms_f, nccl_ms=ms_n, fused_busbw_gbs=sent / ms_f / 1e6,
                         nccl_busbw_gbs=sent / ms_n / 1e6, fused_frac_of_770=sent / ms_f / 1e6 / 770.0)
        mc = bool(ar.buf.multicast_ptr)
        del ar
    if rank == 0:
        print("ALLREDUCE_BW " + json.dumps(dict(world=world, multicast=mc, results=out)), flush=True)
    return ""


CASES = dict(allreduce=case_allreduce, allreduce_bw=case_allreduce_bw, sharded_adamw=case_sharded_adamw, ddp=case_ddp,
             ddp_nccl=lambda d: case_ddp(d, fused=False), rank_exit=case_rank_exit)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True)
    ap.add_argument("--cpu", action="store_true")
    args = ap.parse_args()
    if args.cpu:
        dist.init_process_group("gloo")
        dev = torch.device("cpu")
    else:
        dist_utils.init_distributed("nccl")
        dev = torch.device("cuda", dist_utils.env_local_rank())
    if args.case in CASES:
        fn = CASES[args.case]
    else:
        import selftest_sharded
        fn = getattr(selftest_sharded, "case_" + args.case)
    note = fn(dev)
    from burn_dragon_b200.parallel import symm
    if symm.GUARD_BYTES and args.case != "rank_exit":
        # checked configuration: once every rank has finished its launches, no collective of this case
        # may have written outside the window it was given
        if dev.type == "cuda":
            torch.cuda.synchronize()
        dist.barrier()
        note = f"{note or ''} guards_ok={symm.check_all_canaries()}"
    if args.case != "rank_exit":
        dist.barrier()
    if dist.get_rank() == 0:
        print(f"PASS {args.case} {note or ''}", flush=True)
    if args.case != "rank_exit":
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())

"""Multi-rank self tests of the sharded wrappers (FSDP, neuron TP); started through
`parallel.selftest --case fsdp|tp`."""
from __future__ import annotations

import torch
import torch.distributed as dist

from selftest import _bf16_path


def _bdh(dev, rot="rope", N=128):
    from burn_dragon_b200.models.bdh import BDH, BDHConfig
    torch.manual_seed(0)
    return BDH(BDHConfig(n_layer=2, n_embd=64, n_head=2, n_latent_per_head=N, vocab_size=256, dropout=0.0,
                         rotary_embedding=rot)).to(dev)


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def _fused_modes(dev):
    """Wrapper modes a device can run: the fused path needs GPUs - or, for the host logic of the fully
    sharded state, CPU ranks on the emulated kernel path."""
    from burn_dragon_b200.ops import emulate
    return (True, False) if (dev.type == "cuda" or emulate.active()) else (False,)


def case_fsdp(dev):
    """Sharded optimizer training equals one process training on the concatenated batch, the
    gathered state dict is identical on all ranks, and optimizer state round-trips logically."""
    from burn_dragon_b200.engine.trainer import Trainer
    from burn_dragon_b200.parallel.fsdp import FSDP
    rank, world = dist.get_rank(), dist.get_world_size()
    B, T = 2, 64
    g = torch.Generator().manual_seed(5)
    data = torch.randint(0, 256, (world * B, T + 1), generator=g).to(dev)
    mine = data[rank * B:(rank + 1) * B]
    notes = []
    for fused in _fused_modes(dev):
        m = _bdh(dev)
        w = FSDP(m, lr=1e-2, fused=fused)
        if fused:
            assert w.fused, getattr(w, "fallback_reason", "")
        tr = Trainer(m, lr=1e-2, wrapper=w)
        one = _bdh(dev)
        tr1 = Trainer(one, lr=1e-2)
        for _ in range(3):
            tr.train_step(mine[:, :-1], mine[:, 1:])
            tr1.train_step(data[:, :-1], data[:, 1:])
        sd = w.gather_state_dict()
        tol = 2e-2 if _bf16_path(dev) else 1e-5
        for k, v in one.state_dict().items():
            assert _rel(sd[k], v.cpu()) < tol, (fused, k, _rel(sd[k], v.cpu()))
        osd = w.optimizer.logical_state_dict()
        # one full-size moment per parameter, equal to the unsharded optimizer's
        assert osd["step"] == 3 and set(osd["m"]) == {n for n, _ in one.named_parameters()}
        f1 = tr1.opt.flat
        for i, n in enumerate(f1.names):
            a, b = osd["m"][n].flatten().float(), f1.view(tr1.opt.m, i).cpu().flatten().float()
            cos = torch.dot(a, b) / (a.norm() * b.norm() + 1e-20)
            assert cos > 0.98, (fused, n, cos.item())
        mom = w.state.m if w.state is not None else w.m
        before = mom.clone()
        w.optimizer.load_logical_state_dict(osd)
        assert torch.equal(before, mom)
        if w.state is not None:
            # fully sharded: no rank holds more than 1/world of the fp32 state of the big weights
            pb = w.state.persistent_bytes()
            fp32 = pb["master_fp32"] + pb["moments_fp32"] + pb["gradient_fp32"]
            assert fp32 < pb["unsharded_fp32_equivalent"] / world * 1.1 + 16 * 4 * w.state.small_n, pb
        notes.append(f"fused={w.fused}")
    return " ".join(notes)


def case_accum(dev):
    """Gradient accumulation under the wrappers: two micro-batches of half the rows, one update, equals
    one step on the whole batch (the loss is a mean over tokens, the halves have equal size)."""
    from burn_dragon_b200.engine.trainer import Trainer
    from burn_dragon_b200.parallel.fsdp import FSDP
    from burn_dragon_b200.parallel.tp import NeuronTP
    rank, world = dist.get_rank(), dist.get_world_size()
    B, T = 4, 64
    g = torch.Generator().manual_seed(9)
    notes = []
    for kind in ("fsdp", "tp"):
        data = torch.randint(0, 256, ((world if kind == "fsdp" else 1) * B, T + 1), generator=g).to(dev)
        mine = data[rank * B:(rank + 1) * B] if kind == "fsdp" else data      # TP ranks share the batch
        for fused in _fused_modes(dev):
            sds = []
            for accum in (2, 1):
                m = _bdh(dev, N=128 * world)
                w = FSDP(m, lr=1e-2, fused=fused) if kind == "fsdp" else NeuronTP(m, lr=1e-2, fused=fused)
                tr = Trainer(m, lr=1e-2, wrapper=w, grad_accum=accum)
                for _ in range(2):
                    for part in mine.chunk(accum, dim=0):
                        tr.train_step(part[:, :-1], part[:, 1:])
                assert tr.step_index == 2
                sds.append(w.gather_state_dict())
            tol = 3e-2 if _bf16_path(dev) else 1e-5
            for k in sds[0]:
                assert _rel(sds[0][k], sds[1][k]) < tol, (kind, fused, k, _rel(sds[0][k], sds[1][k]))
            notes.append(f"{kind}:fused={fused}")
    return " ".join(notes)


def case_clip(dev):
    """Global-norm gradient clipping under the wrappers equals clipping in one process: same norm,
    same weights after two clipped steps."""
    from burn_dragon_b200.engine.trainer import Trainer
    from burn_dragon_b200.parallel.fsdp import FSDP
    from burn_dragon_b200.parallel.tp import NeuronTP
    rank, world = dist.get_rank(), dist.get_world_size()
    B, T, clip = 2, 64, 0.05
    g = torch.Generator().manual_seed(11)
    notes = []
    for kind in ("fsdp", "tp"):
        data = torch.randint(0, 256, ((world if kind == "fsdp" else 1) * B, T + 1), generator=g).to(dev)
        mine = data[rank * B:(rank + 1) * B] if kind == "fsdp" else data
        for fused in _fused_modes(dev):
            m, one = _bdh(dev, N=128 * world), _bdh(dev, N=128 * world)
            w = FSDP(m, lr=1e-2, fused=fused) if kind == "fsdp" else NeuronTP(m, lr=1e-2, fused=fused)
            tr = Trainer(m, lr=1e-2, wrapper=w, grad_clip=clip)
            tr1 = Trainer(one, lr=1e-2, grad_clip=clip)
            for _ in range(2):
                tr.train_step(mine[:, :-1], mine[:, 1:])
                tr1.train_step(data[:, :-1], data[:, 1:])
                a, b = float(tr.last_grad_norm), float(tr1.last_grad_norm)
                assert b > 2 * clip, b                               # the clip is active
                assert abs(a - b) < (5e-2 if _bf16_path(dev) else 1e-4) * b, (kind, fused, a, b)
            sd = w.gather_state_dict()
            # (bf16 kernels: Adam normalises the update, so elements whose tiny gradient changes sign
            # between two summation orders move by 2 lr - of the order of the weights themselves)
            tol = 0.15 if _bf16_path(dev) else 1e-5
            for k, v in one.state_dict().items():
                assert _rel(sd[k], v.cpu()) < tol, (kind, fused, k, _rel(sd[k], v.cpu()))
            notes.append(f"{kind}:fused={fused}")
    return " ".join(notes)


def case_tp(dev):
    """Neuron-sharded tensor parallelism computes the same loss and gradients as one process, and
    training with it follows the same loss curve."""
    from burn_dragon_b200.engine.trainer import Trainer
    from burn_dragon_b200.parallel.tp import NeuronTP, unshard_rows
    rank, world = dist.get_rank(), dist.get_world_size()
    B, T = 2, 64
    g = torch.Generator().manual_seed(7)
    data = torch.randint(0, 256, (B, T + 1), generator=g).to(dev)
    x, y = data[:, :-1], data[:, 1:]
    notes = []
    for rot in ("rope", "alibi", "pope"):
        for fused in ((True, "mc_red", "allreduce", False) if dev.type == "cuda" else (False,)):
            full = _bdh(dev, rot, N=128 * world)
            one = _bdh(dev, rot, N=128 * world)
            with torch.no_grad():
                for m in (full, one):
                    m.encoder.mul_(4.0); m.encoder_v.mul_(4.0); m.decoder.mul_(4.0)
            w = NeuronTP(full, lr=1e-3, fused=fused)
            c = one.config
            # one forward / backward: loss and every gradient
            w.opt.zero_grad()
            l_tp = w.shard(x, y)
            l_tp.backward()
            l_one = one(x, y)
            l_one.backward()
            assert abs(l_tp.item() - l_one.item()) < 2e-2 * max(1.0, abs(l_one.item())), (rot, fused, l_tp.item(), l_one.item())
            for name in ("encoder", "encoder_v", "decoder"):
                local = getattr(w.shard, name).grad.detach().contiguous()
                parts = [torch.empty_like(local) for _ in range(world)]
                dist.all_gather(parts, local)
                got = unshard_rows(parts, c.n_head, c.latent_per_head)
                want = getattr(one, name).grad
                cos = torch.dot(got.flatten(), want.flatten()) / (got.norm() * want.norm() + 1e-20)
                assert cos > 0.99 and _rel(got, want) < 0.12, (rot, fused, name, cos.item(), _rel(got, want))
            for a, b in ((w.shard.embed.weight.grad, one.embed.weight.grad), (w.shard.lm_head.grad, one.lm_head.grad)):
                assert _rel(a, b) < 0.12, (rot, fused, _rel(a, b))
            # a few optimizer steps: same loss curve
            one.zero_grad()
            tr = Trainer(full, lr=1e-3, wrapper=w)
            tr1 = Trainer(one, lr=1e-3)
            for _ in range(3):
                a = tr.train_step(x, y)
                b = tr1.train_step(x, y)
            assert abs(a.item() - b.item()) < 3e-2 * max(1.0, abs(b.item())), (rot, fused, a.item(), b.item())
            sd = w.gather_state_dict()
            assert sd["encoder"].shape == one.encoder.shape
            notes.append(f"{rot}:{w.comm.mode}{'+mc' if w.comm.multicast else ''}")
        # the row-normalised forward (`fast_train`) under the same sharding: the scores are summed over
        # the shards before they are normalised (torch path on every device)
        full = _bdh(dev, rot, N=128 * world)
        one = _bdh(dev, rot, N=128 * world)
        with torch.no_grad():
            for m in (full, one):
                m.encoder.mul_(4.0); m.encoder_v.mul_(4.0); m.decoder.mul_(4.0)
        one.use_native = False
        w = NeuronTP(full, lr=1e-3, fused=False)
        w.opt.zero_grad()
        l_tp = w.shard.forward_fast(x, y)
        l_tp.backward()
        l_one = one.forward_fast(x, y)
        l_one.backward()
        tol = 2e-3 if dev.type == "cpu" else 3e-2        # (other summation orders on a GPU)
        assert abs(l_tp.item() - l_one.item()) < tol * max(1.0, abs(l_one.item())), (rot, "fast", l_tp.item(), l_one.item())
        c = one.config
        for name in ("encoder", "encoder_v", "decoder"):
            local = getattr(w.shard, name).grad.detach().contiguous()
            parts = [torch.empty_like(local) for _ in range(world)]
            dist.all_gather(parts, local)
            got, want = unshard_rows(parts, c.n_head, c.latent_per_head), getattr(one, name).grad
            assert _rel(got, want) < tol, (rot, "fast", name, _rel(got, want))
        for a, b in ((w.shard.embed.weight.grad, one.embed.weight.grad), (w.shard.lm_head.grad, one.lm_head.grad)):
            assert _rel(a, b) < tol, (rot, "fast", _rel(a, b))
        tr = Trainer(full, lr=1e-3, wrapper=w, fast_train=True)
        one.zero_grad()
        tr1 = Trainer(one, lr=1e-3, fast_train=True)
        for _ in range(3):
            a = tr.train_step(x, y)
            b = tr1.train_step(x, y)
        assert abs(a.item() - b.item()) < 3 * tol * max(1.0, abs(b.item())), (rot, "fast", a.item(), b.item())
        notes.append(f"{rot}:fast")
    return " ".join(notes)


def _tp_reduce_once(comm, A, Bm, rows, cols, K, bf16):
    from burn_dragon_b200.ops import gemm as G
    buf = comm.begin("t", rows, cols)
    G.gemm(A, Bm, M=rows, N=cols, K=K, flags=comm.flags, out0=buf.view, **buf.kw)
    return comm.end(buf, bf16=bf16)


def case_tp_reduce(dev):
    """GEMM whose epilogue is the cross-rank reduction, every mode against an fp32 matmul + NCCL sum:
    full tiles, ragged rows and columns, fp32 and bf16 results, repeated on the same buffers."""
    from burn_dragon_b200.ops import native
    from burn_dragon_b200.parallel.tp import TPComm
    rank, world = dist.get_rank(), dist.get_world_size()
    notes = []
    for mode in ("rs", "mc_red", "allreduce", False):
        comm = TPComm(dev, None, mode)
        for rows, cols, K in ((1024, 256, 128), (300, 64, 64), (128 * world + 40, 200, 192)):
            for rep in range(2):
                torch.manual_seed(11 * rank + rep + rows)
                A = (torch.randn(rows, K, device=dev) * 0.5).to(torch.bfloat16)
                Bm = (torch.randn(cols, K, device=dev) * 0.5).to(torch.bfloat16)
                want = A.float() @ Bm.float().t()
                dist.all_reduce(want)
                for bf16 in (False, True):
                    native.clear_status()
                    got = _tp_reduce_once(comm, A, Bm, rows, cols, K, bf16).float()
                    torch.cuda.synchronize()
                    assert native.status_code() == 0, "peer flag wait timed out"
                    tol = 6e-2 if bf16 else 2e-3
                    err = (got - want).abs().max().item()
                    assert err < tol * max(1.0, want.abs().max().item()), (mode, rows, cols, K, bf16, err)
        notes.append(str(comm.mode))
    return " ".join(notes)


def case_tp_reduce_bw(dev):
    """Device-timed GEMM + cross-rank reduction of its [rows, D] fp32 partial sums (bf16 result), the
    shape of one attention-output reduction: every mode, max over ranks, with the GEMM alone for
    reference and the NVLink roofline (bytes a GPU must receive for an fp32 reduce-scatter plus a
    bf16 all-gather, over 770 GB/s)."""
    import json
    from burn_dragon_b200.ops import gemm as G
    from burn_dragon_b200.parallel import dist_utils
    from burn_dragon_b200.parallel.tp import TPComm
    rank, world = dist.get_rank(), dist.get_world_size()
    rows, cols, K = 65536, 1024, 1024
    torch.manual_seed(rank)
    A = (torch.randn(rows, K, device=dev) * 0.1).to(torch.bfloat16)
    Bm = (torch.randn(cols, K, device=dev) * 0.1).to(torch.bfloat16)
    local = torch.zeros(rows, cols, device=dev)

    def timed(fn, iters=8):
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

    out = dict(world=world, rows=rows, cols=cols, K=K,
               gemm_only_ms=timed(lambda: G.gemm(A, Bm, M=rows, N=cols, K=K, flags=G.F_OUT_F32, out0=local)))
    for mode in ("rs", "mc_red", "allreduce", False):
        comm = TPComm(dev, None, mode)
        out[str(comm.mode) + "_ms"] = timed(lambda: _tp_reduce_once(comm, A, Bm, rows, cols, K, True))
        del comm
    nbytes = rows * cols * (4 + 2) * (world - 1) / world
    out["nvlink_roof_ms"] = nbytes / 770e9 * 1e3
    out["gemm_flops"] = 2.0 * rows * cols * K
    if rank == 0:
        print("TP_REDUCE_BW " + json.dumps(out), flush=True)
    return ""


def case_cp(dev):
    """Context parallel forward == single-device forward over the concatenated sequence: logits of
    every segment, the state after the sequence, and a second call that continues from that state."""
    from burn_dragon_b200.parallel.cp import ContextParallel
    rank, world = dist.get_rank(), dist.get_world_size()
    T = 64
    notes = []
    for rot in ("alibi", "rope", "pope"):
        m = _bdh(dev, rot).eval()
        for p in m.parameters():
            dist.broadcast(p.data, src=0)
        g = torch.Generator().manual_seed(3)
        toks = torch.randint(0, 256, (2, 2 * world * T), generator=g).to(dev)
        half = world * T
        with torch.no_grad():
            ref_state = m.init_state()
            ref1 = m.forward_with_state(toks[:, :half], ref_state)
            ref2 = m.forward_with_state(toks[:, half:], ref_state)
            cp = ContextParallel(m)
            st = m.init_state()
            mine1 = cp.forward_with_state(toks[:, rank * T:(rank + 1) * T].contiguous(), st)
            assert st.position == half
            mine2 = cp.forward_with_state(toks[:, half + rank * T:half + (rank + 1) * T].contiguous(), st)
            assert st.position == 2 * half
            st_p, last = cp.prefill(toks[:, :half])
        tol = 5e-2 if _bf16_path(dev) else 1e-4
        assert _rel(mine1, ref1[:, rank * T:(rank + 1) * T]) < tol, (rot, "first", _rel(mine1, ref1[:, rank * T:(rank + 1) * T]))
        assert _rel(mine2, ref2[:, rank * T:(rank + 1) * T]) < tol, (rot, "second", _rel(mine2, ref2[:, rank * T:(rank + 1) * T]))
        for a, b in zip(st.layers, ref_state.layers):
            assert _rel(a.rho, b.rho) < tol, (rot, "state", _rel(a.rho, b.rho))
        assert _rel(last, ref1[:, -1]) < tol and st_p.position == half
        notes.append(rot)
    return " ".join(notes)


def case_ckpt(dev):
    """Checkpoint / resume under the sharded wrappers: two steps, save (weights and optimizer state in
    the unsharded layout, gathered by all ranks, written by rank 0), load into a fresh differently
    initialised model + wrapper, one more step == three uninterrupted steps."""
    import tempfile
    from burn_dragon_b200.engine import checkpoint as CK
    from burn_dragon_b200.engine.trainer import Trainer
    from burn_dragon_b200.parallel.fsdp import FSDP
    from burn_dragon_b200.parallel.tp import NeuronTP
    rank, world = dist.get_rank(), dist.get_world_size()
    g = torch.Generator().manual_seed(11)
    data = torch.randint(0, 256, (2, 65), generator=g).to(dev)
    x, y = data[:, :-1], data[:, 1:]
    notes = []
    for kind in ("fsdp", "tp"):
        def make(seed):
            torch.manual_seed(seed)
            m = _bdh(dev, "rope", N=128 * world)
            if seed:
                with torch.no_grad():
                    for p in m.parameters():
                        p.add_(torch.randn_like(p) * 0.01)
            w = FSDP(m, lr=1e-2) if kind == "fsdp" else NeuronTP(m, lr=1e-2)
            return m, w, Trainer(m, lr=1e-2, wrapper=w)

        m_a, w_a, t_a = make(0)
        for _ in range(3):
            loss_a = t_a.train_step(x, y)
        want = w_a.gather_state_dict()

        m_b, w_b, t_b = make(0)
        for _ in range(2):
            t_b.train_step(x, y)
        weights, opt_state = CK.gather_for_checkpoint(t_b, w_b)
        box = [tempfile.mkdtemp() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        if rank == 0:
            CK.save_checkpoint(box[0], 1, m_b, t_b, None, logical_state=weights, optimizer_state=opt_state)
        dist.barrier()
        m_c, w_c, t_c = make(5)
        mp, sp, ep = CK.resolve_checkpoint(box[0])
        CK.load_checkpoint(m_c, mp, sp, t_c, None)
        w_c.sync_from_model()
        assert t_c.step_index == 2 and ep == 1
        loss_c = t_c.train_step(x, y)
        got = w_c.gather_state_dict()
        tol = 2e-2 if _bf16_path(dev) else 1e-5
        assert abs(loss_a.item() - loss_c.item()) < tol * max(1.0, abs(loss_a.item())), (kind, loss_a.item(), loss_c.item())
        for k in want:
            assert _rel(got[k].float(), want[k].float()) < tol, (kind, k, _rel(got[k].float(), want[k].float()))
        notes.append(kind)
        dist.barrier()
    return " ".join(notes)


def case_cp_train(dev):
    """Context-parallel training: sequences split over the ranks, loss and every parameter gradient equal
    the single-process ones over the whole sequences (the gradients of later segments reach earlier
    ranks through the differentiable state hand-off)."""
    from burn_dragon_b200.parallel.cp import ContextParallel
    rank, world = dist.get_rank(), dist.get_world_size()
    T = 32
    notes = []
    for rot in ("alibi", "rope", "pope"):
        m = _bdh(dev, rot)
        m.use_native = False                    # this is a torch-path feature
        for p in m.parameters():
            dist.broadcast(p.data, src=0)
        g = torch.Generator().manual_seed(9)
        data = torch.randint(0, 256, (2, world * T + 1), generator=g).to(dev)
        x, y = data[:, :-1], data[:, 1:]
        m.zero_grad()
        want = m(x, y, mode="parallel")
        want.backward()
        ref = {n: p.grad.clone() for n, p in m.named_parameters()}
        m.zero_grad()
        cp = ContextParallel(m)
        sl = slice(rank * T, (rank + 1) * T)
        loss = cp.loss(x[:, sl].contiguous(), y[:, sl].contiguous())
        loss.backward()
        cp.reduce_gradients()
        total = loss.detach().clone()
        dist.all_reduce(total)
        assert abs(total.item() / world - want.item()) < 1e-5, (rot, total.item() / world, want.item())
        for n, p in m.named_parameters():
            assert _rel(p.grad, ref[n]) < 1e-4, (rot, n, _rel(p.grad, ref[n]))
        notes.append(rot)
    return " ".join(notes)


def case_cp_train_kernels(dev):
    """Context-parallel training on the kernel path: every rank trains its slice of the sequences on the
    kernels (or their emulation), the layer's own forward / backward pass hands the states on and their
    gradients back, once with one segment per rank and once with the rank's slice cut into two segments.
    Loss and gradients against the single-process torch definition over the whole sequences, at the
    tolerance of bf16 activations."""
    from burn_dragon_b200.ops import fused_bdh
    from burn_dragon_b200.parallel.cp import ContextParallel
    rank, world = dist.get_rank(), dist.get_world_size()
    T = 128
    notes = []
    for rot in ("alibi", "rope", "pope"):
        for chunk in (None, 64):
            m = _bdh(dev, rot)
            with torch.no_grad():
                m.encoder.mul_(4.0); m.encoder_v.mul_(4.0); m.decoder.mul_(4.0)
            for p in m.parameters():
                dist.broadcast(p.data, src=0)
            g = torch.Generator().manual_seed(9)
            data = torch.randint(0, 256, (2, world * T + 1), generator=g).to(dev)
            x, y = data[:, :-1], data[:, 1:]
            m.zero_grad()
            m.use_native = False
            want = m(x, y, mode="parallel")
            want.backward()
            ref = {n: p.grad.clone() for n, p in m.named_parameters()}
            m.zero_grad()
            m.use_native = True
            m.attention_chunk = chunk
            cp = ContextParallel(m)
            sl = slice(rank * T, (rank + 1) * T)
            xs, ys = x[:, sl].contiguous(), y[:, sl].contiguous()
            assert fused_bdh.can_run(m, xs, None), "the kernel path must take this case"
            loss = cp.loss(xs, ys)
            loss.backward()
            cp.reduce_gradients()
            total = loss.detach().clone()
            dist.all_reduce(total)
            assert abs(total.item() / world - want.item()) < 2e-2, (rot, chunk, total.item() / world, want.item())
            for n, p in m.named_parameters():
                cos = torch.nn.functional.cosine_similarity(p.grad.flatten(), ref[n].flatten(), dim=0).item()
                assert cos > 0.99 and _rel(p.grad, ref[n]) < 0.12, (rot, chunk, n, cos, _rel(p.grad, ref[n]))
            notes.append(f"{rot}/{chunk}")
    return " ".join(notes)


def _ag_fill(op, seed):
    """Every rank writes its own rows of the gathered operand; returns the whole matrix (the same on every
    rank, from the seeds) for the oracle."""
    parts = []
    for r in range(op.world):
        g = torch.Generator().manual_seed(seed * 100 + r)
        parts.append((torch.randn(op.rows, op.K, generator=g) * 0.5).to(torch.bfloat16))
    op.shard.copy_(parts[op.rank].to(op.full.device))
    return torch.cat(parts, 0).to(op.full.device)


def case_ag_gemm(dev):
    """All-gather -> GEMM as one kernel (`parallel/seqpar.py`): token shards written by every rank, gathered by
    the GEMM's own warps over peer loads, against an fp32 matmul over the whole matrix; plain and ReLU
    epilogues, three rounds with fresh data (the counters, barriers and buffers are reused), and the NCCL
    baseline of the same product."""
    from burn_dragon_b200.ops import gemm as G
    from burn_dragon_b200.ops import native
    from burn_dragon_b200.parallel.seqpar import GatheredOperand
    world = dist.get_world_size()
    M, K, N = 256 * world, 256, 512
    op = GatheredOperand(M, K, dev)
    g = torch.Generator().manual_seed(5)
    w = (torch.randn(N, K, generator=g) * 0.2).to(torch.bfloat16).to(dev)
    notes = []
    for rnd in range(3):
        A = _ag_fill(op, rnd)
        want = A.float() @ w.float().t()
        out = torch.zeros(M, N, device=dev, dtype=torch.bfloat16)
        native.clear_status()
        if rnd == 1:
            op.gemm(w, N=N, epi=G.EPI_RELU, out0=out, theta=0.1)
            want = torch.relu(want - 0.1)
        else:
            op.gemm(w, N=N, out0=out)
        op.release()
        torch.cuda.synchronize()
        assert native.status_code() == 0, "a bounded wait ran out"
        assert torch.equal(op.full, A), "the local copy holds every rank's rows after the launch"
        assert _rel(out, want) < 1e-2, (rnd, _rel(out, want))
        out2 = torch.zeros_like(out)
        op.shard.copy_(A[op.rank * op.rows:(op.rank + 1) * op.rows])
        if rnd == 1:
            op.gemm_nccl(w, N=N, epi=G.EPI_RELU, out0=out2, theta=0.1)
        else:
            op.gemm_nccl(w, N=N, out0=out2)
        op.release()
        assert _rel(out2, want) < 1e-2
        notes.append(f"{_rel(out, want):.1e}")
    return " ".join(notes)


def case_ag_gemm_bw(dev):
    """The encoder product of the tensor-parallel configuration with its token rows sharded: [16384, 1024] bf16
    activations (1/world of the rows per rank) times this rank's [32768, 1024] slice of the neurons, ReLU
    epilogue. Fused (gather inside the GEMM) against NCCL all-gather + GEMM, device-timed, max over ranks."""
    import json
    from burn_dragon_b200.ops import gemm as G
    from burn_dragon_b200.ops import native
    from burn_dragon_b200.parallel.seqpar import GatheredOperand
    rank, world = dist.get_rank(), dist.get_world_size()
    M, K, N = 16384, 1024, 32768
    op = GatheredOperand(M, K, dev)
    w = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)
    out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    A = _ag_fill(op, 1)

    def timed(fn, n=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / n], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    def fused():
        op.gemm(w, N=N, epi=G.EPI_RELU, out0=out, theta=0.0)
        op.release()

    def nccl():
        op.gemm_nccl(w, N=N, epi=G.EPI_RELU, out0=out, theta=0.0)
        op.release()

    def alone():
        G.gemm(op.full, w, M=M, N=N, K=K, epi=G.EPI_RELU, out0=out, theta=0.0)

    native.clear_status()
    res = dict(world=world, fused_ms=timed(fused), nccl_ms=timed(nccl), gemm_alone_ms=timed(alone),
               gathered_mb=(world - 1) / world * M * K * 2 / 1e6)
    assert native.status_code() == 0
    want = torch.relu(A.float()[:512] @ w.float()[:512].t())
    fused()
    torch.cuda.synchronize()
    assert _rel(out[:512, :512], want) < 1e-2
    if rank == 0:
        print("AG_GEMM_BW " + json.dumps(res), flush=True)
    return ""

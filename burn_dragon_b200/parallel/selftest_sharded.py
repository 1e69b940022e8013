"""Multi-rank self tests of the sharded wrappers (FSDP, neuron TP); started through
`parallel.selftest --case fsdp|tp`."""
from __future__ import annotations

import torch
import torch.distributed as dist


def _bdh(dev, rot="rope", N=128):
    from ..models.bdh import BDH, BDHConfig
    torch.manual_seed(0)
    return BDH(BDHConfig(n_layer=2, n_embd=64, n_head=2, n_latent_per_head=N, vocab_size=256, dropout=0.0,
                         rotary_embedding=rot)).to(dev)


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def case_fsdp(dev):
    """Sharded optimizer training equals one process training on the concatenated batch, the
    gathered state dict is identical on all ranks, and optimizer state round-trips logically."""
    from ..engine.trainer import Trainer
    from .fsdp import FSDP
    rank, world = dist.get_rank(), dist.get_world_size()
    B, T = 2, 64
    g = torch.Generator().manual_seed(5)
    data = torch.randint(0, 256, (world * B, T + 1), generator=g).to(dev)
    mine = data[rank * B:(rank + 1) * B]
    notes = []
    for fused in ((True, False) if dev.type == "cuda" else (False,)):
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
        tol = 2e-2 if dev.type == "cuda" else 1e-5
        for k, v in one.state_dict().items():
            assert _rel(sd[k], v.cpu()) < tol, (fused, k, _rel(sd[k], v.cpu()))
        osd = w.optimizer.logical_state_dict()
        assert osd["m"].numel() == w.numel and osd["step"] == 3
        w.optimizer.load_logical_state_dict(osd)
        notes.append(f"fused={w.fused}")
    return " ".join(notes)


def case_tp(dev):
    """Neuron-sharded tensor parallel training equals single-process training on the same batch."""
    from ..engine.trainer import Trainer
    from .tp import NeuronTP
    rank, world = dist.get_rank(), dist.get_world_size()
    B, T = 2, 64
    g = torch.Generator().manual_seed(7)
    data = torch.randint(0, 256, (B, T + 1), generator=g).to(dev)
    notes = []
    for rot in ("rope", "alibi", "pope"):
        for fused in ((True, False) if dev.type == "cuda" else (False,)):
            full = _bdh(dev, rot, N=128 * world)
            one = _bdh(dev, rot, N=128 * world)
            w = NeuronTP(full, lr=1e-2, fused=fused)
            tr = Trainer(full, lr=1e-2, wrapper=w)
            tr1 = Trainer(one, lr=1e-2)
            for _ in range(3):
                l_tp = tr.train_step(data[:, :-1], data[:, 1:])
                l_one = tr1.train_step(data[:, :-1], data[:, 1:])
            tol = 3e-2 if dev.type == "cuda" else 1e-5
            assert abs(l_tp.item() - l_one.item()) < tol * max(1.0, abs(l_one.item())), (rot, fused, l_tp.item(), l_one.item())
            sd = w.gather_state_dict()
            for k, v in one.state_dict().items():
                assert _rel(sd[k], v.cpu()) < tol, (rot, fused, k, _rel(sd[k], v.cpu()))
            notes.append(f"{rot}:{'fused' if w.fused else 'nccl'}")
    return " ".join(notes)

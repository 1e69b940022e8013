import pytest
import torch

from burn_dragon_b200.models.bdh_graph import BDHGraph, BDHGraphConfig
from burn_dragon_b200.ops import native

pytestmark = pytest.mark.gpu


def test_block_ell_encoder_matches_masked_dense():
    torch.manual_seed(0)
    g = BDHGraph(BDHGraphConfig(n_layer=1, n_embd=256, n_head=2, n_latent_per_head=512, vocab_size=64, dropout=0.0,
                                graph_block=64, graph_density=0.5)).cuda()
    cur = torch.randn(200, 256, device="cuda")
    n0 = native.launch_count()
    got = g.encode_sparse(cur)
    assert native.launch_count() == n0 + 1
    want = torch.relu(cur.to(torch.bfloat16).float() @ g.encoder.to(torch.bfloat16).float().t())
    assert torch.allclose(got.float(), want, atol=3e-2, rtol=2e-2)


def test_graph_model_trains_on_kernel_path_with_masks_intact():
    torch.manual_seed(0)
    g = BDHGraph(BDHGraphConfig(n_layer=2, n_embd=64, n_head=2, n_latent_per_head=128, vocab_size=256, dropout=0.0,
                                rotary_embedding="rope", graph_block=64, graph_density=0.5)).cuda()
    from burn_dragon_b200.engine.trainer import Trainer
    tr = Trainer(g, lr=1e-2)
    tok = torch.randint(0, 256, (2, 65), device="cuda")
    l0 = float(tr.train_step(tok[:, :-1], tok[:, 1:]))
    for _ in range(4):
        l1 = float(tr.train_step(tok[:, :-1], tok[:, 1:]))
    assert l1 < l0
    dead = ~g._expand(g.encoder_blocks)
    assert (g.encoder[dead] == 0).all()

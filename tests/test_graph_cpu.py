import torch

from burn_dragon_b200.models.bdh import BDH, BDHConfig
from burn_dragon_b200.models.bdh_graph import BDHGraph, BDHGraphConfig, block_mask_to_ell, random_block_mask
from burn_dragon_b200.ops.block_sparse import BlockPattern1d, BlockPattern2d


def _cfg(**kw):
    base = dict(n_layer=2, n_embd=16, n_head=2, n_latent_per_head=16, vocab_size=32, dropout=0.0,
                rotary_embedding="rope", graph_block=8, graph_density=0.5)
    base.update(kw)
    return BDHGraphConfig(**base)


def test_dense_limit_equals_bdh():
    torch.manual_seed(0)
    g = BDHGraph(_cfg(graph_density=1.0))
    torch.manual_seed(0)
    d = BDH(BDHConfig(**{k: v for k, v in _cfg().__dict__.items() if not k.startswith("graph_")}))
    d.load_state_dict(g.state_dict(), strict=False)
    tok = torch.randint(0, 32, (2, 9))
    assert g.graph_density() == 1.0
    assert torch.allclose(g(tok), d(tok), atol=1e-6)


def test_masked_weights_stay_zero_through_training():
    torch.manual_seed(0)
    g = BDHGraph(_cfg())
    dead = ~g._expand(g.encoder_blocks)
    assert dead.any() and (g.encoder[dead] == 0).all()
    opt = torch.optim.AdamW(g.parameters(), lr=1e-2, weight_decay=0.1)
    tok = torch.randint(0, 32, (2, 9))
    for _ in range(3):
        loss = g(tok[:, :-1], tok[:, 1:])
        opt.zero_grad(); loss.backward(); opt.step()
    assert (g.encoder[dead] == 0).all() and (g.decoder[~g._expand(g.decoder_blocks)] == 0).all()
    assert g.edge_count() == int((g.encoder_blocks.sum() + g.encoder_v_blocks.sum() + g.decoder_blocks.sum())) * 64


def test_ell_layout_and_sparse_encoder_matches_dense():
    m = random_block_mask(4, 6, 0.5, 1)
    assert (m.sum(1) == 3).all()
    ell = block_mask_to_ell(m)
    assert ell.shape == (4, 3) and all(m[r, c] for r in range(4) for c in ell[r].tolist())
    g = BDHGraph(_cfg())
    cur = torch.randn(5, 16)
    want = torch.relu(cur.to(torch.bfloat16).float() @ g.encoder.to(torch.bfloat16).float().t())
    assert torch.allclose(g.encode_sparse(cur).float(), want, atol=2e-2)


def test_block_patterns_behaviour():
    p = BlockPattern1d.from_blocks(3, [0, 2])
    assert p.mask(8).flatten().tolist() == [1, 1, 1, 0, 0, 0, 1, 1]
    assert BlockPattern1d.dense(0).block_size == 1 and not BlockPattern1d.dense(4).is_sparse()
    d2 = BlockPattern2d.dense(4)
    assert d2.is_active(2, 1) and not d2.is_active(1, 2) and list(d2.iter_cols(2, 5)) == [0, 1, 2]
    s2 = BlockPattern2d.from_pairs(4, [(0, 0), (2, 0), (2, 2), (1, 3)])
    assert list(s2.iter_cols(2, 5)) == [0, 2] and list(s2.iter_cols(1, 5)) == []     # never beyond the diagonal


def test_latent_block_mask_and_time_pairs_in_model():
    from burn_dragon_b200.ops.block_sparse import BlockSparseConfig
    torch.manual_seed(0)
    cfg = BDHConfig(n_layer=1, n_embd=16, n_head=2, n_latent_per_head=8, vocab_size=32, dropout=0.0)
    cfg.block_sparse = BlockSparseConfig(BlockPattern1d.from_blocks(4, [0]), BlockPattern2d.from_pairs(2, [(0, 0), (1, 1), (2, 2)]))
    m = BDH(cfg).eval()
    tok = torch.randint(0, 32, (1, 6))
    out, _, (x, y, xy) = m._layer_torch(torch.randn(1, 1, 6, 16), 0, None, "parallel")
    assert (x[..., 4:] == 0).all() and (y[..., 4:] == 0).all()
    assert m.forward_fast(tok).shape == (1, 6, 32)

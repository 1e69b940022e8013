"""Op-level equivalences the reference asserts in tests/fused_kernel_tests.rs, restated on this
framework's definitions: the ReLU low-rank op against its hand composition, and blocked attention
(row-normalised mode, block pairs) against the dense quadratic form for RoPE and PoPE."""
import pytest
import torch

from burn_dragon_b200.ops import reference as R
from burn_dragon_b200.ops.block_sparse import BlockPattern1d, BlockPattern2d


def test_relu_lowrank_with_bias_threshold_and_block_mask():
    torch.manual_seed(0)
    B, T, D, H, N = 2, 5, 4, 2, 9
    x = torch.randn(B, 1, T, D)
    w = torch.randn(H, D, N)
    bias = torch.randn(1, H, 1, N)
    pat = BlockPattern1d.from_blocks(3, [0, 2])
    got = R.relu_lowrank(x, w, bias, 0.25, pat.mask(N))
    want = torch.relu(torch.einsum("bztd,hdn->bhtn", x, w) + bias - 0.25)
    want[..., 3:6] = 0
    assert torch.allclose(got, want, atol=1e-5, rtol=1e-5)


def _blocked_rownorm(q, v, block):
    """Row-normalised attention evaluated block by block (what the reference's blocked op does with
    ALiBi off): accumulate |S| row sums and S V over the causal column blocks, then divide."""
    B, H, T, N = q.shape
    out = torch.zeros(B, H, T, v.shape[-1])
    norm = torch.zeros(B, H, T, 1)
    pat = BlockPattern2d.dense(block)
    nb = (T + block - 1) // block
    for r in range(nb):
        rs = slice(r * block, min((r + 1) * block, T))
        for c in pat.iter_cols(r, nb):
            cs = slice(c * block, min((c + 1) * block, T))
            S = q[:, :, rs] @ q[:, :, cs].transpose(-1, -2)
            if r == c:
                S = torch.tril(S, -1)
            norm[:, :, rs] += S.abs().sum(-1, keepdim=True)
            out[:, :, rs] += S @ v[:, :, cs].expand(B, H, -1, -1)
    return out / (norm + R.ROW_NORM_EPS)


@pytest.mark.parametrize("rot", ["rope", "pope"])
def test_blocked_attention_equals_dense(rot):
    torch.manual_seed(1)
    B, H, T, N, Dv = 1, 2, 6, 8, 6
    x = torch.relu(torch.randn(B, H, T, N))
    v = torch.randn(B, 1, T, Dv)
    q = R.rotate(x, rot, R.build_freqs(N, 65536.0, rot), 0)
    dense = R.attention_rownorm(q, v, None)
    assert torch.allclose(_blocked_rownorm(q, v, 3), dense, atol=1e-4, rtol=1e-4)
    pairs = BlockPattern2d.dense(3).pairs(2)
    assert torch.allclose(R.attention_rownorm(q, v, None, pairs, 3), dense, atol=1e-6)


def test_rownorm_alibi_bias_is_masked_and_visible():
    torch.manual_seed(2)
    x = torch.relu(torch.randn(1, 2, 2, 4)) + 0.1
    v = torch.randn(1, 1, 2, 3)
    slopes = R.alibi_slopes(2)
    with_bias = R.attention_rownorm(x, v, slopes)
    without = R.attention_rownorm(x, v, None)
    assert torch.all(with_bias[:, :, 0] == 0)                  # first token attends to nothing
    assert not torch.allclose(with_bias[:, :, 1], without[:, :, 1])


def test_rope_is_norm_preserving_and_pope_doubles_latent():
    x = torch.randn(2, 2, 5, 8)
    f = R.build_freqs(8, 65536.0, "rope")
    assert f[0] == f[1] and f[2] == f[3] and f[0] > f[2]
    q = R.rotate(x, "rope", f, 3)
    assert torch.allclose(q.norm(dim=-1), x.norm(dim=-1), atol=1e-5)
    p = R.rotate(x, "pope", R.build_freqs(8, 65536.0, "pope"), 0)
    assert p.shape[-1] == 16
    mag = torch.nn.functional.softplus(x)
    assert torch.allclose(p[..., :8] ** 2 + p[..., 8:] ** 2, mag ** 2, atol=1e-5)
    assert torch.equal(R.rotate(x, "alibi", f, 7), x)

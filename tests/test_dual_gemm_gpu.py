"""The chained-GEMM kernel (`csrc/dual_gemm_sm100.cuh`) against its fp32 torch statement
(`ops.dual_gemm.dual_reference`), for its three epilogues, on toy shapes and on one layer of the
base configuration (H = 4, N = 8192 neurons per head, D = 256, T = 512)."""
import pytest
import torch

from burn_dragon_b200.ops import dual_gemm as DG
from burn_dragon_b200.ops import gemm as G
from burn_dragon_b200.ops import native

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.float().flatten(), b.float().flatten()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def _bf(*shape, scale=1.0, gen=None):
    return (torch.randn(*shape, device="cuda", generator=gen) * scale).to(torch.bfloat16)


def _case(kind, B, T, H, N, D, gen, drop_p=0.0):
    """Operands of one launch of each kind, as the fused stack builds them."""
    M, HN = B * T, H * N
    kw = dict(M=M, H=H, n_per_head=N, N2=D, T=T)
    if kind == "fwd":
        lna = _bf(H * M, D, gen=gen)
        ev, dec = _bf(HN, D, scale=D ** -0.5, gen=gen), _bf(HN, D, scale=0.05, gen=gen)
        x = torch.relu(_bf(M, HN, gen=gen))
        args = (lna, ev, dec)
        kw.update(K1=D, epi=G.EPI_RELU_GATE, a1_b=T, a1_h=M, in0=x, theta=0.1, drop_p=drop_p, drop_seed=1234)
        out = torch.empty(M, D, device="cuda", dtype=torch.bfloat16)
    elif kind == "gate_bwd":
        dmlp = _bf(M, D, gen=gen)
        dec, ev = _bf(HN, D, scale=D ** -0.5, gen=gen), _bf(HN, D, scale=0.05, gen=gen)
        x = torch.relu(_bf(M, HN, gen=gen))
        xy = (x.float() * torch.relu(_bf(M, HN, gen=gen)).float()).to(torch.bfloat16)
        args = (dmlp, dec, ev)
        kw.update(K1=D, epi=G.EPI_GATE_BWD, group_per_head=True, a1_b=T, a1_h=0, in0=x, in1=xy,
                  out1=torch.empty(M, HN, device="cuda", dtype=torch.bfloat16), alpha=1.25, out_h_stride=M)
        out = torch.empty(H * M, D, device="cuda", dtype=torch.bfloat16)
    else:
        rope = kind == "dq_rope"
        Gs = _bf(B * H * T, T, scale=T ** -0.5, gen=gen)
        q = _bf(M, HN, gen=gen)
        enc = _bf(HN, D, scale=0.05, gen=gen)
        dxg = _bf(M, HN, gen=gen)
        closed = torch.rand(M, HN, device="cuda", generator=gen) < 0.5
        dxg = torch.where(closed, torch.full_like(dxg, -0.0), dxg)
        table = None
        if rope:
            freqs = torch.rand(N // 2, device="cuda", generator=gen) * 0.3
            table = G.rope_table(0, T, freqs)
        args = (Gs, q, enc)
        kw.update(K1=T, epi=G.EPI_DQ_BWD, flags=(G.F_ROPE | G.F_TABLE) if rope else 0, a1_b=H * T, a1_h=T, b1_mn=True,
                  b1_b=T, in0=dxg, in1=table, accumulate=True)
        out = torch.randn(M, D, device="cuda", generator=gen)
    return args, kw, out


def _run_both(kind, B, T, H, N, D, drop_p=0.0, max_ctas=0):
    gen = torch.Generator(device="cuda").manual_seed(7)
    args, kw, out = _case(kind, B, T, H, N, D, gen, drop_p)
    M, HN = B * T, H * N
    p_k = torch.full((M, HN), float("nan"), device="cuda", dtype=torch.bfloat16)
    p_r = torch.empty_like(p_k)
    out_k, out_r = out.clone(), out.clone()
    kw_k, kw_r = dict(kw), dict(kw)
    if kw.get("out1") is not None:
        kw_k["out1"] = torch.full_like(kw["out1"], float("nan"))
        kw_r["out1"] = torch.empty_like(kw["out1"])
    native.clear_status()
    DG.dual(*args, p_k, out_k, max_ctas=max_ctas, **kw_k)
    torch.cuda.synchronize()
    assert native.status_code() == 0
    DG.dual_reference(*args, p_r, out_r, **kw_r)
    return p_k, p_r, out_k, out_r, kw_k.get("out1"), kw_r.get("out1")


@pytest.mark.parametrize("kind", ["fwd", "gate_bwd", "dq_rope", "dq_plain"])
@pytest.mark.parametrize("shape", [(2, 128, 2, 128, 64), (2, 256, 2, 256, 128), (1, 384, 3, 384, 256)])
def test_dual_gemm_matches_the_fp32_statement(kind, shape):
    p_k, p_r, out_k, out_r, o1_k, o1_r = _run_both(kind, *shape)
    assert not torch.isnan(p_k.float()).any()
    assert _rel(p_k, p_r) < 1e-2, _rel(p_k, p_r)
    assert _rel(out_k, out_r) < 1e-2, _rel(out_k, out_r)
    if o1_k is not None:
        assert not torch.isnan(o1_k.float()).any()
        assert _rel(o1_k, o1_r) < 1e-2
        # the -0.0 markers of closed gates are exact
        assert torch.equal(o1_k.view(torch.int16) == -32768, o1_r.view(torch.int16) == -32768)
    if kind == "fwd":
        # zeros of the gate are exact zeros: the sparsity pattern of x*y is not perturbed by rounding
        agree = ((p_k == 0) == (p_r == 0)).float().mean().item()
        assert agree > 0.999, agree


def test_dual_gemm_dropout_uses_the_same_mask_as_the_single_gemm_kernel():
    p_k, p_r, out_k, out_r, _, _ = _run_both("fwd", 2, 128, 2, 256, 64, drop_p=0.25)
    assert _rel(p_k, p_r) < 1e-2 and _rel(out_k, out_r) < 1e-2
    assert abs((p_k == 0).float().mean().item() - (p_r == 0).float().mean().item()) < 1e-3


@pytest.mark.parametrize("kind", ["fwd", "gate_bwd", "dq_rope"])
def test_dual_gemm_work_split_does_not_change_the_result(kind):
    """Any number of CTAs walks the same units; P is bit-identical and the output sums agree to fp32 rounding."""
    ref = _run_both(kind, 2, 256, 2, 512, 128)
    for ctas in (1, 7, 33):
        got = _run_both(kind, 2, 256, 2, 512, 128, max_ctas=ctas)
        assert torch.equal(got[0].view(torch.int16), ref[0].view(torch.int16)), ctas
        assert _rel(got[2], ref[2]) < 2e-3, (ctas, _rel(got[2], ref[2]))


@pytest.mark.parametrize("kind", ["fwd", "gate_bwd", "dq_rope"])
def test_dual_gemm_base_configuration_layer(kind):
    """One layer's launch at the base configuration's shapes (two sequences instead of 32)."""
    p_k, p_r, out_k, out_r, o1_k, o1_r = _run_both(kind, 2, 512, 4, 8192, 256)
    assert _rel(p_k, p_r) < 1e-2
    assert _rel(out_k, out_r) < 1e-2, _rel(out_k, out_r)
    if o1_k is not None:
        assert _rel(o1_k, o1_r) < 1e-2

"""CUDA SSD chunk scan against the literal recurrence."""
import pytest
import torch

from burn_dragon_b200.ops import native
from burn_dragon_b200.ops import ssd as SSD

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,with_h0", [(64, False), (192, True), (100, True)])
def test_ssd_cuda_matches_sequential(T, with_h0):
    torch.manual_seed(0)
    B, H, P, N = 2, 3, 64, 128
    xw = torch.randn(B, T, H, P, device="cuda") * 0.5
    loga = -torch.rand(B, T, H, device="cuda") * 0.2
    Bm, Cm = torch.randn(B, T, N, device="cuda") * 0.3, torch.randn(B, T, N, device="cuda") * 0.3
    h0 = torch.randn(B, H, N, P, device="cuda") if with_h0 else None
    y_ref, h_ref = SSD.ssd_sequential(xw.double(), loga.double(), Bm.double(), Cm.double(),
                                      h0.double() if with_h0 else None)
    y, h = SSD.ssd_cuda(xw, loga, Bm, Cm, h0, tensor_cores=False)
    torch.cuda.synchronize()
    assert torch.allclose(y.double(), y_ref, atol=2e-3, rtol=1e-3)
    assert torch.allclose(h.double(), h_ref, atol=2e-3, rtol=1e-3)
    # the tensor-core kernel rounds its operands to bf16: compared as a whole-tensor relative error
    native.clear_status()
    y_tc, h_tc = SSD.ssd_cuda(xw, loga, Bm, Cm, h0, tensor_cores=True)
    torch.cuda.synchronize()
    assert native.status_code() == 0
    rel = ((y_tc.double() - y_ref).norm() / y_ref.norm()).item()
    assert rel < 1e-2, rel
    assert torch.allclose(h_tc.double(), h_ref, atol=2e-3, rtol=1e-3)      # the states stay fp32
    y2, h2 = SSD.ssd(xw, loga, Bm, Cm, h0)          # dispatcher picks the (tensor-core) kernels when no grad is needed
    assert torch.equal(y2, y_tc)


def test_mamba2_model_uses_kernels_for_prefill():
    from burn_dragon_b200.models.mamba import MambaConfig, MambaLM
    torch.manual_seed(0)
    m = MambaLM(MambaConfig(version=2, n_layer=2, d_model=128, vocab_size=256)).cuda().eval()
    tok = torch.randint(0, 256, (2, 128), device="cuda")
    n0 = native.launch_count()
    with torch.no_grad():
        st = m.init_state()
        a = m.forward_with_state(tok, st)
    assert native.launch_count() > n0
    lg = m(tok[:, :], None)                          # grad-enabled path: torch chunked form
    assert ((a - lg.detach()).norm() / lg.detach().norm()).item() < 2e-2


def test_dual_form_backward_on_the_device_matches_the_written_out_oracle():
    """`ssd_dual` with the chunk-scan kernels under it (y and d xw come from the kernels) against the
    written-out float64 oracle of the gradients."""
    torch.manual_seed(0)
    B, T, H, P, N = 2, 200, 3, 64, 128
    xw = (torch.randn(B, T, H, P, device="cuda") * 0.5).requires_grad_()
    loga = (-torch.rand(B, T, H, device="cuda") * 0.2).requires_grad_()
    Bm = (torch.randn(B, T, N, device="cuda") * 0.3).requires_grad_()
    Cm = (torch.randn(B, T, N, device="cuda") * 0.3).requires_grad_()
    dy = torch.randn(B, T, H, P, device="cuda") * 0.1
    before = native.launch_count()
    y, _ = SSD.ssd_dual(xw, loga, Bm, Cm)
    got = torch.autograd.grad(y, (xw, loga, Bm, Cm), dy)
    assert native.launch_count() >= before + 2, "forward and the dual scan both run the kernels"
    with torch.no_grad():
        want = SSD.ssd_backward_sequential(xw.double(), loga.double(), Bm.double(), Cm.double(), dy.double())
    for g, w, name in zip(got, want, ("xw", "loga", "B", "C")):
        # y and d xw come from the tensor-core kernels (bf16 operands): whole-tensor relative error
        assert ((g.double() - w).norm() / w.norm()).item() < 2e-2, name


def test_decode_step_kernel_matches_the_recurrence():
    torch.manual_seed(0)
    B, H, P, N = 5, 3, 64, 128
    xw = torch.randn(B, 1, H, P, device="cuda")
    loga = -torch.rand(B, 1, H, device="cuda")
    Bm, Cm = torch.randn(B, 1, N, device="cuda"), torch.randn(B, 1, N, device="cuda")
    h0 = torch.randn(B, H, N, P, device="cuda")
    y_ref, h_ref = SSD.ssd_sequential(xw.double(), loga.double(), Bm.double(), Cm.double(), h0.double())
    n0 = native.launch_count()
    y, h = SSD.ssd(xw, loga, Bm, Cm, h0)
    assert native.launch_count() == n0 + 1
    assert torch.allclose(y.double(), y_ref, atol=1e-4, rtol=1e-4) and torch.allclose(h.double(), h_ref, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("k,with_bias", [(4, True), (3, False)])
def test_conv1d_silu_kernels_match_torch_autograd(k, with_bias):
    from burn_dragon_b200.ops import mamba_ops as MO
    torch.manual_seed(0)
    B, T, C = 3, 200, 330                                  # channel count that is no multiple of the block width
    seq = torch.randn(B, T + k - 1, C, device="cuda", requires_grad=True)
    w = (torch.randn(C, k, device="cuda") * 0.5).requires_grad_()
    b = (torch.randn(C, device="cuda") * 0.1).requires_grad_() if with_bias else None
    dout = torch.randn(B, T, C, device="cuda")
    n0 = native.launch_count()
    out = MO.conv1d_silu(seq, w, b)
    got = torch.autograd.grad(out, [t for t in (seq, w, b) if t is not None], dout)
    assert native.launch_count() == n0 + 2, "one kernel entry per direction"
    ref = MO.conv1d_silu_reference(seq.double(), w.double(), b.double() if with_bias else None)
    want = torch.autograd.grad(ref, [t for t in (seq, w, b) if t is not None], dout.double())
    assert torch.allclose(out.double(), ref, atol=1e-5, rtol=1e-5)
    for g, r in zip(got, want):
        assert ((g.double() - r).norm() / r.norm()).item() < 1e-5


@pytest.mark.parametrize("D", [256, 1000])
def test_gated_rmsnorm_kernels_match_torch_autograd(D):
    from burn_dragon_b200.ops import mamba_ops as MO
    torch.manual_seed(0)
    rows = 777
    v = torch.randn(rows, D, device="cuda", requires_grad=True)
    z = torch.randn(rows, D, device="cuda", requires_grad=True)
    w = (1 + 0.1 * torch.randn(D, device="cuda")).requires_grad_()
    dout = torch.randn(rows, D, device="cuda")
    out = MO.gated_rmsnorm(v, z, w)
    got = torch.autograd.grad(out, (v, z, w), dout)
    ref = MO.gated_rmsnorm_reference(v.double(), z.double(), w.double())
    want = torch.autograd.grad(ref, (v, z, w), dout.double())
    assert torch.allclose(out.double(), ref, atol=1e-4, rtol=1e-4)
    for g, r, name in zip(got, want, "vzw"):
        assert ((g.double() - r).norm() / r.norm()).item() < 1e-4, name


def test_mamba2_training_step_runs_its_elementwise_parts_on_kernels():
    """Loss and gradients of a Mamba-2 model with conv + SiLU, the SSD scan and the gated RMSNorm on this
    library's kernels against the same model on torch ops only."""
    from burn_dragon_b200.models.mamba import MambaConfig, MambaLM
    import burn_dragon_b200.ops.mamba_ops as MO
    torch.manual_seed(0)
    m = MambaLM(MambaConfig(version=2, n_layer=2, d_model=128, vocab_size=256)).cuda()
    tok = torch.randint(0, 256, (2, 129), device="cuda")
    n0 = native.launch_count()
    loss = m(tok[:, :-1], tok[:, 1:])
    loss.backward()
    assert native.launch_count() - n0 >= 2 * (2 + 2 + 2), "conv, scan and norm kernels in both directions, per layer"
    got = {n: p.grad.clone() for n, p in m.named_parameters()}
    m.zero_grad()
    keep = MO._on_kernels
    MO._on_kernels = lambda *ts: False
    SSD_dual = SSD._DUAL
    SSD._DUAL = "0"
    try:
        ref = m(tok[:, :-1], tok[:, 1:])
        ref.backward()
    finally:
        MO._on_kernels = keep
        SSD._DUAL = SSD_dual
    assert abs(loss.item() - ref.item()) < 2e-2
    for n, p in m.named_parameters():
        rel = ((got[n] - p.grad).norm() / (p.grad.norm() + 1e-12)).item()
        assert rel < 5e-2, (n, rel)

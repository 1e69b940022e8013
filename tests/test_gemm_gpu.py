"""tcgen05 GEMM and its fused epilogues against the fp32 torch statement of the same contract."""
import pytest
import torch

from burn_dragon_b200.ops import gemm as G
from burn_dragon_b200.ops import native

pytestmark = pytest.mark.gpu


def _rand(r, c, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(r, c, device="cuda", generator=g) * scale).to(torch.bfloat16)


def _check(got, want, tol=2e-2):
    got, want = got.float(), want.float()
    err = (got - want).abs().max().item()
    ref = want.abs().max().item() + 1e-6
    assert err <= tol * ref + 1e-3, f"max abs err {err} (ref max {ref})"


def _run_both(kw, outs):
    """Run the kernel (staged-TMA epilogue where eligible, then the per-thread epilogue) and the
    reference on clones of the outputs; return list of (kernel, reference) pairs for both runs."""
    r_outs = {n: t.clone() for n, t in outs.items()}
    G.gemm_reference(**kw, **r_outs)
    pairs = []
    for tma in (True, False):
        native.clear_status()
        k_outs = {n: t.clone() for n, t in outs.items()}
        G.gemm(**kw, **k_outs, tma_epilogue=tma)
        torch.cuda.synchronize()
        assert native.status_code() == 0, "kernel reported a wait timeout"
        pairs += [(k_outs[n], r_outs[n]) for n in outs]
    return pairs


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (384, 768, 192), (200, 328, 136)])
def test_store_majors(a_mn, b_mn, M, N, K):
    a = _rand(K, M, seed=1) if a_mn else _rand(M, K, seed=1)
    b = _rand(K, N, seed=2) if b_mn else _rand(N, K, seed=2)
    kw = dict(a=a, b=b, M=M, N=N, K=K, a_mn=a_mn, b_mn=b_mn, epi=G.EPI_STORE)
    for k, r in _run_both(kw, dict(out0=torch.zeros(M, N, device="cuda", dtype=torch.bfloat16))):
        _check(k, r)


@pytest.mark.parametrize("bn", [128, 256])
def test_store_f32_accumulate(bn):
    M, N, K = 256, 256, 512
    a, b = _rand(K, M, seed=3), _rand(K, N, seed=4)
    out = torch.randn(M, N, device="cuda")
    kw = dict(a=a, b=b, M=M, N=N, K=K, a_mn=True, b_mn=True, epi=G.EPI_STORE, flags=G.F_OUT_F32 | G.F_ACCUM,
              alpha=0.5, bn=bn)
    for k, r in _run_both(kw, dict(out0=out)):
        _check(k, r, tol=1e-2)


def test_long_k_pipeline():
    # many k-blocks and many tiles per CTA exercise the smem ring and both accumulators
    M, N, K = 1024, 1024, 4096
    a, b = _rand(M, K, 0.1, seed=5), _rand(N, K, 0.1, seed=6)
    kw = dict(a=a, b=b, M=M, N=N, K=K, epi=G.EPI_STORE, max_ctas=3)
    for k, r in _run_both(kw, dict(out0=torch.zeros(M, N, device="cuda", dtype=torch.bfloat16))):
        _check(k, r)


def test_batched_offsets():
    # z0 = head (column window of A, row window of B), z1 = batch (row window of A)
    H, Bb, T, Nh, D = 2, 3, 128, 256, 64
    a = _rand(Bb * T, D, seed=7)            # cur [M, D]
    w = _rand(H * Nh, D, seed=8)            # weights [H*N, D]
    out = torch.zeros(Bb * T, H * Nh, device="cuda", dtype=torch.bfloat16)
    kw = dict(a=a, b=w, M=T, N=Nh, K=D, nz=(H, Bb), a_off=(0, T, 0, 0), b_off=(Nh, 0, 0, 0),
              c_off=(0, T, Nh, 0), epi=G.EPI_STORE)
    for k, r in _run_both(kw, dict(out0=out)):
        _check(k, r)
    _check(out.copy_(_run_both(kw, dict(out0=out))[0][0]), (a.float() @ w.float().t()))


@pytest.mark.parametrize("rot", ["none", "rope", "rope_table", "pope"])
def test_relu_rotary(rot):
    M, N, K, T, Nh = 256, 512, 128, 64, 256
    a, w = _rand(M, K, seed=9), _rand(N, K, 0.2, seed=10)
    freqs = (1.0 / (65536.0 ** (torch.arange(Nh, device="cuda").div(2, rounding_mode="floor") * 2 / Nh))) / 6.283185307
    flags = {"none": 0, "rope": G.F_ROPE, "rope_table": G.F_ROPE | G.F_TABLE, "pope": G.F_POPE}[rot]
    outs = dict(out0=torch.zeros(M, N, device="cuda", dtype=torch.bfloat16))
    kw = dict(a=a, b=w, M=M, N=N, K=K, epi=G.EPI_RELU, flags=flags, theta=0.1, T=T, pos0=5, n_per_head=Nh,
              freqs=(freqs[0::2] if rot.startswith("rope") else freqs).float().contiguous())
    if rot == "rope_table":
        kw["in0"] = G.rope_table(5, T, kw["freqs"])
    if rot.startswith("rope"):
        outs["out1"] = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    if rot == "pope":
        # per-head layout [real Nh | imag Nh]; run one head per z0
        outs["out1"] = torch.zeros(M, 2 * N, device="cuda", dtype=torch.bfloat16)
        kw.update(N=Nh, nz=(N // Nh, 1), b_off=(Nh, 0, 0, 0), c_off=(0, 0, Nh, 0), o1_off=(2 * Nh, 0, Nh))
    for k, r in _run_both(kw, outs):
        _check(k, r)


@pytest.mark.parametrize("drop_p", [0.0, 0.25])
def test_relu_gate(drop_p):
    M, N, K = 256, 512, 128
    a, w, x = _rand(M, K, seed=11), _rand(N, K, 0.2, seed=12), _rand(M, N, seed=13).relu()
    kw = dict(a=a, b=w, M=M, N=N, K=K, epi=G.EPI_RELU_GATE, in0=x, drop_p=drop_p, drop_seed=1234567)
    if drop_p:
        keep = G.dropout_keep_mask(1234567, 0, M, N, drop_p, "cuda")
        assert abs(keep.float().mean().item() - (1 - drop_p)) < 0.01
    outs = dict(out0=torch.zeros(M, N, device="cuda", dtype=torch.bfloat16),
                out1=torch.zeros(M, N, device="cuda", dtype=torch.bfloat16))
    for k, r in _run_both(kw, outs):
        _check(k, r)


@pytest.mark.parametrize("bn", [128, 256])
@pytest.mark.parametrize("upper", [False, True])
def test_causal_decay(bn, upper):
    H, Bb, T, Nh = 2, 2, 512, 128
    q = _rand(Bb * T, H * Nh, 0.3, seed=14)
    slopes = torch.tensor([0.05, 0.02], device="cuda")
    out = torch.full((Bb * H * T, T), 7.0, device="cuda", dtype=torch.bfloat16)
    kw = dict(a=q, b=q, M=T, N=T, K=Nh, nz=(H, Bb), a_off=(0, T, Nh, 0), b_off=(0, T, Nh, 0),
              c_off=(T, H * T, 0, 0), epi=G.EPI_CAUSAL, flags=G.F_UPPER if upper else 0, slopes=slopes,
              causal_tiles=2 if upper else 1, bn=bn)
    for k, r in _run_both(kw, dict(out0=out)):
        _check(k, r)


def test_causal_k_value_product():
    # a = S V with S lower-triangular: only k < m0+128 is contracted
    Bb, T, D = 2, 512, 256
    S = torch.tril(_rand(Bb * T, T, 0.2, seed=15).float().reshape(Bb, T, T), -1).reshape(Bb * T, T).to(torch.bfloat16)
    V = _rand(Bb * T, D, seed=16)
    out = torch.zeros(Bb * T, D, device="cuda", dtype=torch.bfloat16)
    kw = dict(a=S, b=V, M=T, N=D, K=T, b_mn=True, nz=(1, Bb), a_off=(0, T, 0, 0), b_off=(0, 0, 0, T),
              c_off=(0, T, 0, 0), epi=G.EPI_STORE, causal_k=1)
    for k, r in _run_both(kw, dict(out0=out)):
        _check(k, r)
    want = torch.bmm(S.float().reshape(Bb, T, T), V.float().reshape(Bb, T, D)).reshape(Bb * T, D)
    G.gemm(**kw, out0=out)
    _check(out, want)


def test_gate_bwd():
    M, N, K = 256, 512, 128
    g, w = _rand(M, K, seed=17), _rand(N, K, 0.2, seed=18)
    x, y = _rand(M, N, seed=19).relu(), _rand(M, N, seed=20).relu()
    xy = (x.float() * y.float()).to(torch.bfloat16)
    kw = dict(a=g, b=w, M=M, N=N, K=K, epi=G.EPI_GATE_BWD, in0=x, in1=xy)
    outs = dict(out0=torch.zeros(M, N, device="cuda", dtype=torch.bfloat16),
                out1=torch.zeros(M, N, device="cuda", dtype=torch.bfloat16))
    pairs = _run_both(kw, outs)
    for k, r in pairs:
        _check(k, r)
    # closed gates carry the -0.0 marker, open ones never do
    dxg = pairs[1][0]
    marker = dxg.view(torch.int16) == -32768
    assert torch.equal(marker, x <= 0)
    # and the result equals the definition with the true y
    want = torch.where(x > 0, (g.float() @ w.float().t()) * y.float(), torch.zeros(M, N, device="cuda"))
    _check(dxg, want, tol=3e-2)


@pytest.mark.parametrize("rope", ["none", "sincos", "table"])
def test_dq_bwd(rope):
    T, N, Nh = 256, 512, 256
    gs = _rand(T, T, 0.2, seed=21)
    q = _rand(T, N, seed=22)
    x, dxg = _rand(T, N, seed=23).relu(), _rand(T, N, seed=24)
    dxg = torch.where(x > 0, dxg, torch.full_like(dxg, -0.0))
    freqs = ((1.0 / (65536.0 ** (torch.arange(Nh, device="cuda").div(2, rounding_mode="floor") * 2 / Nh)))
             / 6.283185307)[0::2].float().contiguous()
    flags = {"none": 0, "sincos": G.F_ROPE, "table": G.F_ROPE | G.F_TABLE}[rope]
    kw = dict(a=gs, b=q, M=T, N=N, K=T, b_mn=True, epi=G.EPI_DQ_BWD, flags=flags, in0=dxg,
              in1=G.rope_table(3, T, freqs) if rope == "table" else None, T=T, pos0=3, n_per_head=Nh, freqs=freqs)
    for k, r in _run_both(kw, dict(out0=torch.zeros(T, N, device="cuda", dtype=torch.bfloat16))):
        _check(k, r)


@pytest.mark.parametrize("rope", ["none", "table"])
def test_dq_bwd_over_segments_with_two_contractions_in_one_epilogue(rope):
    """Chunk-state attention's dq: every (head, segment) problem covers C rows of a sequence of T positions
    (the rotary table row is the position of the OUTPUT row), and two products meet in the epilogue: the
    first launch keeps the -0.0 markers of closed gates in its output (`F_KEEP_MARK`), the second takes that
    output as its gate-gradient input."""
    T, C, N, Nh, K2 = 256, 128, 512, 256, 128
    J = T // C
    gs = _rand(T, C, 0.2, seed=21)                  # J blocks of [C, C]
    q = _rand(T, N, seed=22)
    x2, r2 = _rand(T, K2, 0.3, seed=25), _rand(J * N, K2, 0.3, seed=26)
    x, dxg = _rand(T, N, seed=23).relu(), _rand(T, N, seed=24)
    dxg = torch.where(x > 0, dxg, torch.full_like(dxg, -0.0))
    freqs = ((1.0 / (65536.0 ** (torch.arange(Nh, device="cuda").div(2, rounding_mode="floor") * 2 / Nh)))
             / 6.283185307)[0::2].float().contiguous()
    flags = G.F_ROPE | G.F_TABLE if rope == "table" else 0
    table = G.rope_table(3, T, freqs) if rope == "table" else None
    common = dict(M=C, N=N, nz=(1, J), c_off=(0, C, 0, 0), epi=G.EPI_DQ_BWD, in1=table, T=T, pos0=3, n_per_head=Nh,
                  freqs=freqs)
    first = dict(a=x2, b=r2, K=K2, a_off=(0, C, 0, 0), b_off=(0, N, 0, 0), flags=flags | G.F_KEEP_MARK, in0=dxg, **common)
    pairs = _run_both(first, dict(out0=torch.zeros(T, N, device="cuda", dtype=torch.bfloat16)))
    for k, r in pairs:
        _check(k, r)
        assert torch.equal(k.view(torch.int16) == -32768, x <= 0), "exactly the closed gates carry the marker"
    mid = pairs[0][0]
    second = dict(a=gs, b=q, K=C, b_mn=True, a_off=(0, C, 0, 0), b_off=(0, 0, 0, C), flags=flags, in0=mid, **common)
    for k, r in _run_both(second, dict(out0=torch.zeros(T, N, device="cuda", dtype=torch.bfloat16))):
        _check(k, r)
        assert not (k.view(torch.int16) == -32768).any()


def test_store_reversed_row_decay_with_atomics():
    """`F_ROWDECAY_REV`: row m of a segment of T rows scaled by exp(-slope * (T - m)), per head, the heads'
    tiles added into one fp32 output (gradient of a segment state w.r.t. the values)."""
    H, C, Np, D = 3, 128, 256, 64
    q = _rand(C, H * Np, 0.3, seed=31)
    st = _rand(H * Np, D, 0.3, seed=32)
    slopes = torch.tensor([0.05, 0.01, 0.002], device="cuda")
    out = torch.randn(C, D, device="cuda")
    kw = dict(a=q, b=st, M=C, N=D, K=Np, b_mn=True, nz=(H, 1), a_off=(0, 0, Np, 0), b_off=(0, 0, Np, 0),
              flags=G.F_OUT_F32 | G.F_ATOMIC | G.F_ROWDECAY_REV, slopes=slopes, T=C)
    for k, r in _run_both(kw, dict(out0=out)):
        _check(k, r, tol=1e-2)


@pytest.mark.parametrize("world", [2, 4])
def test_gather_inside_the_gemm_with_every_rank_on_one_gpu(world):
    """The all-gather -> GEMM kernel with the ranks emulated on one GPU: every "rank" has its own copy of the
    [M, K] buffer holding only its own rows; the launches run one after the other (no launch waits for
    another), each pulling the other copies' rows into its own with the kernel's peer-load path, waiting on
    its arrival counters and multiplying from its local copy."""
    M, K, N = 256 * world, 192, 384
    rows = M // world
    A = _rand(M, K, 0.5, seed=41)
    w = _rand(N, K, 0.3, seed=42)
    want = A.float() @ w.float().t()
    copies = []
    for r in range(world):
        c = torch.zeros(M, K, device="cuda", dtype=torch.bfloat16)
        c[r * rows:(r + 1) * rows] = A[r * rows:(r + 1) * rows]
        copies.append(c)
    ptrs = [c.data_ptr() for c in copies]
    for r in range(world):
        # a later rank's launch finds rows in the earlier ranks' copies that those ranks gathered: same values
        arrived = torch.zeros(M // 128, device="cuda", dtype=torch.int32)
        out = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
        native.clear_status()
        G.gemm(copies[r], w, M=M, N=N, K=K, out0=out, gather_ptrs=ptrs, gather_rows=rows, gather_rank=r,
               gather_arrived=arrived)
        torch.cuda.synchronize()
        assert native.status_code() == 0
        assert torch.equal(copies[r], A), "the local copy holds every rank's rows afterwards"
        own = arrived.view(world, -1)[r]
        assert int(own.max()) == 0 and int(arrived.sum()) > 0, "own blocks are not copied, the others are counted"
        _check(out, want)


@pytest.mark.parametrize("bn", [128, 256])
def test_causal_tile_predicate_skips_tiles(bn):
    """`tile_skip`: output tiles flagged in the byte map are neither computed nor written (they keep what the
    output held), the others are the ordinary causal product - with the staged and the per-thread epilogue,
    which must stay in step with the producer and the MMA issuer over the skipped tiles."""
    T, K = 1024, 128
    q = _rand(2 * T, K, 0.3, seed=91)
    tm, tn = T // 128, T // bn
    g = torch.Generator().manual_seed(3)
    skip = (torch.rand(tm, tn, generator=g) < 0.5).to(torch.uint8).cuda()
    slopes = torch.tensor([0.01, 0.002], device="cuda")
    kw = dict(a=q, b=q, M=T, N=T, K=K, nz=(2, 1), a_off=(T, 0, 0, 0), b_off=(T, 0, 0, 0), c_off=(T, 0, 0, 0),
              epi=G.EPI_CAUSAL, slopes=slopes, causal_tiles=1, bn=bn, tile_skip=skip)
    base = torch.full((2 * T, T), 7.0, device="cuda", dtype=torch.bfloat16)
    for k, r in _run_both(kw, dict(out0=base)):
        _check(k, r)
        blocks = k.view(2, tm, 128, tn, bn)
        for mi in range(tm):
            for ni in range(tn):
                if int(skip[mi, ni]) and ni * bn <= mi * 128 + 127:
                    assert float((blocks[:, mi, :, ni] - 7.0).abs().max()) == 0.0, "a skipped tile was written"


def test_reduce_scatter_epilogue_and_gather_with_two_ranks_on_one_gpu():
    """The tensor-parallel reduction with both ranks emulated on one GPU: each "rank" has its own slot buffer,
    output buffer and flag words; rank r's GEMM stores its partial tiles into slot r of the owner's buffer
    (`F_PEER_RS`), then each rank's `gather_blocks` sums the slots of the rows it owns and stores the sum into
    every rank's output. The launches run one after the other, so the flag words are written ahead of time
    with a value every barrier of the call accepts (no launch waits for a later one)."""
    world, M, N, K = 2, 512, 256, 1024
    block_rows = M // world
    a = [_rand(M, K, 0.3, seed=51 + r) for r in range(world)]
    w = [_rand(K, N, 0.3, seed=61 + r) for r in range(world)]
    want = sum(a[r].float() @ w[r].float() for r in range(world))
    slots = [torch.zeros(world * block_rows, N, device="cuda") for _ in range(world)]
    outs = [torch.zeros(M, N, device="cuda") for _ in range(world)]
    epoch = 3
    flags = [torch.full((4096,), 2 * epoch + 2, device="cuda", dtype=torch.int32) for _ in range(world)]
    native.clear_status()
    for r in range(world):
        G.gemm(a[r], w[r], M=M, N=N, K=K, b_mn=True, flags=G.F_OUT_F32 | G.F_PEER_RS, out0=slots[r],
               peer_ptrs=[t.data_ptr() for t in slots], peer_rows=block_rows, peer_rank=r)
    for r in range(world):
        native.ops.gather_blocks(slots[r], [t.data_ptr() for t in slots], [t.data_ptr() for t in flags],
                                 [t.data_ptr() for t in outs], 0, False, r, world, block_rows * N, epoch, 8)
    torch.cuda.synchronize()
    assert native.status_code() == 0
    for o in outs:
        _check(o, want, tol=1e-2)


def test_fully_sharded_step_with_two_ranks_on_one_gpu():
    """The fully sharded data-parallel step with both ranks emulated on one GPU: each rank's weight-gradient
    GEMM adds its tiles into the OWNER's fp32 gradient slice from its epilogue (`F_PEER_RS | F_ATOMIC`), then
    each rank's `shard_adamw_ag` applies AdamW to its slice, stores the bf16 rows into every rank's working
    copy and clears the slice. Sequential launches; the flag words are written ahead of time."""
    world, R, D, Mtok = 2, 512, 256, 1024          # weight [R, D]; R / world rows per rank
    rpr = R // world
    torch.manual_seed(0)
    W0 = torch.randn(R, D, device="cuda") * 0.1
    x = [_rand(Mtok, R, 0.3, seed=71 + r) for r in range(world)]        # dX-like [tokens, R]
    c = [_rand(Mtok, D, 0.3, seed=81 + r) for r in range(world)]        # cur-like [tokens, D]
    grad = sum(x[r].float().t() @ c[r].float() for r in range(world))   # sum over the ranks' batches
    acc = [torch.zeros(rpr, D, device="cuda") for _ in range(world)]    # each rank's gradient slice
    ptrs = [t.data_ptr() for t in acc]
    native.clear_status()
    for r in range(world):
        G.gemm(x[r], c[r], M=R, N=D, K=Mtok, a_mn=True, b_mn=True, flags=G.F_OUT_F32 | G.F_ATOMIC | G.F_PEER_RS,
               out0=acc[r], peer_ptrs=ptrs, peer_rows=rpr, peer_rank=r)
    torch.cuda.synchronize()
    for r in range(world):
        _check(acc[r], grad[r * rpr:(r + 1) * rpr], tol=1e-2)
    master = [W0[r * rpr:(r + 1) * rpr].clone().contiguous() for r in range(world)]
    m = [torch.zeros(rpr, D, device="cuda") for _ in range(world)]
    v = [torch.zeros(rpr, D, device="cuda") for _ in range(world)]
    shadow = [torch.zeros(R, D, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    epoch = 5
    flags = [torch.full((4096,), 2 * epoch + 2, device="cuda", dtype=torch.int32) for _ in range(world)]
    lr, b1, b2, eps, wd, scale = 1e-2, 0.9, 0.999, 1e-8, 0.1, 1.0 / world
    g_kept = [a.clone() for a in acc]
    for r in range(world):
        native.ops.shard_adamw_ag([t.data_ptr() for t in flags], [t.data_ptr() for t in shadow], r, world, acc[r],
                                  master[r], m[r], v[r], [0, rpr * D], [r * rpr * D], lr, b1, b2, eps, wd, 1, scale,
                                  epoch, 8)
    torch.cuda.synchronize()
    assert native.status_code() == 0
    for r in range(world):
        g = g_kept[r] * scale
        m_ref, v_ref = (1 - b1) * g, (1 - b2) * g * g
        w_ref = W0[r * rpr:(r + 1) * rpr] * (1 - lr * wd) - lr * (m_ref / (1 - b1)) / ((v_ref / (1 - b2)).sqrt() + eps)
        assert torch.allclose(master[r], w_ref, atol=1e-5, rtol=1e-4)
        assert float(acc[r].abs().max()) == 0.0, "the gradient slice is cleared for the next step"
        for sh in shadow:                                            # every rank's working copy got these rows
            assert torch.allclose(sh[r * rpr:(r + 1) * rpr].float(), w_ref, atol=2e-3, rtol=1e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("alibi", [True, False])
def test_rownorm_attention_matches_reference(alibi):
    """forward_fast attention (bias + L1 row normalisation): kernels against the fp32 torch statement,
    forward and both gradients."""
    from burn_dragon_b200.ops import reference as R
    from burn_dragon_b200.ops import rownorm_attention as RA
    torch.manual_seed(3)
    B, H, T, N, D = 2, 3, 256, 128, 64
    q = (torch.randn(B, H, T, N, device="cuda") * 0.3).relu().requires_grad_(True)
    v = torch.randn(B, 1, T, D, device="cuda").requires_grad_(True)
    slopes = torch.tensor([0.5, 0.25, 0.125], device="cuda") if alibi else None
    assert RA.can_run(q, v)
    a = RA.attention_rownorm(q, v, slopes)
    g = torch.randn_like(a)
    a.backward(g)
    dq, dv = q.grad.clone(), v.grad.clone()
    q.grad = v.grad = None
    # the reference sees the same bf16-rounded operands
    qr = q.detach().to(torch.bfloat16).float().requires_grad_(True)
    vr = v.detach().to(torch.bfloat16).float().requires_grad_(True)
    ar = R.attention_rownorm(qr, vr, slopes)
    ar.backward(g)

    def rel(x, y):
        return ((x - y).norm() / (y.norm() + 1e-12)).item()

    assert rel(a, ar) < 2e-2, rel(a, ar)
    assert rel(dv, vr.grad) < 3e-2, rel(dv, vr.grad)
    assert rel(dq, qr.grad) < 3e-2, rel(dq, qr.grad)


@pytest.mark.gpu
def test_forward_fast_uses_kernels_and_matches_torch():
    from burn_dragon_b200.models.bdh import BDH, BDHConfig
    torch.manual_seed(0)
    m = BDH(BDHConfig(n_layer=2, n_embd=64, n_head=2, n_latent_per_head=128, vocab_size=256, dropout=0.0)).cuda()
    toks = torch.randint(0, 256, (2, 128), device="cuda")
    n0 = native.launch_count()
    got = m.forward_fast(toks)
    assert native.launch_count() > n0
    m.use_native = False
    want = m.forward_fast(toks)
    assert ((got - want).norm() / want.norm()).item() < 3e-2


def test_tile_to_cta_assignment_does_not_change_a_bit():
    """Race check by schedule variation: every output tile is produced by one CTA with a fixed K order,
    so the same launch run with the full grid, with 7 CTAs (many tiles per CTA, other neighbours in
    time) and with 1 CTA (fully serial) has to give bit-identical outputs; a missing barrier between
    pipeline stages or accumulator buffers would show up as a difference."""
    M, N, K = 1024, 2048, 512
    a, b = _rand(M, K, seed=11), _rand(N, K, seed=12)
    x = _rand(M, N, seed=13)
    outs = []
    for ctas in (0, 7, 1):
        native.clear_status()
        y, xy = (torch.empty(M, N, device="cuda", dtype=torch.bfloat16) for _ in range(2))
        G.gemm(a, b, M=M, N=N, K=K, epi=G.EPI_RELU_GATE, in0=x, out0=y, out1=xy, theta=0.1, max_ctas=ctas)
        torch.cuda.synchronize()
        assert native.status_code() == 0
        outs.append((y, xy))
    for y, xy in outs[1:]:
        assert torch.equal(y, outs[0][0]) and torch.equal(xy, outs[0][1])


def test_relu_lowrank_with_bias_and_block_mask_on_the_kernel():
    """relu(x W^T + b - theta) * block mask: the bias is added in the GEMM epilogue, the blocks the pattern
    switches off are never computed (reference: src/kernel/relu_lowrank.rs:7-37)."""
    from burn_dragon_b200.ops import lowrank, reference as R
    from burn_dragon_b200.ops.block_sparse import BlockPattern1d
    torch.manual_seed(0)
    M, D, H, N = 256, 64, 2, 256
    x = (torch.randn(M, D, device="cuda")).to(torch.bfloat16)
    w = (torch.randn(H * N, D, device="cuda") * 0.2).to(torch.bfloat16)
    bias = torch.randn(H * N, device="cuda") * 0.3
    pat = BlockPattern1d.from_blocks(64, [0, 2])
    for b in (None, bias):
        for p in (None, pat):
            got = lowrank.relu_lowrank(x, w, b, 0.1, p, n_head=H).float()
            mask = p.mask(N, device="cuda") if p is not None else None
            want = R.relu_lowrank(x.float().view(1, 1, M, D), w.float().view(H, N, D).transpose(1, 2),
                                  b.view(1, H, 1, N) if b is not None else None, 0.1, mask)      # [1, H, M, N]
            want = want[0].permute(1, 0, 2).reshape(M, H * N)
            assert (got - want).norm() / want.norm() < 5e-3
            if p is not None:
                assert float(got.view(M, H, N)[:, :, 64:128].abs().max()) == 0.0

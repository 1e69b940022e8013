"""Small, self-terminating workloads for kernel profiling and roofline timing:

    python tests/profile_cases.py --case dq_bwd [--launches 3] [--time]

Each case launches one kernel of the BDH layer a few times on a reduced batch of the base
configuration (8 sequences instead of 32: inputs still exceed the 126 MB L2, the device holds a few
GB). With `--time` the case is timed with CUDA events (after warm-up, L2 flushed by the size of the
working set) and a JSON line with achieved bytes/s and FLOP/s against the measured peaks is printed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from burn_dragon_b200.ops import gemm as G
from burn_dragon_b200.ops import dual_gemm as DG
from burn_dragon_b200.ops import native

B, T, H, N, D = 8, 512, 4, 8192, 256
M, HN = B * T, H * N


def _rnd(r, c, s=1.0):
    return (torch.randn(r, c, device="cuda") * s).to(torch.bfloat16)


def build(case: str):
    """-> (callable, flops, algorithmic bytes)"""
    cur, W = _rnd(M, D), _rnd(HN, D, 0.02)
    x = torch.zeros(M, HN, device="cuda", dtype=torch.bfloat16)
    q = torch.zeros_like(x)
    act = _rnd(M, HN, 0.1).relu()
    freqs = ((1.0 / (65536.0 ** (torch.arange(N, device="cuda").div(2, rounding_mode="floor") * 2 / N)))
             / 6.283185307).float()[0::2].contiguous()
    tab = G.rope_table(0, T, freqs)
    S = _rnd(B * H * T, T, 0.1)
    big = 2.0 * M * HN          # bytes of one [M, H*N] bf16 tensor
    gemm_fl = 2.0 * M * HN * D
    att_fl = 2.0 * B * H * T * T * N
    cases = {
        "enc_rope": (lambda: G.gemm(cur, W, M=M, N=HN, K=D, epi=G.EPI_RELU, flags=G.F_ROPE | G.F_TABLE, in0=tab,
                                    out0=x, out1=q, T=T, n_per_head=N, freqs=freqs), gemm_fl, 2 * big),
        "ygate": (lambda: G.gemm(cur, W, M=M, N=HN, K=D, epi=G.EPI_RELU_GATE, flags=G.F_NO_OUT0, in0=act, out1=q),
                  gemm_fl, 2 * big),
        "gate_bwd": (lambda: G.gemm(cur, W, M=M, N=HN, K=D, epi=G.EPI_GATE_BWD, in0=act, in1=act, out0=x, out1=q),
                     gemm_fl, 4 * big),
        "dq_bwd": (lambda: G.gemm(S, act, M=T, N=N, K=T, b_mn=True, nz=(H, B), a_off=(T, H * T, 0, 0),
                                  b_off=(N, 0, 0, T), c_off=(0, T, N, 0), epi=G.EPI_DQ_BWD,
                                  flags=G.F_ROPE | G.F_TABLE, in0=act, in1=tab, T=T, n_per_head=N, freqs=freqs,
                                  out0=x), att_fl, 3 * big),
        "scores": (lambda: G.gemm(act, act, M=T, N=T, K=N, nz=(H, B), a_off=(0, T, N, 0), b_off=(0, T, N, 0),
                                  c_off=(T, H * T, 0, 0), epi=G.EPI_CAUSAL, causal_tiles=1, out0=S),
                   att_fl / 2, big),
        "decoder": (lambda: G.gemm(act, W, M=M, N=D, K=HN, b_mn=True, out0=cur), gemm_fl, big),
        "wgrad": (lambda: G.gemm(act, cur, M=HN, N=D, K=M, a_mn=True, b_mn=True, flags=G.F_OUT_F32 | G.F_ACCUM,
                                 out0=torch.zeros(HN, D, device="cuda")), gemm_fl, big),
    }
    if case.startswith("dual_"):
        # the chained-GEMM kernels at the base configuration's shapes (8 sequences); bytes = the [M, H*N] tensors
        # each launch has to move once, FLOPs = both GEMMs
        lna, xy, dmlp = _rnd(H * M, D), torch.empty(M, HN, device="cuda", dtype=torch.bfloat16), _rnd(M, D)
        mlp = torch.empty(M, D, device="cuda", dtype=torch.bfloat16)
        dlna = torch.empty(H * M, D, device="cuda", dtype=torch.bfloat16)
        dcur = torch.zeros(M, D, device="cuda")
        W2 = _rnd(HN, D, 0.02)
        ctas = int(os.environ.get("BDH_CASE_CTAS", "0"))       # 0: one CTA per SM
        dual = {
            "dual_fwd": (lambda: DG.dual(lna, W, W2, xy, mlp, M=M, H=H, n_per_head=N, K1=D, N2=D, T=T,
                                         epi=G.EPI_RELU_GATE, a1_b=T, a1_h=M, in0=act, max_ctas=ctas), 2 * gemm_fl, 2 * big),
            "dual_gate_bwd": (lambda: DG.dual(dmlp, W, W2, xy, dlna, M=M, H=H, n_per_head=N, K1=D, N2=D, T=T,
                                              epi=G.EPI_GATE_BWD, group_per_head=True, a1_b=T, a1_h=0, in0=act,
                                              in1=act, out1=q, out_h_stride=M, max_ctas=ctas), 2 * gemm_fl, 4 * big),
            "dual_dq_bwd": (lambda: DG.dual(S, act, W2, xy, dcur, M=M, H=H, n_per_head=N, K1=T, N2=D, T=T,
                                            epi=G.EPI_DQ_BWD, flags=G.F_ROPE | G.F_TABLE, a1_b=H * T, a1_h=T,
                                            b1_mn=True, b1_b=T, in0=act, in1=tab, accumulate=True, max_ctas=ctas),
                            att_fl + gemm_fl, 3 * big),
        }
        return dual[case]
    if case == "ag_gemm":
        # the all-gather -> GEMM kernel with two ranks emulated on one GPU: this launch is "rank 0", its peer's
        # rows live in a second buffer on the same device (the copy path, counters and tile order are the real
        # ones; the link is not). [8192, 1024] x [8192, 1024]^T, ReLU epilogue.
        Mg, Kg, Ng = 8192, 1024, 8192
        full = [_rnd(Mg, Kg, 0.3) for _ in range(2)]
        wg = _rnd(Ng, Kg, 0.05)
        outg = torch.empty(Mg, Ng, device="cuda", dtype=torch.bfloat16)
        arrived = torch.zeros(Mg // 128, device="cuda", dtype=torch.int32)

        def run():
            arrived.zero_()
            G.gemm(full[0], wg, M=Mg, N=Ng, K=Kg, epi=G.EPI_RELU, out0=outg, theta=0.0,
                   gather_ptrs=[t.data_ptr() for t in full], gather_rows=Mg // 2, gather_rank=0, gather_arrived=arrived)
        return run, 2.0 * Mg * Ng * Kg, 2.0 * (Mg * Ng + Mg * Kg + Ng * Kg)
    if case == "decode_state":
        # the decode state update for 64 streams of the base model: fp32 state [64, 4, 8192, 256] = 2.1 GB, half of
        # the query entries zero (their state rows are skipped); bytes = the rows that are read and written
        Bd = 64
        qd = _rnd(Bd, HN, 0.1).relu()
        cd = _rnd(Bd, D)
        rho = torch.zeros(Bd, H, N, D, device="cuda")
        ad = torch.zeros(H * Bd, D, device="cuda")
        live = float((qd != 0).float().mean())
        return (lambda: native.ops.decode_state_update(qd, cd, rho, ad, None)), 4.0 * Bd * HN * D * live, \
            2.0 * 4.0 * Bd * HN * D * live
    if case in ("rownorm_fwd", "fast_attention"):
        # forward_fast attention at T = 2048 (B 8, H 4, N 2048, D 256): scores are 268 MB in bf16
        from burn_dragon_b200.ops import rownorm_attention as RA
        Bf, Tf, Nf = 8, 2048, 2048
        if case == "rownorm_fwd":
            Sc = _rnd(Bf * H * Tf, Tf, 0.1)
            rn = torch.empty(Bf * H * Tf, device="cuda")
            # strictly causal rows: half of the matrix is read and written once
            return (lambda: native.ops.rownorm_fwd(Sc, rn, Tf)), 0.0, 2.0 * Sc.numel()
        qf = (_rnd(Bf * H * Tf, Nf, 0.1).relu().view(Bf, H, Tf, Nf)).requires_grad_(True)
        vf = _rnd(Bf * Tf, D).view(Bf, 1, Tf, D).requires_grad_(True)
        sl = torch.tensor([1.0, 0.5, 0.25, 0.125], device="cuda")
        go = torch.randn(Bf, H, Tf, D, device="cuda", dtype=torch.bfloat16)

        def fwd_bwd():
            qf.grad = vf.grad = None
            RA.attention_rownorm(qf, vf, sl).backward(go)
        # scores + G (causal halves) and the four T x T x N products of dq count as executed FLOPs
        fl = 2.0 * Bf * H * Tf * Tf * (Nf + D) + 2.0 * Bf * H * Tf * Tf * (D + D) + 2.0 * 2.0 * Bf * H * Tf * Tf * Nf
        return fwd_bwd, fl, 0.0
    return cases[case]


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True)
    ap.add_argument("--launches", type=int, default=3)
    ap.add_argument("--time", action="store_true")
    args = ap.parse_args()
    native.load()
    torch.manual_seed(0)
    fn, flops, nbytes = build(args.case)
    for _ in range(args.launches):
        fn()
    torch.cuda.synchronize()
    assert native.status_code() == 0
    if args.time:
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(10)]
        for a, b in evs:
            a.record()
            fn()
            b.record()
        torch.cuda.synchronize()
        ms = sorted(a.elapsed_time(b) for a, b in evs)[5]
        peaks = {}
        p = os.path.join(os.path.dirname(__file__), "..", "MEASURED_PEAKS.json")
        if os.path.exists(p):
            peaks = json.load(open(p))
        hbm, tf = peaks.get("hbm_gbs", 6650.0), peaks.get("bf16_tflops", 1590.0)
        print(json.dumps(dict(case=args.case, ms=ms, gbs=nbytes / ms / 1e6, tflops=flops / ms / 1e9,
                              frac_hbm=nbytes / ms / 1e6 / hbm, frac_tensor=flops / ms / 1e9 / tf,
                              peaks="measured" if peaks else "fallback")))
    else:
        print("ok")
    return 0


if __name__ == "__main__":
    sys.exit(main())

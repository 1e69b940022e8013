"""The allocation-free SSD entry point (`bdh_ssd_chunk_scan_static`), called through its exported C
symbol the way a host application without a device allocator would call it: raw device pointers
for inputs and outputs, no scratch argument. Its results must equal the regular entry point's,
which is handed caller-allocated scratch, on two consecutive calls (the built-in scratch is shared
and keeps the previous call's contents). Collected last so a failure here cannot hide others."""
import ctypes

import pytest
import torch

from burn_dragon_b200 import build as _build

pytestmark = pytest.mark.gpu


def _lib():
    lib = ctypes.CDLL(str(_build.ensure_built()))
    fp, vp, ci = ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int
    lib.bdh_ssd_chunk_scan_static.restype = ci
    lib.bdh_ssd_chunk_scan_static.argtypes = [fp, fp, fp, fp, fp, fp, ci, ci, ci, vp]
    lib.bdh_ssd_chunk_scan.restype = ci
    lib.bdh_ssd_chunk_scan.argtypes = [fp, fp, fp, fp, fp, fp, fp, fp, ci, ci, ci, vp]
    return lib


def _inputs(B, T, H, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    r = lambda *s: torch.randn(*s, device="cuda", generator=g)
    return (r(B, T, H, 64) * 0.5, -torch.rand(B, T, H, device="cuda", generator=g) * 0.2, r(B, T, 128) * 0.3,
            r(B, T, 128) * 0.3, r(B, H, 128, 64))


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def test_static_scratch_entry_matches_regular_entry_twice():
    lib = _lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, (B, T, H) in enumerate([(2, 192, 3), (1, 256, 8)]):
        xw, loga, Bm, Cm, h0 = _inputs(B, T, H, seed=call)
        C = T // 64
        # regular entry point: scratch comes from the caller
        h_ref, y_ref = h0.clone(), torch.empty(B, T, H, 64, device="cuda")
        states = torch.empty(B, C, H, 128, 64, device="cuda")
        decay = torch.empty(B, C, H, device="cuda")
        rc = lib.bdh_ssd_chunk_scan(_p(xw), _p(loga), _p(Bm), _p(Cm), _p(h_ref), _p(states), _p(decay), _p(y_ref),
                                    B, T, H, stream)
        assert rc == 0
        # allocation-free entry point: inputs and outputs only
        h_new, y_new = h0.clone(), torch.full((B, T, H, 64), float("nan"), device="cuda")
        rc = lib.bdh_ssd_chunk_scan_static(_p(xw), _p(loga), _p(Bm), _p(Cm), _p(h_new), _p(y_new), B, T, H, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.allclose(y_new, y_ref, atol=2e-3, rtol=1e-3)
        assert torch.allclose(h_new, h_ref, atol=2e-3, rtol=1e-3)


def test_static_scratch_entry_rejects_oversized_problem():
    lib = _lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    B, T, H = 4, 64 * 33, 4                      # 4 * 33 * 4 = 528 chunk-heads > 512
    xw, loga, Bm, Cm, h0 = _inputs(B, T, H, seed=9)
    y = torch.zeros(B, T, H, 64, device="cuda")
    rc = lib.bdh_ssd_chunk_scan_static(_p(xw), _p(loga), _p(Bm), _p(Cm), _p(h0), _p(y), B, T, H, stream)
    torch.cuda.synchronize()
    assert rc == 7                               # BDH_ERR_TOO_LARGE, nothing launched
    assert float(y.abs().sum()) == 0.0

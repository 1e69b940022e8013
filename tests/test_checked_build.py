"""The bounds-checked build of the extension (`csrc/debug_bounds.cuh`, `python -m burn_dragon_b200.build
--checked`): data-dependent indices are compared with their extents, the first violation is recorded
for the host, nothing traps. The reference has no counterpart (safe Rust; its CI runs clippy,
.github/workflows/clippy.yml:36-37)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _toolkit():
    import shutil
    return shutil.which("nvcc") or os.path.exists("/usr/local/cuda/bin/nvcc")


needs_nvcc = pytest.mark.skipif(not _toolkit(), reason="no CUDA toolkit: the extension cannot be compiled here")


@needs_nvcc
def test_checked_library_builds_and_differs_only_in_the_instrumented_files():
    from burn_dragon_b200 import build
    lib = build.build(checked=True, verbose=False)
    assert lib == build.LIB_CHECKED and lib.exists() and build.is_current(checked=True)
    instrumented = sorted(p.stem for p in build.CSRC.glob("*.cu") if build._instrumented(p))
    assert instrumented == ["graph", "rowwise"]
    for stem in instrumented:
        assert (build.OBJ / f"{stem}.checked.o").exists()
    # the record readers, one library per process (both register `torch.ops.bdh` when loaded): the
    # unchecked library answers zeros; the checked one, which has to synchronise, reports the failed
    # call on a machine without a device instead of crashing
    probe = ("import ctypes, sys, torch\nlib = ctypes.CDLL(sys.argv[1])\nout = (ctypes.c_longlong * 5)(9, 9, 9, 9, 9)\n"
             "rc = lib.bdh_bounds_record_rowwise(out, 0)\nprint('RC', rc, list(out), int(torch.cuda.is_available()))\n")

    def run(path):
        r = subprocess.run([sys.executable, "-c", probe, str(path)], capture_output=True, text=True, timeout=600, cwd=ROOT)
        assert r.returncode == 0, r.stderr[-1500:]
        return r.stdout.strip().splitlines()[-1]
    assert run(build.LIB).startswith("RC 0 [0, 0, 0, 0, 0]")
    line = run(lib)
    assert line.startswith("RC 0 [1, 0, 0, 0, 0]") if line.endswith(" 1") else not line.startswith("RC 0 "), line


@needs_nvcc
def test_checked_library_is_the_one_loaded_on_request():
    code = ("import torch\nfrom burn_dragon_b200.ops import native\nassert native.load()\n"
            "assert hasattr(torch.ops.bdh, 'bounds_records')\n"
            "import re\nmaps = open('/proc/self/maps').read()\n"
            "assert '_C_checked.so' in maps and not re.search(r'/_C\\.so', maps)\nprint('ok')\n")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600, cwd=ROOT,
                       env=dict(os.environ, PYTHONPATH=ROOT, BDH_CHECKED_KERNELS="1"))
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout[-1500:] + r.stderr[-1500:]


_DEVICE_CASE = r"""
import torch
from burn_dragon_b200.ops import native
ops = native.ops
dev = "cuda"
V, D, rows = 64, 128, 32
emb = torch.randn(V, D, device=dev).bfloat16()
cur = torch.empty(rows, D, device=dev, dtype=torch.bfloat16)
tok = torch.randint(0, V, (rows,), device=dev)
ops.embed_ln_fwd(tok, emb, cur)
assert native.bounds_violations() == [], "clean run"
bad = tok.clone(); bad[3] = V + 5
ops.embed_ln_fwd(bad, emb, cur)
v = native.bounds_violations()
assert len(v) == 1 and v[0]["index"] == V + 5 and v[0]["extent"] == V and v[0]["where"] == 3, v
assert "embed_ln_fwd" in v[0]["site"]
# the violating row was clamped exactly as the unchecked kernel clamps it
ok = tok.clone(); ok[3] = V - 1
want = torch.empty_like(cur); ops.embed_ln_fwd(ok, emb, want)
assert torch.equal(cur, want)
assert native.bounds_violations() == [], "the record was cleared"
logits = torch.randn(rows, V, device=dev)
tgt = torch.randint(0, V, (rows,), device=dev); tgt[5] = -100; tgt[7] = 999
loss = torch.empty(rows, device=dev)
ops.cross_entropy(logits, tgt, loss, None, 1.0)
v = native.bounds_violations()
assert len(v) == 1 and v[0]["index"] == 999 and v[0]["where"] == 7 and float(loss[7]) == 0.0 and float(loss[5]) == 0.0, v
assert native.status_code() == 0
print("PASS checked_build")
"""


@pytest.mark.gpu
def test_checked_kernels_record_out_of_range_ids_on_the_device():
    """Out-of-range token / target ids under the checked build: recorded with their row, handled as
    the unchecked kernels handle them (clamped / ignored), no fault. Child process: the checked
    library and the regular one cannot both register `torch.ops.bdh` in one process."""
    r = subprocess.run([sys.executable, "-c", _DEVICE_CASE], capture_output=True, text=True, timeout=600, cwd=ROOT,
                       env=dict(os.environ, PYTHONPATH=ROOT, BDH_CHECKED_KERNELS="1"))
    assert r.returncode == 0 and "PASS checked_build" in r.stdout, r.stdout[-1500:] + r.stderr[-1500:]


def test_host_side_extent_check_of_a_launch():
    """`gemm.check_extents`: the operand / output windows of the last batch index must lie inside
    their tensors (it runs for every launch of the emulated kernel path, so the CPU tests of that path
    also prove the offsets of every launch of a training step, prefill and decode step)."""
    import torch
    from burn_dragon_b200.ops import gemm as G
    H, B, T, Np, D = 2, 3, 64, 128, 32
    q = torch.zeros(B * T, H * Np, dtype=torch.bfloat16)
    S = torch.zeros(B * H * T, T, dtype=torch.bfloat16)
    good = dict(M=T, N=T, K=Np, nz=(H, B), a_off=(0, T, Np, 0), b_off=(0, T, Np, 0), c_off=(T, H * T, 0, 0),
                epi=G.EPI_CAUSAL, out0=S)
    G.check_extents(q, q, **good)
    with pytest.raises(ValueError, match="out0"):
        G.check_extents(q, q, **{**good, "c_off": (T, H * T + 1, 0, 0)})
    with pytest.raises(ValueError, match="window of `a`"):
        G.check_extents(q, q, **{**good, "K": Np + 64})
    with pytest.raises(ValueError, match="negative"):
        G.check_extents(q, q, **{**good, "b_off": (0, -T, Np, 0)})
    with pytest.raises(ValueError, match="needs `out1`"):
        G.check_extents(q, q, M=B * T, N=B * T, K=H * Np, epi=G.EPI_RELU_GATE, in0=q, out0=q)
    # an MN-major operand is indexed [k, mn]
    v = torch.zeros(B * T, D, dtype=torch.bfloat16)
    rho = torch.zeros(B * H * Np, D)
    G.check_extents(q, v, M=Np, N=D, K=T, a_mn=True, b_mn=True, nz=(H, B), a_off=(Np, 0, 0, T), b_off=(0, 0, 0, T),
                    c_off=(Np, H * Np, 0, 0), flags=G.F_OUT_F32, out0=rho)
    with pytest.raises(ValueError, match="window of `b`"):
        G.check_extents(q, v, M=Np, N=D, K=T, a_mn=True, b_mn=True, nz=(H, B), a_off=(Np, 0, 0, T), b_off=(0, 0, 0, T + 1),
                        c_off=(Np, H * Np, 0, 0), flags=G.F_OUT_F32, out0=rho)


def test_guard_words_around_symmetric_buffers():
    """Checked configuration of `parallel.symm.SymmetricBuffer`: guards with a canary pattern on both
    sides of the window every rank (and every peer pointer) addresses; a write past the window is
    found afterwards. The allocator is replaced by host memory here."""
    import torch
    from burn_dragon_b200.parallel import symm

    class HostBuffer(symm.SymmetricBuffer):
        def _allocate(self, numel, dtype, device):
            raw = torch.zeros(numel, dtype=dtype)
            return raw, [raw.data_ptr(), raw.data_ptr() + 4096], 1 << 20, 0, 2

    class Group:
        group_name = "g"

    plain = HostBuffer(100, torch.float32, "cpu", Group(), guard_bytes=0)
    assert plain.raw.numel() == 100 and plain.tensor.data_ptr() == plain.raw.data_ptr()
    assert plain.ptrs[0] == plain.raw.data_ptr() and plain.multicast_ptr == 1 << 20 and plain.check_canaries() == []
    for dtype, numel in ((torch.bfloat16, 101), (torch.float32, 64), (torch.int32, 7)):
        b = HostBuffer(numel, dtype, "cpu", Group(), guard_bytes=256)
        item = b.raw.element_size()
        assert b.tensor.numel() == numel and b.tensor.data_ptr() == b.raw.data_ptr() + 256
        assert b.ptrs == [b.raw.data_ptr() + 256, b.raw.data_ptr() + 4096 + 256] and b.multicast_ptr == (1 << 20) + 256
        assert all(p % 16 == 0 for p in (b.ptrs[0] - b.raw.data_ptr(), b._guards()[1].data_ptr() - b.raw.data_ptr()))
        b.tensor.fill_(3)
        assert b.check_canaries() == [] and symm.check_all_canaries() >= 1
        b.raw[b.raw.numel() - 256 // item] = 1                      # first element past the (padded) window
        bad = b.check_canaries()
        assert len(bad) == 1 and bad[0][:2] == ("above", 0)
        with pytest.raises(RuntimeError, match="guard words overwritten"):
            symm.check_all_canaries()
        b.raw[256 // item - 1] = 1                                  # last element before the window
        assert {x[0] for x in b.check_canaries()} == {"below", "above"}
        del b

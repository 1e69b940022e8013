"""In-tree build of the sm_100a extension (`burn_dragon_b200/_C.so`).

`python -m burn_dragon_b200.build` compiles every `.cu` under `csrc/` with
`nvcc -gencode arch=compute_100a,code=sm_100a`, the torch binding with g++, and links them into
one shared object next to the package. nvcc cross-compiles, so this works on a machine without
a GPU. A content hash of the sources is stored beside the library; `ensure_built()` rebuilds
only when the hash differs, so a prebuilt library copied to another machine is used as is.

`python -m burn_dragon_b200.build --checked` also links `_C_checked.so`: the same sources, with the
files that include `csrc/debug_bounds.cuh` compiled under `-DBDH_DEBUG_BOUNDS` (data-dependent
indices are checked and the first violation is recorded; nothing traps). `BDH_CHECKED_KERNELS=1`
makes `ops.native` load that library instead of `_C.so`.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "_obj"
LIB = PKG / "_C.so"
HOST_LIB = PKG / "_host.so"
HOST_SRC = CSRC / "host"
STAMP = PKG / "_C.hash"
LIB_CHECKED = PKG / "_C_checked.so"
STAMP_CHECKED = PKG / "_C_checked.hash"
CHECK_FLAG = "-DBDH_DEBUG_BOUNDS"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def _sources():
    cu = sorted(CSRC.glob("*.cu"))
    cpp = sorted(CSRC.glob("*.cpp"))
    hdr = sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")))
    return cu, cpp, hdr


def source_hash() -> str:
    cu, cpp, hdr = _sources()
    h = hashlib.sha256()
    for p in cu + cpp + hdr + sorted(HOST_SRC.glob("*.cpp")):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_current(checked: bool = False) -> bool:
    if checked:
        return (LIB_CHECKED.exists() and STAMP_CHECKED.exists()
                and STAMP_CHECKED.read_text().strip() == source_hash())
    return (LIB.exists() and HOST_LIB.exists() and STAMP.exists()
            and STAMP.read_text().strip() == source_hash())


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; cannot build the sm_100a extension")
    return cand


def _run(cmd, log: Path):
    r = subprocess.run(cmd, capture_output=True, text=True)
    log.write_text(" ".join(map(str, cmd)) + "\n" + r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"build step failed: {' '.join(map(str, cmd))}\n{r.stdout}\n{r.stderr}")
    return r


def _instrumented(src: Path) -> bool:
    """Does this source compile differently under the checked build?"""
    text = src.read_text()
    return "debug_bounds.cuh" in text or "BDH_DEBUG_BOUNDS" in text


def build(force: bool = False, verbose: bool = True, checked: bool = False) -> Path:
    """Compile and link the extension. Returns the path of the shared object. `checked` links the
    bounds-checked variant: the regular objects, except that the instrumented sources are compiled
    again with the check flag."""
    if checked:
        build(force=force, verbose=verbose)           # the regular objects are reused
    if not force and is_current(checked):
        return LIB_CHECKED if checked else LIB
    import torch
    from torch.utils import cpp_extension as ce

    OBJ.mkdir(exist_ok=True)
    cu, cpp, _ = _sources()
    inc = [f"-I{p}" for p in ce.include_paths("cuda")] + [f"-I{sysconfig.get_paths()['include']}", f"-I{CSRC}"]
    abi = f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"
    nvcc = _nvcc()
    jobs, objects = [], []
    for src in cu:
        again = checked and _instrumented(src)
        obj = OBJ / (src.stem + (".checked.o" if again else ".o"))
        objects.append(obj)
        if checked and not again:
            continue
        jobs.append(([nvcc, *NVCC_FLAGS, *([CHECK_FLAG] if again else []), f"-I{CSRC}", "-I/usr/local/cuda/include",
                      "-c", str(src), "-o", str(obj)], OBJ / (obj.stem + ".log")))
    for src in cpp:
        obj = OBJ / (src.stem + ".o")
        objects.append(obj)
        if checked:
            continue
        jobs.append((["g++", "-O2", "-std=c++17", "-fPIC", abi, "-DTORCH_API_INCLUDE_EXTENSION_H", *inc, "-c", str(src),
                      "-o", str(obj)], OBJ / (src.stem + ".log")))
    with cf.ThreadPoolExecutor(max_workers=max(1, min(8, len(jobs)))) as ex:
        futs = [ex.submit(_run, cmd, log) for cmd, log in jobs]
        for f in futs:
            f.result()
    tlib = Path(torch.__file__).parent / "lib"
    cuda_lib = Path("/usr/local/cuda/lib64")
    lib = LIB_CHECKED if checked else LIB
    link = ["g++", "-shared", "-o", str(lib), *[str(o) for o in objects], f"-L{tlib}", f"-L{cuda_lib}",
            "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-lcudart",
            f"-Wl,-rpath,{tlib}", f"-Wl,-rpath,{cuda_lib}"]
    _run(link, OBJ / ("link_checked.log" if checked else "link.log"))
    if checked:
        STAMP_CHECKED.write_text(source_hash())
    else:
        # host-only helpers: plain C ABI, no torch / CUDA dependency
        _run(["g++", "-O3", "-std=c++17", "-fPIC", "-shared", "-pthread", "-o", str(HOST_LIB),
              *[str(p) for p in sorted(HOST_SRC.glob("*.cpp"))]], OBJ / "host.log")
        STAMP.write_text(source_hash())
    if verbose:
        print(f"built {lib}")
    return lib


def ensure_built(checked: bool = False) -> Path:
    return build(force=False, verbose=False, checked=checked)


def ptxas_report() -> str:
    """Registers / spills per kernel, from the logs of the last build."""
    out = []
    for log in sorted(OBJ.glob("*.log")):
        for line in log.read_text().splitlines():
            if "Compiling entry" in line or "registers" in line or "spill" in line:
                out.append(f"{log.stem}: {line.strip()}")
    return "\n".join(out)


if __name__ == "__main__":
    build(force="--force" in sys.argv, checked="--checked" in sys.argv)
    if "--ptxas" in sys.argv:
        print(ptxas_report())

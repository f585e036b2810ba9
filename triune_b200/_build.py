"""In-tree build of the native code.

Two artefacts are produced next to the Python sources so they travel with the tree:

* ``triune_b200/_C.so``            torch extension with every sm_100a kernel (nvcc, ``-gencode
                                   arch=compute_100a,code=sm_100a``) and its bindings;
* ``triune_b200/libtriune_core.so`` C-ABI engine library (arena, CUDA-graph lifecycle, pinned staging ring,
                                   CPU fast paths) loadable through ``ctypes`` or from other languages.

The build is incremental (mtime based) and needs no GPU: nvcc cross-compiles.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = CSRC / "_obj"
EXT_SO = PKG / "_C.so"
CORE_SO = PKG / "libtriune_core.so"
NOALLOC_SO = PKG / "libtriune_noalloc.so"

NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _cuda_home() -> str:
    for c in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if c and Path(c, "bin", "nvcc").exists():
            return c
    nv = shutil.which("nvcc")
    if nv:
        return str(Path(nv).resolve().parent.parent)
    raise RuntimeError("nvcc not found; set CUDA_HOME")


def _torch_flags():
    import torch
    from torch.utils import cpp_extension as ce

    inc = [f"-I{p}" for p in ce.include_paths()] + [f"-I{sysconfig.get_paths()['include']}"]
    abi = int(torch.compiled_with_cxx11_abi())
    defs = [f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H"]
    libdir = str(Path(torch.__file__).parent / "lib")
    return inc, defs, libdir


def _newest_header_mtime() -> float:
    m = 0.0
    for ext in ("*.cuh", "*.h", "*.hpp"):
        for p in CSRC.rglob(ext):
            m = max(m, p.stat().st_mtime)
    return m


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"command failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    if verbose and (r.stdout.strip() or r.stderr.strip()):
        print(r.stdout, r.stderr, flush=True)
    return r


def build_extension(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    cuda = _cuda_home()
    nvcc = str(Path(cuda, "bin", "nvcc"))
    inc, defs, torch_lib = _torch_flags()
    OBJ.mkdir(parents=True, exist_ok=True)
    hdr_m = _newest_header_mtime()
    sources = sorted(p for p in CSRC.rglob("*.cu") if "engine" not in p.parts and p.name != "gla_noalloc.cu") + sorted(
        p for p in CSRC.rglob("*.cpp") if "engine" not in p.parts
    )
    jobs = []
    objs = []
    for src in sources:
        obj = OBJ / (src.relative_to(CSRC).as_posix().replace("/", "__") + ".o")
        objs.append(obj)
        stale = force or (not obj.exists()) or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_m)
        if not stale:
            continue
        if src.suffix == ".cu":
            cmd = (
                [nvcc, "-c", str(src), "-o", str(obj)]
                + NVCC_ARCH
                + ["-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr", "--use_fast_math"]
                + ["-Xcompiler", "-fPIC", f"-I{cuda}/include", f"-I{CSRC}"]
            )
            if ptxas_info:
                cmd += ["-Xptxas", "-v"]
        else:
            cmd = (
                ["g++", "-c", str(src), "-o", str(obj), "-O2", "-std=c++17", "-fPIC", "-w"]
                + inc
                + defs
                + [f"-I{cuda}/include", f"-I{CSRC}"]
            )
        jobs.append(cmd)
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            results = list(ex.map(lambda c: _run(c, verbose), jobs))
        if ptxas_info:
            for r in results:
                if r.stderr.strip():
                    print(r.stderr)
    need_link = force or jobs or not EXT_SO.exists() or any(o.stat().st_mtime > EXT_SO.stat().st_mtime for o in objs)
    if need_link:
        cmd = (
            ["g++", "-shared", "-o", str(EXT_SO)]
            + [str(o) for o in objs]
            + [f"-L{torch_lib}", "-lc10", "-ltorch", "-ltorch_cpu", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda"]
            + [f"-L{cuda}/lib64", "-lcudart", f"-Wl,-rpath,{torch_lib}", f"-Wl,-rpath,{cuda}/lib64"]
        )
        _run(cmd, verbose)
    return EXT_SO


def build_core(force: bool = False, verbose: bool = False) -> Path:
    """C-ABI engine library: plain C++ plus one small .cu, no torch dependency."""
    cuda = _cuda_home()
    nvcc = str(Path(cuda, "bin", "nvcc"))
    eng = CSRC / "engine"
    sources = sorted(eng.glob("*.cpp")) + sorted(eng.glob("*.cu"))
    if not sources:
        return CORE_SO
    newest = max([p.stat().st_mtime for p in sources] + [p.stat().st_mtime for p in eng.glob("*.h")])
    if not force and CORE_SO.exists() and CORE_SO.stat().st_mtime >= newest:
        return CORE_SO
    cmd = (
        [nvcc, "-shared", "-o", str(CORE_SO)]
        + [str(s) for s in sources]
        + NVCC_ARCH
        + ["-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC,-mavx2,-mfma,-fopenmp", f"-I{eng}", f"-I{CSRC}"]
        + ["-lcudart", "-lgomp", "-ldl"]
    )
    _run(cmd, verbose)
    return CORE_SO


def build_noalloc(force: bool = False, verbose: bool = False) -> Path:
    """Allocation-free C entry point over the GLA kernels (no torch dependency; loadable with ctypes)."""
    cuda = _cuda_home()
    nvcc = str(Path(cuda, "bin", "nvcc"))
    srcs = [CSRC / "gla" / "gla_noalloc.cu", CSRC / "gla" / "gla_kernels.cu"]
    deps = srcs + [CSRC / "gla" / "gla_noalloc.h", CSRC / "gla" / "gla.cuh", CSRC / "common" / "ptx.cuh",
                   CSRC / "common" / "tma_desc.h", CSRC / "common" / "per_device.h", CSRC / "gla" / "gla_tiles.cuh"]
    newest = max(p.stat().st_mtime for p in deps)
    if not force and NOALLOC_SO.exists() and NOALLOC_SO.stat().st_mtime >= newest:
        return NOALLOC_SO
    cmd = ([nvcc, "-shared", "-o", str(NOALLOC_SO)] + [str(s) for s in srcs] + NVCC_ARCH
           + ["-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr", "--use_fast_math", "-Xcompiler", "-fPIC",
              f"-I{CSRC}", "-lcudart"])
    _run(cmd, verbose)
    return NOALLOC_SO


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_extension(force=force, verbose=verbose)
    build_core(force=force, verbose=verbose)
    build_noalloc(force=force, verbose=verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print("built", EXT_SO, CORE_SO if CORE_SO.exists() else "")

"""Build the C-ABI shared library with nvcc, in-tree.

    python -m latentserve_b200.build          # -> latentserve_b200/_C/libls_b200.so

One `nvcc -shared` over the `.cu` files in `csrc/`, for sm_100a only. No GPU is
needed to build (nvcc cross-compiles). The library is rebuilt when any source
is newer than it. The reference compiles its kernels at run time with NVRTC
through CuPy (kernels/cuda/paged_decode_cuda.py:77-102); here the build is an
explicit, ahead-of-time step so that the `.so` can be loaded by anything that
speaks the C ABI.
"""

from __future__ import annotations

import os
import pathlib
import shutil
import subprocess
import sys

HERE = pathlib.Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OUT_DIR = HERE / "_C"
LIB = OUT_DIR / "libls_b200.so"
SOURCES = ("paged_decode.cu", "kv_write.cu", "page_select.cu", "fused_elementwise.cu",
           "skinny_gemm.cu")
ARCH_FLAGS = ("-gencode", "arch=compute_100a,code=sm_100a")


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the library is CUDA-only and has no other build")


def sources() -> list[pathlib.Path]:
    return [CSRC / s for s in SOURCES if (CSRC / s).exists()]


def needs_build() -> bool:
    if not LIB.exists():
        return True
    built = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh"))
    return any(p.stat().st_mtime > built for p in deps)


def build(force: bool = False, verbose: bool = False, ptxas_verbose: bool = False) -> pathlib.Path:
    if not force and not needs_build():
        return LIB
    OUT_DIR.mkdir(exist_ok=True)
    cmd = [nvcc_path(), "-shared", "-Xcompiler", "-fPIC", "-O3", "-std=c++17", "-lineinfo",
           *ARCH_FLAGS, "-I", str(CSRC)]
    if ptxas_verbose:
        cmd += ["-Xptxas", "-v"]
    # Developer knobs for measurement builds: LS_NVCC_EXTRA adds compiler flags (e.g.
    # '-DLS_LOADS_ONLY': the decode kernels' pages land and nothing is computed -- the
    # ceiling of their access pattern), LS_LIB_OUT writes the result elsewhere, to be
    # loaded through LATENTSERVE_B200_LIB instead of the product library.
    cmd += os.environ.get("LS_NVCC_EXTRA", "").split()
    out = os.environ.get("LS_LIB_OUT") or str(LIB)
    cmd += [str(s) for s in sources()] + ["-o", out]
    if verbose:
        print(" ".join(cmd), file=sys.stderr)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed ({res.returncode}):\n{res.stdout}\n{res.stderr}")
    if verbose or ptxas_verbose:
        sys.stderr.write(res.stdout + res.stderr)
    return pathlib.Path(out)


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose=True, ptxas_verbose="--ptxas" in sys.argv)
    print(path)

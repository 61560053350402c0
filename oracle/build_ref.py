"""Compile the reference's own CUDA decode kernels for sm_100a, from the sources
where they lie in a LatentServe checkout, into `oracle/_ref/` (git-ignored).

    python oracle/build_ref.py [/path/to/LatentServe]

Test / measurement infrastructure only: `bench.py` times the resulting kernel on
the same GPU, beside this library's, as "the reference's kernel on this box".
Nothing of the product loads it. No reference source is copied: nvcc reads the
`.cu` files in place, with the defines the reference passes to NVRTC
(kernels/cuda/paged_decode_cuda.py:84-110: HEAD_DIM, NREP, PAGE, TOKG, ASYM,
HAS_RES, MIN_BLOCKS).
"""

from __future__ import annotations

import os
import pathlib
import shutil
import subprocess
import sys
from typing import Optional

HERE = pathlib.Path(__file__).resolve().parent
OUT = HERE / "_ref"
# (output name, source under kernels/cuda, extra defines)
TARGETS = (
    ("paged_decode_fp16.cubin", "paged_decode_fp16.cu", ()),
    ("paged_decode_int8.cubin", "paged_decode_int8.cu", ("-DASYM=0", "-DHAS_RES=1", "-DMIN_BLOCKS=12")),
    # page_bounds_update, page_index, page_index_heads and paged_sparse_fp16 in one module
    # (kernels/cuda/paged_sparse.py:43-57 passes PAGES_PER_WARP = 16)
    ("paged_sparse_fp16.cubin", "paged_sparse_fp16.cu", ("-DPAGES_PER_WARP=16",)),
)
COMMON = ("-DHEAD_DIM=128", "-DNREP=6", "-DPAGE=16", "-DTOKG=4")


def reference_checkout() -> Optional[pathlib.Path]:
    """A LatentServe source checkout, if one is at hand: the directory
    `LATENTSERVE_REFERENCE` names, else a `reference` directory beside this
    repository. None when neither holds the kernel sources."""
    for cand in (os.environ.get("LATENTSERVE_REFERENCE"), HERE.parent.parent / "reference"):
        if cand and (pathlib.Path(cand) / "kernels" / "cuda" / "paged_decode_fp16.cu").is_file():
            return pathlib.Path(cand)
    return None


def build(reference_root=None) -> list[pathlib.Path]:
    root = pathlib.Path(reference_root) if reference_root else reference_checkout()
    if root is None:
        raise FileNotFoundError("no LatentServe checkout: set LATENTSERVE_REFERENCE")
    src_dir = root / "kernels" / "cuda"
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not src_dir.is_dir():
        raise FileNotFoundError(f"no LatentServe checkout at {root}")
    OUT.mkdir(exist_ok=True)
    built = []
    for name, src, extra in TARGETS:
        out = OUT / name
        cmd = [nvcc, "-cubin", "-arch=sm_100a", "-O3", "-std=c++17", *COMMON, *extra, str(src_dir / src),
               "-o", str(out)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{res.stderr}")
        built.append(out)
    return built


if __name__ == "__main__":
    for path in build(*sys.argv[1:2]):
        print(path)

"""Install a LatentServe checkout, unmodified, into `baseline/_ref/` (git-ignored).

    python baseline/install_reference.py [/path/to/LatentServe]

`tests/test_gpu_dropin.py` imports the installed tree on the GPU machine and
drives this library through the reference's own model, caches and graph runner
(`dropin.install()` patches its kernel modules in place). Nothing of the product
imports it. The checkout is copied to a temporary directory first because a
build writes into its source tree, and dependencies are left alone: the tests
need torch and transformers only, which the environment has.
"""

from __future__ import annotations

import pathlib
import shutil
import subprocess
import sys
import tempfile

HERE = pathlib.Path(__file__).resolve().parent
OUT = HERE / "_ref"
sys.path.insert(0, str(HERE.parent))


def install(reference_root=None) -> pathlib.Path:
    from oracle.build_ref import reference_checkout

    root = pathlib.Path(reference_root) if reference_root else reference_checkout()
    if root is None:
        raise FileNotFoundError("no LatentServe checkout: set LATENTSERVE_REFERENCE")
    with tempfile.TemporaryDirectory() as tmp:
        src = pathlib.Path(tmp) / "latentserve"
        shutil.copytree(root, src, ignore=shutil.ignore_patterns(".git", "results", "notebooks", "docs"))
        if OUT.exists():
            shutil.rmtree(OUT)
        cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
               "--quiet", "--target", str(OUT), str(src)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"pip install failed:\n{res.stdout}\n{res.stderr}")
    return OUT


if __name__ == "__main__":
    print(install(*sys.argv[1:2]))

"""The C-ABI library builds, loads, and exports every symbol the header declares.
No kernel is launched here (no GPU in this test tier)."""

import ctypes
import pathlib
import re

from latentserve_b200 import _lib, build

ROOT = pathlib.Path(__file__).resolve().parents[1]


def _declared():
    text = (ROOT / "include" / "latentserve_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\bint\s+(ls_\w+)\s*\(", text)))


def test_library_builds_for_sm100a_only():
    path = build.build()
    assert path.exists() and path.suffix == ".so"
    assert "arch=compute_100a,code=sm_100a" in " ".join(build.ARCH_FLAGS)


def test_every_declared_symbol_is_exported_and_prototyped():
    declared = _declared()
    assert len(declared) >= 11
    handle = ctypes.CDLL(str(build.build()))
    for name in declared:
        assert hasattr(handle, name), f"{name} declared in the header but not exported"
    assert declared == _lib.exported_symbols(), "ctypes prototypes and header disagree"


def test_prototype_arity_matches_the_header():
    text = (ROOT / "include" / "latentserve_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    for name, args in re.findall(r"\bint\s+(ls_\w+)\s*\(([^;]*?)\)\s*;", text, flags=re.S):
        n = len([a for a in args.split(",") if a.strip()])
        assert n == len(_lib._PROTOTYPES[name]), f"{name}: header has {n} parameters"


def test_argument_validation_needs_no_gpu():
    lib = _lib.lib()
    assert lib.ls_decode_slots(16, 148) == 164
    # Null tensors are rejected before anything touches a device.
    rc = lib.ls_combine(0, 0, 0, 0, 0, 1, 2, 6, 0, 0, 0, 0)
    assert rc == -1
    rc = lib.ls_topk_pages(0, 0, 1, 2, 64, 8, 0, 0, 0, 0, 0)
    assert rc == -1

"""The drop-in installer against an importable LatentServe tree. Skipped where
no such tree is on the path (the library itself never needs one)."""

import importlib
import os
import pathlib
import sys

import pytest
import torch

from oracle.build_ref import reference_checkout

# A source checkout if one is at hand, else the copy installed under baseline/_ref.
REF = str(reference_checkout() or pathlib.Path(__file__).resolve().parents[1] / "baseline" / "_ref")
have_reference = os.path.isdir(os.path.join(REF, "kernels", "cuda"))
pytestmark = pytest.mark.skipif(not have_reference, reason="no LatentServe tree to install into")


@pytest.fixture()
def reference_on_path():
    sys.path.insert(0, REF)
    sys.dont_write_bytecode = True
    try:
        yield
    finally:
        from latentserve_b200 import dropin

        dropin.uninstall()
        sys.path.remove(REF)


def test_install_replaces_and_uninstall_restores(reference_on_path):
    from latentserve_b200 import dropin, int8_write, paged_decode_cuda, paged_sparse

    pdc = importlib.import_module("kernels.cuda.paged_decode_cuda")
    rps = importlib.import_module("kernels.cuda.paged_sparse")
    riw = importlib.import_module("kernels.cuda.int8_write")
    rpd = importlib.import_module("kernels.gqa.paged_decode")
    original = (pdc.paged_decode_cuda, rps.sparse_attention, riw.decode_write, rpd.decode_backend())
    names = dropin.install()
    assert "kernels.cuda.paged_decode_cuda.paged_decode_cuda" in names
    assert pdc.paged_decode_cuda is paged_decode_cuda.paged_decode_cuda
    assert pdc.eligible is paged_decode_cuda.eligible
    assert rps.sparse_attention is paged_sparse.sparse_attention and rps.select is paged_sparse.select
    assert riw.decode_write is int8_write.decode_write
    assert rpd.decode_backend() == "cuda"
    dropin.uninstall()
    assert (pdc.paged_decode_cuda, rps.sparse_attention, riw.decode_write,
            rpd.decode_backend()) == original


def test_reference_cpu_route_is_untouched_after_install(reference_on_path):
    """CPU tensors never reach this library: the reference's dispatcher keeps
    serving them from its own torch reference, with the same result."""
    from latentserve_b200 import dropin, synthetic

    rpd = importlib.import_module("kernels.gqa.paged_decode")
    case = synthetic.dense_case([130, 48], seed=2)
    t = {k: torch.from_numpy(v) for k, v in case.items()}
    before = rpd.paged_decode_attention(t["q"].float(), t["k_pool"], t["v_pool"], t["block_tables"],
                                        t["seq_lens"])
    dropin.install()
    after = rpd.paged_decode_attention(t["q"].float(), t["k_pool"], t["v_pool"], t["block_tables"],
                                       t["seq_lens"])
    assert torch.equal(before, after)


def test_signatures_match_the_reference(reference_on_path):
    import inspect

    from latentserve_b200 import int8_write, paged_decode, paged_decode_cuda, paged_sparse

    pairs = [("kernels.cuda.paged_decode_cuda", paged_decode_cuda, ["eligible", "paged_decode_cuda",
                                                                    "choose_splits"]),
             ("kernels.cuda.paged_sparse", paged_sparse, ["budget", "budgets", "rebuild_bounds",
                                                          "update_bounds", "page_scores",
                                                          "page_scores_mass", "select", "sparse_decode",
                                                          "sparse_attention"]),
             ("kernels.cuda.int8_write", int8_write, ["eligible", "decode_write"]),
             ("kernels.gqa.paged_decode", paged_decode, ["set_decode_backend", "decode_backend",
                                                         "paged_decode_attention"])]
    for mod_name, mine, names in pairs:
        ref = importlib.import_module(mod_name)
        for name in names:
            want = list(inspect.signature(getattr(ref, name)).parameters)
            got = list(inspect.signature(getattr(mine, name)).parameters)
            assert got[:len(want)] == want, f"{mod_name}.{name}: {got} vs {want}"

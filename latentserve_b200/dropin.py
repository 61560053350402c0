"""Install this library's kernels behind an importable LatentServe tree.

    import latentserve_b200.dropin as dropin
    dropin.install()          # reference on sys.path (its root is the import root)

After `install()`, the reference's own host code — `GQAAttention.forward`
(model/attention/gqa.py:283-344), `PagedKVCache.write/_update_bounds`
(cache/paged_cache.py:398-461), `Int8PagedKVCache.write`
(cache/int8_paged_cache.py:722-736), `ServingEngine` and `runtime/cuda_graph.py`
— reaches the sm_100a kernels through the module attributes it already looks
up at call time:

    kernels.cuda.paged_decode_cuda : eligible, paged_decode_cuda, choose_splits
    kernels.cuda.paged_sparse      : budget, budgets, rebuild_bounds, update_bounds, page_scores,
                                     page_scores_mass, select, sparse_decode, sparse_attention
    kernels.cuda.int8_write        : eligible, decode_write, ENABLED
    kernels.gqa.paged_decode       : decode backend set to "cuda"

Nothing of the reference is copied or edited; `uninstall()` restores every
attribute. The reference's CPU route (`paged_decode_reference`) is untouched:
it belongs to the reference, and CPU tensors never reach this library
(`eligible` is False for them).
"""

from __future__ import annotations

import importlib

from latentserve_b200 import int8_write, paged_decode_cuda, paged_sparse

_PATCHES = {
    "kernels.cuda.paged_decode_cuda": (paged_decode_cuda, ("eligible", "paged_decode_cuda",
                                                           "choose_splits")),
    "kernels.cuda.paged_sparse": (paged_sparse, ("budget", "budgets", "rebuild_bounds",
                                                 "update_bounds", "page_scores", "page_scores_mass",
                                                 "select", "sparse_decode", "sparse_attention")),
    "kernels.cuda.int8_write": (int8_write, ("eligible", "decode_write")),
}
_SAVED: dict = {}


def install(set_backend: bool = True) -> list[str]:
    """Patch the reference modules in place; returns the names replaced."""
    done = []
    for mod_name, (source, names) in _PATCHES.items():
        target = importlib.import_module(mod_name)
        for name in names:
            _SAVED.setdefault((mod_name, name), getattr(target, name))
            setattr(target, name, getattr(source, name))
            done.append(f"{mod_name}.{name}")
    if set_backend:
        pd = importlib.import_module("kernels.gqa.paged_decode")
        _SAVED.setdefault(("kernels.gqa.paged_decode", "_backend"), pd.decode_backend())
        pd.set_decode_backend("cuda")
    return done


def uninstall() -> None:
    for (mod_name, name), value in list(_SAVED.items()):
        target = importlib.import_module(mod_name)
        if name == "_backend":
            target.set_decode_backend(value)
        else:
            setattr(target, name, value)
    _SAVED.clear()

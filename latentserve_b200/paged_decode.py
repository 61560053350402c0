"""Entry point of the decode-attention path.

Mirrors the reference dispatcher `kernels/gqa/paged_decode.py`
(`set_decode_backend` :491-494, `decode_backend` :497-498,
`paged_decode_attention` :709-829) with one backend: the sm_100a kernels of
this library. There is no Triton backend and no CPU path here; a CPU tensor,
`force_reference=True`, or an ineligible layout raises instead of quietly
running something else.
"""

from __future__ import annotations

from typing import Optional

import torch

from latentserve_b200 import _lib
from latentserve_b200 import paged_decode_cuda as pdc

_BACKEND = {"decode": "cuda"}


def set_decode_backend(name: str) -> None:
    if name != "cuda":
        raise ValueError(f"unknown decode backend {name!r}: this library has only 'cuda'")
    _BACKEND["decode"] = name


def decode_backend() -> str:
    return _BACKEND["decode"]


def paged_decode_attention(
    q: torch.Tensor,
    k_pool: torch.Tensor,
    v_pool: torch.Tensor,
    block_tables: torch.Tensor,
    seq_lens: torch.Tensor,
    k_scale: Optional[torch.Tensor] = None,
    v_scale: Optional[torch.Tensor] = None,
    k_zero: Optional[torch.Tensor] = None,
    v_zero: Optional[torch.Tensor] = None,
    num_splits: Optional[int] = None,
    softmax_scale: Optional[float] = None,
    max_seq_len: Optional[int] = None,
    force_reference: bool = False,
    k_residual: Optional[torch.Tensor] = None,
    res_rows: Optional[torch.Tensor] = None,
    pages_per_iter: Optional[int] = None,
    num_warps: Optional[int] = None,
    num_stages: Optional[int] = None,
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """q [B, H_kv, N_REP, D]; pools [num_blocks, PAGE, H_kv, D]; block_tables
    [B, max_pages] int32; seq_lens [B] int32 -> [B, H_kv, N_REP, D].

    `num_splits` is ignored, as the reference's "cuda" backend ignores it
    (kernels/gqa/paged_decode.py:750-762); `pages_per_iter`, `num_warps` and
    `num_stages` tuned the reference's Triton kernels and have no meaning here.
    `out` (not in the reference's signature) makes the kernel write the result
    there instead of into the library's persistent scratch.
    """
    if force_reference:
        raise RuntimeError("latentserve_b200 carries no reference implementation to force")
    # A cache in fused-append mode has left this layer's new K / V rows here instead of
    # launching its append: they ride on the attention launch.
    k_new = v_new = None
    if _PENDING_APPENDS:
        pending = _PENDING_APPENDS.pop(k_pool.data_ptr(), None)
        if pending is not None:
            k_new, v_new = pending
    # A decode loop makes the same call every step (persistent pools, tables,
    # lengths, projection buffers), so a validated call is remembered by the
    # addresses and layouts of its tensors and repeated as one library call.
    key = (q.data_ptr(), q.shape, q.stride(), q.dtype,
           k_pool.data_ptr(), k_pool.shape, k_pool.stride(), k_pool.dtype,
           v_pool.data_ptr(), v_pool.stride(),
           block_tables.data_ptr(), block_tables.shape, block_tables.stride(), block_tables.dtype,
           seq_lens.data_ptr(), seq_lens.shape, seq_lens.dtype, softmax_scale, pdc.dense_launch_flags(),
           pdc.int8_loader_flags(),
           _ident(k_scale), _ident(v_scale), _ident(k_zero), _ident(v_zero), _ident(k_residual),
           _ident(res_rows), _ident(out), _ident(k_new), _ident(v_new))
    plan = _PLANS.get(key)
    if plan is None:
        if not q.is_cuda:
            raise RuntimeError("latentserve_b200 has no CPU path: tensors must be on a CUDA device")
        if not pdc.eligible(q, k_pool, k_scale, k_residual, v_scale=v_scale, k_zero=k_zero,
                            v_zero=v_zero, res_rows=res_rows):
            raise ValueError(
                "layout not supported by the sm_100a kernels: need fp16 q with head_dim 128, <= 8 query "
                "rows per KV head, page 16, fp16 or INT8 pools with 16-byte aligned rows")
        plan = pdc.plan_decode(q, k_pool, v_pool, block_tables, seq_lens, softmax_scale=softmax_scale,
                               k_scale=k_scale, v_scale=v_scale, k_zero=k_zero, v_zero=v_zero,
                               k_residual=k_residual, res_rows=res_rows, out=out, k_new=k_new, v_new=v_new)
        if len(_PLANS) >= _PLAN_LIMIT:
            _PLANS.clear()
        _PLANS[key] = plan
    fn, args, out, dev_index = plan
    _lib.check(fn(*args, _lib.raw_stream(dev_index)), "paged_decode_attention")
    return out


_PLANS: dict = {}
_PLAN_LIMIT = 4096
# k_pool address -> (k_new, v_new) of a cache.write() whose append was left to the next
# attention call on that pool (PagedKVCache.enable_fused_append).
_PENDING_APPENDS: dict = {}


def defer_append(k_pool: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor) -> None:
    _PENDING_APPENDS[k_pool.data_ptr()] = (k_new, v_new)


def take_pending_append(k_pool: torch.Tensor):
    """The rows left for `k_pool` by `defer_append`, if no attention call took them."""
    return _PENDING_APPENDS.pop(k_pool.data_ptr(), None)


def _ident(t: Optional[torch.Tensor]):
    return None if t is None else (t.data_ptr(), t.shape, t.stride(), t.dtype)

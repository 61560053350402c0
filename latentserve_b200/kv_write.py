"""Decode-step KV append for the fp16 paged cache — host side.

`append_fp16` is what `PagedKVCache.write()` does for one new token per
sequence (cache/paged_cache.py:398-417 in the reference: two `index_copy_`
scatters, then `page_bounds_update` when page bounds are on) as one launch.
`update_bounds_only` is the reference's stand-alone `update_bounds`
(kernels/cuda/paged_sparse.py:88-101).
"""

from __future__ import annotations

from typing import Optional

import torch

from latentserve_b200 import _lib


def _rows(t: torch.Tensor) -> torch.Tensor:
    """[B, H, 1, D] or [B, H, D] -> a [B, H, D] view (no copy)."""
    if t.dim() == 4:
        if t.shape[2] != 1:
            raise ValueError("the append kernels take one token per sequence")
        t = t[:, :, 0]
    if t.dim() != 3 or t.stride(-1) != 1:
        raise ValueError("K/V rows must be [B, H, D] with unit-stride channels")
    return t


def append_fp16(k: torch.Tensor, v: torch.Tensor, slots: torch.Tensor, flat_k: torch.Tensor,
                flat_v: torch.Tensor, kmin: Optional[torch.Tensor] = None,
                kmax: Optional[torch.Tensor] = None, page: int = 16) -> None:
    """k, v [B, H, 1, D] fp16 (views of the projection output are fine);
    slots [B] int64 flat token slots; flat_k / flat_v [num_blocks * page, H, D];
    kmin / kmax [num_blocks, H, D] or None."""
    if not k.is_cuda:
        raise RuntimeError("latentserve_b200 has no CPU path: tensors must be on a CUDA device")
    kr, vr = _rows(k), _rows(v)
    b, h, d = kr.shape
    if slots.dtype != torch.int64 or slots.numel() < b or (slots.numel() > 1 and slots.stride(-1) != 1):
        raise ValueError("slots must be a contiguous int64 vector with one entry per sequence")
    if flat_k.stride() != flat_v.stride() or flat_k.stride(-1) != 1:
        raise ValueError("K and V pools must share one layout with unit-stride channels")
    sb = (kmin.stride(0), kmin.stride(1)) if kmin is not None else (0, 0)
    rc = _lib.lib().ls_kv_append_fp16(
        kr.data_ptr(), vr.data_ptr(), slots.data_ptr(), flat_k.data_ptr(), flat_v.data_ptr(),
        _lib.ptr(kmin), _lib.ptr(kmax), b, h, d, page, flat_k.shape[0],
        kr.stride(0), kr.stride(1), vr.stride(0), vr.stride(1),
        flat_k.stride(0), flat_k.stride(1), sb[0], sb[1], _lib.current_stream(k.device))
    _lib.check(rc, "append_fp16")


def update_bounds_only(k_new: torch.Tensor, slots: torch.Tensor, kmin: torch.Tensor,
                       kmax: torch.Tensor, page: int = 16) -> None:
    """Page bounds for rows that something else already scattered."""
    kr = _rows(k_new)
    b, h, d = kr.shape
    rc = _lib.lib().ls_kv_append_fp16(
        kr.data_ptr(), 0, slots.data_ptr(), 0, 0, kmin.data_ptr(), kmax.data_ptr(),
        b, h, d, page, kmin.shape[0] * page,
        kr.stride(0), kr.stride(1), 0, 0, 0, 0, kmin.stride(0), kmin.stride(1),
        _lib.current_stream(kr.device))
    _lib.check(rc, "update_bounds")

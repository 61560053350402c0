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


def _rows(t: torch.Tensor):
    """[B, H, 1, D] or [B, H, D] -> (B, H, D, batch stride, head stride) of the
    row view, without building it (its address is the tensor's own)."""
    shape, stride = t.shape, t.stride()
    if len(shape) == 4:
        if shape[2] != 1:
            raise ValueError("the append kernels take one token per sequence")
        b, h, _, d = shape
        sb, sh, _, sd = stride
    elif len(shape) == 3:
        (b, h, d), (sb, sh, sd) = shape, stride
    else:
        raise ValueError("K/V rows must be [B, H, D] with unit-stride channels")
    if sd != 1:
        raise ValueError("K/V rows must be [B, H, D] with unit-stride channels")
    return b, h, d, sb, sh


def append_fp16(k: torch.Tensor, v: torch.Tensor, slots: torch.Tensor, flat_k: torch.Tensor,
                flat_v: torch.Tensor, kmin: Optional[torch.Tensor] = None,
                kmax: Optional[torch.Tensor] = None, page: int = 16) -> None:
    """k, v [B, H, 1, D] fp16 (views of the projection output are fine);
    slots [B] int64 flat token slots; flat_k / flat_v [num_blocks * page, H, D];
    kmin / kmax [num_blocks, H, D] or None."""
    if not k.is_cuda:
        raise RuntimeError("latentserve_b200 has no CPU path: tensors must be on a CUDA device")
    b, h, d, ksb, ksh = _rows(k)
    _, _, _, vsb, vsh = _rows(v)
    if slots.dtype != torch.int64 or slots.numel() < b or (slots.numel() > 1 and slots.stride(-1) != 1):
        raise ValueError("slots must be a contiguous int64 vector with one entry per sequence")
    fk_stride = flat_k.stride()
    if fk_stride != flat_v.stride() or fk_stride[-1] != 1:
        raise ValueError("K and V pools must share one layout with unit-stride channels")
    sb = (kmin.stride(0), kmin.stride(1)) if kmin is not None else (0, 0)
    rc = _lib.lib().ls_kv_append_fp16(
        k.data_ptr(), v.data_ptr(), slots.data_ptr(), flat_k.data_ptr(), flat_v.data_ptr(),
        _lib.ptr(kmin), _lib.ptr(kmax), b, h, d, page, flat_k.shape[0],
        ksb, ksh, vsb, vsh, fk_stride[0], fk_stride[1], sb[0], sb[1], _lib.current_stream(k.device))
    _lib.check(rc, "append_fp16")


def update_bounds_only(k_new: torch.Tensor, slots: torch.Tensor, kmin: torch.Tensor,
                       kmax: torch.Tensor, page: int = 16) -> None:
    """Page bounds for rows that something else already scattered."""
    b, h, d, ksb, ksh = _rows(k_new)
    rc = _lib.lib().ls_kv_append_fp16(
        k_new.data_ptr(), 0, slots.data_ptr(), 0, 0, kmin.data_ptr(), kmax.data_ptr(),
        b, h, d, page, kmin.shape[0] * page,
        ksb, ksh, 0, 0, 0, 0, kmin.stride(0), kmin.stride(1),
        _lib.current_stream(k_new.device))
    _lib.check(rc, "update_bounds")

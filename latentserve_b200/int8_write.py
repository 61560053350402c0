"""INT8 cache writes on the sm_100a kernels — host side.

`eligible` / `decode_write` mirror the reference's `kernels/cuda/int8_write.py`
(:53-58, :61-81): one launch per layer quantises V per (token, head) and
scatters it, and copies K into the fp16 residual. `finalize_blocks` is the
kernel form of `Int8PagedKVCache._finalize_blocks`
(cache/int8_paged_cache.py:670-699): a completed K page quantised per
(block, head, channel) straight out of the residual rows, no gather.

Both are bit-exact against the reference's arithmetic as it runs on a GPU,
where `t / 127` is `t * fp32(1/127)`: the reciprocals are formed here, on the
host, in fp32, exactly as PyTorch forms them.
"""

from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from latentserve_b200 import _lib

ENABLED = True


def eligible(k: torch.Tensor, v: torch.Tensor) -> bool:
    """One token per sequence, fp16, head_dim 128, channels unit-stride."""
    return (ENABLED and k.is_cuda and v.is_cuda and k.dtype == v.dtype == torch.float16
            and k.dim() == 4 and k.shape[2] == 1 and v.shape[2] == 1 and k.shape[-1] == 128
            and k.stride(-1) == 1 and v.stride(-1) == 1
            and all(s % 4 == 0 for s in (*k.stride()[:2], *v.stride()[:2]))
            and k.data_ptr() % 8 == 0 and v.data_ptr() % 8 == 0)


def _reciprocal(x: float) -> float:
    """fp32(1) / fp32(x): the reciprocal PyTorch multiplies by for `t / x`."""
    return float(np.float32(1.0) / np.float32(x))


def decode_write(k, v, slots, res_idx, flat_v, flat_v_scale, flat_v_zero, k_res, *,
                 asym: bool, eps: float, qmax: float, levels: float, offset: float) -> None:
    """k, v [B, H, 1, D] fp16; slots, res_idx [B] int64 flat indices;
    flat_v [S, H, D] int8, flat_v_scale / flat_v_zero [S, H] fp32 (contiguous);
    k_res [R, H, D] fp16 (contiguous)."""
    b, h, _, d = k.shape
    if not (flat_v.is_contiguous() and flat_v_scale.is_contiguous() and k_res.is_contiguous()):
        raise ValueError("the flat V pool, its scales and the residual must be contiguous")
    if slots.dtype != torch.int64 or res_idx.dtype != torch.int64:
        raise ValueError("slots and residual indices must be int64")
    rc = _lib.lib().ls_int8_decode_write(
        k.data_ptr(), v.data_ptr(), slots.data_ptr(), res_idx.data_ptr(), flat_v.data_ptr(),
        flat_v_scale.data_ptr(), _lib.ptr(flat_v_zero), k_res.data_ptr(),
        b, h, d, flat_v.shape[0], k_res.shape[0],
        k.stride(0), k.stride(1), v.stride(0), v.stride(1),
        int(asym), eps, qmax, _reciprocal(qmax), levels, _reciprocal(levels), offset,
        _lib.current_stream(k.device))
    _lib.check(rc, "int8 decode_write")


def finalize_blocks(k_residual: torch.Tensor, res_rows: torch.Tensor, block_ids: torch.Tensor,
                    k_pool: torch.Tensor, k_scale: torch.Tensor,
                    k_zero: Optional[torch.Tensor] = None, *, eps: float, qmax: float,
                    levels: float, offset: float) -> None:
    """Quantise residual rows `res_rows` [N] (int64) of `k_residual`
    [max_batch, 16, H, D] fp16 into physical blocks `block_ids` [N] (int64) of
    `k_pool` [num_blocks, 16, H, D] int8, one step per (block, head, channel)
    into `k_scale` [num_blocks, H, D] (and `k_zero` when asymmetric)."""
    n = int(res_rows.numel())
    if n == 0:
        return
    if res_rows.dtype != torch.int64 or block_ids.dtype != torch.int64 or block_ids.numel() != n:
        raise ValueError("res_rows and block_ids must be int64 vectors of one length")
    if k_residual.stride(-1) != 1 or k_pool.stride(-1) != 1 or k_scale.stride(-1) != 1:
        raise ValueError("channels must be unit-stride")
    asym = k_zero is not None
    if asym and k_zero.stride() != k_scale.stride():
        raise ValueError("k_zero must share k_scale's layout")
    rc = _lib.lib().ls_int8_finalize_blocks(
        k_residual.data_ptr(), res_rows.data_ptr(), block_ids.data_ptr(), k_pool.data_ptr(),
        k_scale.data_ptr(), _lib.ptr(k_zero), n, k_pool.shape[2], k_pool.shape[3], k_pool.shape[1],
        k_residual.shape[0], k_pool.shape[0],
        k_residual.stride(0), k_residual.stride(1), k_residual.stride(2),
        k_pool.stride(0), k_pool.stride(1), k_pool.stride(2),
        k_scale.stride(0), k_scale.stride(1),
        int(asym), eps, qmax, _reciprocal(qmax), levels, _reciprocal(levels), offset,
        _lib.current_stream(k_pool.device))
    _lib.check(rc, "int8 finalize_blocks")


def finalize_layers(k_residual: torch.Tensor, res_rows: torch.Tensor, block_ids: torch.Tensor,
                    count: int, k_pool: torch.Tensor, k_scale: torch.Tensor,
                    k_zero: Optional[torch.Tensor] = None, *, eps: float, qmax: float,
                    levels: float, offset: float) -> None:
    """`finalize_blocks` for every layer in one launch: `k_residual`
    [layers, max_batch, 16, H, D], `k_pool` [layers, num_blocks, 16, H, D],
    `k_scale` / `k_zero` [layers, num_blocks, H, D]; the first `count` entries of
    `res_rows` / `block_ids` (int64, device) apply to every layer."""
    if count == 0:
        return
    if res_rows.dtype != torch.int64 or block_ids.dtype != torch.int64 or min(
            res_rows.numel(), block_ids.numel()) < count:
        raise ValueError("res_rows and block_ids must be int64 vectors of at least `count` entries")
    if k_residual.dim() != 5 or k_pool.dim() != 5 or k_scale.dim() != 4 or k_pool.shape[0] != k_residual.shape[0]:
        raise ValueError("finalize_layers takes layer-stacked tensors")
    if k_residual.stride(-1) != 1 or k_pool.stride(-1) != 1 or k_scale.stride(-1) != 1:
        raise ValueError("channels must be unit-stride")
    asym = k_zero is not None
    if asym and k_zero.stride() != k_scale.stride():
        raise ValueError("k_zero must share k_scale's layout")
    rc = _lib.lib().ls_int8_finalize_layers(
        k_residual.data_ptr(), res_rows.data_ptr(), block_ids.data_ptr(), k_pool.data_ptr(),
        k_scale.data_ptr(), _lib.ptr(k_zero), count, k_pool.shape[0], k_pool.shape[3], k_pool.shape[4],
        k_pool.shape[2], k_residual.shape[1], k_pool.shape[1],
        k_residual.stride(0), k_residual.stride(1), k_residual.stride(2), k_residual.stride(3),
        k_pool.stride(0), k_pool.stride(1), k_pool.stride(2), k_pool.stride(3),
        k_scale.stride(0), k_scale.stride(1), k_scale.stride(2),
        int(asym), eps, qmax, _reciprocal(qmax), levels, _reciprocal(levels), offset,
        _lib.current_stream(k_pool.device))
    _lib.check(rc, "int8 finalize_layers")


def finalize_pending(k_residual: torch.Tensor, res_rows: torch.Tensor, block_ids: torch.Tensor,
                     state: torch.Tensor, k_pool: torch.Tensor, k_scale: torch.Tensor,
                     k_zero: Optional[torch.Tensor] = None, *, eps: float, qmax: float,
                     levels: float, offset: float) -> None:
    """`finalize_layers` with the number of pages on the device: `state` int32 [2]
    holds (pages to finalise, 0); the kernel finalises the first state[0] entries of
    `res_rows` / `block_ids` in every layer and sets state[0] back to zero. Always one
    launch of a fixed grid (sized by the lists' capacity), so it can be a node of a
    captured decode step; a step with nothing to finalise costs one read per CTA."""
    if res_rows.dtype != torch.int64 or block_ids.dtype != torch.int64:
        raise ValueError("res_rows and block_ids must be int64 vectors")
    if state.dtype != torch.int32 or state.numel() < 2 or not state.is_contiguous():
        raise ValueError("state must be a contiguous int32 tensor of two entries")
    if k_residual.dim() != 5 or k_pool.dim() != 5 or k_scale.dim() != 4 or k_pool.shape[0] != k_residual.shape[0]:
        raise ValueError("finalize_pending takes layer-stacked tensors")
    if k_residual.stride(-1) != 1 or k_pool.stride(-1) != 1 or k_scale.stride(-1) != 1:
        raise ValueError("channels must be unit-stride")
    asym = k_zero is not None
    if asym and k_zero.stride() != k_scale.stride():
        raise ValueError("k_zero must share k_scale's layout")
    rc = _lib.lib().ls_int8_finalize_pending(
        k_residual.data_ptr(), res_rows.data_ptr(), block_ids.data_ptr(), state.data_ptr(),
        k_pool.data_ptr(), k_scale.data_ptr(), _lib.ptr(k_zero),
        min(res_rows.numel(), block_ids.numel()), k_pool.shape[0], k_pool.shape[3], k_pool.shape[4],
        k_pool.shape[2], k_residual.shape[1], k_pool.shape[1],
        k_residual.stride(0), k_residual.stride(1), k_residual.stride(2), k_residual.stride(3),
        k_pool.stride(0), k_pool.stride(1), k_pool.stride(2), k_pool.stride(3),
        k_scale.stride(0), k_scale.stride(1), k_scale.stride(2),
        int(asym), eps, qmax, _reciprocal(qmax), levels, _reciprocal(levels), offset,
        _lib.current_stream(k_pool.device))
    _lib.check(rc, "int8 finalize_pending")

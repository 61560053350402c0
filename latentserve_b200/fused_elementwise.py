"""RMSNorm, SiLU * up and RoPE (+ KV append) on the sm_100a kernels — host side.

`rms_norm`, `fused_add_rms_norm`, `silu_and_mul` mirror the reference's
`kernels/fused_elementwise.py` (:190-226): same names, arguments and fp16
rounding. `rope_append` has no single counterpart there: it is the reference's
`rope_qk` (:229-252) and the cache's `write()` in one launch, reading q, k, v
straight from the fused QKV projection row (see `PagedKVCache.rope_write`).
fp16 CUDA tensors only; anything else raises.
"""

from __future__ import annotations

import torch

from latentserve_b200 import _lib


def _rows(t: torch.Tensor) -> torch.Tensor:
    t2 = t.reshape(-1, t.shape[-1])
    if not (t2.is_cuda and t2.dtype == torch.float16 and t2.stride(-1) == 1):
        raise ValueError("fused element-wise kernels take fp16 CUDA rows with unit-stride channels")
    return t2


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    x2 = _rows(x)
    y = torch.empty_like(x2)
    rc = _lib.lib().ls_rms_norm(x2.data_ptr(), 0, weight.data_ptr(), y.data_ptr(), 0, x2.shape[0],
                                x2.shape[1], eps, x2.stride(0), 0, y.stride(0), 0,
                                _lib.current_stream(x.device))
    _lib.check(rc, "rms_norm")
    return y.reshape(x.shape)


def fused_add_rms_norm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float):
    """(norm(residual + x), residual + x) in one kernel."""
    x2, r2 = _rows(x), _rows(residual)
    y, res_out = torch.empty_like(x2), torch.empty_like(x2)
    rc = _lib.lib().ls_rms_norm(x2.data_ptr(), r2.data_ptr(), weight.data_ptr(), y.data_ptr(),
                                res_out.data_ptr(), x2.shape[0], x2.shape[1], eps, x2.stride(0),
                                r2.stride(0), y.stride(0), res_out.stride(0),
                                _lib.current_stream(x.device))
    _lib.check(rc, "fused_add_rms_norm")
    return y.reshape(x.shape), res_out.reshape(x.shape)


def silu_and_mul(gate_up: torch.Tensor) -> torch.Tensor:
    gu = _rows(gate_up)
    inter = gu.shape[-1] // 2
    out = torch.empty((gu.shape[0], inter), dtype=gu.dtype, device=gu.device)
    rc = _lib.lib().ls_silu_mul(gu.data_ptr(), out.data_ptr(), gu.shape[0], inter, gu.stride(0),
                                out.stride(0), _lib.current_stream(gu.device))
    _lib.check(rc, "silu_and_mul")
    return out.reshape(*gate_up.shape[:-1], inter)


def rope_append_fp16(qkv, cos, sin, positions, slots, q_out, flat_k, flat_v, kmin, kmax,
                     q_heads: int, kv_heads: int, page: int = 16) -> None:
    """qkv [B, (q_heads + 2 kv_heads) * 128] fp16 (q, k, v head order); cos, sin
    [max_pos, 128] fp16; positions, slots [B] int64; q_out [B, q_heads * 128] fp16;
    flat_k / flat_v [num_slots, kv_heads, 128]; kmin / kmax [num_blocks, kv_heads, 128] or None."""
    b = qkv.shape[0]
    sb = (kmin.stride(0), kmin.stride(1)) if kmin is not None else (0, 0)
    rc = _lib.lib().ls_rope_append_fp16(
        qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), positions.data_ptr(), slots.data_ptr(),
        q_out.data_ptr(), flat_k.data_ptr(), flat_v.data_ptr(), _lib.ptr(kmin), _lib.ptr(kmax),
        b, q_heads, kv_heads, 128, page, cos.shape[0], flat_k.shape[0], qkv.stride(0), cos.stride(0),
        q_out.stride(0), flat_k.stride(0), flat_k.stride(1), sb[0], sb[1],
        _lib.current_stream(qkv.device))
    _lib.check(rc, "rope_append_fp16")


def rope_append_int8(qkv, cos, sin, positions, slots, res_idx, q_out, flat_v, flat_v_scale,
                     flat_v_zero, k_res, q_heads: int, kv_heads: int, *, asym: bool, eps: float,
                     qmax: float, levels: float, offset: float, kmin=None, kmax=None) -> None:
    """As above for the INT8 cache: flat_v int8 [num_slots, kv_heads, 128], its fp32
    scales (and zero points) [num_slots, kv_heads], k_res fp16 [rows, kv_heads, 128]
    with res_idx [B] int64; all contiguous."""
    from latentserve_b200.int8_write import _reciprocal

    rc = _lib.lib().ls_rope_append_int8(
        qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), positions.data_ptr(), slots.data_ptr(),
        res_idx.data_ptr(), q_out.data_ptr(), flat_v.data_ptr(), flat_v_scale.data_ptr(),
        _lib.ptr(flat_v_zero), k_res.data_ptr(), _lib.ptr(kmin), _lib.ptr(kmax), qkv.shape[0], q_heads,
        kv_heads, 128, cos.shape[0], flat_v.shape[0], k_res.shape[0], qkv.stride(0), cos.stride(0),
        q_out.stride(0), kmin.stride(0) if kmin is not None else 0,
        kmin.stride(1) if kmin is not None else 0, int(asym),
        eps, qmax, _reciprocal(qmax), levels, _reciprocal(levels), offset,
        _lib.current_stream(qkv.device))
    _lib.check(rc, "rope_append_int8")


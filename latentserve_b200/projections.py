"""Decode-step projections on the weight-streaming kernel (`ls_skinny_gemm`).

In the reference the four projections of a decoder layer are Hugging Face
`nn.Linear` modules (cuBLAS) run by `LatentServeQwen._run_layers`
(model/latentserve_qwen.py:397-451), with RMSNorm, the residual add and
SiLU * up as separate (optionally Triton-fused) element-wise launches
(kernels/fused_elementwise.py:194-232). For a decode batch of tens of rows each
projection is a stream of weights through HBM, and the element-wise launches
around it are latency-floor kernels; `linear` folds them into the projection:

    qkv      = linear(s, w_qkv, b_qkv, norm_weight=ln1, row_sumsq=ss)
    s, ss    = linear(attn, w_o, add_residual=s, want_sumsq=True)    # s = residual stream
    act      = linear(s, w_gate_up, norm_weight=ln2, row_sumsq=ss, swiglu=True)
    s, ss    = linear(act, w_down, add_residual=s, want_sumsq=True)

(`row_sumsq` hands the norm its row statistics from the projection that wrote
the row; without it the kernel reads the whole rows itself, and can add a
`residual` in front of the norm.)

Rounding follows the unfused model code (fp16 where Hugging Face rounds to
fp16, fp32 accumulation in the product), so results agree with
`fused_elementwise` + `torch.matmul` to fp16 rounding of the accumulation
order; the GPU tests state the tolerance.
"""

from __future__ import annotations

from typing import Optional

import torch

from latentserve_b200 import _lib
from latentserve_b200 import paged_decode_cuda as pdc

GEMM_NORM, GEMM_SWIGLU = 1, 2
MAX_ROWS = 32
TILE_ROWS = 32


def _rows_pad(m: int) -> int:
    return 16 if m <= 16 else 32


MAX_CHUNKS_PER_CTA = 48             # 8 warps x 6 chunks whose activations a warp keeps in registers


def choose_splits(device: torch.device, tiles: int, k: int, m: int = 16) -> int:
    """Slices of K across CTAs: enough that tiles x splits fills the CTAs the device
    holds at once (without going past it, which would leave a second, nearly empty
    wave), every warp still gets a 32-wide chunk, and a CTA's slice is at most 48
    chunks."""
    chunks = k // 32
    if chunks <= MAX_CHUNKS_PER_CTA and tiles >= 32:
        # A short K on a few dozen CTAs streams faster than the same matrix cut into
        # slices whose partial sums meet in global memory (measured: 4.9 vs 7.0 us
        # for 1536 x 1536).
        return 1
    resident = (2 if m <= 16 else 1) * pdc.sm_count(device)
    splits = max(1, min(resident // tiles, chunks // 8 if chunks >= 8 else 1))
    return max(splits, -(-chunks // MAX_CHUNKS_PER_CTA))


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, *,
           norm_weight: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
           row_sumsq: Optional[torch.Tensor] = None, add_residual: Optional[torch.Tensor] = None,
           want_sumsq: bool = False, eps: float = 1e-6, swiglu: bool = False,
           out: Optional[torch.Tensor] = None, splits: Optional[int] = None):
    """x [M, K] fp16 (M <= 32), w [N, K] fp16 -> [M, N] fp16 (or [M, N / 2] with
    `swiglu`).

    Front: with `norm_weight`, x is RMS-normalised first -- after adding
    `residual`, when given (the return value is then (out, x + residual)), or
    with the row statistics in `row_sumsq` (as returned by `want_sumsq`).
    Back: `add_residual` [M, N] is added to the fp16-rounded product;
    `want_sumsq` also returns per-row partial sums of squares of the output
    ([64, N / 32] fp32: row r's partials are contiguous), for the next call's
    `row_sumsq`."""
    if not x.is_cuda:
        raise RuntimeError("latentserve_b200 has no CPU path: tensors must be on a CUDA device")
    if x.dim() != 2 or w.dim() != 2 or x.dtype != torch.float16 or w.dtype != torch.float16:
        raise ValueError("linear takes fp16 x [M, K] and w [N, K]")
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k or x.stride(1) != 1 or w.stride(1) != 1:
        raise ValueError("x and w must share K and have unit-stride rows")
    if m > MAX_ROWS:
        raise ValueError(f"linear streams weights for at most {MAX_ROWS} rows, got {m}")
    if (residual is not None or row_sumsq is not None) and norm_weight is None:
        raise ValueError("residual / row_sumsq belong to the norm: pass norm_weight as well")
    if residual is not None and row_sumsq is not None:
        raise ValueError("row_sumsq describes x itself: it cannot be combined with a residual")
    if residual is not None and (residual.shape != x.shape or residual.dtype != x.dtype
                                 or residual.stride(1) != 1):
        raise ValueError("residual must match x")
    if row_sumsq is not None and (row_sumsq.dtype != torch.float32 or row_sumsq.dim() != 2
                                  or row_sumsq.shape[0] != 64 or not row_sumsq.is_contiguous()):
        raise ValueError("row_sumsq must be the contiguous fp32 [64, tiles] tensor want_sumsq returns")
    if row_sumsq is not None and row_sumsq.shape[1] * 32 != k:
        raise ValueError("row_sumsq does not describe rows of this K")
    if bias is not None and (bias.shape != (n,) or bias.dtype != x.dtype or not bias.is_contiguous()):
        raise ValueError("bias must be a contiguous fp16 [N] vector")
    if swiglu and (bias is not None or add_residual is not None or want_sumsq):
        raise ValueError("the SwiGLU epilogue takes no bias, residual or row statistics")
    if add_residual is not None and (add_residual.shape != (m, n) or add_residual.dtype != x.dtype
                                     or add_residual.stride(1) != 1):
        raise ValueError("add_residual must be fp16 [M, N] with unit-stride rows")
    mode = (GEMM_NORM if norm_weight is not None else 0) | (GEMM_SWIGLU if swiglu else 0)
    mode |= pdc.launch_flags()
    tiles = n // 32
    n_out = n // 2 if swiglu else n
    if out is None:
        out = torch.empty((m, n_out), dtype=x.dtype, device=x.device)
    elif out.shape != (m, n_out) or out.dtype != x.dtype or out.stride(1) != 1:
        raise ValueError("out has the wrong shape, dtype or layout")
    res_out = torch.empty_like(x) if residual is not None else None
    sumsq = torch.empty((64, tiles), dtype=torch.float32, device=x.device) if want_sumsq else None
    if splits is None:
        splits = choose_splits(x.device, tiles, k, m)
    part = counters = None
    if splits > 1:
        part = pdc.scratch("gemm_part", (tiles * splits * _rows_pad(m) * 32,), torch.float32, x.device)
        counters = pdc.scratch("gemm_counters", (tiles,), torch.int32, x.device, zero=True)
    ptr = _lib.ptr
    rc = _lib.lib().ls_skinny_gemm(
        x.data_ptr(), ptr(residual), ptr(norm_weight), ptr(res_out), ptr(row_sumsq),
        row_sumsq.shape[1] if row_sumsq is not None else 0, w.data_ptr(), ptr(bias),
        ptr(add_residual), ptr(sumsq), out.data_ptr(), ptr(part), ptr(counters), m, n, k, splits, mode,
        eps, x.stride(0), residual.stride(0) if residual is not None else 0,
        res_out.stride(0) if res_out is not None else 0, w.stride(0),
        add_residual.stride(0) if add_residual is not None else 0, out.stride(0),
        _lib.current_stream(x.device))
    _lib.check(rc, "linear")
    extra = tuple(t for t in (res_out, sumsq) if t is not None)
    return (out, *extra) if extra else out


def qkv_rope_append(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], cos: torch.Tensor,
                    sin: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, q_out: torch.Tensor,
                    flat_k: torch.Tensor, flat_v: torch.Tensor, kmin: Optional[torch.Tensor],
                    kmax: Optional[torch.Tensor], q_heads: int, kv_heads: int, *,
                    norm_weight: Optional[torch.Tensor] = None, row_sumsq: Optional[torch.Tensor] = None,
                    eps: float = 1e-6, splits: Optional[int] = None) -> None:
    """The fused QKV projection of a decode step with RoPE and the fp16 cache append
    in its epilogue: what `linear(x, w, bias, norm_weight=..., row_sumsq=...)`
    followed by `fused_elementwise.rope_append_fp16` writes (rotated q into `q_out`
    [M, q_heads * 128], rotated k and v at `slots` [M] int64 of the flat pools
    [num_slots, kv_heads, 128], the page bounds when given), bit for bit, in one
    launch. w [(q_heads + 2 kv_heads) * 128, K] in q, k, v head order; cos, sin
    [max_pos, 128] fp16; positions [M] int64."""
    if not x.is_cuda:
        raise RuntimeError("latentserve_b200 has no CPU path: tensors must be on a CUDA device")
    if x.dim() != 2 or w.dim() != 2 or x.dtype != torch.float16 or w.dtype != torch.float16:
        raise ValueError("qkv_rope_append takes fp16 x [M, K] and w [N, K]")
    m, k = x.shape
    n = (q_heads + 2 * kv_heads) * 128
    if w.shape != (n, k) or x.stride(1) != 1 or w.stride(1) != 1:
        raise ValueError("w must be [(q_heads + 2 kv_heads) * 128, K] with unit-stride rows, as x")
    if m > MAX_ROWS:
        raise ValueError(f"the streaming projection takes at most {MAX_ROWS} rows, got {m}")
    if row_sumsq is not None and norm_weight is None:
        raise ValueError("row_sumsq belongs to the norm: pass norm_weight as well")
    if row_sumsq is not None and (row_sumsq.dtype != torch.float32 or row_sumsq.dim() != 2
                                  or row_sumsq.shape[0] != 64 or not row_sumsq.is_contiguous()
                                  or row_sumsq.shape[1] * 32 != k):
        raise ValueError("row_sumsq must be the contiguous fp32 [64, K / 32] tensor want_sumsq returns")
    if bias is not None and (bias.shape != (n,) or bias.dtype != x.dtype or not bias.is_contiguous()):
        raise ValueError("bias must be a contiguous fp16 [N] vector")
    if flat_k.dtype != torch.float16 or flat_v.dtype != torch.float16 or flat_k.shape != flat_v.shape \
            or flat_k.stride() != flat_v.stride() or flat_k.stride(2) != 1:
        raise ValueError("flat_k / flat_v must be fp16 [num_slots, kv_heads, 128] views of one layout")
    if (kmin is None) != (kmax is None):
        raise ValueError("kmin and kmax come together")
    if q_out.shape != (m, q_heads * 128) or q_out.dtype != x.dtype or q_out.stride(1) != 1:
        raise ValueError("q_out must be fp16 [M, q_heads * 128] with unit-stride rows")
    if positions.dtype != torch.int64 or slots.dtype != torch.int64 or positions.numel() < m \
            or slots.numel() < m:
        raise ValueError("positions and slots must be int64 [M]")
    tiles = n // 32
    if splits is None:
        splits = choose_splits(x.device, tiles, k, m)
    part = counters = None
    if splits > 1:
        part = pdc.scratch("gemm_part", (tiles * splits * _rows_pad(m) * 32,), torch.float32, x.device)
        counters = pdc.scratch("gemm_counters", (tiles,), torch.int32, x.device, zero=True)
    mode = (GEMM_NORM if norm_weight is not None else 0) | pdc.launch_flags()
    ptr = _lib.ptr
    sb = (kmin.stride(0), kmin.stride(1)) if kmin is not None else (0, 0)
    rc = _lib.lib().ls_qkv_rope_append_fp16(
        x.data_ptr(), ptr(norm_weight), ptr(row_sumsq), row_sumsq.shape[1] if row_sumsq is not None else 0,
        w.data_ptr(), ptr(bias), cos.data_ptr(), sin.data_ptr(), positions.data_ptr(), slots.data_ptr(),
        q_out.data_ptr(), flat_k.data_ptr(), flat_v.data_ptr(), ptr(kmin), ptr(kmax), ptr(part),
        ptr(counters), m, q_heads, kv_heads, 128, 16, k, splits, mode, eps, cos.shape[0], flat_k.shape[0],
        x.stride(0), w.stride(0), cos.stride(0), q_out.stride(0), flat_k.stride(0), flat_k.stride(1),
        sb[0], sb[1], _lib.current_stream(x.device))
    _lib.check(rc, "qkv_rope_append")

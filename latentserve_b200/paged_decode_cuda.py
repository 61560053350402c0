"""Paged decode attention on the sm_100a kernels — host side.

Mirrors the reference's `kernels/cuda/paged_decode_cuda.py` (`eligible` :112-141,
`choose_splits` :197-199, `paged_decode_cuda` :202-252): same names, same
argument meaning, same exceptions, so it can stand in for that module. What
differs is underneath: the kernels are ahead-of-time compiled CUDA behind a C
ABI (`_lib`), the split merge is a CUDA kernel of this library rather than
Triton, and nothing is filled before a launch.

Work is not split per sequence. The batch's pages are laid on one axis and cut
into `num_chunks` equal pieces (csrc/decode_sched.cuh), so `num_splits` keeps
its place in the signature but only as an upper bound on how finely the axis is
cut; the result does not depend on it beyond fp32 rounding.
"""

from __future__ import annotations

import math
import os
from typing import Optional

import torch

from latentserve_b200 import _lib

IMPL_MMA, IMPL_SIMT = 0, 1          # tensor-core kernel / CUDA-core kernel (fp16 pools)
LAUNCH_PROGRAMMATIC = 0x100         # see LS_LAUNCH_PROGRAMMATIC in the header
EARLY_PAGES = 0x800                 # see LS_EARLY_PAGES (dense entry points only)
# Decode launches use programmatic dependent launch when this is set: the
# kernel's prologue (which reads only seq_lens and block_tables) overlaps the
# tail of the previous kernel on the stream. Safe wherever that previous kernel
# does not write those two tensors -- in a LatentServe layer it is the KV
# append. Off unless asked for (LATENTSERVE_B200_PDL=1 or set_programmatic_launch).
_PROGRAMMATIC = {"on": os.environ.get("LATENTSERVE_B200_PDL", "0") == "1"}
LOAD_CP_ASYNC, LOAD_TMA = 0x200, 0x400   # see LS_LOAD_CP_ASYNC / LS_LOAD_TMA in the header
LOAD_TMA_SPLIT_KV = 0x1000                # see LS_LOAD_TMA_SPLIT_KV (INT8 entry points)
# "auto": TMA tile copies for INT8 pools, per-lane cp.async for fp16 pools (the
# faster form of each); "tma" / "cp_async" force one (same results; for
# comparison and for the tests).
_LOADER = {"name": os.environ.get("LATENTSERVE_B200_LOADER", "auto")}
ROWS_PER_PARTIAL = 8                # query rows a partial holds (GQA ratio <= 8)
MIN_CHUNK_PAGES = 8                 # never cut the page axis finer than this
CTAS_PER_SM = 2                     # resident CTAs per SM the kernels are sized for
# ... and for the INT8 kernel (must match LS_INT8_CTAS the library was built with)
INT8_CTAS_PER_SM = int(os.environ.get("LATENTSERVE_B200_INT8_CTAS", "3"))
MAX_BATCH = 1024

_SCRATCH: dict = {}
_SM_COUNT: dict = {}


def set_programmatic_launch(on: bool, early_pages: bool = True) -> None:
    _PROGRAMMATIC["on"] = bool(on)
    _PROGRAMMATIC["early"] = bool(early_pages)


def launch_flags() -> int:
    return LAUNCH_PROGRAMMATIC if _PROGRAMMATIC["on"] else 0


def dense_launch_flags() -> int:
    """Flags of the dense decode entry points: with programmatic launch on, old
    pages are requested ahead of the dependency wait as well (the caches of this
    package and of LatentServe write only the newest token between steps)."""
    on = _PROGRAMMATIC["on"] and _PROGRAMMATIC.get("early", True)
    return (LAUNCH_PROGRAMMATIC | EARLY_PAGES) if on else launch_flags()


def set_loader(name: str) -> None:
    if name not in ("auto", "tma", "tma_split_kv", "cp_async"):
        raise ValueError(f"unknown page loader {name!r}")
    _LOADER["name"] = name


def loader_flags() -> int:
    return {"auto": 0, "tma": LOAD_TMA, "tma_split_kv": LOAD_TMA, "cp_async": LOAD_CP_ASYNC}[_LOADER["name"]]


def int8_loader_flags() -> int:
    """The loader flags of the INT8 entry points: `tma_split_kv` asks for a page's K and V
    tiles by one copy each (what pools more than 2^40 bytes apart get by themselves)."""
    return loader_flags() | (LOAD_TMA_SPLIT_KV if _LOADER["name"] == "tma_split_kv" else 0)


def scratch(key, shape, dtype, device, zero: bool = False) -> torch.Tensor:
    """Persistent scratch, one buffer per (name, shape, dtype, device), never
    replaced: a captured CUDA graph keeps its addresses valid
    (reference: kernels/gqa/paged_decode.py:501-517)."""
    full_key = (key, tuple(shape), dtype, str(device))
    buf = _SCRATCH.get(full_key)
    if buf is None:
        buf = (torch.zeros if zero else torch.empty)(shape, dtype=dtype, device=device)
        _SCRATCH[full_key] = buf
    return buf


def sm_count(device: torch.device) -> int:
    dev = device.index if device.index is not None else torch.cuda.current_device()
    if dev not in _SM_COUNT:
        _SM_COUNT[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
    return _SM_COUNT[dev]


def _aligned(t: torch.Tensor, nbytes: int) -> bool:
    return (t.stride(-1) == 1 and t.data_ptr() % nbytes == 0
            and all((st * t.element_size()) % nbytes == 0 for st in t.stride()[:-1]))


def eligible(q: torch.Tensor, k_pool: torch.Tensor, k_scale=None, k_residual=None,
             v_scale=None, k_zero=None, v_zero=None, res_rows=None) -> bool:
    """What the kernels handle: fp16 queries, head_dim 128, page 16, at most 8
    query rows per KV head, fp16 or INT8 pools, and 16-byte aligned rows."""
    if not (q.is_cuda and q.dtype == torch.float16 and q.dim() == 4 and q.shape[-1] == 128
            and q.shape[2] <= ROWS_PER_PARTIAL and q.shape[0] <= MAX_BATCH
            and k_pool.dim() == 4 and k_pool.shape[1] == 16 and _aligned(q, 16)):
        return False
    if k_pool.dtype == torch.float16:
        return k_scale is None and k_residual is None and _aligned(k_pool, 16)
    if k_pool.dtype != torch.int8:
        return False
    if k_scale is None or v_scale is None or not _aligned(k_pool, 16):
        return False
    if k_scale.dtype != torch.float32 or v_scale.dtype != torch.float32 or not _aligned(k_scale, 16):
        return False
    if (k_zero is None) != (v_zero is None):
        return False
    if k_zero is not None and (k_zero.dtype != torch.float32 or k_zero.stride() != k_scale.stride()
                               or v_zero.stride() != v_scale.stride() or not _aligned(k_zero, 16)):
        return False
    if (k_residual is None) != (res_rows is None):
        return False
    if k_residual is not None and (k_residual.dtype != torch.float16 or not _aligned(k_residual, 16)
                                   or res_rows.dtype != torch.int32):
        return False
    return True


def choose_chunks(device: torch.device, kv_heads: int, num_splits: Optional[int] = None,
                  batch: int = 1, ctas_per_sm: int = CTAS_PER_SM) -> int:
    """Pieces the batch's page axis is cut into: one per resident CTA column
    (grid = chunks x KV heads fills every SM `CTAS_PER_SM` times). A caller's
    `num_splits` caps it at batch x num_splits."""
    chunks = max(1, (ctas_per_sm * sm_count(device)) // max(1, kv_heads))
    if num_splits:
        chunks = max(1, min(chunks, batch * num_splits))
    return chunks


def choose_splits(batch: int, kv_heads: int, num_pages: int) -> int:
    """Kept for callers of the reference's name: partial slots per sequence at
    most. The kernels derive the real cut on the device."""
    return max(1, min(num_pages, 128))


def seg_len(batch: int, kv_heads: int) -> int:
    """int32 entries of the bookkeeping scratch: per-sequence slot ranges, the
    error flag, and one arrival counter per (sequence, KV head)."""
    return 2 * batch + 2 + batch * kv_heads


def seg_scratch(tag: str, batch: int, kv_heads: int, device) -> torch.Tensor:
    """The bookkeeping scratch of one (batch, KV heads) shape. Its layout depends
    on the batch size (slot ranges in [0, 2B), the error flag at [2B], arrival
    counters from [2B + 2)), and the arrival counters must read zero when a launch
    starts, so the buffer is keyed by the shape, never by its flat length: (5, 2)
    and (2, 8) are both 22 ints long, and one's slot ranges would be the other's
    counters."""
    return scratch(f"{tag}_seg_b{batch}_h{kv_heads}", (seg_len(batch, kv_heads),), torch.int32,
                   device, zero=True)


def _partials(q: torch.Tensor, chunks: int, tag: str):
    b, h = q.shape[0], q.shape[1]
    slots = b + chunks
    acc = scratch(tag + "_acc", (slots, h, ROWS_PER_PARTIAL, 128), torch.float32, q.device)
    m = scratch(tag + "_m", (slots, h, ROWS_PER_PARTIAL), torch.float32, q.device)
    l = scratch(tag + "_l", (slots, h, ROWS_PER_PARTIAL), torch.float32, q.device)
    seg = seg_scratch(tag, b, h, q.device)
    return acc, m, l, seg


def error_flag(device, batch: int, kv_heads: int = 2, tag: str = "cuda") -> int:
    """1 if a launch at this batch size met a block id (or residual row)
    outside its pool and skipped it. Reading it synchronises; for tests."""
    seg = _SCRATCH.get((f"{tag}_seg_b{batch}_h{kv_heads}", (seg_len(batch, kv_heads),), torch.int32,
                        str(torch.device(device))))
    return 0 if seg is None else int(seg[2 * batch].item())


def paged_decode_cuda(q, k_pool, v_pool, block_tables, seq_lens, max_seq_len: int,
                      num_splits: Optional[int] = None,
                      softmax_scale: Optional[float] = None,
                      k_scale=None, v_scale=None, k_zero=None, v_zero=None,
                      k_residual=None, res_rows=None,
                      min_blocks: Optional[int] = None, impl: int = IMPL_MMA,
                      merge: bool = True) -> Optional[torch.Tensor]:
    """q [B, H_kv, N_REP, 128] fp16; pools [num_blocks, 16, H_kv, 128] fp16 or int8;
    block_tables [B, max_pages] int32; seq_lens [B] int32 -> [B, H_kv, N_REP, 128] fp16.

    `max_seq_len` and `min_blocks` are accepted for signature parity; extents
    come from `seq_lens` on the device. The returned tensor is persistent
    scratch, valid until the next call with the same shapes. `merge=False`
    stops at the partial states (no output is written) and returns None.
    """
    fn, args, out, dev_index = plan_decode(q, k_pool, v_pool, block_tables, seq_lens, num_splits,
                                           softmax_scale, k_scale, v_scale, k_zero, v_zero,
                                           k_residual, res_rows, impl, merge)
    _lib.check(fn(*args, _lib.raw_stream(dev_index)), "paged_decode_cuda")
    return out if merge else None


def append_rows_ok(k_new: torch.Tensor, v_new: torch.Tensor, q: torch.Tensor) -> bool:
    """Whether the step's new K / V rows ([B, H, 1, 128] or [B, H, 128], fp16) can ride
    on the attention launch: unit-stride channels, 16-byte aligned rows."""
    def ok(t):
        return (t.is_cuda and t.dtype == torch.float16 and t.dim() in (3, 4) and t.shape[0] == q.shape[0]
                and t.shape[1] == q.shape[1] and t.shape[-1] == 128 and (t.dim() == 3 or t.shape[2] == 1)
                and t.stride(-1) == 1 and t.data_ptr() % 16 == 0 and t.stride(0) % 8 == 0
                and t.stride(1) % 8 == 0)
    return ok(k_new) and ok(v_new)


def plan_decode(q, k_pool, v_pool, block_tables, seq_lens, num_splits=None, softmax_scale=None,
                k_scale=None, v_scale=None, k_zero=None, v_zero=None, k_residual=None, res_rows=None,
                impl: int = IMPL_MMA, merge: bool = True, out: Optional[torch.Tensor] = None,
                k_new: Optional[torch.Tensor] = None, v_new: Optional[torch.Tensor] = None):
    """Validate one decode call and bind its arguments: returns (entry point,
    argument tuple without the stream, output tensor, device index). The tuple
    holds raw addresses, so it is valid for as long as the tensors it was built
    from are alive and unmoved -- which is how a decode loop calls this path
    (persistent pools, tables, lengths and projection buffers)."""
    if not q.is_cuda:
        raise RuntimeError("latentserve_b200 has no CPU path: tensors must be on a CUDA device")
    b, h_kv, n_rep, d = q.shape
    if q.stride(-1) != 1 or k_pool.stride(-1) != 1 or v_pool.stride() != k_pool.stride():
        raise ValueError("the CUDA kernel needs unit-stride head dims and matching K/V pools")
    if block_tables.dtype != torch.int32 or seq_lens.dtype != torch.int32:
        raise ValueError("block tables and sequence lengths must be int32")
    if block_tables.stride(-1) != 1 or (seq_lens.numel() > 1 and seq_lens.stride(0) != 1):
        raise ValueError("block tables and sequence lengths must be contiguous rows")
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
    int8 = k_pool.dtype == torch.int8
    chunks = choose_chunks(q.device, h_kv, num_splits, b, INT8_CTAS_PER_SM if int8 else CTAS_PER_SM)
    tag = "cuda_i8" if int8 else "cuda"
    acc, m, l, seg = _partials(q, chunks, tag)
    if out is None:
        out = scratch(tag + "_out", (b, h_kv, n_rep, d), q.dtype, q.device)
    elif (out.shape != q.shape or out.dtype != q.dtype or out.device != q.device
          or out.stride(-1) != 1):
        raise ValueError("out must be an fp16 [B, H_kv, N_REP, 128] tensor on q's device with "
                         "unit-stride channels")
    out_ptr = out.data_ptr() if merge else 0
    lib = _lib.lib()
    ptr = _lib.ptr
    dev_index = q.device.index if q.device.index is not None else torch.cuda.current_device()
    if int8:
        if k_scale is None or v_scale is None:
            raise ValueError("INT8 pools need k_scale and v_scale")
        res_st = k_residual.stride()[:3] if k_residual is not None else (0, 0, 0)
        fn = lib.ls_paged_decode_int8
        args = (
            ptr(q), ptr(k_pool), ptr(v_pool), ptr(block_tables), ptr(seq_lens),
            ptr(k_scale), ptr(v_scale), ptr(k_zero), ptr(v_zero), ptr(k_residual), ptr(res_rows),
            ptr(acc), ptr(m), ptr(l), ptr(seg), out_ptr,
            b, h_kv, n_rep, d, k_pool.shape[1], block_tables.stride(0), k_pool.shape[0],
            0 if k_residual is None else k_residual.shape[0], chunks, MIN_CHUNK_PAGES,
            dense_launch_flags() | int8_loader_flags(),
            q.stride(0), q.stride(1), q.stride(2),
            k_pool.stride(0), k_pool.stride(1), k_pool.stride(2),
            k_scale.stride(0), k_scale.stride(1),
            v_scale.stride(0), v_scale.stride(1), v_scale.stride(2),
            *res_st, out.stride(0), out.stride(1), out.stride(2), scale)
    elif k_new is not None:
        # The step's append rides on the launch (fp16 pools, dense): see the header.
        if k_scale is not None or k_residual is not None:
            raise ValueError("fp16 pools take no scales or residual")
        if v_new is None or not append_rows_ok(k_new, v_new, q):
            raise ValueError("the new K / V rows must be fp16 [B, H, (1,) 128] with 16-byte aligned rows")
        fn = lib.ls_paged_decode_append_fp16
        args = (
            ptr(q), ptr(k_new), ptr(v_new), ptr(k_pool), ptr(v_pool), ptr(block_tables), ptr(seq_lens),
            ptr(acc), ptr(m), ptr(l), ptr(seg), out_ptr,
            b, h_kv, n_rep, d, k_pool.shape[1], block_tables.stride(0), k_pool.shape[0],
            chunks, MIN_CHUNK_PAGES, impl | dense_launch_flags() | (loader_flags() & ~LOAD_TMA),
            q.stride(0), q.stride(1), q.stride(2),
            k_new.stride(0), k_new.stride(1), v_new.stride(0), v_new.stride(1),
            k_pool.stride(0), k_pool.stride(1), k_pool.stride(2),
            out.stride(0), out.stride(1), out.stride(2), scale)
    else:
        if k_scale is not None or k_residual is not None:
            raise ValueError("fp16 pools take no scales or residual")
        fn = lib.ls_paged_decode_fp16
        args = (
            ptr(q), ptr(k_pool), ptr(v_pool), ptr(block_tables), ptr(seq_lens),
            ptr(acc), ptr(m), ptr(l), ptr(seg), out_ptr,
            b, h_kv, n_rep, d, k_pool.shape[1], block_tables.stride(0), k_pool.shape[0],
            chunks, MIN_CHUNK_PAGES, impl | dense_launch_flags() | loader_flags(),
            q.stride(0), q.stride(1), q.stride(2),
            k_pool.stride(0), k_pool.stride(1), k_pool.stride(2),
            out.stride(0), out.stride(1), out.stride(2), scale)
    return fn, args, out, dev_index

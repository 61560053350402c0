"""Run the reference's own CUDA decode kernels (compiled by `oracle/build_ref.py`
into `oracle/_ref/*.cubin`) on the current GPU, launched the way the reference's
host code launches them (kernels/cuda/paged_decode_cuda.py:202-252: grid
(B, splits, H), one warp per program, partial states `[B, H, S, 16, D]` /
`[B, H, S, 16]`, m filled with -inf and l with 0 before every launch), and merged
with the torch form of its combine (kernels/gqa/paged_decode.py:689-706).

Test / measurement infrastructure: used by the GPU tests (to check that the
kernel is driven correctly) and by `bench.py`'s baseline leg (to time "the
reference's kernel on this box"). The product never imports this module.
"""

from __future__ import annotations

import ctypes
import math
import pathlib
from typing import Optional

import torch

REF_DIR = pathlib.Path(__file__).resolve().parent / "_ref"
TARGET_WARPS, MAX_SPLITS = 960, 128          # kernels/cuda/paged_decode_cuda.py:41-42
_FUNCS: dict = {}


def available(name: str = "paged_decode_fp16") -> bool:
    return (REF_DIR / f"{name}.cubin").exists()


def _check(res):
    err = res[0]
    if int(err) != 0:
        raise RuntimeError(f"CUDA driver error {err}")
    return res[1] if len(res) == 2 else res[1:]


def _function(name: str, module: Optional[str] = None):
    """Kernel `name` of `oracle/_ref/<module>.cubin` (module = name by default)."""
    from cuda.bindings import driver

    dev = torch.cuda.current_device()
    key = (name, module or name, dev)
    if key not in _FUNCS:
        torch.cuda.init()
        torch.zeros(1, device="cuda")                      # make sure the primary context is current
        data = (REF_DIR / f"{module or name}.cubin").read_bytes()
        mod = _check(driver.cuModuleLoadData(data))
        _FUNCS[key] = (mod, _check(driver.cuModuleGetFunction(mod, name.encode())))
    return _FUNCS[key][1]


def choose_splits(batch: int, kv_heads: int, num_pages: int) -> int:
    """The reference's rule (kernels/cuda/paged_decode_cuda.py:197-199)."""
    return max(1, min(num_pages, MAX_SPLITS, -(-TARGET_WARPS // max(1, batch * kv_heads))))


class RefDecode:
    """Scratch + argument list for one (shape, pools) combination; `launch()`
    enqueues the fills and the kernel on torch's current stream."""

    def __init__(self, q, k_pool, v_pool, block_tables, seq_lens, max_seq_len: int,
                 softmax_scale: Optional[float] = None, k_scale=None, v_scale=None, k_residual=None,
                 res_rows=None):
        b, h, r, d = q.shape
        self.int8 = k_pool.dtype == torch.int8
        self.name = "paged_decode_int8" if self.int8 else "paged_decode_fp16"
        self.fn = _function(self.name)
        num_pages = -(-max_seq_len // k_pool.shape[1])
        self.splits = choose_splits(b, h, num_pages)
        self.shape = (b, h, r, d)
        dev = q.device
        self.acc = torch.empty((b, h, self.splits, 16, d), dtype=torch.float32, device=dev)
        self.m = torch.empty((b, h, self.splits, 16), dtype=torch.float32, device=dev)
        self.l = torch.empty((b, h, self.splits, 16), dtype=torch.float32, device=dev)
        scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
        P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
        vals = [q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), block_tables.data_ptr(),
                seq_lens.data_ptr(), self.acc.data_ptr(), self.m.data_ptr(), self.l.data_ptr()]
        types = [P] * 8
        if self.int8:
            vals += [k_scale.data_ptr(), v_scale.data_ptr(), 0, 0,
                     k_residual.data_ptr() if k_residual is not None else 0,
                     res_rows.data_ptr() if res_rows is not None else 0]
            types += [P] * 6
        vals += [block_tables.shape[1], self.splits, *q.stride()[:3], *k_pool.stride()[:3]]
        types += [I, I] + [L] * 6
        if self.int8:
            res_st = k_residual.stride()[:3] if k_residual is not None else (0, 0, 0)
            vals += [*k_scale.stride()[:2], *v_scale.stride()[:3], *res_st]
            types += [L] * 8
        vals += [*self.acc.stride()[:4], *self.m.stride()[:3], scale]
        types += [L] * 7 + [F]
        self.params = (tuple(vals), tuple(types))
        self.keep = (q, k_pool, v_pool, block_tables, seq_lens, k_scale, v_scale, k_residual, res_rows)

    def launch(self) -> None:
        from cuda.bindings import driver

        b, h, _, _ = self.shape
        self.m.fill_(float("-inf"))                        # the reference fills both on every call
        self.l.zero_()
        stream = torch.cuda.current_stream().cuda_stream
        _check(driver.cuLaunchKernel(self.fn, b, self.splits, h, 32, 1, 1, 0, stream, self.params, 0))

    def combine(self) -> torch.Tensor:
        """out = sum_s acc_s e^(m_s - M) / max(sum_s l_s e^(m_s - M), 1e-20)  (torch form of the merge)."""
        r = self.shape[2]
        m, l, acc = self.m[..., :r], self.l[..., :r], self.acc[..., :r, :]
        mg = m.amax(dim=2, keepdim=True)
        w = torch.where(torch.isinf(mg) & (mg < 0), torch.zeros_like(m), torch.exp(m - mg))
        den = (l * w).sum(dim=2).clamp_min(1e-20)
        return ((acc * w.unsqueeze(-1)).sum(dim=2) / den.unsqueeze(-1)).to(torch.float16)


class RefSparse:
    """The reference's sparse trio for one layer call, as its host code runs it
    (kernels/cuda/paged_sparse.py:104-123, 164-168, 185-251): `page_index` (grid
    (B, H, ceil(max_pages / 64)), 128 threads), `torch.topk(sorted=True)` with the
    cast to int32, then `paged_sparse_fp16` (grid (B, splits, H), one warp) after
    the fills of its m / l scratch. `launch()` enqueues all of it on torch's current
    stream; `combine()` is the torch form of the merge (the reference's is Triton)."""

    def __init__(self, q, k_pool, v_pool, block_tables, seq_lens, kmin, kmax, ratio: float,
                 max_seq_len: int, recent: int = 2, softmax_scale: Optional[float] = None):
        b, h, r, d = q.shape
        self.shape = (b, h, r, d)
        self.index_fn = _function("page_index", "paged_sparse_fp16")
        self.attend_fn = _function("paged_sparse_fp16")
        self.max_pages = block_tables.shape[1]
        pages = min(self.max_pages, -(-max_seq_len // k_pool.shape[1]))
        self.k = pages if ratio >= 1.0 else min(pages, max(recent + 1, math.ceil(ratio * pages)))
        self.splits = max(1, min(choose_splits(b, h, self.k), self.k))
        dev = q.device
        self.scores = torch.empty((b, h, self.max_pages), dtype=torch.float32, device=dev)
        self.acc = torch.empty((b, h, self.splits, 16, d), dtype=torch.float32, device=dev)
        self.m = torch.empty((b, h, self.splits, 16), dtype=torch.float32, device=dev)
        self.l = torch.empty((b, h, self.splits, 16), dtype=torch.float32, device=dev)
        self.sel = torch.zeros((b, h, self.k), dtype=torch.int32, device=dev)
        scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
        P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
        self.index_params = (
            (q.data_ptr(), kmin.data_ptr(), kmax.data_ptr(), block_tables.data_ptr(), seq_lens.data_ptr(),
             self.scores.data_ptr(), self.max_pages, recent, *q.stride()[:3], *kmin.stride()[:2],
             *self.scores.stride()[:2]),
            (P,) * 6 + (I, I) + (L,) * 7)
        self.attend_params = (
            (q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), block_tables.data_ptr(),
             seq_lens.data_ptr(), self.sel.data_ptr(), float(ratio), recent, self.acc.data_ptr(),
             self.m.data_ptr(), self.l.data_ptr(), self.max_pages, self.k, self.splits, *q.stride()[:3],
             *k_pool.stride()[:3], *self.sel.stride()[:2], *self.acc.stride()[:4], *self.m.stride()[:3],
             scale),
            (P,) * 6 + (F, I) + (P,) * 3 + (I,) * 3 + (L,) * 15 + (F,))
        self.keep = (q, k_pool, v_pool, block_tables, seq_lens, kmin, kmax)

    def launch(self) -> None:
        from cuda.bindings import driver

        b, h, _, _ = self.shape
        stream = torch.cuda.current_stream().cuda_stream
        grid_z = -(-self.max_pages // 64)
        _check(driver.cuLaunchKernel(self.index_fn, b, h, grid_z, 128, 1, 1, 0, stream, self.index_params, 0))
        self.sel.copy_(torch.topk(self.scores, self.k, dim=-1, sorted=True).indices)    # topk + cast to int32
        self.m.fill_(float("-inf"))
        self.l.zero_()
        _check(driver.cuLaunchKernel(self.attend_fn, b, self.splits, h, 32, 1, 1, 0, stream,
                                     self.attend_params, 0))

    combine = RefDecode.combine

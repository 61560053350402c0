"""Page-sparse decode attention on the sm_100a kernels — host side.

Mirrors the reference's `kernels/cuda/paged_sparse.py` (`budget` :74-78,
`rebuild_bounds` :81-85, `update_bounds` :88-101, `page_scores` :104-123,
`page_scores_mass` :126-161, `select` :164-168, `budgets` :171-182,
`sparse_decode` :185-219, `sparse_attention` :222-251): index, select, attend.

Two differences a caller can observe, both tightenings:
  * `select` is this library's own top-k kernel and its order is fully
    specified: score descending, ties to the lower page index (the reference
    calls `torch.topk`, whose tie order is unspecified);
  * the scores it ranks are reproducible bit for bit on a CPU (the kernel keeps
    the reference kernel's fp32 evaluation order).
"""

from __future__ import annotations

import math
from typing import Optional

import torch

from latentserve_b200 import _lib
from latentserve_b200 import paged_decode_cuda as pdc


def budget(ratio: float, max_pages: int, recent: int = 2) -> int:
    """Pages kept per (sequence, KV head): at least the sink and recent ones."""
    if ratio >= 1.0:
        return max_pages
    return min(max_pages, max(recent + 1, math.ceil(ratio * max_pages)))


def budgets(seq_lens: torch.Tensor, ratio: float, recent: int = 2, page: int = 16) -> torch.Tensor:
    """Per-sequence page budget for its current length, as the sparse kernel
    computes it on the device (float32 product, then ceil). -> int32 [B]."""
    pages = (seq_lens.to(torch.int64) + page - 1) // page
    if ratio >= 1.0:
        return pages.to(torch.int32)
    prod = torch.tensor(ratio, dtype=torch.float32, device=pages.device) * pages.to(torch.float32)
    n = torch.ceil(prod).to(torch.int64).clamp(min=recent + 1)
    return torch.minimum(n, pages).to(torch.int32)


def rebuild_bounds(k_pool: torch.Tensor, kmin: torch.Tensor, kmax: torch.Tensor) -> None:
    """Every block's bounds from the pool, over all rows of the page. For
    set-up and tests; a live cache maintains them as it appends."""
    kmin.copy_(k_pool.amin(dim=1))
    kmax.copy_(k_pool.amax(dim=1))


def update_bounds(k_new: torch.Tensor, slots: torch.Tensor, kmin: torch.Tensor,
                  kmax: torch.Tensor, page: int = 16) -> None:
    """k_new [B, H, D] (or [B, H, 1, D]) just written at flat `slots` [B]:
    reset the page's bounds at offset 0, widen them otherwise. Bounds only —
    the cache's own append does the scatter and this update in one launch."""
    from latentserve_b200 import kv_write

    kv_write.update_bounds_only(k_new, slots, kmin, kmax, page)


def page_scores(q, kmin, kmax, block_tables, seq_lens, recent: int = 2) -> torch.Tensor:
    """-> [B, H, max_pages] fp32: bound per page, +inf forced for the first and
    the `recent` last pages, -inf past the end."""
    b, h, n_rep, d = q.shape
    max_pages = block_tables.shape[1]
    scores = pdc.scratch("sparse_scores", (b, h, max_pages), torch.float32, q.device)
    rc = _lib.lib().ls_page_index(
        q.data_ptr(), kmin.data_ptr(), kmax.data_ptr(), block_tables.data_ptr(),
        seq_lens.data_ptr(), scores.data_ptr(), b, h, n_rep, d, 16, max_pages,
        block_tables.stride(0), kmin.shape[0], recent,
        q.stride(0), q.stride(1), q.stride(2), kmin.stride(0), kmin.stride(1),
        scores.stride(0), scores.stride(1), _lib.current_stream(q.device))
    _lib.check(rc, "page_scores")
    return scores


def page_scores_mass(q, kmin, kmax, block_tables, seq_lens, recent: int = 2,
                     softmax_scale: Optional[float] = None, page: int = 16) -> torch.Tensor:
    """Summed-mass scores [B, H, max_pages]: each query head's bounds turned
    into estimated attention weights (softmax over pages of bound * scale +
    log(tokens in the page)) and summed over the group. The per-head bounds
    come from this library's kernel; the small softmax over pages is torch, as
    in the reference."""
    b, h, n_rep, d = q.shape
    max_pages = block_tables.shape[1]
    heads = pdc.scratch("sparse_heads", (b, h, n_rep, max_pages), torch.float32, q.device)
    rc = _lib.lib().ls_page_index_heads(
        q.data_ptr(), kmin.data_ptr(), kmax.data_ptr(), block_tables.data_ptr(),
        seq_lens.data_ptr(), heads.data_ptr(), b, h, n_rep, d, page, max_pages,
        block_tables.stride(0), kmin.shape[0],
        q.stride(0), q.stride(1), q.stride(2), kmin.stride(0), kmin.stride(1),
        heads.stride(0), heads.stride(1), heads.stride(2), _lib.current_stream(q.device))
    _lib.check(rc, "page_scores_mass")
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
    idx = torch.arange(max_pages, device=q.device)
    lens = seq_lens.to(torch.int64)[:, None]
    counts = (lens - idx[None, :] * page).clamp(0, page).to(torch.float32)
    logits = heads * scale + torch.log(counts)[:, None, None, :]
    score = torch.softmax(logits, dim=-1).sum(dim=2)
    pages = (lens + page - 1) // page
    forced = (idx[None, :] == 0) | ((idx[None, :] >= pages - recent) & (idx[None, :] < pages))
    score = torch.where(forced[:, None, :], torch.full_like(score, float("inf")), score)
    return torch.where((idx[None, :] >= pages)[:, None, :],
                       torch.full_like(score, float("-inf")), score)


def select(scores: torch.Tensor, k: int, sorted: bool = True) -> torch.Tensor:
    """Top-k pages per (sequence, head) -> int32 [B, H, k], always ordered:
    score descending, ties to the lower page index."""
    b, h, n = scores.shape
    if not 0 < k <= n:
        raise ValueError(f"k must be in [1, {n}], got {k}")
    if scores.stride(-1) != 1 or scores.dtype != torch.float32:
        raise ValueError("scores must be fp32 with a unit-stride page axis")
    sel = pdc.scratch("sparse_sel", (b, h, k), torch.int32, scores.device)
    rc = _lib.lib().ls_topk_pages(scores.data_ptr(), sel.data_ptr(), b, h, n, k,
                                  scores.stride(0), scores.stride(1), sel.stride(0), sel.stride(1),
                                  _lib.current_stream(scores.device))
    _lib.check(rc, "select")
    return sel


def select_for_attention(scores: torch.Tensor, seq_lens: torch.Tensor, k: int, ratio: Optional[float],
                         recent: int = 2) -> torch.Tensor:
    """The pages `sparse_decode(..., ratio=ratio)` would attend out of
    `select(scores, k)`: per (sequence, head) the n best pages, n = that
    sequence's own budget, in ascending page order, then -1 up to k. Same set as
    the first n entries of the sorted selection (ties to the lower page), without
    sorting the row. -> int32 [B, H, k]."""
    b, h, n = scores.shape
    if not 0 < k <= n:
        raise ValueError(f"k must be in [1, {n}], got {k}")
    if scores.stride(-1) != 1 or scores.dtype != torch.float32:
        raise ValueError("scores must be fp32 with a unit-stride page axis")
    if seq_lens.dtype != torch.int32:
        raise ValueError("sequence lengths must be int32")
    sel = pdc.scratch("sparse_sel_set", (b, h, k), torch.int32, scores.device)
    rc = _lib.lib().ls_select_pages(scores.data_ptr(), seq_lens.data_ptr(), sel.data_ptr(), b, h, n, k,
                                    0.0 if ratio is None else float(ratio), recent,
                                    scores.stride(0), scores.stride(1), sel.stride(0), sel.stride(1),
                                    _lib.current_stream(scores.device))
    _lib.check(rc, "select_for_attention")
    return sel


def index_and_select(q, kmin, kmax, block_tables, seq_lens, k: int, ratio: Optional[float],
                     recent: int = 2):
    """`page_scores` then `select_for_attention` behind one library call. Same
    scores, same pages. -> (scores fp32 [B, H, max_pages], sel int32 [B, H, k]). With
    programmatic launch on (`paged_decode_cuda.set_programmatic_launch`) the page
    bounds are requested while the previous kernel of the stream drains; they are
    never a sequence's last page's, the only bounds a decode step's append changes."""
    b, h, n_rep, d = q.shape
    max_pages = block_tables.shape[1]
    if not 0 < k <= max_pages:
        raise ValueError(f"k must be in [1, {max_pages}], got {k}")
    if seq_lens.dtype != torch.int32 or block_tables.dtype != torch.int32:
        raise ValueError("block tables and sequence lengths must be int32")
    scores = pdc.scratch("sparse_scores", (b, h, max_pages), torch.float32, q.device)
    sel = pdc.scratch("sparse_sel_set", (b, h, k), torch.int32, q.device)
    rc = _lib.lib().ls_page_index_select(
        q.data_ptr(), kmin.data_ptr(), kmax.data_ptr(), block_tables.data_ptr(), seq_lens.data_ptr(),
        scores.data_ptr(), sel.data_ptr(), b, h, n_rep, d, 16, max_pages,
        block_tables.stride(0), kmin.shape[0], recent, k, 0.0 if ratio is None else float(ratio),
        pdc.dense_launch_flags(), q.stride(0), q.stride(1), q.stride(2), kmin.stride(0), kmin.stride(1),
        scores.stride(0), scores.stride(1), sel.stride(0), sel.stride(1), _lib.current_stream(q.device))
    _lib.check(rc, "index_and_select")
    return scores, sel


def sparse_decode(q, k_pool, v_pool, block_tables, seq_lens, sel,
                  num_splits: Optional[int] = None,
                  softmax_scale: Optional[float] = None,
                  ratio: Optional[float] = None, recent: int = 2,
                  k_scale=None, v_scale=None, k_residual=None, res_rows=None) -> torch.Tensor:
    """Attention over the pages in `sel` [B, H, K] only. With `ratio`, each
    sequence attends the first n entries its own length is owed (computed on
    the device); entries that are not pages of the sequence are skipped.
    INT8 pools (symmetric; an extension, the reference's sparse path is fp16
    only) take `k_scale`, `v_scale` and, for the still-filling last page,
    `k_residual` / `res_rows`, as `paged_decode_attention` does."""
    if not q.is_cuda:
        raise RuntimeError("latentserve_b200 has no CPU path: tensors must be on a CUDA device")
    b, h, n_rep, d = q.shape
    if q.stride(-1) != 1 or k_pool.stride(-1) != 1 or v_pool.stride() != k_pool.stride():
        raise ValueError("the CUDA kernel needs unit-stride head dims and matching K/V pools")
    if sel.dtype != torch.int32 or sel.stride(-1) != 1:
        raise ValueError("the selection must be int32 with a unit-stride last axis")
    if block_tables.dtype != torch.int32 or seq_lens.dtype != torch.int32:
        raise ValueError("block tables and sequence lengths must be int32")
    num_sel = sel.shape[-1]
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
    int8 = k_pool.dtype == torch.int8
    chunks = pdc.choose_chunks(q.device, h, num_splits, b,
                               pdc.INT8_CTAS_PER_SM if int8 else pdc.CTAS_PER_SM)
    tag = "sparse_i8" if int8 else "sparse"
    acc, m, l, seg = pdc._partials(q, chunks, tag)
    out = pdc.scratch(tag + "_out", (b, h, n_rep, d), q.dtype, q.device)
    flags = pdc.launch_flags() | (pdc.int8_loader_flags() if int8 else pdc.loader_flags())
    ratio_f = 0.0 if ratio is None else float(ratio)
    ptr = _lib.ptr
    if int8:
        if not pdc.eligible(q, k_pool, k_scale, k_residual, v_scale=v_scale, res_rows=res_rows):
            raise ValueError("INT8 pools need fp32 k_scale / v_scale (and k_residual with res_rows) in the "
                             "layouts paged_decode_attention takes")
        res_st = k_residual.stride()[:3] if k_residual is not None else (0, 0, 0)
        rc = _lib.lib().ls_paged_sparse_int8(
            sel.data_ptr(), ratio_f, recent, num_sel, sel.stride(0), sel.stride(1),
            q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), block_tables.data_ptr(),
            seq_lens.data_ptr(), k_scale.data_ptr(), v_scale.data_ptr(), 0, 0, ptr(k_residual),
            ptr(res_rows), acc.data_ptr(), m.data_ptr(), l.data_ptr(), seg.data_ptr(), out.data_ptr(),
            b, h, n_rep, d, k_pool.shape[1], block_tables.stride(0), k_pool.shape[0],
            0 if k_residual is None else k_residual.shape[0], chunks, pdc.MIN_CHUNK_PAGES, flags,
            q.stride(0), q.stride(1), q.stride(2),
            k_pool.stride(0), k_pool.stride(1), k_pool.stride(2),
            k_scale.stride(0), k_scale.stride(1),
            v_scale.stride(0), v_scale.stride(1), v_scale.stride(2),
            *res_st, out.stride(0), out.stride(1), out.stride(2), scale,
            _lib.current_stream(q.device))
    else:
        if k_scale is not None or k_residual is not None:
            raise ValueError("fp16 pools take no scales or residual")
        rc = _lib.lib().ls_paged_sparse_fp16(
            q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), block_tables.data_ptr(),
            seq_lens.data_ptr(), sel.data_ptr(), ratio_f, recent,
            acc.data_ptr(), m.data_ptr(), l.data_ptr(), seg.data_ptr(), out.data_ptr(),
            b, h, n_rep, d, k_pool.shape[1], block_tables.stride(0), k_pool.shape[0], num_sel,
            chunks, pdc.MIN_CHUNK_PAGES, flags,
            q.stride(0), q.stride(1), q.stride(2),
            k_pool.stride(0), k_pool.stride(1), k_pool.stride(2),
            sel.stride(0), sel.stride(1), out.stride(0), out.stride(1), out.stride(2),
            scale, _lib.current_stream(q.device))
    _lib.check(rc, "sparse_decode")
    return out


def sparse_attention(q, k_pool, v_pool, block_tables, seq_lens, kmin, kmax,
                     ratio: float = 0.25, recent: int = 2,
                     num_splits: Optional[int] = None, max_seq_len: Optional[int] = None,
                     softmax_scale: Optional[float] = None,
                     scoring: str = "bounds", k_scale=None, v_scale=None, k_residual=None,
                     res_rows=None) -> torch.Tensor:
    """Index, select, attend. ratio >= 1 still runs all three. The budget
    follows `max_seq_len` (the context) when given, else the table's width.
    The INT8 arguments are passed through to `sparse_decode`."""
    page = k_pool.shape[1]
    pages = block_tables.shape[1] if max_seq_len is None else min(
        block_tables.shape[1], -(-max_seq_len // page))
    k = budget(ratio, pages, recent)
    # The reference sorts (`select(scores, k, sorted=True)`) and lets each sequence attend the
    # first n entries it is owed; the same n pages are picked here without the sort, and for
    # the bounds scoring by the index kernel itself.
    if scoring == "mass":
        scores = page_scores_mass(q, kmin, kmax, block_tables, seq_lens, recent, softmax_scale,
                                  page=page)
        sel = select_for_attention(scores, seq_lens, k, ratio, recent)
    elif scoring == "bounds":
        _, sel = index_and_select(q, kmin, kmax, block_tables, seq_lens, k, ratio, recent)
    else:
        raise ValueError(f"unknown scoring {scoring!r}")
    return sparse_decode(q, k_pool, v_pool, block_tables, seq_lens, sel, num_splits,
                         softmax_scale, ratio=ratio, recent=recent, k_scale=k_scale, v_scale=v_scale,
                         k_residual=k_residual, res_rows=res_rows)

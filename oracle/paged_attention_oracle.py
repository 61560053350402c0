"""CPU oracle for the paged decode-attention path. TEST INFRASTRUCTURE ONLY.

Nothing in `latentserve_b200/` imports this file; only `tests/`,
`__graft_entry__.smoke()` and `bench.py`'s CPU-baseline leg do, and only as the
checker. It restates, in numpy, the algorithm of the reference's own CPU route:

    paged_decode_blockwise   kernels/gqa/paged_decode.py:151-269  (block walk, online softmax,
                                                                   split merge, INT8 dequant, residual)
    paged_decode             the same function evaluated as gather-then-softmax
                             (cache/paged_cache.py:486-506 + model/attention/gqa.py:157-188)
    combine_splits           kernels/gqa/paged_decode.py:689-706
    quantize_v_rows          cache/int8_paged_cache.py:738-766 (V: per token, head)
    quantize_k_blocks        cache/int8_paged_cache.py:670-699 (K: per block, head, channel)
    page_min_max             cache/paged_cache.py:467-484, kernels/cuda/paged_sparse.py:81-85
    page_scores              kernels/cuda/paged_sparse_fp16.cu:78-130 (kernel evaluation order)
                             == model/attention/sparse.py:57-74 page_bounds(...).amax up to rounding
    budget / budgets         kernels/cuda/paged_sparse.py:74-78, 171-182
    select                   kernels/cuda/paged_sparse.py:164-168 with ties fixed to the lower index
    sparse_decode            kernels/cuda/paged_sparse_fp16.cu:205-364 (which entries are attended)

Pinned: `tests/test_oracle_golden.py` checks every function here against
fixtures under `tests/golden/` that were produced by importing the reference
itself (`tests/golden/make_golden.py`). One point cannot be pinned on a CPU and
is stated instead: on a GPU, PyTorch evaluates `t / 127` as `t * fp32(1/127)`
(the reference documents and reproduces this, kernels/cuda/int8_write.cu:16-22),
so `quantize_*` take `reciprocal=True` for the GPU arithmetic and
`reciprocal=False` for the CPU arithmetic that the fixtures hold.
"""

from __future__ import annotations

import math

import numpy as np

F32 = np.float32
PAGE = 16


def _f32(x):
    return np.asarray(x, dtype=F32)


# ---------------------------------------------------------------------------
# Dequantisation (kernels/gqa/paged_decode.py:122-148)
def dequant_k(k_q, scale, zero):
    """k_q [PAGE, D]; scale / zero [D] of this (block, head)."""
    if scale is None:
        return _f32(k_q)
    out = _f32(k_q) * _f32(scale)[None, :]
    return out + _f32(zero)[None, :] if zero is not None else out


def dequant_v(v_q, scale, zero):
    """v_q [PAGE, D]; scale / zero [PAGE] of this (block, head)."""
    if scale is None:
        return _f32(v_q)
    out = _f32(v_q) * _f32(scale)[:, None]
    return out + _f32(zero)[:, None] if zero is not None else out


def _page_kv(i, head, p, num_pages, k_pool, v_pool, tables, k_scale, v_scale, k_zero, v_zero,
             k_residual, res_rows):
    blk = int(tables[i, p])
    if k_residual is not None and p == num_pages - 1:
        k = _f32(k_residual[int(res_rows[i]), :, head])
    else:
        k = dequant_k(k_pool[blk, :, head], None if k_scale is None else k_scale[blk, head],
                      None if k_zero is None else k_zero[blk, head])
    v = dequant_v(v_pool[blk, :, head], None if v_scale is None else v_scale[blk, :, head],
                  None if v_zero is None else v_zero[blk, :, head])
    return k, v


def combine_splits(part_acc, part_m, part_l):
    """part_acc [S, R, D]; part_m / part_l [S, R] -> [R, D]."""
    m_g = part_m.max(axis=0)
    with np.errstate(invalid="ignore"):
        w = np.where(np.isinf(m_g)[None, :], F32(0), np.exp(part_m - m_g[None, :])).astype(F32)
    l_t = (part_l * w).sum(axis=0)
    acc = (part_acc * w[:, :, None]).sum(axis=0)
    return acc / np.maximum(l_t, F32(1e-20))[:, None]


def paged_decode_blockwise(q, k_pool, v_pool, tables, lens, k_scale=None, v_scale=None,
                           k_zero=None, v_zero=None, num_splits=1, softmax_scale=None,
                           k_residual=None, res_rows=None):
    """The reference algorithm step for step, in fp32. Python loops: small cases only.
    q [B, H, R, D] -> fp32 [B, H, R, D]."""
    b, h_kv, n_rep, d = q.shape
    scale = F32(softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d))
    out = np.zeros((b, h_kv, n_rep, d), dtype=F32)
    for i in range(b):
        length = int(lens[i])
        num_pages = (length + PAGE - 1) // PAGE
        pps = max(1, (num_pages + num_splits - 1) // num_splits)
        for head in range(h_kv):
            qi = _f32(q[i, head])
            accs, ms, ls = [], [], []
            for s in range(num_splits):
                lo, hi = s * pps, min(s * pps + pps, num_pages)
                if lo >= hi:
                    continue
                m_i = np.full(n_rep, -np.inf, dtype=F32)
                l_i = np.zeros(n_rep, dtype=F32)
                acc = np.zeros((n_rep, d), dtype=F32)
                for p in range(lo, hi):
                    k, v = _page_kv(i, head, p, num_pages, k_pool, v_pool, tables, k_scale,
                                    v_scale, k_zero, v_zero, k_residual, res_rows)
                    valid = (p * PAGE + np.arange(PAGE)) < length
                    qk = (qi @ k.T) * scale
                    qk = np.where(valid[None, :], qk, F32(-np.inf))
                    m_new = np.maximum(m_i, qk.max(axis=-1))
                    with np.errstate(invalid="ignore"):
                        alpha = np.where(np.isinf(m_new), F32(0), np.exp(m_i - m_new)).astype(F32)
                        pw = np.where(valid[None, :], np.exp(qk - m_new[:, None]), F32(0)).astype(F32)
                    # Rows past the end may hold anything; they carry zero weight.
                    v = np.where(valid[:, None], v, F32(0))
                    l_i = l_i * alpha + pw.sum(axis=-1)
                    acc = acc * alpha[:, None] + pw @ v
                    m_i = m_new
                accs.append(acc)
                ms.append(m_i)
                ls.append(l_i)
            if accs:
                out[i, head] = combine_splits(np.stack(accs), np.stack(ms), np.stack(ls))
    return out


def gather_sequence(i, k_pool, v_pool, tables, lens, k_scale=None, v_scale=None, k_zero=None,
                    v_zero=None, k_residual=None, res_rows=None):
    """Dequantised K, V of sequence i as [H, L, D] fp32 (vectorised)."""
    length = int(lens[i])
    num_pages = (length + PAGE - 1) // PAGE
    blocks = np.asarray(tables[i, :num_pages], dtype=np.int64)
    k = _f32(k_pool[blocks])                                   # [P, PAGE, H, D]
    v = _f32(v_pool[blocks])
    if k_scale is not None:
        k = k * _f32(k_scale[blocks])[:, None]
        if k_zero is not None:
            k = k + _f32(k_zero[blocks])[:, None]
        v = v * _f32(v_scale[blocks])[..., None]
        if v_zero is not None:
            v = v + _f32(v_zero[blocks])[..., None]
    if k_residual is not None and num_pages > 0:
        k[num_pages - 1] = _f32(k_residual[int(res_rows[i])])
    hh, dd = k.shape[2], k.shape[3]
    k = k.reshape(num_pages * PAGE, hh, dd)[:length].transpose(1, 0, 2)
    v = v.reshape(num_pages * PAGE, hh, dd)[:length].transpose(1, 0, 2)
    return k, v


def _softmax_attend(qi, k, v, scale, keep=None):
    """qi [R, D], k / v [L, D], keep [L] bool or None -> [R, D] fp32."""
    if k.shape[0] == 0:
        return np.zeros((qi.shape[0], v.shape[1]), dtype=F32)
    s = (qi @ k.T) * scale
    if keep is not None:
        if not keep.any():
            return np.zeros((qi.shape[0], v.shape[1]), dtype=F32)
        s = np.where(keep[None, :], s, F32(-np.inf))
    s = s - s.max(axis=-1, keepdims=True)
    p = np.exp(s).astype(F32)
    v = np.where(np.isfinite(v), v, F32(0)) if keep is not None else v
    return (p @ v) / p.sum(axis=-1, keepdims=True)


def paged_decode(q, k_pool, v_pool, tables, lens, k_scale=None, v_scale=None, k_zero=None,
                 v_zero=None, softmax_scale=None, k_residual=None, res_rows=None):
    """Same function as `paged_decode_blockwise`, evaluated as gather-then-softmax
    in fp32. q [B, H, R, D] -> fp32 [B, H, R, D]."""
    b, h_kv, n_rep, d = q.shape
    scale = F32(softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d))
    out = np.zeros((b, h_kv, n_rep, d), dtype=F32)
    for i in range(b):
        if int(lens[i]) <= 0:
            continue
        k, v = gather_sequence(i, k_pool, v_pool, tables, lens, k_scale, v_scale, k_zero, v_zero,
                               k_residual, res_rows)
        for head in range(h_kv):
            out[i, head] = _softmax_attend(_f32(q[i, head]), k[head], v[head], scale)
    return out


# ---------------------------------------------------------------------------
# Quantize-on-write (bit-exact targets)
def _recip(x, reciprocal):
    return (F32(1.0) / F32(x)) if reciprocal else None


def _fit_sym(amax, eps, qmax, reciprocal):
    floor = np.maximum(amax, F32(eps))
    return (floor * _recip(qmax, True)) if reciprocal else (floor / F32(qmax))


def _fit_asym(lo, hi, eps, levels, reciprocal):
    span = hi - lo
    step = (span * _recip(levels, True)) if reciprocal else (span / F32(levels))
    return np.maximum(step, F32(eps))


def quantize_v_rows(v, asym=False, eps=1e-8, qmax=127.0, levels=255.0, offset=128.0,
                    reciprocal=True):
    """v [..., D] fp16 -> (int8 [..., D], step fp32 [...], zero fp32 [...] or None):
    one step per row, fitted and applied in fp32, round-half-to-even."""
    x = _f32(v)
    if not asym:
        step = _fit_sym(np.abs(x).max(axis=-1), eps, qmax, reciprocal)
        q = np.clip(np.rint(x / step[..., None]), -F32(qmax), F32(qmax)).astype(np.int8)
        return q, step.astype(F32), None
    lo, hi = x.min(axis=-1), x.max(axis=-1)
    step = _fit_asym(lo, hi, eps, levels, reciprocal)
    u = np.clip(np.rint((x - lo[..., None]) / step[..., None]), F32(0), F32(levels))
    q = (u - F32(offset)).astype(np.int8)
    zero = lo + F32(offset) * step
    return q, step.astype(F32), zero.astype(F32)


def quantize_k_blocks(data, asym=False, eps=1e-8, qmax=127.0, levels=255.0, offset=128.0,
                      reciprocal=True):
    """data [N, PAGE, H, D] fp16 -> (int8 [N, PAGE, H, D], step [N, H, D], zero or None):
    one step per (block, head, channel), fitted over the page's tokens."""
    f = _f32(data)
    if not asym:
        step = _fit_sym(np.abs(f).max(axis=1), eps, qmax, reciprocal)
        q = np.clip(np.rint(f / step[:, None]), -F32(qmax), F32(qmax)).astype(np.int8)
        return q, step.astype(F32), None
    lo, hi = f.min(axis=1), f.max(axis=1)
    step = _fit_asym(lo, hi, eps, levels, reciprocal)
    u = np.clip(np.rint((f - lo[:, None]) / step[:, None]), F32(0), F32(levels))
    q = (u - F32(offset)).astype(np.int8)
    zero = lo + F32(offset) * step
    return q, step.astype(F32), zero.astype(F32)


# ---------------------------------------------------------------------------
# Page bounds, scores, selection
def page_min_max(k_rows):
    """k_rows [n, H, D] fp16, the written rows of one page -> (min, max) [H, D] fp16."""
    return k_rows.min(axis=0), k_rows.max(axis=0)


def page_scores(q, kmin, kmax, tables, lens, recent=2, max_pages=None):
    """Quest bound per page in the sparse indexer's exact fp32 order:
    lane l sums channels 4l..4l+3 left to right from 0, then an xor butterfly
    over the 32 lanes (offsets 16, 8, 4, 2, 1), then max over query rows.
    q [B, H, R, 128] fp16; kmin / kmax [num_blocks, H, 128] fp16 -> fp32 [B, H, max_pages]."""
    b, h_kv, n_rep, d = q.shape
    assert d == 128
    max_pages = tables.shape[1] if max_pages is None else max_pages
    scores = np.full((b, h_kv, max_pages), -np.inf, dtype=F32)
    lanes = np.arange(32)
    for i in range(b):
        np_i = (int(lens[i]) + PAGE - 1) // PAGE
        np_i = min(np_i, max_pages)
        if np_i == 0:
            continue
        blocks = np.asarray(tables[i, :np_i], dtype=np.int64)
        for head in range(h_kv):
            qf = _f32(q[i, head])                                  # [R, 128]
            lo = _f32(kmin[blocks, head])                          # [P, 128]
            hi = _f32(kmax[blocks, head])
            m = np.maximum(qf[None] * lo[:, None], qf[None] * hi[:, None])   # [P, R, 128]
            m = m.reshape(np_i, n_rep, 32, 4)
            s = np.zeros((np_i, n_rep, 32), dtype=F32)
            for j in range(4):
                s = s + m[..., j]
            for off in (16, 8, 4, 2, 1):
                s = s + s[..., lanes ^ off]
            best = s[..., 0].max(axis=1)                           # [P]
            pages = np.arange(np_i)
            forced = (pages == 0) | (pages >= np_i - recent)
            scores[i, head, :np_i] = np.where(forced, F32(np.inf), best)
    return scores


def budget(ratio, max_pages, recent=2):
    if ratio >= 1.0:
        return max_pages
    return min(max_pages, max(recent + 1, math.ceil(ratio * max_pages)))


def budgets(lens, ratio, recent=2):
    """Per-sequence count the sparse kernel attends: float32 product, then ceil."""
    pages = (np.asarray(lens, dtype=np.int64) + PAGE - 1) // PAGE
    if ratio >= 1.0:
        return pages.astype(np.int32)
    prod = F32(ratio) * pages.astype(F32)
    n = np.maximum(np.ceil(prod).astype(np.int64), recent + 1)
    return np.minimum(n, pages).astype(np.int32)


def select(scores, k):
    """Indices of the k largest per row, score descending, ties to the lower
    index: a stable descending sort. scores [..., P] -> int32 [..., k]."""
    order = np.argsort(-scores.astype(np.float64), axis=-1, kind="stable")
    return order[..., :k].astype(np.int32)


def sparse_decode(q, k_pool, v_pool, tables, lens, sel, ratio=None, recent=2, softmax_scale=None,
                  k_scale=None, v_scale=None, k_residual=None, res_rows=None):
    """Attention over the first n entries of sel[b, h] that are pages of the
    sequence (n = the sequence's own budget when `ratio` is given, else all).
    -> fp32 [B, H, R, D]. With the INT8 arguments the rows are dequantised as in
    `paged_decode` (the reference has no INT8 sparse kernel; the definition is
    the same masked softmax over the same dequantised rows)."""
    b, h_kv, n_rep, d = q.shape
    scale = F32(softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d))
    out = np.zeros((b, h_kv, n_rep, d), dtype=F32)
    num_sel = sel.shape[-1]
    counts = budgets(lens, ratio, recent) if ratio is not None and ratio > 0 else None
    for i in range(b):
        length = int(lens[i])
        num_pages = (length + PAGE - 1) // PAGE
        if num_pages == 0:
            continue
        n = num_sel if counts is None else min(int(counts[i]), num_sel)
        k, v = gather_sequence(i, k_pool, v_pool, tables, lens, k_scale, v_scale, None, None, k_residual,
                               res_rows)
        for head in range(h_kv):
            keep = np.zeros(length, dtype=bool)
            for p in sel[i, head, :n]:
                if 0 <= p < num_pages:
                    keep[p * PAGE:min(length, (p + 1) * PAGE)] = True
            out[i, head] = _softmax_attend(_f32(q[i, head]), k[head], v[head], scale, keep)
    return out


# ---------------------------------------------------------------------------
# The timed CPU baseline: the reference's gather-then-softmax decode route
# (PagedKVCache.read, cache/paged_cache.py:486-506, then GQAAttention._attend,
# model/attention/gqa.py:157-188) restated with torch CPU ops so that it uses
# every host thread, as the reference's CPU route does. fp16 pools only.
def paged_decode_torch_cpu(q, k_pool, v_pool, tables, lens, softmax_scale=None):
    """torch CPU tensors in, fp32 [B, H, R, D] out. Ragged batches are padded
    to the longest sequence and masked, as the reference's padding mask does."""
    import torch

    b, h_kv, n_rep, d = q.shape
    page = k_pool.shape[1]
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
    max_len = int(lens.max())
    pos = torch.arange(max_len)
    pages = pos // page
    slots = tables[:, pages].long() * page + (pos % page)[None, :]          # [B, L]
    flat_k = k_pool.reshape(-1, h_kv, d)
    flat_v = v_pool.reshape(-1, h_kv, d)
    k = flat_k[slots].permute(0, 2, 1, 3).float()                           # [B, H, L, D]
    v = flat_v[slots].permute(0, 2, 1, 3).float()
    scores = torch.matmul(q.float(), k.transpose(2, 3)) * scale             # [B, H, R, L]
    keep = pos[None, :] < lens[:, None].long()
    scores = scores.masked_fill(~keep[:, None, None, :], float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    v = torch.where(keep[:, None, :, None], v, torch.zeros_like(v))
    return torch.matmul(probs, v)


# ---------------------------------------------------------------------------
# The per-layer element-wise ops around attention, with the fp16 rounding
# sequence of the reference's torch forms (kernels/fused_elementwise.py:75-107).
F16 = np.float16


def _r16(x):
    """Round fp32 values to fp16 and return them as fp32: one model-dtype rounding."""
    return np.asarray(x, dtype=F32).astype(F16).astype(F32)


def rms_norm(x, weight, eps, residual=None):
    """x, residual [rows, n] fp16, weight [n] fp16 -> (y fp16, summed residual fp16 or None).
    kernels/fused_elementwise.py:75-86 (`rms_norm_ref`, `fused_add_rms_norm_ref`)."""
    s = None
    h = _f32(x)
    if residual is not None:
        s = _r16(_f32(residual) + h)
        h = s
    var = (h * h).mean(axis=-1, keepdims=True, dtype=F32)
    normed = _r16(h * (F32(1) / np.sqrt(var + F32(eps))))
    y = (_f32(weight) * normed).astype(F16)
    return y, None if s is None else s.astype(F16)


def silu_and_mul(gate_up):
    """[rows, 2 * inter] fp16 -> [rows, inter] fp16. kernels/fused_elementwise.py:89-91."""
    inter = gate_up.shape[-1] // 2
    g, u = _f32(gate_up[..., :inter]), _f32(gate_up[..., inter:])
    act = _r16(g / (F32(1) + np.exp(-g)))
    return (act * u).astype(F16)


def rope(x, cos, sin):
    """x [..., heads, 128] fp16, cos / sin broadcastable [..., 1, 128] fp16 -> fp16:
    x * cos + rotate_half(x) * sin with every product and the sum rounded to fp16.
    kernels/fused_elementwise.py:94-107 (`rope_qk_ref`)."""
    half = x.shape[-1] // 2
    xf, c, s = _f32(x), _f32(cos), _f32(sin)
    rot = np.concatenate([-xf[..., half:], xf[..., :half]], axis=-1)
    return (_r16(xf * c) + _r16(rot * s)).astype(F16)

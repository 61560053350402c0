"""The weight-streaming projection kernel (`ls_skinny_gemm`) against fp32 torch
products, with and without the fused RMSNorm / residual / SiLU * up.

Floating-point parity: fp16 operands, fp32 accumulation, one fp16 rounding of
the result. Against an fp32 product of the same fp16 operands the bound is one
fp16 rounding (2^-11 relative) plus the accumulation-order noise of an fp32 sum
over K <= 8960 terms, stated below as |got - want| <= 2e-3 * scale + 1.5e-3 * |want|,
scale = the typical magnitude of the outputs.
"""

import numpy as np
import pytest
import torch

from latentserve_b200 import fused_elementwise as fe
from latentserve_b200 import projections as pj
from tests.gpu_util import device

pytestmark = pytest.mark.gpu


def _rand(shape, scale, seed, dev):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).half().to(dev)


def _close(got, want):
    got, want = got.float(), want.float()
    scale = want.abs().mean().item() + 1e-6
    err = (got - want).abs()
    bound = 2e-3 * scale + 1.5e-3 * want.abs()
    assert torch.isfinite(got).all()
    assert bool((err <= bound).all()), f"max err {err.max().item():.3e}, scale {scale:.3e}"


def _gamma(k, seed, dev):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (1 + 0.1 * torch.randn(k, generator=g)).half().to(dev)


def _normed64(s, gamma, eps=1e-6):
    """RMSNorm of fp16 rows in fp64, nothing rounded."""
    sd = s.double()
    return sd * torch.rsqrt((sd * sd).mean(-1, keepdim=True) + eps) * gamma.double()


def _as_accurate(got, separate, exact):
    """The fused call applies the row factor 1 / rms after the product, so its
    rounding differs from the separate-kernel route (which rounds the normalised
    row to fp16 twice before the product). Both are measured against the
    unrounded fp64 result: the fused call must be as close to it as the separate
    kernels are, and close in absolute terms."""
    err_got = (got.double() - exact).abs()
    err_sep = (separate.double() - exact).abs()
    assert torch.isfinite(got).all()
    assert err_got.pow(2).mean().sqrt().item() <= 1.1 * err_sep.pow(2).mean().sqrt().item() + 1e-7
    assert err_got.max().item() <= 1.5 * err_sep.max().item() + 1e-4
    scale = exact.abs().mean().item()
    assert bool((err_got <= 1e-2 * scale + 1e-2 * exact.abs()).all()), err_got.max().item()


# (N, K) of the Qwen2.5-1.5B projections plus small odd ones.
SHAPES = [(2048, 1536), (1536, 1536), (1536, 8960), (17920, 1536), (64, 32), (96, 160), (4768, 1536)]


@pytest.mark.parametrize("m", [1, 5, 16, 17, 32])
@pytest.mark.parametrize("n,k", SHAPES)
def test_plain_product(m, n, k):
    dev = device()
    x, w = _rand((m, k), 1.0, 1, dev), _rand((n, k), 0.05, 2, dev)
    want = x.float() @ w.float().t()
    _close(pj.linear(x, w), want)


@pytest.mark.parametrize("m", [3, 16, 29])
def test_bias_and_strided_rows(m):
    dev = device()
    n, k = 2048, 1536
    xbig = _rand((m, k + 64), 1.0, 3, dev)
    x = xbig[:, 32:32 + k]                                       # row stride k + 64, offset 64 bytes
    w, b = _rand((n, k), 0.05, 4, dev), _rand((n,), 1.0, 5, dev)
    want = x.float() @ w.float().t() + b.float()
    _close(pj.linear(x, w, b), want)


@pytest.mark.parametrize("splits", [1, 2, 3, 6, 48])  # K = 1536: 48 chunks
def test_split_k_is_deterministic_and_agrees(splits):
    dev = device()
    x, w = _rand((16, 1536), 1.0, 6, dev), _rand((1536, 1536), 0.05, 7, dev)
    a = pj.linear(x, w, splits=splits).clone()
    for _ in range(5):
        assert torch.equal(pj.linear(x, w, splits=splits), a)    # same bits every launch
    _close(a, x.float() @ w.float().t())


@pytest.mark.parametrize("m", [1, 16, 31])
@pytest.mark.parametrize("with_residual", [False, True])
def test_norm_prologue(m, with_residual):
    dev = device()
    n, k = 2048, 1536
    x, r = _rand((m, k), 2.0, 8, dev), _rand((m, k), 3.0, 9, dev)
    gamma = _gamma(k, 40, dev)
    w, b = _rand((n, k), 0.05, 10, dev), _rand((n,), 0.5, 11, dev)
    if with_residual:
        h, s = fe.fused_add_rms_norm(x, r, gamma, 1e-6)
        got, s_got = pj.linear(x, w, b, norm_weight=gamma, residual=r, eps=1e-6)
        assert torch.equal(s_got, s)                              # x + residual: bit-exact
    else:
        h, s = fe.rms_norm(x, gamma, 1e-6), x
        got = pj.linear(x, w, b, norm_weight=gamma, eps=1e-6)
    separate = (h.float() @ w.float().t() + b.float()).half()
    _as_accurate(got, separate, _normed64(s, gamma) @ w.double().t() + b.double())


@pytest.mark.parametrize("m", [2, 16, 32])
def test_norm_prologue_and_swiglu_epilogue(m):
    dev = device()
    inter, k = 8960, 1536
    x, r = _rand((m, k), 1.0, 12, dev), _rand((m, k), 1.0, 13, dev)
    gamma = _gamma(k, 40, dev)
    w = _rand((2 * inter, k), 0.03, 14, dev)
    h, s = fe.fused_add_rms_norm(x, r, gamma, 1e-6)
    gu = (h.float() @ w.float().t()).half()
    want = fe.silu_and_mul(gu)
    got, s_got = pj.linear(x, w, norm_weight=gamma, residual=r, eps=1e-6, swiglu=True)
    assert torch.equal(s_got, s)
    assert got.shape == (m, inter)
    gu64 = _normed64(s, gamma) @ w.double().t()
    exact = gu64[:, :inter] * torch.sigmoid(gu64[:, :inter]) * gu64[:, inter:]
    _as_accurate(got, want, exact)


@pytest.mark.parametrize("m", [1, 16, 17, 32])
def test_residual_epilogue_feeds_the_next_norm(m):
    """o_proj-style call: product + residual with row statistics, then a normed
    projection that takes those statistics instead of reading the rows."""
    dev = device()
    x, r = _rand((m, 1536), 1.0, 23, dev), _rand((m, 1536), 2.0, 24, dev)
    w1, w2 = _rand((1536, 1536), 0.05, 25, dev), _rand((2048, 1536), 0.05, 26, dev)
    gamma = _gamma(1536, 41, dev)
    s, ss = pj.linear(x, w1, add_residual=r, want_sumsq=True)
    want_s = ((x.float() @ w1.float().t()).half().float() + r.float())
    _close(s, want_s)
    assert ss.shape == (64, 48)
    got_sq = ss.sum(1)[:m]
    want_sq = (s.float() ** 2).sum(1)                             # of the values actually stored
    assert torch.allclose(got_sq, want_sq, rtol=1e-5, atol=0)
    y = pj.linear(s, w2, norm_weight=gamma, row_sumsq=ss, eps=1e-6)
    separate = (fe.rms_norm(s, gamma, 1e-6).float() @ w2.float().t()).half()
    _as_accurate(y, separate, _normed64(s, gamma) @ w2.double().t())
    # ... and the same bits as the kernel computing the statistics itself would give,
    # up to the summation order of the squares (1 fp16 ulp of the normalised input).
    y2 = pj.linear(s, w2, norm_weight=gamma, eps=1e-6)
    _close(y2, y.float())


def test_swiglu_without_norm():
    dev = device()
    x, w = _rand((16, 512), 1.0, 15, dev), _rand((2 * 256, 512), 0.05, 16, dev)
    want = fe.silu_and_mul((x.float() @ w.float().t()).half())
    got = pj.linear(x, w, swiglu=True)
    err = (got.float() - want.float()).abs()
    assert bool((err <= 2e-3 * want.float().abs().mean() + 3e-3 * want.float().abs()).all())


def test_argument_errors():
    dev = device()
    x, w = _rand((4, 48), 1.0, 17, dev), _rand((64, 48), 1.0, 18, dev)
    with pytest.raises(ValueError):
        pj.linear(x, w)                                          # K not a multiple of 32
    x, w = _rand((4, 64), 1.0, 19, dev), _rand((40, 64), 1.0, 20, dev)
    with pytest.raises(ValueError):
        pj.linear(x, w)                                          # N not a multiple of 32
    x, w = _rand((33, 64), 1.0, 21, dev), _rand((64, 64), 1.0, 22, dev)
    with pytest.raises(ValueError):
        pj.linear(x, w)                                          # more than 32 rows
    with pytest.raises(ValueError):
        pj.linear(x[:4], w, residual=x[:4])                      # residual without a norm
    with pytest.raises(RuntimeError):
        pj.linear(x[:4].cpu(), w.cpu())


@pytest.mark.parametrize("m", [1, 16, 17, 32])
@pytest.mark.parametrize("norm", ["none", "rows", "stats"])
def test_qkv_projection_with_rope_and_append_equals_the_two_launches(m, norm):
    """`qkv_rope_append` against `linear` followed by `rope_append_fp16`: every byte it
    writes (rotated q, K and V pool rows, page bounds) is the same, rows with an
    out-of-range position or slot are left alone in the same way."""
    dev = device()
    hq, hk, k, max_pos, blocks = 12, 2, 1536, 640, 40
    n = (hq + 2 * hk) * 128
    x = _rand((m, k), 1.0, 50, dev)
    w, bias = _rand((n, k), 0.05, 51, dev), _rand((n,), 0.3, 52, dev)
    gamma = _gamma(k, 53, dev)
    g = torch.Generator(device="cpu").manual_seed(54)
    ang = torch.rand(max_pos, 64, generator=g) * 6.28
    cos = torch.cat([ang.cos(), ang.cos()], dim=1).half().to(dev)
    sin = torch.cat([ang.sin(), ang.sin()], dim=1).half().to(dev)
    positions = torch.randint(0, max_pos, (m,), generator=g).to(dev)
    perm = torch.randperm(blocks, generator=g)[:m]
    slots = (perm * 16 + torch.randint(0, 16, (m,), generator=g)).to(dev)
    if m >= 16:
        slots[3] = slots[3] // 16 * 16                 # first row of a page: bounds are reset
        slots[5] = -1                                  # nothing appended for this row
        positions[7] = max_pos                         # out of range: q and k of this row untouched
    kwargs = {}
    if norm != "none":
        kwargs["norm_weight"] = gamma
    if norm == "stats":
        # statistics as an o_proj-style call leaves them: x is that call's output
        x0, w0 = _rand((m, k), 1.0, 55, dev), _rand((k, k), 0.05, 56, dev)
        x, ss = pj.linear(x0, w0, add_residual=_rand((m, k), 1.0, 57, dev), want_sumsq=True)
        kwargs["row_sumsq"] = ss

    def fresh():
        gen = torch.Generator(device="cpu").manual_seed(58)
        pool = lambda: torch.randn(blocks * 16, hk, 128, generator=gen).half().to(dev)
        return pool(), pool(), pool() - 1.0, pool() + 1.0, torch.full((m, hq * 128), 7.0, device=dev).half()

    k1, v1, mn1, mx1, q1 = fresh()
    qkv = pj.linear(x, w, bias, **kwargs)
    fe.rope_append_fp16(qkv, cos, sin, positions, slots, q1, k1, v1, mn1.view(blocks, 16, hk, 128)[:, 0],
                        mx1.view(blocks, 16, hk, 128)[:, 0], hq, hk)
    k2, v2, mn2, mx2, q2 = fresh()
    pj.qkv_rope_append(x, w, bias, cos, sin, positions, slots, q2, k2, v2,
                       mn2.view(blocks, 16, hk, 128)[:, 0], mx2.view(blocks, 16, hk, 128)[:, 0], hq, hk, **kwargs)
    assert torch.equal(q2, q1)
    assert torch.equal(k2, k1) and torch.equal(v2, v1)
    assert torch.equal(mn2, mn1) and torch.equal(mx2, mx1)
    # ... and without bounds
    k3, v3, _, _, q3 = fresh()
    pj.qkv_rope_append(x, w, bias, cos, sin, positions, slots, q3, k3, v3, None, None, hq, hk, **kwargs)
    assert torch.equal(q3, q1) and torch.equal(k3, k1) and torch.equal(v3, v1)

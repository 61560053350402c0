"""RMSNorm, SiLU * up and RoPE + append kernels against the oracle's
restatements of the reference's torch forms (kernels/fused_elementwise.py:75-107;
the reference checks its Triton kernels the same way, tests/test_fused_elementwise.py)."""

import numpy as np
import pytest
import torch

from latentserve_b200 import cache as lc
from latentserve_b200 import fused_elementwise as fe
from oracle import paged_attention_oracle as orc
from tests.gpu_util import device

pytestmark = pytest.mark.gpu


def _dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).to(device())


def _ulps(a: torch.Tensor, b: np.ndarray) -> np.ndarray:
    """Distance in fp16 steps between two fp16 arrays (same-sign values)."""
    x = a.cpu().numpy().view(np.int16).astype(np.int32)
    y = b.view(np.int16).astype(np.int32)
    return np.abs(x - y)


@pytest.mark.parametrize("rows,n", [(16, 1536), (3, 256), (64, 8960)])
def test_rms_norm_and_residual_add(rows, n):
    rng = np.random.default_rng(rows + n)
    x = (rng.standard_normal((rows, n)) * 3).astype(np.float16)
    r = (rng.standard_normal((rows, n)) * 2).astype(np.float16)
    w = (1 + 0.1 * rng.standard_normal(n)).astype(np.float16)
    want, _ = orc.rms_norm(x, w, 1e-6)
    got = fe.rms_norm(_dev(x), _dev(w), 1e-6)
    # The row's sum of squares is added in another order: the inverse norm can differ in
    # its last fp32 bit, which moves the normalised value by one fp16 step, rarely; the
    # multiply by the weight can turn that into two steps of the result.
    d = _ulps(got, want)
    assert d.max() <= 2 and np.mean(d > 0) < 0.02
    want, want_sum = orc.rms_norm(x, w, 1e-6, residual=r)
    got, got_sum = fe.fused_add_rms_norm(_dev(x), _dev(r), _dev(w), 1e-6)
    assert np.array_equal(got_sum.cpu().numpy(), want_sum)
    d = _ulps(got, want)
    assert d.max() <= 2 and np.mean(d > 0) < 0.02


def test_rms_norm_matches_the_reference_fixture(golden_dir):
    g = np.load(golden_dir / "elementwise.npz")
    got, got_sum = fe.fused_add_rms_norm(_dev(g["x"]), _dev(g["r"]), _dev(g["w"]), 1e-6)
    assert np.array_equal(got_sum.cpu().numpy(), g["add_rms_sum"])
    assert _ulps(got, g["add_rms"]).max() <= 2
    assert _ulps(fe.rms_norm(_dev(g["x"]), _dev(g["w"]), 1e-6), g["rms"]).max() <= 2


def test_silu_and_mul(golden_dir):
    rng = np.random.default_rng(5)
    gu = (rng.standard_normal((16, 2 * 8960)) * 2).astype(np.float16)
    d = _ulps(fe.silu_and_mul(_dev(gu)), orc.silu_and_mul(gu))
    # exp() differs in the last fp32 bit: silu moves by one fp16 step, rarely, and the
    # multiply by `up` can make that two steps of the product.
    assert d.max() <= 2 and np.mean(d > 0) < 0.01
    g = np.load(golden_dir / "elementwise.npz")
    assert _ulps(fe.silu_and_mul(_dev(g["gu"])), g["silu_mul"]).max() <= 2


def _rope_inputs(b, rng, max_pos=300):
    qkv = rng.standard_normal((b, 16 * 128)).astype(np.float16)
    half = 64
    inv = 1e6 ** (-np.arange(half, dtype=np.float32) / half)
    ang = np.arange(max_pos, dtype=np.float32)[:, None] * inv[None, :]
    ang = np.concatenate([ang, ang], -1)
    return qkv, np.cos(ang).astype(np.float16), np.sin(ang).astype(np.float16)


def test_rope_append_fp16_is_bit_exact_and_updates_bounds():
    dev = device()
    rng = np.random.default_rng(9)
    spec = lc.KVCacheSpec(num_layers=1, num_kv_heads=2, head_dim=128, max_seq_len=256,
                          max_batch_size=3, device="cuda")
    cache = lc.PagedKVCache(spec, num_blocks=40)
    cache.enable_page_bounds()
    history = [[] for _ in range(3)]
    start = [0, 5, 17]
    for i, n in enumerate(start):                       # unequal positions per sequence
        for _ in range(n):
            cache.tables[i].append(1)
    _, cos, sin = _rope_inputs(3, rng)
    for step in range(20):
        qkv, _, _ = _rope_inputs(3, rng)
        cache.advance(1, slots=[0, 1, 2])
        pos = np.asarray([n - 1 for n in cache.seq_lens], dtype=np.int64)
        q_out = torch.zeros(3, 12 * 128, dtype=torch.float16, device=dev)
        wide = torch.zeros(3, 16 * 128 + 64, dtype=torch.float16, device=dev)    # a strided row
        wide[:, : 16 * 128] = _dev(qkv)
        cache.rope_write(0, wide[:, : 16 * 128], _dev(cos), _dev(sin), _dev(pos), q_out, 12)
        heads = qkv.reshape(3, 16, 128)
        c, s = cos[pos][:, None, :], sin[pos][:, None, :]
        assert np.array_equal(q_out.cpu().numpy().reshape(3, 12, 128), orc.rope(heads[:, :12], c, s))
        want_k = orc.rope(heads[:, 12:14], c, s)
        for i in range(3):
            slot = cache.tables[i].slot(int(pos[i]))
            assert np.array_equal(cache.k_pool[0].view(-1, 2, 128)[slot].cpu().numpy(), want_k[i])
            assert np.array_equal(cache.v_pool[0].view(-1, 2, 128)[slot].cpu().numpy(), heads[i, 14:16])
            history[i].append((slot, want_k[i]))
    kmin, kmax = cache.page_bounds(0)
    for i in range(3):
        by_block = {}
        for slot, k in history[i]:
            by_block.setdefault(slot // 16, []).append((slot % 16, k))
        for blk, rows in by_block.items():
            if min(o for o, _ in rows) != 0:
                continue                                # page began before this test wrote into it
            stack = np.stack([k for _, k in rows])
            assert np.array_equal(kmin[blk].cpu().numpy(), stack.min(0))
            assert np.array_equal(kmax[blk].cpu().numpy(), stack.max(0))


@pytest.mark.parametrize("asym", [False, True])
def test_rope_append_int8_is_bit_exact(asym):
    dev = device()
    rng = np.random.default_rng(11)
    spec = lc.KVCacheSpec(num_layers=1, num_kv_heads=2, head_dim=128, max_seq_len=256,
                          max_batch_size=4, device="cuda")
    cache = lc.Int8PagedKVCache(spec, num_blocks=40, asymmetric=asym)
    _, cos, sin = _rope_inputs(4, rng)
    for step in range(19):                              # crosses a page boundary: finalize runs too
        qkv, _, _ = _rope_inputs(4, rng)
        qkv[:, 14 * 128:] *= np.float16(10.0 ** rng.uniform(-2, 1))
        cache.advance(1, slots=[0, 1, 2, 3])
        pos = np.asarray([n - 1 for n in cache.seq_lens], dtype=np.int64)
        q_out = torch.zeros(4, 12 * 128, dtype=torch.float16, device=dev)
        cache.rope_write(0, _dev(qkv), _dev(cos), _dev(sin), _dev(pos), q_out, 12)
        heads = qkv.reshape(4, 16, 128)
        c, s = cos[pos][:, None, :], sin[pos][:, None, :]
        assert np.array_equal(q_out.cpu().numpy().reshape(4, 12, 128), orc.rope(heads[:, :12], c, s))
        want_k = orc.rope(heads[:, 12:14], c, s)
        vq, vs, vz = orc.quantize_v_rows(heads[:, 14:16], asym=asym, reciprocal=True)
        for i in range(4):
            slot = cache.tables[i].slot(int(pos[i]))
            assert np.array_equal(cache.residual(0)[i, int(pos[i]) % 16].cpu().numpy(), want_k[i])
            assert np.array_equal(cache.v_pool[0].view(-1, 2, 128)[slot].cpu().numpy(), vq[i])
            assert np.array_equal(cache.v_scale_pool[0].view(-1, 2)[slot].cpu().numpy(), vs[i])
            if asym:
                assert np.array_equal(cache.v_zero_pool[0].view(-1, 2)[slot].cpu().numpy(), vz[i])


def test_wrong_dtypes_and_layouts_raise():
    dev = device()
    x = torch.zeros(4, 1536, device=dev)                # fp32
    w = torch.ones(1536, dtype=torch.float16, device=dev)
    with pytest.raises(ValueError):
        fe.rms_norm(x, w, 1e-6)
    with pytest.raises(ValueError):
        fe.rms_norm(torch.zeros(4, 1532, dtype=torch.float16, device=dev), w[:1532], 1e-6)   # n % 8
    with pytest.raises(ValueError):
        fe.silu_and_mul(torch.zeros(4, 20, dtype=torch.float16))                             # CPU

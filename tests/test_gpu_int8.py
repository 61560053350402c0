"""INT8 path on the GPU: quantize-on-write and page finalisation bit-exact,
INT8 decode attention against the oracle on the dequantised cache (cases follow
the reference's tests/test_phase16_int8.py:70-141, tests/test_cuda_decode.py:174-212,
tests/test_phase14_int8_graph.py:73-167)."""

import numpy as np
import pytest
import torch

from latentserve_b200 import cache as lc
from latentserve_b200 import int8_write as iw
from latentserve_b200 import paged_decode_cuda as pdc
from oracle import paged_attention_oracle as orc
from tests.gpu_util import close, device

pytestmark = pytest.mark.gpu
CONSTS = dict(eps=1e-8, qmax=127.0, levels=255.0, offset=128.0)


def _torch_formula(v, asym):
    """The reference cache's V arithmetic as torch ops, run ON THE GPU
    (cache/int8_paged_cache.py:738-766): the second oracle for bit-exactness."""
    v_f = v.to(torch.float32)
    if asym:
        lo, hi = v_f.amin(dim=-1, keepdim=True), v_f.amax(dim=-1, keepdim=True)
        step = ((hi - lo) / 255).clamp_min(1e-8)
        u = torch.clamp(torch.round((v_f - lo) / step), 0, 255)
        return (u - 128).to(torch.int8), step.squeeze(-1), (lo + 128 * step).squeeze(-1)
    step = v_f.abs().amax(dim=-1, keepdim=True).clamp_min(1e-8) / 127
    return torch.clamp(torch.round(v_f / step), -127, 127).to(torch.int8), step.squeeze(-1), None


@pytest.mark.parametrize("asym", [False, True])
def test_decode_write_is_bit_exact(asym):
    dev = device()
    rng = np.random.default_rng(5)
    b, h, d = 256, 2, 128
    mag = np.logspace(-3, 2, b)[:, None, None, None]
    v_np = (rng.standard_normal((b, h, 1, d)) * mag).astype(np.float16)
    v_np[3] = 0                                              # all-zero rows: the eps floor
    k_np = rng.standard_normal((b, h, 1, d)).astype(np.float16)
    slots_np = rng.permutation(4 * b)[:b].astype(np.int64)
    v, k = torch.from_numpy(v_np).to(dev), torch.from_numpy(k_np).to(dev)
    slots = torch.from_numpy(slots_np).to(dev)
    res_idx = torch.arange(b, device=dev)
    flat_v = torch.zeros(4 * b, h, d, dtype=torch.int8, device=dev)
    flat_s = torch.zeros(4 * b, h, device=dev)
    flat_z = torch.zeros(4 * b, h, device=dev) if asym else None
    k_res = torch.zeros(b, h, d, dtype=torch.float16, device=dev)
    iw.decode_write(k, v, slots, res_idx, flat_v, flat_s, flat_z, k_res, asym=asym, **CONSTS)
    torch.cuda.synchronize()
    # Oracle 1: the numpy restatement with the GPU's reciprocal multiply.
    want_q, want_s, want_z = orc.quantize_v_rows(v_np[:, :, 0], asym=asym, reciprocal=True)
    assert np.array_equal(flat_v[slots].cpu().numpy(), want_q)
    assert np.array_equal(flat_s[slots].cpu().numpy(), want_s), "scales differ: check the reciprocal"
    if asym:
        assert np.array_equal(flat_z[slots].cpu().numpy(), want_z)
    assert torch.equal(k_res, k[:, :, 0])
    # Oracle 2: the reference's torch ops on this GPU.
    tq, ts, tz = _torch_formula(v[:, :, 0], asym)
    assert torch.equal(flat_v[slots], tq) and torch.equal(flat_s[slots], ts)
    if asym:
        assert torch.equal(flat_z[slots], tz)
    # Slots nothing wrote stay untouched.
    mask = torch.ones(4 * b, dtype=torch.bool, device=dev)
    mask[slots] = False
    assert (flat_v[mask] == 0).all()


@pytest.mark.parametrize("asym", [False, True])
def test_decode_write_takes_strided_projection_views(asym):
    dev = device()
    g = torch.Generator(device=dev).manual_seed(2)
    qkv = torch.randn(5, 1, 2 * 2 * 128 + 64, dtype=torch.float16, device=dev, generator=g)
    k = qkv[:, :, :256].view(5, 1, 2, 128).transpose(1, 2)      # [B, H, 1, D], non-contiguous
    v = qkv[:, :, 256:512].view(5, 1, 2, 128).transpose(1, 2)
    assert iw.eligible(k, v)
    slots = torch.tensor([9, 3, 0, 31, 17], device=dev)
    flat_v = torch.zeros(32, 2, 128, dtype=torch.int8, device=dev)
    flat_s = torch.zeros(32, 2, device=dev)
    flat_z = torch.zeros(32, 2, device=dev) if asym else None
    k_res = torch.zeros(8, 2, 128, dtype=torch.float16, device=dev)
    iw.decode_write(k, v, slots, torch.arange(5, device=dev), flat_v, flat_s, flat_z, k_res,
                    asym=asym, **CONSTS)
    want_q, want_s, _ = orc.quantize_v_rows(v[:, :, 0].cpu().numpy(), asym=asym)
    assert np.array_equal(flat_v[slots].cpu().numpy(), want_q)
    assert np.array_equal(flat_s[slots].cpu().numpy(), want_s)
    assert torch.equal(k_res[:5], k[:, :, 0])


@pytest.mark.parametrize("asym", [False, True])
def test_finalize_blocks_is_bit_exact(asym):
    dev = device()
    rng = np.random.default_rng(9)
    rows, h, d, nb = 12, 2, 128, 40
    res_np = (rng.standard_normal((rows, 16, h, d)) * np.logspace(-2, 1.5, rows)[:, None, None, None]
              ).astype(np.float16)
    res_np[2, :, 0, 5] = 0                                   # an all-zero channel
    res = torch.from_numpy(res_np).to(dev)
    pick = torch.tensor([7, 0, 11, 2, 5], device=dev)
    ids = torch.tensor([3, 39, 17, 0, 21], device=dev)
    k_pool = torch.zeros(nb, 16, h, d, dtype=torch.int8, device=dev)
    k_scale = torch.ones(nb, h, d, device=dev)
    k_zero = torch.zeros(nb, h, d, device=dev) if asym else None
    iw.finalize_blocks(res, pick, ids, k_pool, k_scale, k_zero, **CONSTS)
    torch.cuda.synchronize()
    want_q, want_s, want_z = orc.quantize_k_blocks(res_np[pick.cpu().numpy()], asym=asym)
    assert np.array_equal(k_pool[ids].cpu().numpy(), want_q)
    assert np.array_equal(k_scale[ids].cpu().numpy(), want_s)
    if asym:
        assert np.array_equal(k_zero[ids].cpu().numpy(), want_z)
    # Second oracle: the reference's torch ops on this GPU (cache/int8_paged_cache.py:683-699).
    f = res[pick].to(torch.float32)
    if asym:
        lo, hi = f.amin(dim=1), f.amax(dim=1)
        step = ((hi - lo) / 255).clamp_min(1e-8)
        q = (torch.clamp(torch.round((f - lo.unsqueeze(1)) / step.unsqueeze(1)), 0, 255) - 128).to(torch.int8)
        assert torch.equal(k_zero[ids], lo + 128 * step)
    else:
        step = f.abs().amax(dim=1).clamp_min(1e-8) / 127
        q = torch.clamp(torch.round(f / step.unsqueeze(1)), -127, 127).to(torch.int8)
    assert torch.equal(k_pool[ids], q) and torch.equal(k_scale[ids], step)
    untouched = torch.ones(nb, dtype=torch.bool, device=dev)
    untouched[ids] = False
    assert (k_pool[untouched] == 0).all() and (k_scale[untouched] == 1).all()


def _golden_state(g, asym, dev):
    t = {k: torch.from_numpy(np.ascontiguousarray(g[k])).to(dev)
         for k in ("q", "k_pool", "v_pool", "k_scale", "v_scale", "k_residual", "res_rows",
                   "block_tables", "seq_lens")}
    if asym:
        t["k_zero"] = torch.from_numpy(g["k_zero"]).to(dev)
        t["v_zero"] = torch.from_numpy(g["v_zero"]).to(dev)
    return t


@pytest.mark.parametrize("name,asym", [("int8_sym", False), ("int8_asym", True)])
def test_int8_decode_matches_the_reference_on_its_own_cache_state(name, asym, golden_dir):
    """Pools, scales, residual and tables exactly as the reference cache left
    them; expected output from the reference's paged_decode_reference."""
    g = np.load(golden_dir / f"{name}.npz")
    t = _golden_state(g, asym, device())
    got = pdc.paged_decode_cuda(
        t["q"], t["k_pool"], t["v_pool"], t["block_tables"], t["seq_lens"], int(g["seq_lens"].max()),
        k_scale=t["k_scale"], v_scale=t["v_scale"], k_zero=t.get("k_zero"), v_zero=t.get("v_zero"),
        k_residual=t["k_residual"], res_rows=t["res_rows"])
    close(got, g["out"])


def _random_int8_case(lens, asym, residual, seed):
    rng = np.random.default_rng(seed)
    h, d = 2, 128
    pages = max(1, -(-max(lens) // 16))
    nb = len(lens) * pages + 3
    k_f = (rng.standard_normal((nb, 16, h, d)) + (0.7 if asym else 0.0)).astype(np.float16)
    v_f = (rng.standard_normal((nb, 16, h, d)) * 1.5).astype(np.float16)
    kq, ks, kz = orc.quantize_k_blocks(k_f, asym=asym)
    vq, vs, vz = orc.quantize_v_rows(v_f.transpose(0, 1, 2, 3), asym=asym)     # per (blk, tok, head)
    case = dict(k_pool=kq, v_pool=vq, k_scale=ks, v_scale=vs)
    if asym:
        case.update(k_zero=kz, v_zero=vz)
    case["block_tables"] = rng.permutation(nb)[: len(lens) * pages].reshape(len(lens), pages).astype(np.int32)
    case["seq_lens"] = np.asarray(lens, dtype=np.int32)
    case["q"] = rng.standard_normal((len(lens), h, 6, d)).astype(np.float16)
    if residual:
        case["k_residual"] = rng.standard_normal((len(lens) + 2, 16, h, d)).astype(np.float16)
        case["res_rows"] = rng.permutation(len(lens) + 2)[: len(lens)].astype(np.int32)   # not the identity
    return case


@pytest.fixture(params=["tma", "cp_async"])
def loader(request):
    """Both page-loading forms of the INT8 kernel (TMA tiles for symmetric pools,
    per-lane cp.async otherwise or on request)."""
    pdc.set_loader(request.param)
    yield request.param
    pdc.set_loader("auto")


@pytest.mark.parametrize("asym", [False, True])
@pytest.mark.parametrize("residual", [False, True])
@pytest.mark.parametrize("splits", [None, 1, 3])
def test_int8_decode_matches_the_oracle(asym, residual, splits, loader):
    lens = [1024, 300, 61, 17, 1, 32, 0]
    case = _random_int8_case(lens, asym, residual, seed=21)
    extra = {k: case[k] for k in ("k_scale", "v_scale", "k_zero", "v_zero", "k_residual", "res_rows")
             if k in case}
    want = orc.paged_decode(case["q"], case["k_pool"], case["v_pool"], case["block_tables"],
                            case["seq_lens"], **extra)
    dev = device()
    t = {k: torch.from_numpy(np.ascontiguousarray(v)).to(dev) for k, v in case.items()}
    got = pdc.paged_decode_cuda(
        t["q"], t["k_pool"], t["v_pool"], t["block_tables"], t["seq_lens"], max(lens),
        num_splits=splits, k_scale=t["k_scale"], v_scale=t["v_scale"], k_zero=t.get("k_zero"),
        v_zero=t.get("v_zero"), k_residual=t.get("k_residual"), res_rows=t.get("res_rows"))
    close(got, want)
    assert pdc.error_flag(dev, len(lens), tag="cuda_i8") == 0


@pytest.mark.parametrize("seed", range(4))
def test_int8_decode_on_seeded_random_batches(seed, loader):
    """Random batch sizes and lengths over symmetric and asymmetric pools with residuals:
    the oracle's result wherever the page axis is cut."""
    rng = np.random.default_rng(700 + seed)
    batch = int(rng.integers(1, 25))
    lens = rng.integers(0, 500, size=batch)
    lens[rng.integers(0, batch)] = int(rng.integers(1500, 4000))
    for edge in (16, 17, 32, 1):
        lens[rng.integers(0, batch)] = edge
    lens = [int(x) for x in lens]
    asym = bool(seed % 2)
    case = _random_int8_case(lens, asym, True, seed=seed + 50)
    extra = {k: case[k] for k in ("k_scale", "v_scale", "k_zero", "v_zero", "k_residual", "res_rows")
             if k in case}
    want = orc.paged_decode(case["q"], case["k_pool"], case["v_pool"], case["block_tables"],
                            case["seq_lens"], **extra)
    dev = device()
    t = {k: torch.from_numpy(np.ascontiguousarray(v)).to(dev) for k, v in case.items()}
    got = pdc.paged_decode_cuda(
        t["q"], t["k_pool"], t["v_pool"], t["block_tables"], t["seq_lens"], max(max(lens), 1),
        k_scale=t["k_scale"], v_scale=t["v_scale"], k_zero=t.get("k_zero"), v_zero=t.get("v_zero"),
        k_residual=t["k_residual"], res_rows=t["res_rows"])
    close(got, want)
    assert pdc.error_flag(dev, batch, tag="cuda_i8") == 0


@pytest.mark.parametrize("strided_scales", [False, True])
def test_int8_pools_that_are_views_of_larger_tensors(strided_scales, loader):
    """Pools with head stride 128 inside a 3-head allocation (tensor maps describe them;
    with strided V scales the TMA loader does not apply and the cp.async form runs)."""
    lens = [500, 77, 16]
    case = _random_int8_case(lens, False, True, seed=41)
    extra = {k: case[k] for k in ("k_scale", "v_scale", "k_residual", "res_rows")}
    want = orc.paged_decode(case["q"], case["k_pool"], case["v_pool"], case["block_tables"],
                            case["seq_lens"], **extra)
    dev = device()
    t = {k: torch.from_numpy(np.ascontiguousarray(v)).to(dev) for k, v in case.items()}
    nb = t["k_pool"].shape[0]

    def widen(x, axis):                                          # same values, one spare head alongside
        shape = list(x.shape)
        shape[axis] += 1
        big = torch.full(shape, 3, dtype=x.dtype, device=dev)
        view = big.narrow(axis, 0, x.shape[axis])
        view.copy_(x)
        return view

    k_pool, v_pool = widen(t["k_pool"], 2), widen(t["v_pool"], 2)
    k_scale = widen(t["k_scale"], 1)
    v_scale = widen(t["v_scale"], 2) if strided_scales else t["v_scale"]
    assert not k_pool.is_contiguous() and k_pool.shape == (nb, 16, 2, 128)
    got = pdc.paged_decode_cuda(t["q"], k_pool, v_pool, t["block_tables"], t["seq_lens"], max(lens),
                                k_scale=k_scale, v_scale=v_scale, k_residual=t["k_residual"],
                                res_rows=t["res_rows"])
    close(got, want)


def test_int8_loaders_agree_bit_for_bit():
    """TMA tiles (K and V of a page by one copy, or by one each) and per-lane cp.async feed
    the same arithmetic."""
    lens = [2000, 777, 16, 15, 1]
    case = _random_int8_case(lens, False, True, seed=23)
    dev = device()
    t = {k: torch.from_numpy(np.ascontiguousarray(v)).to(dev) for k, v in case.items()}
    outs = {}
    for name in ("tma", "tma_split_kv", "cp_async"):
        pdc.set_loader(name)
        try:
            outs[name] = pdc.paged_decode_cuda(
                t["q"], t["k_pool"], t["v_pool"], t["block_tables"], t["seq_lens"], max(lens),
                k_scale=t["k_scale"], v_scale=t["v_scale"], k_residual=t["k_residual"],
                res_rows=t["res_rows"]).clone()
        finally:
            pdc.set_loader("auto")
    assert torch.equal(outs["tma"], outs["cp_async"])
    assert torch.equal(outs["tma_split_kv"], outs["cp_async"])      # K and V tiles by a copy each



@pytest.mark.parametrize("order", ["k_first", "v_first"])
def test_int8_k_and_v_tiles_by_one_copy_whatever_the_pools_address_order(order):
    """The TMA loader fetches a page's K and V tiles with one copy of a tensor map that spans
    both pools (outermost stride = their distance). K below V and V below K both give the
    cp.async form's bits."""
    lens = [1500, 333, 48, 16, 5]
    case = _random_int8_case(lens, False, True, seed=29)
    dev = device()
    t = {k: torch.from_numpy(np.ascontiguousarray(v)).to(dev) for k, v in case.items()}
    n = t["k_pool"].numel()
    gap = 4096
    arena = torch.zeros(2 * n + gap + 64, dtype=torch.int8, device=dev)
    base = (-arena.data_ptr()) % 16                           # first 16-byte aligned element
    lo = arena[base: base + n].view(t["k_pool"].shape)
    hi = arena[base + n + gap: base + 2 * n + gap].view(t["k_pool"].shape)
    k_pool, v_pool = (hi, lo) if order == "v_first" else (lo, hi)
    k_pool.copy_(t["k_pool"])
    v_pool.copy_(t["v_pool"])
    outs = {}
    for name in ("tma", "cp_async"):
        pdc.set_loader(name)
        try:
            outs[name] = pdc.paged_decode_cuda(
                t["q"], k_pool, v_pool, t["block_tables"], t["seq_lens"], max(lens),
                k_scale=t["k_scale"], v_scale=t["v_scale"], k_residual=t["k_residual"],
                res_rows=t["res_rows"]).clone()
        finally:
            pdc.set_loader("auto")
    assert torch.equal(outs["tma"], outs["cp_async"])
    assert pdc.error_flag(dev, len(lens), tag="cuda_i8") == 0

@pytest.mark.parametrize("ratio", [None, 0.5])
def test_int8_sparse_decode_matches_the_oracle(ratio, loader):
    """Attention over a page list on INT8 pools (an extension: the reference's sparse
    kernel is fp16 only) against masked softmax over the dequantised rows."""
    from latentserve_b200 import paged_sparse as ps

    lens = [700, 333, 64, 17, 0]
    case = _random_int8_case(lens, False, True, seed=31)
    rng = np.random.default_rng(32)
    pages = -(-max(lens) // 16)
    sel = np.stack([np.stack([rng.permutation(pages)[:24] for _ in range(2)]) for _ in lens]).astype(np.int32)
    sel[0, 0, 3] = -1                                            # not a page: skipped
    if 20 not in sel[1, 1]:
        sel[1, 1, 0] = 20                                        # the sequence's last page (K from the residual)
    sel[2, :, 5] = pages + 7                                     # past the table: skipped
    extra = {k: case[k] for k in ("k_scale", "v_scale", "k_residual", "res_rows")}
    want = orc.sparse_decode(case["q"], case["k_pool"], case["v_pool"], case["block_tables"],
                             case["seq_lens"], sel, ratio=ratio, **extra)
    dev = device()
    t = {k: torch.from_numpy(np.ascontiguousarray(v)).to(dev) for k, v in case.items()}
    got = ps.sparse_decode(t["q"], t["k_pool"], t["v_pool"], t["block_tables"], t["seq_lens"],
                           torch.from_numpy(sel).to(dev), ratio=ratio, k_scale=t["k_scale"],
                           v_scale=t["v_scale"], k_residual=t["k_residual"], res_rows=t["res_rows"])
    close(got, want)


def test_int8_cache_with_page_bounds_runs_the_sparse_pipeline():
    """Int8PagedKVCache keeping page bounds of the exact K: index + select + INT8
    attention at a full budget equals the dense INT8 attention; bounds equal the
    fp16 cache's for the same tokens."""
    from latentserve_b200 import cache as lc, paged_decode as pd, paged_sparse as ps

    dev = device()
    spec = lc.KVCacheSpec(num_layers=1, num_kv_heads=2, head_dim=128, max_seq_len=256,
                          max_batch_size=2, device="cuda")
    c8, c16 = lc.Int8PagedKVCache(spec, num_blocks=40), lc.PagedKVCache(spec, num_blocks=40)
    c8.enable_page_bounds()
    c16.enable_page_bounds()
    rng = np.random.default_rng(33)
    for i, n in enumerate([70, 37]):
        k = torch.from_numpy(rng.standard_normal((1, 2, n, 128)).astype(np.float16)).to(dev)
        v = torch.from_numpy(rng.standard_normal((1, 2, n, 128)).astype(np.float16)).to(dev)
        for c in (c8, c16):
            c.advance(n, slots=[i])
            c.write(0, k, v)
    for _ in range(12):                                          # decode steps across a page boundary
        k = torch.from_numpy(rng.standard_normal((2, 2, 1, 128)).astype(np.float16)).to(dev)
        v = torch.from_numpy(rng.standard_normal((2, 2, 1, 128)).astype(np.float16)).to(dev)
        for c in (c8, c16):
            c.advance(1, slots=[0, 1])
            c.write(0, k, v)
    # Same tokens, same block ids (both allocators hand out blocks in the same order).
    assert c8.tables[0].blocks == c16.tables[0].blocks and c8.tables[1].blocks == c16.tables[1].blocks
    used = sorted(set(c8.tables[0].blocks + c8.tables[1].blocks))
    assert torch.equal(c8.kmin[0][used], c16.kmin[0][used]) and torch.equal(c8.kmax[0][used], c16.kmax[0][used])
    q = torch.from_numpy(rng.standard_normal((2, 2, 6, 128)).astype(np.float16)).to(dev)
    tables, lens = c8.block_tables_tensor(2), c8.seq_lens_tensor(2)
    args = dict(k_scale=c8.k_scale_pool[0], v_scale=c8.v_scale_pool[0], k_residual=c8.residual(0),
                res_rows=c8.residual_rows_tensor(2))
    dense = pd.paged_decode_attention(q, c8.k_pool[0], c8.v_pool[0], tables, lens, max_seq_len=c8.max_len,
                                      **args).clone()
    full = ps.sparse_attention(q, c8.k_pool[0], c8.v_pool[0], tables, lens, c8.kmin[0], c8.kmax[0],
                               ratio=1.0, max_seq_len=c8.max_len, **args)
    assert (full.float() - dense.float()).abs().max() <= 2e-3


def test_int8_stale_scales_and_rows_are_never_read(loader):
    lens = [100, 37]
    case = _random_int8_case(lens, False, True, seed=22)
    extra = {k: case[k] for k in ("k_scale", "v_scale", "k_residual", "res_rows")}
    want = orc.paged_decode(case["q"], case["k_pool"], case["v_pool"], case["block_tables"],
                            case["seq_lens"], **extra)
    vs = case["v_scale"].copy()
    res = case["k_residual"].copy()
    for b, L in enumerate(lens):
        last = (L - 1) // 16
        blk = case["block_tables"][b, last]
        vs[blk, L - last * 16:] = np.nan                       # V scales of unwritten tokens
        res[case["res_rows"][b], L - last * 16:] = np.nan      # residual rows past the end
    case.update(v_scale=vs, k_residual=res)
    dev = device()
    t = {k: torch.from_numpy(np.ascontiguousarray(v)).to(dev) for k, v in case.items()}
    got = pdc.paged_decode_cuda(t["q"], t["k_pool"], t["v_pool"], t["block_tables"], t["seq_lens"],
                                max(lens), k_scale=t["k_scale"], v_scale=t["v_scale"],
                                k_residual=t["k_residual"], res_rows=t["res_rows"])
    close(got, want)


@pytest.mark.parametrize("asym", [False, True])
def test_cache_decode_steps_reproduce_the_reference_cache_bytes(asym, golden_dir):
    """Int8PagedKVCache driven exactly as make_golden.py drove the reference's
    cache (prefill 37 / 80 / 16 tokens, then 21 decode steps): every pool byte,
    scale and residual row against the oracle's quantisers in GPU arithmetic
    (the fixture's bytes were produced with CPU division), then attention."""
    name = "int8_asym" if asym else "int8_sym"
    g = np.load(golden_dir / f"{name}.npz")
    dev = device()
    spec = lc.KVCacheSpec(num_layers=1, num_kv_heads=2, head_dim=128, max_seq_len=160,
                          max_batch_size=3, device="cuda")
    cache = lc.Int8PagedKVCache(spec, num_blocks=40, asymmetric=asym)
    prompt, steps = [int(x) for x in g["prompt"]], int(g["steps"])
    fed = [(torch.from_numpy(g[f"fed_k{i}"]).to(dev), torch.from_numpy(g[f"fed_v{i}"]).to(dev))
           for i in range(3)]
    for i, n in enumerate(prompt):
        cache.advance(n, slots=[i])
        cache.write(0, fed[i][0][None, :, :n], fed[i][1][None, :, :n])
    for s in range(steps):
        cache.advance(1, slots=[0, 1, 2])
        k = torch.stack([fed[i][0][:, prompt[i] + s] for i in range(3)])[:, :, None]
        v = torch.stack([fed[i][1][:, prompt[i] + s] for i in range(3)])[:, :, None]
        cache.write(0, k, v)
    q = torch.from_numpy(g["q"]).to(dev)
    got = pdc.paged_decode_cuda(
        q, cache.k_pool[0], cache.v_pool[0], cache.block_tables_tensor(3), cache.seq_lens_tensor(3),
        cache.max_len, k_scale=cache.k_scale_pool[0], v_scale=cache.v_scale_pool[0],
        k_zero=cache.k_zero_pool[0] if asym else None, v_zero=cache.v_zero_pool[0] if asym else None,
        k_residual=cache.residual(0), res_rows=cache.residual_rows_tensor(3))
    assert cache.seq_lens == [int(x) for x in g["seq_lens"]]
    tables = cache.block_tables_tensor(3).cpu().numpy()
    for i, L in enumerate(cache.seq_lens):
        fk, fv = g[f"fed_k{i}"], g[f"fed_v{i}"]
        vq, vstep, _ = orc.quantize_v_rows(fv, asym=asym, reciprocal=True)
        for pos in range(L):
            blk, off = int(tables[i, pos // 16]), pos % 16
            assert np.array_equal(cache.v_pool[0][blk, off].cpu().numpy(), vq[:, pos])
            assert np.array_equal(cache.v_scale_pool[0][blk, off].cpu().numpy(), vstep[:, pos])
        done = L // 16 if L % 16 else L // 16 - 1
        for p in range(done):
            kq, kstep, _ = orc.quantize_k_blocks(fk[:, p * 16:(p + 1) * 16].transpose(1, 0, 2)[None],
                                                 asym=asym, reciprocal=True)
            blk = int(tables[i, p])
            assert np.array_equal(cache.k_pool[0][blk].cpu().numpy(), kq[0])
            assert np.array_equal(cache.k_scale_pool[0][blk].cpu().numpy(), kstep[0])
        tail0 = (L - 1) // 16 * 16
        assert np.array_equal(cache.residual(0)[i, :L - tail0].cpu().numpy(),
                              fk[:, tail0:L].transpose(1, 0, 2))
    # Attention over the cache's own state against the oracle on that state. (The
    # fixture's output is for CPU-arithmetic scales: GPU arithmetic moves a few
    # codes by one step, which shifts the output by up to 1e-2 in the asymmetric
    # case, so it is only a loose cross-check here.)
    extra = dict(k_scale=cache.k_scale_pool[0], v_scale=cache.v_scale_pool[0],
                 k_residual=cache.residual(0), res_rows=cache.residual_rows_tensor(3))
    if asym:
        extra.update(k_zero=cache.k_zero_pool[0], v_zero=cache.v_zero_pool[0])
    want = orc.paged_decode(g["q"], cache.k_pool[0].cpu().numpy(), cache.v_pool[0].cpu().numpy(), tables,
                            cache.seq_lens_tensor(3).cpu().numpy(),
                            **{k: v.cpu().numpy() for k, v in extra.items()})
    close(got, want)
    close(got, g["out"], atol=2e-2)


def test_finalize_pending_reads_its_count_on_the_device_and_consumes_it_once():
    """The in-step form of page finalisation: same bytes as the host-counted launch,
    the count comes from device memory, and a second launch without a new list
    changes nothing even though the residual has moved on."""
    dev = device()
    rng = np.random.default_rng(19)
    layers, rows, h, d, nb = 3, 6, 2, 128, 24
    res = torch.from_numpy((rng.standard_normal((layers, rows, 16, h, d)) * 2).astype(np.float16)).to(dev)
    pick = torch.tensor([4, 1, 5, 0, 0, 0], device=dev)              # capacity 6, three in use
    ids = torch.tensor([7, 23, 2, 0, 0, 0], device=dev)
    consts = CONSTS
    want_pool = torch.zeros(layers, nb, 16, h, d, dtype=torch.int8, device=dev)
    want_scale = torch.ones(layers, nb, h, d, device=dev)
    iw.finalize_layers(res, pick, ids, 3, want_pool, want_scale, None, **consts)
    pool, scale = torch.zeros_like(want_pool), torch.ones_like(want_scale)
    state = torch.tensor([3, 0, 0, 0], dtype=torch.int32, device=dev)
    iw.finalize_pending(res, pick, ids, state, pool, scale, None, **consts)
    torch.cuda.synchronize()
    assert torch.equal(pool, want_pool) and torch.equal(scale, want_scale)
    assert state.tolist()[:2] == [0, 0]                              # consumed, arrivals reset
    res.mul_(0.5)                                                    # the residual moves on
    iw.finalize_pending(res, pick, ids, state, pool, scale, None, **consts)
    torch.cuda.synchronize()
    assert torch.equal(pool, want_pool) and torch.equal(scale, want_scale)
    # A count past the lists' capacity is clamped; out-of-range entries are skipped.
    state.copy_(torch.tensor([99, 0, 0, 0], dtype=torch.int32))
    ids[3:] = torch.tensor([nb + 5, -1, 10_000_000], device=dev)
    iw.finalize_pending(res, pick, ids, state, pool, scale, None, **consts)
    torch.cuda.synchronize()
    untouched = torch.ones(nb, dtype=torch.bool, device=dev)
    untouched[ids[:3]] = False
    assert (pool[:, untouched] == 0).all() and state.tolist()[:2] == [0, 0]


def _int8_decode_loop(programmatic: bool, graphed: bool, in_step: bool, steps: int = 44):
    """Prefill four sequences, then `steps` decode steps of two layers (write +
    attention per layer) over an Int8PagedKVCache; returns every step's outputs and
    the cache in its final state, and the last step's queries."""
    from latentserve_b200 import paged_decode as pd

    dev = device()
    layers, batch = 2, 4
    spec = lc.KVCacheSpec(num_layers=layers, num_kv_heads=2, head_dim=128, max_seq_len=1024,
                          max_batch_size=batch, device="cuda")
    cache = lc.Int8PagedKVCache(spec, num_blocks=4 * 64 + 8)
    if in_step:
        cache.enable_finalize_in_step()
    g = torch.Generator(device=dev).manual_seed(77)
    for i, n in enumerate([700, 333, 130, 47]):                      # 47: completes a page at once
        cache.advance(n, slots=[i])
        for layer in range(layers):
            k = torch.randn(1, 2, n, 128, dtype=torch.float16, device=dev, generator=g)
            v = torch.randn(1, 2, n, 128, dtype=torch.float16, device=dev, generator=g)
            cache.write(layer, k, v)
    feed_k = torch.randn(steps, layers, batch, 2, 1, 128, dtype=torch.float16, device=dev, generator=g)
    feed_v = torch.randn(steps, layers, batch, 2, 1, 128, dtype=torch.float16, device=dev, generator=g)
    feed_q = torch.randn(steps, layers, batch, 2, 6, 128, dtype=torch.float16, device=dev, generator=g)
    k_in, v_in, q_in = feed_k[0].clone(), feed_v[0].clone(), feed_q[0].clone()
    out = torch.zeros(layers, batch, 2, 6, 128, dtype=torch.float16, device=dev)

    def body():
        for layer in range(layers):
            cache.write(layer, k_in[layer], v_in[layer])
            pd.paged_decode_attention(
                q_in[layer], cache.k_pool[layer], cache.v_pool[layer], cache.block_tables_tensor(batch),
                cache.seq_lens_tensor(batch), k_scale=cache.k_scale_pool[layer],
                v_scale=cache.v_scale_pool[layer], max_seq_len=1024, k_residual=cache.residual(layer),
                res_rows=cache.residual_rows_tensor(batch), out=out[layer])

    pdc.set_programmatic_launch(programmatic, early_pages=True)
    pd.set_decode_backend("cuda")
    outs, graph = [], None
    try:
        for s in range(steps):
            cache.advance(1, batch_size=batch)
            k_in.copy_(feed_k[s]); v_in.copy_(feed_v[s]); q_in.copy_(feed_q[s])
            if graphed and graph is None:
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    body()                                           # warm-up run of this very step
                torch.cuda.current_stream().wait_stream(side)
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    body()
            if graph is not None:
                graph.replay()
            else:
                body()
            outs.append(out.clone())
        torch.cuda.synchronize()
    finally:
        pdc.set_programmatic_launch(False)
    assert pdc.error_flag(dev, batch, tag="cuda_i8") == 0
    return outs, cache, feed_q[-1]


def test_int8_programmatic_launch_with_early_pages_across_page_finalisation(loader):
    """44 steps take every sequence across two or three page boundaries, so pages are
    quantised (rewritten) between steps while the next attention launch is already
    requesting old pages ahead of its dependency wait. Outputs and cache bytes must
    equal the plain-launch run bit for bit: eager, replayed from a graph, and with
    the finalisation inside the captured step."""
    base, c0, last_q = _int8_decode_loop(programmatic=False, graphed=False, in_step=False)
    for programmatic, graphed, in_step in [(True, False, False), (True, True, False),
                                           (True, True, True), (False, True, True),
                                           (True, False, True)]:
        got, c1, _ = _int8_decode_loop(programmatic, graphed, in_step)
        for s, (a, b) in enumerate(zip(base, got)):
            assert torch.equal(a, b), f"step {s} differs (programmatic={programmatic}, " \
                                      f"graphed={graphed}, in_step={in_step})"
        assert torch.equal(c0._k_pool_all, c1._k_pool_all) and torch.equal(c0._k_scale_all, c1._k_scale_all)
        assert all(torch.equal(a, b) for a, b in zip(c0.v_pool, c1.v_pool))
    # The reference run itself against the oracle on the cache's final state.
    layer = 1
    want = orc.paged_decode(
        last_q[layer].cpu().numpy(),
        c0.k_pool[layer].cpu().numpy(), c0.v_pool[layer].cpu().numpy(),
        c0.block_tables_tensor(4).cpu().numpy(), c0.seq_lens_tensor(4).cpu().numpy(),
        k_scale=c0.k_scale_pool[layer].cpu().numpy(), v_scale=c0.v_scale_pool[layer].cpu().numpy(),
        k_residual=c0.residual(layer).cpu().numpy(), res_rows=c0.residual_rows_tensor(4).cpu().numpy())
    close(base[-1][layer], want)


def test_int8_asymmetric_pools_at_long_contexts():
    """Asymmetric pools (zero points) at contexts where every CTA walks hundreds of pages and
    chunks span sequences: both loaders agree bit for bit, one sequence against the oracle,
    and a clean error flag."""
    lens = [8192, 5000, 8192 - 3, 300]
    case = _random_int8_case(lens, True, True, seed=31)
    dev = device()
    t = {k: torch.from_numpy(np.ascontiguousarray(v)).to(dev) for k, v in case.items()}
    outs = {}
    for name in ("tma", "cp_async"):
        pdc.set_loader(name)
        try:
            outs[name] = pdc.paged_decode_cuda(
                t["q"], t["k_pool"], t["v_pool"], t["block_tables"], t["seq_lens"], max(lens),
                k_scale=t["k_scale"], v_scale=t["v_scale"], k_zero=t["k_zero"], v_zero=t["v_zero"],
                k_residual=t["k_residual"], res_rows=t["res_rows"]).clone()
        finally:
            pdc.set_loader("auto")
    assert torch.equal(outs["tma"], outs["cp_async"])
    assert pdc.error_flag(dev, len(lens), tag="cuda_i8") == 0
    b = 1
    pages = -(-lens[b] // 16)
    blocks = case["block_tables"][b, :pages]
    row = int(case["res_rows"][b])
    want = orc.paged_decode(
        case["q"][b:b + 1], case["k_pool"][blocks], case["v_pool"][blocks],
        np.arange(pages, dtype=np.int32)[None], np.asarray([lens[b]], dtype=np.int32),
        k_scale=case["k_scale"][blocks], v_scale=case["v_scale"][blocks], k_zero=case["k_zero"][blocks],
        v_zero=case["v_zero"][blocks], k_residual=case["k_residual"][row:row + 1],
        res_rows=np.zeros(1, dtype=np.int32))
    close(outs["tma"][b:b + 1], want)

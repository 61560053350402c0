"""Page-sparse path on the GPU: page bounds, indexer scores and top-k bit-exact
against the oracle; attention over selected pages within tolerance (cases
follow the reference's tests/test_phase14_sparse_kernels.py:73-217 and
tests/test_phase17_policy.py:108-143)."""

import numpy as np
import pytest
import torch

from latentserve_b200 import cache as lc
from latentserve_b200 import kv_write
from latentserve_b200 import paged_decode_cuda as pdc
from latentserve_b200 import paged_sparse as ps
from latentserve_b200 import synthetic
from oracle import paged_attention_oracle as orc
from tests.gpu_util import close, device, on_device

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True, params=["tma", "cp_async"])
def loader(request):
    """Every test runs with both page-loading forms of the kernels (TMA tile
    copies, and per-lane cp.async)."""
    pdc.set_loader(request.param)
    yield request.param
    pdc.set_loader("auto")


def _with_bounds(case):
    t = on_device(case)
    nb, _, h, d = t["k_pool"].shape
    t["kmin"] = torch.empty(nb, h, d, dtype=torch.float16, device=device())
    t["kmax"] = torch.empty_like(t["kmin"])
    ps.rebuild_bounds(t["k_pool"], t["kmin"], t["kmax"])
    return t


def test_bounds_updated_token_by_token_equal_the_true_min_and_max():
    dev = device()
    rng = np.random.default_rng(1)
    h, d, nb = 2, 128, 8
    kmin = torch.full((nb, h, d), 99.0, dtype=torch.float16, device=dev)
    kmax = torch.full_like(kmin, -99.0)
    k_pool = torch.zeros(nb, 16, h, d, dtype=torch.float16, device=dev)
    v_pool = torch.zeros_like(k_pool)
    blocks, rows = [5, 2], {}
    for pos in range(27):
        slot = blocks[pos // 16] * 16 + pos % 16
        k_new = torch.from_numpy(rng.standard_normal((1, h, 1, d)).astype(np.float16)).to(dev)
        v_new = torch.from_numpy(rng.standard_normal((1, h, 1, d)).astype(np.float16)).to(dev)
        kv_write.append_fp16(k_new, v_new, torch.tensor([slot], device=dev), k_pool.view(-1, h, d),
                             v_pool.view(-1, h, d), kmin, kmax)
        rows.setdefault(blocks[pos // 16], []).append((pos % 16, k_new[0, :, 0], v_new[0, :, 0]))
    torch.cuda.synchronize()
    for blk, items in rows.items():
        stack = torch.stack([k for _, k, _ in items])
        assert torch.equal(kmin[blk], stack.amin(0)) and torch.equal(kmax[blk], stack.amax(0))
        for off, k, v in items:
            assert torch.equal(k_pool[blk, off], k) and torch.equal(v_pool[blk, off], v)
    # Stand-alone bounds update (rows scattered by someone else) gives the same.
    kmin2 = torch.full((nb, h, d), 99.0, dtype=torch.float16, device=dev)
    kmax2 = torch.full_like(kmin2, -99.0)
    for blk, items in rows.items():
        for off, k, _ in items:
            ps.update_bounds(k[None], torch.tensor([blk * 16 + off], device=dev), kmin2, kmax2)
    assert torch.equal(kmin2[blocks], kmin[blocks]) and torch.equal(kmax2[blocks], kmax[blocks])


@pytest.mark.parametrize("lens", [[700, 333], [32768, 4096, 17, 1, 0]])
def test_indexer_scores_are_bit_exact(lens):
    case = synthetic.dense_case(lens, seed=11, page_offset_std=0.5)
    t = _with_bounds(case)
    got = ps.page_scores(t["q"], t["kmin"], t["kmax"], t["block_tables"], t["seq_lens"], recent=2)
    want = orc.page_scores(case["q"], t["kmin"].cpu().numpy(), t["kmax"].cpu().numpy(),
                           case["block_tables"], case["seq_lens"], recent=2)
    assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("n_rep", [1, 4, 7, 8])
def test_indexer_scores_are_bit_exact_for_other_group_sizes(n_rep):
    """Groups other than six query heads per KV head take the kernel's general form
    (rows tested against the group size at run time); a warp's span of several items too."""
    case = synthetic.dense_case([2100, 640, 31], n_rep=n_rep, seed=5, page_offset_std=0.5)
    t = _with_bounds(case)
    got = ps.page_scores(t["q"], t["kmin"], t["kmax"], t["block_tables"], t["seq_lens"], recent=2)
    want = orc.page_scores(case["q"], t["kmin"].cpu().numpy(), t["kmax"].cpu().numpy(),
                           case["block_tables"], case["seq_lens"], recent=2)
    assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))


def test_indexer_scores_are_bit_exact_when_a_warp_pair_walks_several_items():
    """More (sequence, head, 128-page) spans than the GPU holds CTAs of the index kernel at
    once: each warp pair then scores several 32-page items, reusing its shared memory."""
    dev = device()
    lens = [20000 - 37 * i for i in range(40)]           # 40 x 2 heads x 10 spans = 800 CTAs at one item each
    pages = -(-max(lens) // 16)
    g = torch.Generator(device=dev).manual_seed(77)
    nb = sum(-(-x // 16) for x in lens) + 3
    kmin = torch.randn(nb, 2, 128, dtype=torch.float16, device=dev, generator=g) - 1.0
    kmax = kmin + torch.rand(nb, 2, 128, dtype=torch.float16, device=dev, generator=g) * 3
    q = torch.randn(len(lens), 2, 6, 128, dtype=torch.float16, device=dev, generator=g)
    perm = torch.randperm(nb, device=dev, generator=g).to(torch.int32)
    tables = torch.zeros(len(lens), pages, dtype=torch.int32, device=dev)
    at = 0
    for i, x in enumerate(lens):
        n = -(-x // 16)
        tables[i, :n] = perm[at:at + n]
        at += n
    seq = torch.tensor(lens, dtype=torch.int32, device=dev)
    got = ps.page_scores(q, kmin, kmax, tables, seq).cpu().numpy()
    rows = [0, 17, 39]                                    # the oracle on three of the sequences
    want = orc.page_scores(q[rows].cpu().numpy(), kmin.cpu().numpy(), kmax.cpu().numpy(),
                           tables[rows].cpu().numpy(), seq[rows].cpu().numpy())
    assert np.array_equal(got[rows].view(np.uint32), want.view(np.uint32))
    # The per-head form of the kernel (summed-mass scoring): the same three sequences scored
    # as part of the big batch and on their own (one item per warp pair) agree bit for bit.
    mass = ps.page_scores_mass(q, kmin, kmax, tables, seq)[rows].clone()
    alone = ps.page_scores_mass(q[rows].contiguous(), kmin, kmax, tables[rows].contiguous(),
                                seq[rows].contiguous())
    assert torch.equal(mass, alone)


def test_indexer_scores_against_the_reference_bounds(golden_dir):
    g = np.load(golden_dir / "sparse.npz")
    lens = [int(x) for x in g["seq_lens"]]
    t = _with_bounds(synthetic.dense_case(lens, seed=11, page_offset_std=0.5))
    scores = ps.page_scores(t["q"], t["kmin"], t["kmax"], t["block_tables"], t["seq_lens"]).cpu().numpy()
    for b, L in enumerate(lens):
        np_ = -(-L // 16)
        mid = slice(1, np_ - 2)
        np.testing.assert_allclose(scores[b, :, mid], g[f"bounds{b}"][:, mid], rtol=1e-4, atol=1e-3)
        assert np.isposinf(scores[b, :, 0]).all() and np.isposinf(scores[b, :, np_ - 2:np_]).all()
        assert np.isneginf(scores[b, :, np_:]).all()


@pytest.mark.parametrize("n,k", [(2048, 1024), (2048, 2048), (700, 44), (33, 3), (1, 1), (257, 256)])
def test_topk_is_bit_exact_with_ties_to_the_lower_index(n, k):
    rng = np.random.default_rng(n + k)
    s = rng.standard_normal((3, 2, n)).astype(np.float32)
    s[..., 0] = np.inf
    if n > 40:
        s[0, 0, 10:30] = s[0, 0, 10]                          # runs of exact ties
        s[1, 1, :] = np.round(s[1, 1, :], 1)                  # many ties everywhere
        s[..., n - n // 4:] = -np.inf                         # pages past the end
        s[..., n - n // 4 - 2:n - n // 4] = np.inf            # recent pages
        s[2, 0, 5] = -0.0
        s[2, 0, 6] = 0.0
    got = ps.select(torch.from_numpy(s).to(device()), k)
    assert np.array_equal(got.cpu().numpy(), orc.select(s, k))


@pytest.mark.parametrize("n,k,ratio", [(2048, 1024, 0.5), (2048, 2048, 1.0), (700, 44, 0.0625), (33, 3, 0.05),
                                       (1, 1, 0.5), (257, 256, None), (8192, 4096, 0.5), (5000, 1250, 0.25)])
def test_selection_without_the_sort_picks_the_same_pages(n, k, ratio):
    """`select_for_attention` against the sorted selection: per sequence the first n
    entries of the sort (n = its own budget), as a set and in ascending page order."""
    rng = np.random.default_rng(n * 7 + k)
    s = rng.standard_normal((4, 2, n)).astype(np.float32)
    lens = np.asarray([n * 16, max(1, n * 16 - 5), max(1, (n // 2) * 16 + 3), 0], dtype=np.int32)
    for b, L in enumerate(lens):                                  # what the indexer would write
        np_ = -(-int(L) // 16)
        s[b, :, np_:] = -np.inf
        if np_:
            s[b, :, 0] = np.inf
            s[b, :, max(0, np_ - 2):np_] = np.inf
    if n > 40:
        s[0, 0, 10:30] = s[0, 0, 10]                              # runs of exact ties
        s[1, 1, : n // 2] = np.round(s[1, 1, : n // 2], 1)        # many ties
        s[2, 0, 5], s[2, 0, 6] = -0.0, 0.0
    dev = device()
    got = ps.select_for_attention(torch.from_numpy(s).to(dev), torch.from_numpy(lens).to(dev), k, ratio)
    got = got.cpu().numpy()
    order = orc.select(s, k)                                      # stable descending sort, first k
    counts = orc.budgets(lens, ratio) if ratio is not None and 0 < ratio < 1 else -(-lens // 16)
    for b in range(4):
        keep = int(min(counts[b], -(-int(lens[b]) // 16), k))
        for h in range(2):
            want = np.sort(order[b, h, :keep])
            assert np.array_equal(got[b, h, :keep], want), (b, h)
            assert (got[b, h, keep:] == -1).all()


def test_selection_threshold_search_takes_both_routes():
    """The wanted score is found in one pass over equal-width buckets when its bucket holds few
    keys, and by the bit-wise search when the bucket is crowded: rows of well spread scores, of
    two values only, of one value, and of a tight cluster around a power of two all select
    exactly the first n entries of the stable sort."""
    n, k, ratio = 2048, 1024, 0.5
    rng = np.random.default_rng(99)
    s = np.empty((5, 2, n), dtype=np.float32)
    s[0] = rng.standard_normal((2, n)) * 40 + 120                 # spread over two binades
    s[1] = np.where(rng.random((2, n)) < 0.5, 3.0, 7.0)           # two values: the bucket is crowded
    s[2] = 1.5                                                    # all equal
    s[3] = 128.0 + rng.integers(-40, 40, size=(2, n)) * 2.0 ** -17    # a cluster straddling 2^7, many ties
    s[4] = rng.standard_normal((2, n)).astype(np.float32) * 1e-30     # tiny magnitudes, both signs
    lens = np.full(5, n * 16, dtype=np.int32)
    s[:, :, 0] = np.inf
    s[:, :, n - 2:] = np.inf
    dev = device()
    got = ps.select_for_attention(torch.from_numpy(s).to(dev), torch.from_numpy(lens).to(dev), k, ratio)
    got = got.cpu().numpy()
    order = orc.select(s, k)
    keep = int(orc.budgets(lens, ratio)[0])
    for b in range(5):
        for h in range(2):
            assert np.array_equal(got[b, h, :keep], np.sort(order[b, h, :keep])), (b, h)
            assert (got[b, h, keep:] == -1).all()


@pytest.mark.parametrize("seed", range(6))
def test_selection_on_seeded_random_rows_and_budgets(seed):
    """Rows of random length, score distribution and budget (spread, heavy ties, clusters around
    powers of two, both signs, tiny and huge magnitudes): the kept pages are the first n of
    the stable descending sort, in ascending page order."""
    rng = np.random.default_rng(1000 + seed)
    n = int(rng.integers(40, 8193))
    batch = 6
    s = np.empty((batch, 2, n), dtype=np.float32)
    for b in range(batch):
        for h in range(2):
            kind = rng.integers(0, 5)
            x = rng.standard_normal(n)
            if kind == 0:
                v = x * 30 + 100
            elif kind == 1:
                v = np.round(x * 3) / 2                                # heavy ties
            elif kind == 2:
                v = 2.0 ** rng.integers(-3, 9) + x * 2.0 ** -12        # a cluster around a power of two
            elif kind == 3:
                v = x * 1e-20
            else:
                v = x * 1e20 * (rng.random(n) < 0.5)                   # half of them exactly zero
            s[b, h] = v.astype(np.float32)
    lens = rng.integers(1, n * 16 + 1, size=batch).astype(np.int32)
    lens[0] = n * 16
    for b, L in enumerate(lens):
        np_ = -(-int(L) // 16)
        s[b, :, np_:] = -np.inf
        s[b, :, 0] = np.inf
        s[b, :, max(0, np_ - 2):np_] = np.inf
    ratio = float(rng.choice([0.0625, 0.25, 0.5, 0.75]))
    k = max(3, int(np.ceil(ratio * n)))
    dev = device()
    got = ps.select_for_attention(torch.from_numpy(s).to(dev), torch.from_numpy(lens).to(dev), k, ratio)
    got = got.cpu().numpy()
    order = orc.select(s, k)
    counts = orc.budgets(lens, ratio)
    for b in range(batch):
        keep = int(min(counts[b], -(-int(lens[b]) // 16), k))
        for h in range(2):
            assert np.array_equal(got[b, h, :keep], np.sort(order[b, h, :keep])), (seed, b, h)
            assert (got[b, h, keep:] == -1).all()


def test_topk_longest_row_and_one_past_it():
    """8192 pages (a 128K context) is the longest row the sort takes."""
    rng = np.random.default_rng(8192)
    s = rng.standard_normal((2, 2, 8192)).astype(np.float32)
    s[0, 1, 100:4000] = 0.25                                   # a long run of ties
    got = ps.select(torch.from_numpy(s).to(device()), 4096)
    assert np.array_equal(got.cpu().numpy(), orc.select(s, 4096))
    with pytest.raises(ValueError):
        ps.select(torch.zeros(1, 2, 8193, device=device()), 16)


def test_selection_end_to_end_is_bit_exact_on_the_sparse_workload_shape():
    """Scores from the kernel, selection from the kernel, against the oracle
    chain, at 2048 pages and a 50 % budget."""
    lens = [32768, 32768]
    case = synthetic.dense_case(lens, seed=17, page_offset_std=0.5)
    t = _with_bounds(case)
    scores = ps.page_scores(t["q"], t["kmin"], t["kmax"], t["block_tables"], t["seq_lens"])
    k = ps.budget(0.5, 2048)
    assert k == 1024
    sel = ps.select(scores, k).cpu().numpy()
    want_scores = orc.page_scores(case["q"], t["kmin"].cpu().numpy(), t["kmax"].cpu().numpy(),
                                  case["block_tables"], case["seq_lens"])
    assert np.array_equal(sel, orc.select(want_scores, k))
    assert (sel[..., :3] == np.asarray([0, 2046, 2047])).all()  # forced pages first, index order


@pytest.mark.parametrize("num_splits", [None, 1, 3])
def test_sparse_kernel_attends_exactly_the_given_pages(num_splits, golden_dir):
    g = np.load(golden_dir / "sparse.npz")
    lens = [int(x) for x in g["seq_lens"]]
    case = synthetic.dense_case(lens, seed=11, page_offset_std=0.5)
    t = on_device(case)
    sel = np.stack([np.stack([p, p[::-1]]) for p in g["picks"]]).astype(np.int32)
    got = ps.sparse_decode(t["q"], t["k_pool"], t["v_pool"], t["block_tables"], t["seq_lens"],
                           torch.from_numpy(sel).to(device()), num_splits=num_splits)
    close(got, g["attend_picks"])


def test_selection_with_invalid_entries_and_per_sequence_budgets():
    lens = [4096, 700, 40, 0]
    ratio = 0.375
    case = synthetic.dense_case(lens, seed=19, page_offset_std=0.5)
    t = _with_bounds(case)
    scores = ps.page_scores(t["q"], t["kmin"], t["kmax"], t["block_tables"], t["seq_lens"])
    k = ps.budget(ratio, 256)
    sel = ps.select(scores, k)
    got = ps.sparse_decode(t["q"], t["k_pool"], t["v_pool"], t["block_tables"], t["seq_lens"], sel,
                           ratio=ratio)
    assert ps.budgets(t["seq_lens"], ratio).tolist() == [96, 17, 3, 0]
    want = orc.sparse_decode(case["q"], case["k_pool"], case["v_pool"], case["block_tables"],
                             case["seq_lens"], sel.cpu().numpy(), ratio=ratio)
    close(got, want)
    # A hand-made list with negative and past-the-end entries is skipped, not read.
    bad = sel.clone()
    bad[:, :, 1] = -1
    bad[:, :, 2] = 1_000_000
    got = ps.sparse_decode(t["q"], t["k_pool"], t["v_pool"], t["block_tables"], t["seq_lens"], bad)
    want = orc.sparse_decode(case["q"], case["k_pool"], case["v_pool"], case["block_tables"],
                             case["seq_lens"], bad.cpu().numpy())
    close(got, want)


def test_full_budget_reproduces_the_dense_kernel():
    case = synthetic.dense_case([1024, 300], seed=3)
    t = _with_bounds(case)
    dense = pdc.paged_decode_cuda(t["q"], t["k_pool"], t["v_pool"], t["block_tables"], t["seq_lens"],
                                  1024).clone()
    sparse = ps.sparse_attention(t["q"], t["k_pool"], t["v_pool"], t["block_tables"], t["seq_lens"],
                                 t["kmin"], t["kmax"], ratio=1.0)
    close(sparse, dense.float().cpu().numpy(), atol=1e-3)


@pytest.mark.parametrize("scoring", ["bounds", "mass"])
def test_sparse_attention_pipeline_at_quarter_budget(scoring):
    lens = [2048, 900]
    case = synthetic.dense_case(lens, seed=23, page_offset_std=0.5)
    t = _with_bounds(case)
    got = ps.sparse_attention(t["q"], t["k_pool"], t["v_pool"], t["block_tables"], t["seq_lens"],
                              t["kmin"], t["kmax"], ratio=0.25, max_seq_len=2048, scoring=scoring)
    if scoring == "bounds":
        scores = orc.page_scores(case["q"], t["kmin"].cpu().numpy(), t["kmax"].cpu().numpy(),
                                 case["block_tables"], case["seq_lens"])
    else:
        scores = ps.page_scores_mass(t["q"], t["kmin"], t["kmax"], t["block_tables"],
                                     t["seq_lens"]).cpu().numpy()
    sel = orc.select(scores, ps.budget(0.25, 128))
    for b, L in enumerate(lens):
        np_ = -(-L // 16)
        n = int(orc.budgets([L], 0.25)[0])
        assert {0, np_ - 2, np_ - 1} <= set(sel[b, 0, :n].tolist())
    want = orc.sparse_decode(case["q"], case["k_pool"], case["v_pool"], case["block_tables"],
                             case["seq_lens"], sel, ratio=0.25)
    close(got, want)


def test_sparse_pipeline_survives_graph_capture():
    case = synthetic.dense_case([1500, 640], seed=29, page_offset_std=0.5)
    t = _with_bounds(case)
    args = (t["q"], t["k_pool"], t["v_pool"], t["block_tables"], t["seq_lens"], t["kmin"], t["kmax"])
    ps.sparse_attention(*args, ratio=0.25)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = ps.sparse_attention(*args, ratio=0.25)
    q2 = np.random.default_rng(2).standard_normal(case["q"].shape).astype(np.float16)
    t["q"].copy_(torch.from_numpy(q2))
    graph.replay()
    torch.cuda.synchronize()
    scores = orc.page_scores(q2, t["kmin"].cpu().numpy(), t["kmax"].cpu().numpy(),
                             case["block_tables"], case["seq_lens"])
    sel = orc.select(scores, ps.budget(0.25, 94))
    want = orc.sparse_decode(q2, case["k_pool"], case["v_pool"], case["block_tables"],
                             case["seq_lens"], sel, ratio=0.25)
    close(out, want)


def test_fp16_cache_decode_steps_with_bounds_and_prefix_sharing():
    """PagedKVCache end to end: prefill, a shared ref-counted prefix, decode
    steps with page bounds on; dense and sparse attention against the oracle
    over the cache's own pools."""
    dev = device()
    rng = np.random.default_rng(31)
    spec = lc.KVCacheSpec(num_layers=2, num_kv_heads=2, head_dim=128, max_seq_len=512,
                          max_batch_size=3, device="cuda")
    cache = lc.PagedKVCache(spec, num_blocks=80)
    cache.enable_page_bounds()

    def rows(b, n):
        return (torch.from_numpy(rng.standard_normal((b, 2, n, 128)).astype(np.float16)).to(dev),
                torch.from_numpy(rng.standard_normal((b, 2, n, 128)).astype(np.float16)).to(dev))

    cache.advance(64, slots=[0])
    for layer in range(2):
        cache.write(layer, *rows(1, 64))
    shared = cache.tables[0].blocks[:2]                        # 32 tokens = 2 full blocks
    cache.attach_prefix(1, shared, 32)
    assert cache.allocator.ref_count(shared[0]) == 2
    cache.advance(21, slots=[1])
    for layer in range(2):
        cache.write(layer, *rows(1, 21))
    for _ in range(19):
        cache.advance(1, slots=[0, 1])
        for layer in range(2):
            cache.write(layer, *rows(2, 1))
    assert cache.seq_lens == [83, 72]
    tables, lens = cache.block_tables_tensor(2), cache.seq_lens_tensor(2)
    assert tables[0, :2].tolist() == tables[1, :2].tolist() == shared
    q = torch.from_numpy(rng.standard_normal((2, 2, 6, 128)).astype(np.float16)).to(dev)
    for layer in range(2):
        k, v = cache.k_pool[layer], cache.v_pool[layer]
        want = orc.paged_decode(q.cpu().numpy(), k.cpu().numpy(), v.cpu().numpy(),
                                tables.cpu().numpy(), lens.cpu().numpy())
        close(pdc.paged_decode_cuda(q, k, v, tables, lens, cache.max_len), want)
        kmin, kmax = cache.page_bounds(layer)
        for b, L in enumerate(cache.seq_lens):
            for p in range(-(-L // 16)):
                blk = int(tables[b, p])
                n = min(16, L - p * 16)
                assert torch.equal(kmin[blk], k[blk, :n].amin(0)) and torch.equal(kmax[blk], k[blk, :n].amax(0))
        got = ps.sparse_attention(q, k, v, tables, lens, kmin, kmax, ratio=0.5, max_seq_len=cache.max_len)
        scores = orc.page_scores(q.cpu().numpy(), kmin.cpu().numpy(), kmax.cpu().numpy(),
                                 tables.cpu().numpy(), lens.cpu().numpy())
        sel = orc.select(scores, ps.budget(0.5, -(-cache.max_len // 16)))
        want = orc.sparse_decode(q.cpu().numpy(), k.cpu().numpy(), v.cpu().numpy(),
                                 tables.cpu().numpy(), lens.cpu().numpy(), sel, ratio=0.5)
        close(got, want)
    cache.free_sequence(0)
    assert cache.allocator.ref_count(shared[0]) == 1           # still held by sequence 1


@pytest.mark.parametrize("lens,ratio", [([700, 333, 64, 17, 0], 0.25), ([32768, 9000], 0.5),
                                        ([65536, 40000, 100], 0.5), ([70000, 5000], 0.25)])
@pytest.mark.parametrize("programmatic", [False, True])
def test_index_and_select_behind_one_call_equals_the_two_calls(lens, ratio, programmatic):
    """Scores and picked pages of `index_and_select` against `page_scores` followed by
    `select_for_attention`, bit for bit: ragged rows, rows of 2048, 4096 and more
    pages, with and without requesting the bounds ahead of the dependency wait, three
    times in a row."""
    dev = device()
    pages = max(1, -(-max(lens) // 16))
    g = torch.Generator(device=dev).manual_seed(len(lens) * 1000 + pages)
    nb = sum(-(-x // 16) for x in lens) + 5
    kmin = torch.randn(nb, 2, 128, dtype=torch.float16, device=dev, generator=g) - 1.0
    kmax = kmin + torch.rand(nb, 2, 128, dtype=torch.float16, device=dev, generator=g) * 3
    q = torch.randn(len(lens), 2, 6, 128, dtype=torch.float16, device=dev, generator=g)
    perm = torch.randperm(nb, device=dev, generator=g).to(torch.int32)
    tables = torch.zeros(len(lens), pages, dtype=torch.int32, device=dev)
    at = 0
    for i, x in enumerate(lens):
        n = -(-x // 16)
        tables[i, :n] = perm[at:at + n]
        at += n
    seq = torch.tensor(lens, dtype=torch.int32, device=dev)
    k = ps.budget(ratio, pages)
    want_scores = ps.page_scores(q, kmin, kmax, tables, seq).clone()
    want_sel = ps.select_for_attention(want_scores, seq, k, ratio).clone()
    pdc.set_programmatic_launch(programmatic, early_pages=True)
    try:
        for _ in range(3):
            scores, sel = ps.index_and_select(q, kmin, kmax, tables, seq, k, ratio)
            assert torch.equal(scores, want_scores)
            assert torch.equal(sel, want_sel)
            sel.fill_(-7)
        torch.cuda.synchronize()
    finally:
        pdc.set_programmatic_launch(False)


def test_rewind_reuses_blocks_and_recomputes_the_landing_pages_bounds():
    """Decode from one prefilled state, rewind, decode again with other tokens
    (the reference's oracle-study use, cache/paged_cache.py:275-303): same blocks, same
    slots, bounds of the page the rewind lands in taken over its remaining rows."""
    dev = device()
    spec = lc.KVCacheSpec(num_layers=1, num_kv_heads=2, head_dim=128, max_seq_len=128, max_batch_size=1,
                          device="cuda")
    cache = lc.PagedKVCache(spec, num_blocks=12)
    cache.enable_page_bounds()
    g = torch.Generator(device=dev).manual_seed(3)
    k = torch.randn(1, 2, 40, 128, dtype=torch.float16, device=dev, generator=g)
    cache.advance(40, slots=[0])
    cache.write(0, k, k)
    blocks = list(cache.tables[0].blocks)
    for _ in range(10):                                   # to 50 tokens: page 3 opened
        cache.advance(1, slots=[0])
        cache.write(0, torch.randn(1, 2, 1, 128, dtype=torch.float16, device=dev, generator=g) * 5,
                    torch.zeros(1, 2, 1, 128, dtype=torch.float16, device=dev))
    cache.rewind(40)
    assert cache.seq_lens == [40] and int(cache.seq_lens_tensor(1)[0]) == 40
    blk = blocks[2]
    assert torch.equal(cache.kmin[0][blk], k[0, :, 32:40].amin(dim=1))
    assert torch.equal(cache.kmax[0][blk], k[0, :, 32:40].amax(dim=1))
    new = torch.randn(1, 2, 1, 128, dtype=torch.float16, device=dev, generator=g)
    cache.advance(1, slots=[0])
    cache.write(0, new, new)
    assert cache.tables[0].blocks[:3] == blocks[:3] and int(cache.seq_lens_tensor(1)[0]) == 41
    assert torch.equal(cache.k_pool[0][blk, 8], new[0, :, 0])
    with pytest.raises(ValueError):
        cache.rewind(99)

"""Dense fp16 paged decode on the GPU against the CPU oracle and the golden
fixtures (cases follow the reference's tests/test_cuda_decode.py:69-122 and
tests/test_phase11_kernel.py:87-135)."""

import numpy as np
import pytest
import torch

from latentserve_b200 import paged_decode as pd
from latentserve_b200 import paged_decode_cuda as pdc
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
IMPLS = [pdc.IMPL_MMA, pdc.IMPL_SIMT]


def _run(t, impl=pdc.IMPL_MMA, splits=None, **kw):
    # max_seq_len is signature parity only; a constant keeps this call free of
    # device reads, so it can run under graph capture.
    return pdc.paged_decode_cuda(t["q"], t["k_pool"], t["v_pool"], t["block_tables"], t["seq_lens"],
                                 t["block_tables"].shape[1] * 16, num_splits=splits, impl=impl, **kw)


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("splits", [None, 1, 3, 64])
def test_matches_the_oracle_on_ragged_lengths(impl, splits):
    case = synthetic.dense_case([1024, 300, 61, 17, 1], seed=0)
    want = orc.paged_decode(case["q"], case["k_pool"], case["v_pool"], case["block_tables"],
                            case["seq_lens"])
    close(_run(on_device(case), impl, splits), want)


@pytest.mark.parametrize("seed", range(6))
def test_matches_the_oracle_on_seeded_random_batches(seed):
    """Batches of random size and lengths (empty sequences, single tokens, page edges, a few
    long ones): wherever the page axis happens to be cut, the result is the oracle's, with
    either loader and with the split count capped or free."""
    rng = np.random.default_rng(500 + seed)
    batch = int(rng.integers(1, 41))
    lens = rng.integers(0, 600, size=batch)
    lens[rng.integers(0, batch)] = int(rng.integers(2000, 6000))       # one long sequence
    for edge in (16, 17, 31, 32, 1):
        lens[rng.integers(0, batch)] = edge
    case = synthetic.dense_case([int(x) for x in lens], seed=seed)
    want = orc.paged_decode(case["q"], case["k_pool"], case["v_pool"], case["block_tables"],
                            case["seq_lens"])
    t = on_device(case)
    for loader in ("cp_async", "tma"):
        pdc.set_loader(loader)
        try:
            close(_run(t, pdc.IMPL_MMA, None), want)
            close(_run(t, pdc.IMPL_MMA, int(rng.integers(1, 9))), want)
        finally:
            pdc.set_loader("auto")
    assert pdc.error_flag(device(), batch) == 0


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("name,make", [
    ("dense_ragged", lambda: synthetic.dense_case([1024, 300, 61, 17, 1], seed=0)),
    ("dense_config1", lambda: synthetic.config1(seed=0)),
    ("dense_edges", lambda: synthetic.dense_case([15, 16, 17, 31, 32, 33, 1], seed=3)),
])
def test_matches_the_reference_golden_outputs(impl, name, make, golden_dir):
    g = np.load(golden_dir / f"{name}.npz")
    close(_run(on_device(make()), impl), g["out_splits1"])


@pytest.mark.parametrize("impl", IMPLS)
def test_final_page_lengths_and_empty_sequences(impl):
    lens = [1, 15, 16, 17, 31, 32, 33, 0, 48, 0]
    case = synthetic.dense_case(lens, seed=4)
    want = orc.paged_decode(case["q"], case["k_pool"], case["v_pool"], case["block_tables"],
                            case["seq_lens"])
    got = _run(on_device(case), impl)
    close(got, want)
    assert (got[7] == 0).all() and (got[9] == 0).all()          # empty sequences give zeros


def test_largest_batch_the_kernels_take_and_one_past_it():
    """1024 sequences (the prefix-sum limit of the scheduler), short and ragged, some empty."""
    rng = np.random.default_rng(12)
    lens = rng.integers(0, 40, size=1024).tolist()
    case = synthetic.dense_case(lens, seed=12)
    want = orc.paged_decode(case["q"], case["k_pool"], case["v_pool"], case["block_tables"],
                            case["seq_lens"])
    close(_run(on_device(case)), want)
    over = synthetic.dense_case([3] * 1025, seed=13)
    with pytest.raises(ValueError):
        _run(on_device(over))


def test_every_sequence_empty_gives_zeros():
    case = synthetic.dense_case([0, 0, 0], seed=14)
    got = _run(on_device(case))
    assert got.shape == (3, 2, 6, 128) and (got == 0).all()


def test_no_cross_sequence_leak_and_stale_rows_are_never_read():
    """Rows past each sequence's end, and every block no table names, hold NaN."""
    lens = [100, 37, 260]
    case = synthetic.dense_case(lens, seed=6)
    want = orc.paged_decode(case["q"], case["k_pool"], case["v_pool"], case["block_tables"],
                            case["seq_lens"])
    k, v = case["k_pool"].copy(), case["v_pool"].copy()
    used = np.zeros(k.shape[:2], dtype=bool)
    for b, L in enumerate(lens):
        for pos in range(L):
            used[case["block_tables"][b, pos // 16], pos % 16] = True
    k[~used] = np.nan
    v[~used] = np.nan
    case.update(k_pool=k, v_pool=v)
    for impl in IMPLS:
        close(_run(on_device(case), impl), want)


def test_other_group_sizes():
    for n_rep in (1, 4, 8):
        case = synthetic.dense_case([200, 33], n_rep=n_rep, seed=8)
        want = orc.paged_decode(case["q"], case["k_pool"], case["v_pool"], case["block_tables"],
                                case["seq_lens"])
        for impl in IMPLS:
            close(_run(on_device(case), impl), want)


def test_four_kv_heads_and_a_strided_query_view():
    case = synthetic.dense_case([500, 130], n_rep=6, h=4, seed=9)
    want = orc.paged_decode(case["q"], case["k_pool"], case["v_pool"], case["block_tables"],
                            case["seq_lens"])
    t = on_device(case)
    # q as the model hands it over: a reshape of a [B, 1, Hq*D] projection slice.
    wide = torch.zeros(2, 1, 4 * 6 * 128 + 512, dtype=torch.float16, device=device())
    wide[:, 0, : 4 * 6 * 128] = t["q"].reshape(2, -1)
    t["q"] = wide[:, 0, : 4 * 6 * 128].view(2, 4, 6, 128)
    assert not t["q"].is_contiguous()
    close(_run(t), want)


def test_dispatch_through_the_entry_point():
    case = synthetic.dense_case([700, 33], seed=10)
    want = orc.paged_decode(case["q"], case["k_pool"], case["v_pool"], case["block_tables"],
                            case["seq_lens"])
    t = on_device(case)
    pd.set_decode_backend("cuda")
    got = pd.paged_decode_attention(t["q"], t["k_pool"], t["v_pool"], t["block_tables"],
                                    t["seq_lens"], max_seq_len=700)
    close(got, want)


def test_softmax_scale_is_honoured():
    case = synthetic.dense_case([300, 90], seed=12)
    want = orc.paged_decode(case["q"], case["k_pool"], case["v_pool"], case["block_tables"],
                            case["seq_lens"], softmax_scale=0.05)
    close(_run(on_device(case), softmax_scale=0.05), want)


def test_survives_cuda_graph_capture_and_reads_current_inputs():
    case = synthetic.dense_case([500, 200], seed=13)
    t = on_device(case)
    _run(t)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = _run(t)
    # New query and a longer second sequence after capture: replay must see both.
    q2 = (np.random.default_rng(1).standard_normal(case["q"].shape)).astype(np.float16)
    t["q"].copy_(torch.from_numpy(q2))
    t["seq_lens"].copy_(torch.tensor([480, 230], dtype=torch.int32))
    graph.replay()
    torch.cuda.synchronize()
    want = orc.paged_decode(q2, case["k_pool"], case["v_pool"], case["block_tables"],
                            np.asarray([480, 230], dtype=np.int32))
    close(out, want)


def test_programmatic_launch_eager_and_under_capture():
    """Back-to-back layer calls launched with programmatic stream serialization
    (each kernel's prologue overlapping the previous kernel's tail, shared
    partial scratch) give the same bits as ordinary launches."""
    dev = device()
    cases = [synthetic.dense_case([3000, 1200, 64, 5], seed=50 + i) for i in range(4)]
    ts = [on_device(c) for c in cases]
    plain = [_run(t).clone() for t in ts]
    pdc.set_programmatic_launch(True)
    try:
        eager = [_run(t).clone() for t in ts]
        torch.cuda.synchronize()
        outs = [torch.empty_like(plain[0]) for _ in ts]
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for t, o in zip(ts, outs):
                o.copy_(_run(t))
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
    finally:
        pdc.set_programmatic_launch(False)
    for a, b, c, case in zip(plain, eager, outs, cases):
        assert torch.equal(a, b) and torch.equal(a, c)
        close(a, orc.paged_decode(case["q"], case["k_pool"], case["v_pool"], case["block_tables"],
                                  case["seq_lens"]))


def test_long_uniform_batch_property_checks():
    """Full-size shape of the benchmark workload (batch 16 x 16K), checked by
    properties that need no CPU pass over 268 MB: (1) permuting which physical
    blocks hold the pages changes nothing; (2) V = const gives that constant;
    (3) one sequence of it against the oracle."""
    dev = device()
    w = synthetic.dense_pools_on_device(16, 16384, 1, dev, seed=2)
    k, v = w["pools"][0]
    q = w["q"][0]
    out = pdc.paged_decode_cuda(q, k, v, w["block_tables"], w["seq_lens"], 16384).clone()
    assert torch.isfinite(out).all()
    # (3) sequence 5 on the CPU
    b = 5
    blocks = w["block_tables"][b].long()
    case_k = k[blocks].cpu().numpy()
    case_v = v[blocks].cpu().numpy()
    tables = np.arange(1024, dtype=np.int32)[None]
    want = orc.paged_decode(q[b:b + 1].cpu().numpy(), case_k, case_v, tables,
                            np.asarray([16384], dtype=np.int32))
    close(out[b:b + 1], want)
    # (1) move every page to a different physical block
    perm = torch.randperm(w["num_blocks"], device=dev)
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(w["num_blocks"], device=dev)
    k2, v2 = k[perm], v[perm]                      # block i of the new pool = old block perm[i]
    tables2 = inv[w["block_tables"].long()].to(torch.int32)
    out2 = pdc.paged_decode_cuda(q, k2, v2, tables2, w["seq_lens"], 16384)
    assert torch.equal(out, out2)
    # (2) constant V
    v.fill_(0.25)
    out3 = pdc.paged_decode_cuda(q, k, v, w["block_tables"], w["seq_lens"], 16384)
    assert torch.allclose(out3.float(), torch.full_like(out3.float(), 0.25), atol=1e-3)


def test_corrupt_block_ids_are_skipped_and_flagged_not_read():
    case = synthetic.dense_case([64, 64], seed=14)
    t = on_device(case)
    t["block_tables"][1, 2] = 10_000_000          # far outside the pool
    out = _run(t)
    torch.cuda.synchronize()
    assert torch.isfinite(out).all()
    assert pdc.error_flag(device(), 2, 2) == 1


def test_batch_shapes_with_equally_long_bookkeeping_do_not_share_it():
    """(5 sequences, 2 KV heads) and (2 sequences, 8 KV heads) both need 22 ints of
    bookkeeping, laid out differently: slot ranges of the first would be arrival
    counters of the second. Each shape has its own buffer, so both calls, in either
    order and repeated, match the oracle."""
    a = synthetic.dense_case([3000, 1500, 900, 2200, 4000], h=2, seed=60)      # several segments each
    b = synthetic.dense_case([3500, 2600], h=8, seed=61)
    assert pdc.seg_len(5, 2) == pdc.seg_len(2, 8)
    ta, tb = on_device(a), on_device(b)
    want_a = orc.paged_decode(a["q"], a["k_pool"], a["v_pool"], a["block_tables"], a["seq_lens"])
    want_b = orc.paged_decode(b["q"], b["k_pool"], b["v_pool"], b["block_tables"], b["seq_lens"])
    for _ in range(2):
        close(_run(ta), want_a)
        close(_run(tb), want_b)
    assert pdc.seg_scratch("cuda", 5, 2, device()).data_ptr() != pdc.seg_scratch("cuda", 2, 8, device()).data_ptr()


def test_partials_then_stand_alone_combine_equal_the_fused_launch():
    from latentserve_b200 import _lib

    case = synthetic.dense_case([4000, 900, 33], seed=16)
    t = on_device(case)
    fused = _run(t).clone()
    assert pdc.paged_decode_cuda(t["q"], t["k_pool"], t["v_pool"], t["block_tables"], t["seq_lens"],
                                 4000, merge=False) is None
    chunks = pdc.choose_chunks(device(), 2, None, 3)
    acc, m, l, seg = pdc._partials(t["q"], chunks, "cuda")
    out = torch.zeros(3, 2, 6, 128, dtype=torch.float16, device=device())
    rc = _lib.lib().ls_combine(acc.data_ptr(), m.data_ptr(), l.data_ptr(), seg.data_ptr(),
                               out.data_ptr(), 3, 2, 6, out.stride(0), out.stride(1), out.stride(2),
                               _lib.current_stream(device()))
    assert rc == 0
    assert torch.equal(out, fused)
    counts = seg[1:6:2].tolist()
    assert counts[0] > 1 and all(c >= 1 for c in counts)      # the long sequence really was split
    assert (seg[2 * 3 + 2:] == 0).all()                        # arrival counters back at zero


def test_layout_violations_raise_value_error():
    case = synthetic.dense_case([64], seed=15)
    t = on_device(case)
    with pytest.raises(ValueError):
        pdc.paged_decode_cuda(t["q"], t["k_pool"], t["v_pool"], t["block_tables"].long(),
                              t["seq_lens"], 64)
    wide = torch.zeros(t["v_pool"].shape[0], 16, 4, 128, dtype=torch.float16, device=device())
    with pytest.raises(ValueError):                   # V pool laid out differently from K
        pdc.paged_decode_cuda(t["q"], t["k_pool"], wide[:, :, :2], t["block_tables"],
                              t["seq_lens"], 64)
    q9 = torch.zeros(1, 2, 9, 128, dtype=torch.float16, device=device())
    assert not pdc.eligible(q9, t["k_pool"])
    with pytest.raises(ValueError):
        pd.paged_decode_attention(q9, t["k_pool"], t["v_pool"], t["block_tables"], t["seq_lens"])


def _decode_loop(fused: bool, programmatic: bool, graphed: bool, steps: int = 20):
    """Prefill three sequences, then `steps` decode steps of two layers through
    PagedKVCache.write + paged_decode_attention; returns every step's outputs and the cache."""
    from latentserve_b200 import cache as lc

    dev = device()
    layers, batch = 2, 3
    spec = lc.KVCacheSpec(num_layers=layers, num_kv_heads=2, head_dim=128, max_seq_len=1024,
                          max_batch_size=batch, device="cuda")
    cache = lc.PagedKVCache(spec, num_blocks=3 * 64 + 4)
    if fused:
        cache.enable_fused_append()
    g = torch.Generator(device=dev).manual_seed(91)
    for i, n in enumerate([700, 47, 15]):        # 47 -> the first step fills a page, the second opens one
        cache.advance(n, slots=[i])
        for layer in range(layers):
            k = torch.randn(1, 2, n, 128, dtype=torch.float16, device=dev, generator=g)
            v = torch.randn(1, 2, n, 128, dtype=torch.float16, device=dev, generator=g)
            cache.write(layer, k, v)
    feed = torch.randn(steps, 3, layers, batch, 2, 6, 128, dtype=torch.float16, device=dev, generator=g)
    k_in = feed[0, 0, :, :, :, :1].clone()       # [layers, B, H, 1, D]
    v_in, q_in = feed[0, 1, :, :, :, :1].clone(), feed[0, 2].clone()
    out = torch.zeros(layers, batch, 2, 6, 128, dtype=torch.float16, device=dev)

    def body():
        for layer in range(layers):
            cache.write(layer, k_in[layer], v_in[layer])
            pd.paged_decode_attention(q_in[layer], cache.k_pool[layer], cache.v_pool[layer],
                                      cache.block_tables_tensor(batch), cache.seq_lens_tensor(batch),
                                      max_seq_len=1024, out=out[layer])

    pdc.set_programmatic_launch(programmatic, early_pages=True)
    pd.set_decode_backend("cuda")
    outs, graph = [], None
    try:
        for s in range(steps):
            cache.advance(1, batch_size=batch)
            k_in.copy_(feed[s, 0, :, :, :, :1]); v_in.copy_(feed[s, 1, :, :, :, :1]); q_in.copy_(feed[s, 2])
            if graphed and graph is None:
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    body()
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
    return outs, cache


def test_append_riding_on_the_attention_launch_changes_nothing():
    """PagedKVCache in fused-append mode: `write()` launches nothing, the attention kernel
    takes each sequence's newest row from the caller's rows and stores it to the pools.
    Outputs of every step and the pools afterwards equal the two-launch route bit for
    bit — eager, replayed from a graph, and with programmatic launch and early page
    requests; a write nobody attended is appended by the next advance()."""
    base, c0 = _decode_loop(fused=False, programmatic=False, graphed=False)
    for programmatic, graphed in [(False, False), (True, False), (True, True)]:
        got, c1 = _decode_loop(True, programmatic, graphed)
        for s, (a, b) in enumerate(zip(base, got)):
            assert torch.equal(a, b), f"step {s} differs (programmatic={programmatic}, graphed={graphed})"
        for layer in range(2):
            assert torch.equal(c0.k_pool[layer], c1.k_pool[layer])
            assert torch.equal(c0.v_pool[layer], c1.v_pool[layer])
    # Rows written but never attended reach the pool at the next advance().
    dev = device()
    g = torch.Generator(device=dev).manual_seed(5)
    k = torch.randn(3, 2, 1, 128, dtype=torch.float16, device=dev, generator=g)
    c1.advance(1, batch_size=3)
    c1.write(0, k, k)
    slots = [c1.tables[i].slot(c1.tables[i].length - 1) for i in range(3)]
    c1.advance(1, batch_size=3)
    torch.cuda.synchronize()
    flat = c1.k_pool[0].view(-1, 2, 128)
    for i, slot in enumerate(slots):
        assert torch.equal(flat[slot], k[i, :, 0])


def test_block_tables_on_the_device_follow_the_host_through_patches_and_row_copies():
    """A decode step that opens a page ships the new block id as a patch inside the
    step's one staging copy; a freed and re-admitted slot, a changed active set and a
    prefill go by whole rows. After every advance() the device rows equal the host's."""
    from latentserve_b200 import cache as lc

    spec = lc.KVCacheSpec(num_layers=1, num_kv_heads=2, head_dim=128, max_seq_len=256,
                          max_batch_size=4, device="cuda")
    cache = lc.PagedKVCache(spec, num_blocks=40)

    def check():
        tables = cache.block_tables_tensor().cpu()
        lens = cache.seq_lens_tensor().cpu().tolist()
        for row, i in enumerate(cache.active_slots()):
            t = cache.tables[i]
            assert lens[row] == t.length
            assert tables[row, :len(t.blocks)].tolist() == t.blocks

    for i, n in enumerate([15, 16, 33, 1]):              # page boundaries at different steps
        cache.advance(n, slots=[i])
        check()
    for step in range(40):
        cache.advance(1, batch_size=4)
        check()
        if step == 17:                                   # slot 1 leaves and comes back shorter
            cache.free_sequence(1)
            cache.advance(5, slots=[1])
            check()
        if step == 25:                                   # another row order
            cache.advance(1, slots=[3, 0, 2])
            check()
    # Running dry in the middle of a step: the rows patched before the failure were never
    # shipped, so they go out as whole rows with the next advance().
    small = lc.PagedKVCache(spec, num_blocks=6)
    for i in range(4):
        small.advance(15, slots=[i])
    small.advance(1, batch_size=4)                       # fills the pages; every row now current
    with pytest.raises(lc.OutOfBlocks):
        small.advance(1, batch_size=4)                   # rows 0 and 1 get blocks, row 2 does not
    assert [t.length for t in small.tables] == [17, 17, 16, 16]
    small.free_sequence(3)
    small.advance(1, slots=[0, 1, 2])
    tables = small.block_tables_tensor().cpu()
    for row, i in enumerate([0, 1, 2]):
        assert len(small.tables[i].blocks) == 2
        assert tables[row, :2].tolist() == small.tables[i].blocks

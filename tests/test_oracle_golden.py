"""The CPU oracle against fixtures produced by the reference itself
(tests/golden/make_golden.py). This is what pins the oracle; the GPU parity
tests then compare the kernels with the oracle."""

import hashlib

import numpy as np
import pytest

from latentserve_b200 import synthetic
from oracle import paged_attention_oracle as orc


def _sha(*arrays):
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


DENSE = {
    "dense_ragged": lambda: synthetic.dense_case([1024, 300, 61, 17, 1], seed=0),
    "dense_config1": lambda: synthetic.config1(seed=0),
    "dense_edges": lambda: synthetic.dense_case([15, 16, 17, 31, 32, 33, 1], seed=3),
}


@pytest.mark.parametrize("name", sorted(DENSE))
def test_dense_oracle_matches_reference_output(name, golden_dir):
    g = np.load(golden_dir / f"{name}.npz")
    c = DENSE[name]()
    assert _sha(c["q"], c["k_pool"], c["v_pool"], c["block_tables"], c["seq_lens"]) == str(
        g["inputs_sha256"]), "input generator drifted: regenerate the fixtures"
    got = orc.paged_decode(c["q"], c["k_pool"], c["v_pool"], c["block_tables"], c["seq_lens"])
    # fp32 evaluation-order differences only (online vs direct softmax).
    np.testing.assert_allclose(got, g["out_splits1"], atol=2e-6, rtol=1e-5)
    np.testing.assert_allclose(got, g["out_splits3"], atol=2e-6, rtol=1e-5)


@pytest.mark.parametrize("splits", [1, 3, 64])
def test_blockwise_restatement_matches_reference_output(splits, golden_dir):
    g = np.load(golden_dir / "dense_edges.npz")
    c = DENSE["dense_edges"]()
    got = orc.paged_decode_blockwise(c["q"], c["k_pool"], c["v_pool"], c["block_tables"],
                                     c["seq_lens"], num_splits=splits)
    np.testing.assert_allclose(got, g["out_splits1"], atol=2e-6, rtol=1e-5)


def test_blockwise_and_gather_forms_agree_on_ragged_lengths():
    c = synthetic.dense_case([300, 61, 17, 1], seed=5)
    a = orc.paged_decode(c["q"], c["k_pool"], c["v_pool"], c["block_tables"], c["seq_lens"])
    b = orc.paged_decode_blockwise(c["q"], c["k_pool"], c["v_pool"], c["block_tables"],
                                   c["seq_lens"], num_splits=4)
    np.testing.assert_allclose(a, b, atol=2e-6, rtol=1e-5)


def _int8_kwargs(g, asym):
    kw = dict(k_scale=g["k_scale"], v_scale=g["v_scale"], k_residual=g["k_residual"],
              res_rows=g["res_rows"])
    if asym:
        kw.update(k_zero=g["k_zero"], v_zero=g["v_zero"])
    return kw


@pytest.mark.parametrize("name,asym", [("int8_sym", False), ("int8_asym", True)])
def test_int8_attention_oracle_matches_reference_output(name, asym, golden_dir):
    g = np.load(golden_dir / f"{name}.npz")
    for fn in (orc.paged_decode, orc.paged_decode_blockwise):
        got = fn(g["q"], g["k_pool"], g["v_pool"], g["block_tables"], g["seq_lens"],
                 **_int8_kwargs(g, asym))
        np.testing.assert_allclose(got, g["out"], atol=3e-6, rtol=1e-5)


@pytest.mark.parametrize("name,asym", [("int8_sym", False), ("int8_asym", True)])
def test_quantizers_reproduce_the_reference_cache_bytes(name, asym, golden_dir):
    """Every V row, every finalised K page and every residual row of a cache
    the reference filled (prefill + 21 deferred-finalize decode steps), bit for
    bit, from the fp16 values that were fed in. CPU arithmetic: true division."""
    g = np.load(golden_dir / f"{name}.npz")
    tables, lens = g["block_tables"], g["seq_lens"]
    for i in range(len(lens)):
        L = int(lens[i])
        fed_k, fed_v = g[f"fed_k{i}"], g[f"fed_v{i}"]              # [H, L, D]
        assert fed_k.shape[1] == L
        q, step, zero = orc.quantize_v_rows(fed_v, asym=asym, reciprocal=False)   # [H, L, D], [H, L]
        for pos in range(L):
            blk, off = int(tables[i, pos // 16]), pos % 16
            assert np.array_equal(g["v_pool"][blk, off], q[:, pos])
            assert np.array_equal(g["v_scale"][blk, off], step[:, pos])
            if asym:
                assert np.array_equal(g["v_zero"][blk, off], zero[:, pos])
        full = L // 16
        # The reference quantises a page in the advance() AFTER it completes, so the
        # page completed by the very last step is still only in the residual.
        done = full if L % 16 else full - 1
        for p in range(done):
            data = fed_k[:, p * 16:(p + 1) * 16].transpose(1, 0, 2)[None]        # [1, 16, H, D]
            kq, kstep, kzero = orc.quantize_k_blocks(data, asym=asym, reciprocal=False)
            blk = int(tables[i, p])
            assert np.array_equal(g["k_pool"][blk], kq[0])
            assert np.array_equal(g["k_scale"][blk], kstep[0])
            if asym:
                assert np.array_equal(g["k_zero"][blk], kzero[0])
        tail0 = (L - 1) // 16 * 16
        row = int(g["res_rows"][i])
        assert np.array_equal(g["k_residual"][row, :L - tail0], fed_k[:, tail0:L].transpose(1, 0, 2))


def test_reciprocal_mode_differs_only_in_the_scale_rounding():
    """GPU arithmetic (multiply by fp32(1/127)) against CPU arithmetic (divide):
    scales differ by at most one ulp, in a few percent of rows."""
    rng = np.random.default_rng(0)
    v = (rng.standard_normal((4096, 128)) * np.logspace(-3, 2, 4096)[:, None]).astype(np.float16)
    _, s_gpu, _ = orc.quantize_v_rows(v, reciprocal=True)
    _, s_cpu, _ = orc.quantize_v_rows(v, reciprocal=False)
    differ = np.mean(s_gpu != s_cpu)
    assert 0.005 < differ < 0.15
    ulps = np.abs(s_gpu.view(np.int32) - s_cpu.view(np.int32))
    assert ulps.max() <= 1


def test_page_scores_match_the_reference_bounds(golden_dir):
    g = np.load(golden_dir / "sparse.npz")
    lens = [int(x) for x in g["seq_lens"]]
    c = synthetic.dense_case(lens, seed=11, page_offset_std=0.5)
    assert _sha(c["q"], c["k_pool"], c["v_pool"], c["block_tables"]) == str(g["inputs_sha256"])
    kmin, kmax = c["k_pool"].min(axis=1), c["k_pool"].max(axis=1)
    scores = orc.page_scores(c["q"], kmin, kmax, c["block_tables"], c["seq_lens"], recent=2)
    for b, L in enumerate(lens):
        np_ = -(-L // 16)
        ref = g[f"bounds{b}"]                                           # [H, P]
        mid = slice(1, np_ - 2)
        np.testing.assert_allclose(scores[b, :, mid], ref[:, mid], rtol=1e-5, atol=1e-4)
        assert np.all(np.isposinf(scores[b, :, 0]))
        assert np.all(np.isposinf(scores[b, :, np_ - 2:np_]))
        assert np.all(np.isneginf(scores[b, :, np_:]))


def test_budgets_match_the_reference(golden_dir):
    g = np.load(golden_dir / "sparse.npz")
    for r, row, per_call in zip(g["ratios"], g["budgets"], g["budget"]):
        assert np.array_equal(orc.budgets(g["probe_lens"], float(r)), row)
        assert [orc.budget(float(r), p) for p in (1, 3, 21, 44, 2048)] == list(per_call)


def test_select_is_a_stable_descending_sort():
    import torch

    rng = np.random.default_rng(3)
    s = rng.standard_normal((3, 2, 200)).astype(np.float32)
    s[..., 0] = np.inf
    s[..., 150:] = -np.inf
    s[0, 0, 40:50] = s[0, 0, 40]                      # a run of ties
    s[..., 120:123] = np.inf
    want = torch.sort(torch.from_numpy(s), dim=-1, descending=True, stable=True).indices[..., :77]
    got = orc.select(s, 77)
    assert np.array_equal(got, want.numpy().astype(np.int32))
    # Where finite scores are distinct, the set equals torch.topk's (the reference's select).
    top = torch.topk(torch.from_numpy(s[1:]), 77, dim=-1).indices.numpy()
    assert np.array_equal(np.sort(got[1:], axis=-1), np.sort(top, axis=-1))


def test_sparse_attention_oracle_matches_the_reference_tests_form(golden_dir):
    g = np.load(golden_dir / "sparse.npz")
    lens = [int(x) for x in g["seq_lens"]]
    c = synthetic.dense_case(lens, seed=11, page_offset_std=0.5)
    picks = g["picks"]
    sel = np.stack([np.stack([p, p[::-1]]) for p in picks]).astype(np.int32)       # [B, H, 6]
    got = orc.sparse_decode(c["q"], c["k_pool"], c["v_pool"], c["block_tables"], c["seq_lens"], sel)
    np.testing.assert_allclose(got, g["attend_picks"], atol=2e-6, rtol=1e-5)


def test_elementwise_restatements_match_the_reference_forms(golden_dir):
    g = np.load(golden_dir / "elementwise.npz")
    y, _ = orc.rms_norm(g["x"], g["w"], 1e-6)
    assert np.array_equal(y, g["rms"])
    y2, s2 = orc.rms_norm(g["x"], g["w"], 1e-6, residual=g["r"])
    assert np.array_equal(y2, g["add_rms"]) and np.array_equal(s2, g["add_rms_sum"])
    act = orc.silu_and_mul(g["gu"])
    # exp() implementations differ in the last fp32 bit: at most one fp16 ulp, rarely.
    assert np.mean(act != g["silu_mul"]) < 2e-3
    np.testing.assert_allclose(act.astype(np.float32), g["silu_mul"].astype(np.float32), rtol=1e-3, atol=1e-6)
    q = orc.rope(g["q"].reshape(3, 12, 128), g["cos"].reshape(3, 1, 128), g["sin"].reshape(3, 1, 128))
    k = orc.rope(g["k"].reshape(3, 2, 128), g["cos"].reshape(3, 1, 128), g["sin"].reshape(3, 1, 128))
    assert np.array_equal(q.reshape(3, 1, -1), g["rope_q"]) and np.array_equal(k.reshape(3, 1, -1), g["rope_k"])


@pytest.mark.parametrize("name", sorted(DENSE))
def test_the_timed_cpu_baseline_is_the_same_function(name, golden_dir):
    """`paged_decode_torch_cpu` is what bench.py times as the CPU baseline and as the
    reference arm: pinned to the reference's own output and to the numpy oracle, on
    ragged batches (padding and masking included)."""
    import torch

    g = np.load(golden_dir / f"{name}.npz")
    c = DENSE[name]()
    got = orc.paged_decode_torch_cpu(*(torch.from_numpy(c[k]) for k in
                                       ("q", "k_pool", "v_pool", "block_tables", "seq_lens"))).numpy()
    np.testing.assert_allclose(got, g["out_splits1"], atol=5e-6, rtol=1e-5)
    want = orc.paged_decode(c["q"], c["k_pool"], c["v_pool"], c["block_tables"], c["seq_lens"])
    np.testing.assert_allclose(got, want, atol=5e-6, rtol=1e-5)


def test_the_timed_cpu_baseline_honours_the_softmax_scale_and_a_compact_pool():
    """The bench hands it a pool renumbered to the sample's own blocks."""
    import torch

    c = synthetic.dense_case([200, 77, 16], seed=5)
    blocks = c["block_tables"].reshape(-1)
    compact = dict(c, k_pool=c["k_pool"][blocks], v_pool=c["v_pool"][blocks],
                   block_tables=np.arange(blocks.size, dtype=np.int32).reshape(c["block_tables"].shape))
    got = orc.paged_decode_torch_cpu(*(torch.from_numpy(compact[k]) for k in
                                       ("q", "k_pool", "v_pool", "block_tables", "seq_lens")),
                                     softmax_scale=0.05).numpy()
    want = orc.paged_decode(c["q"], c["k_pool"], c["v_pool"], c["block_tables"], c["seq_lens"],
                            softmax_scale=0.05)
    np.testing.assert_allclose(got, want, atol=5e-6, rtol=1e-5)

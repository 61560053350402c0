"""INT8 and page-sparse decode at the sizes the benchmark runs them at.

The small cases elsewhere check the arithmetic; these check what only shows at
full size — chunks that span several sequences, hundreds of CTAs, page rings
that wrap thousands of times — through properties that need no CPU pass over
hundreds of megabytes: one sequence (or one head of it) against the CPU oracle,
invariance under moving every page to another physical block, the two page
loaders agreeing bit for bit, and a clean error flag. Shapes: 32 sequences of
8K-32K tokens over INT8 pools written by the quantize-on-write kernels,
8 x 32 768 tokens at a 50 % page budget, and that budget over INT8 pools (cases follow the reference's
tests/test_cuda_decode.py:174-212 and tests/test_phase14_sparse_kernels.py:110-147).
"""

import numpy as np
import pytest
import torch

from latentserve_b200 import paged_decode_cuda as pdc
from latentserve_b200 import paged_sparse as ps
from latentserve_b200 import synthetic
from oracle import paged_attention_oracle as orc
from tests.gpu_util import close, device

pytestmark = pytest.mark.gpu


def _int8_call(w, layer, tables=None, q=None):
    L = w["layers"][layer]
    return pdc.paged_decode_cuda(w["q"][layer] if q is None else q, L["k_pool"], L["v_pool"],
                                 w["block_tables"] if tables is None else tables, w["seq_lens"], 32768,
                                 k_scale=L["k_scale"], v_scale=L["v_scale"], k_residual=L["k_residual"],
                                 res_rows=w["res_rows"])


def test_int8_batch_of_32_long_ragged_sequences():
    dev = device()
    rng = np.random.default_rng(7)
    lens = rng.integers(8192, 32769, size=32).tolist()
    lens[3] = 32768                      # a full last page
    lens[11] = 8192 + 1                  # a last page of one token
    w = synthetic.int8_pools_on_device(lens, 1, dev, seed=5)
    # Residual rows that are not the identity, as a serving cache hands them out.
    res_perm = torch.randperm(32, device=dev)
    L = w["layers"][0]
    L["k_residual"] = L["k_residual"][torch.argsort(res_perm)].contiguous()
    w["res_rows"] = res_perm.to(torch.int32)
    outs = {}
    for name in ("tma", "cp_async"):
        pdc.set_loader(name)
        try:
            outs[name] = _int8_call(w, 0).clone()
        finally:
            pdc.set_loader("auto")
    torch.cuda.synchronize()
    out = outs["tma"]
    assert torch.isfinite(out).all()
    assert torch.equal(outs["tma"], outs["cp_async"])
    assert pdc.error_flag(dev, 32, tag="cuda_i8") == 0
    # One long and one short sequence against the oracle, on their own pages only.
    for b in (int(np.argmax(lens)), 11):
        pages = -(-lens[b] // 16)
        blocks = w["block_tables"][b, :pages].long()
        row = int(w["res_rows"][b])
        want = orc.paged_decode(
            w["q"][0][b:b + 1].cpu().numpy(), L["k_pool"][blocks].cpu().numpy(),
            L["v_pool"][blocks].cpu().numpy(), np.arange(pages, dtype=np.int32)[None],
            np.asarray([lens[b]], dtype=np.int32), k_scale=L["k_scale"][blocks].cpu().numpy(),
            v_scale=L["v_scale"][blocks].cpu().numpy(),
            k_residual=L["k_residual"][row:row + 1].cpu().numpy(), res_rows=np.zeros(1, dtype=np.int32))
        close(out[b:b + 1], want)
    # Every page moved to another physical block: same bits out.
    nb = w["num_blocks"]
    perm = torch.randperm(nb, device=dev)
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(nb, device=dev)
    moved = dict(w)
    moved["layers"] = [dict(L, k_pool=L["k_pool"][perm], v_pool=L["v_pool"][perm],
                            k_scale=L["k_scale"][perm], v_scale=L["v_scale"][perm])]
    out2 = _int8_call(moved, 0, tables=inv[w["block_tables"].long()].to(torch.int32))
    assert torch.equal(out, out2)


def test_sparse_attention_at_8_by_32k_half_budget():
    dev = device()
    batch, context, ratio = 8, 32768, 0.5
    w = synthetic.sparse_pools_on_device(batch, context, 1, dev, seed=3)
    k, v = w["pools"][0]
    kmin, kmax = w["bounds"][0]
    q, tables, lens = w["q"][0], w["block_tables"], w["seq_lens"]
    pages = context // 16
    keep = ps.budget(ratio, pages)
    assert keep == 1024
    got = ps.sparse_attention(q, k, v, tables, lens, kmin, kmax, ratio=ratio, max_seq_len=context).clone()
    assert torch.isfinite(got).all()
    # The pages it attended are the first `keep` of the deterministic sort ...
    scores = ps.page_scores(q, kmin, kmax, tables, lens)
    sel = ps.select(scores, keep).clone()
    picked = ps.select_for_attention(scores, lens, keep, ratio)
    assert torch.equal(torch.sort(sel, dim=-1).values, torch.sort(picked, dim=-1).values)
    by_list = ps.sparse_decode(q, k, v, tables, lens, sel, ratio=ratio)
    assert (by_list.float() - got.float()).abs().max() <= 2e-3      # same pages, another visiting order
    # ... and one (sequence, head) of it against masked softmax on the CPU.
    b, head = 5, 1
    blocks = tables[b].long()
    want = orc.sparse_decode(q[b:b + 1].cpu().numpy(), k[blocks].cpu().numpy(), v[blocks].cpu().numpy(),
                             np.arange(pages, dtype=np.int32)[None], np.asarray([context], dtype=np.int32),
                             sel[b:b + 1].cpu().numpy(), ratio=ratio)
    close(got[b:b + 1, head], want[:, head])
    # The indexer's scores for that row, bit for bit.
    want_scores = orc.page_scores(q[b:b + 1].cpu().numpy(), kmin[blocks].cpu().numpy(),
                                  kmax[blocks].cpu().numpy(), np.arange(pages, dtype=np.int32)[None],
                                  np.asarray([context], dtype=np.int32))
    assert np.array_equal(scores[b:b + 1].cpu().numpy(), want_scores)
    assert np.array_equal(sel[b:b + 1].cpu().numpy(), orc.select(want_scores, keep))
    # A full budget visits every page in order: the dense kernel's bits.
    full = ps.sparse_attention(q, k, v, tables, lens, kmin, kmax, ratio=1.0, max_seq_len=context)
    dense = pdc.paged_decode_cuda(q, k, v, tables, lens, context)
    assert torch.equal(full, dense)


def test_int8_sparse_attention_at_8_by_32k_half_budget():
    """The decode kernel's page-list mode on INT8 pools (a combination the reference never
    built) at the sparse workload's size: 8 sequences of up to 32 768 tokens over pools written
    by the quantize-on-write kernels, each (sequence, head) attending its own half of the pages."""
    dev = device()
    lens = [32768, 32768 - 7, 30001, 32768, 16400, 32768, 9000, 32768]
    w = synthetic.int8_pools_on_device(lens, 1, dev, seed=13)
    L = w["layers"][0]
    q, tables, seq = w["q"][0], w["block_tables"], w["seq_lens"]
    pages = -(-max(lens) // 16)
    keep = pages // 2
    g = torch.Generator(device=dev).manual_seed(5)
    sel = torch.full((len(lens), 2, keep), -1, dtype=torch.int32, device=dev)
    for b, n in enumerate(lens):
        np_ = -(-n // 16)
        for h in range(2):                                # page 0, the two last pages, a random rest
            take = min(keep, np_)
            mid = torch.randperm(np_ - 3, device=dev, generator=g)[: take - 3] + 1
            picked = torch.cat([torch.tensor([0, np_ - 2, np_ - 1], device=dev), mid]).sort().values
            sel[b, h, :take] = picked.to(torch.int32)
    extra = dict(k_scale=L["k_scale"], v_scale=L["v_scale"], k_residual=L["k_residual"], res_rows=w["res_rows"])
    outs = {}
    for name in ("tma", "cp_async"):
        pdc.set_loader(name)
        try:
            outs[name] = ps.sparse_decode(q, L["k_pool"], L["v_pool"], tables, seq, sel, **extra).clone()
        finally:
            pdc.set_loader("auto")
    torch.cuda.synchronize()
    got = outs["tma"]
    assert torch.isfinite(got).all()
    assert torch.equal(outs["tma"], outs["cp_async"])
    # One long and one short sequence against masked softmax over the dequantised rows, on
    # their own pages only.
    for b in (2, 6):
        np_ = -(-lens[b] // 16)
        blocks = tables[b, :np_].long()
        row = int(w["res_rows"][b])
        want = orc.sparse_decode(
            q[b:b + 1].cpu().numpy(), L["k_pool"][blocks].cpu().numpy(), L["v_pool"][blocks].cpu().numpy(),
            np.arange(np_, dtype=np.int32)[None], np.asarray([lens[b]], dtype=np.int32),
            sel[b:b + 1].cpu().numpy(), k_scale=L["k_scale"][blocks].cpu().numpy(),
            v_scale=L["v_scale"][blocks].cpu().numpy(),
            k_residual=L["k_residual"][row:row + 1].cpu().numpy(), res_rows=np.zeros(1, dtype=np.int32))
        close(got[b:b + 1], want)
    # Every page selected, in order: the dense INT8 kernel's result (the lists of the shorter
    # sequences carry entries past their end, so the page axis is cut elsewhere and the partial
    # sums meet in another order: equal to rounding, not to the bit).
    full = torch.arange(pages, dtype=torch.int32, device=dev).expand(len(lens), 2, pages).contiguous()
    dense = pdc.paged_decode_cuda(q, L["k_pool"], L["v_pool"], tables, seq, max(lens), **extra)
    everything = ps.sparse_decode(q, L["k_pool"], L["v_pool"], tables, seq, full, **extra)
    assert (everything.float() - dense.float()).abs().max() <= 2e-3


def test_append_riding_on_the_attention_launch_at_16_by_16k():
    """The fused-append cache mode at the benchmark's size: three decode steps of 16 sequences
    at ~16 384 tokens (one of them opening a new page), two layers, through
    `PagedKVCache.write` + `paged_decode_attention` with the append riding on the attention
    launch and with a launch of its own: same outputs and same pools, bit for bit."""
    import random

    from latentserve_b200 import cache as lc
    from latentserve_b200 import paged_decode as pd

    dev = device()
    batch, context, layers = 16, 16384 - 1, 2            # the second step opens page 1024
    spec = lc.KVCacheSpec(num_layers=layers, num_kv_heads=2, head_dim=128, max_seq_len=context + 64,
                          max_batch_size=batch, device="cuda")
    need = -(-(context + 64) // 16)
    g = torch.Generator(device=dev).manual_seed(3)
    seed_pools = [(torch.randn(int(1.1 * batch * need), 16, 2, 128, dtype=torch.float16, device=dev, generator=g),
                   torch.randn(int(1.1 * batch * need), 16, 2, 128, dtype=torch.float16, device=dev, generator=g))
                  for _ in range(layers)]
    feed = torch.randn(3, layers, batch, 2, 8, 128, dtype=torch.float16, device=dev, generator=g)

    def run(fused):
        cache = lc.PagedKVCache(spec, num_blocks=int(1.1 * batch * need))
        for layer in range(layers):
            cache.k_pool[layer].copy_(seed_pools[layer][0])
            cache.v_pool[layer].copy_(seed_pools[layer][1])
        random.Random(0).shuffle(cache.allocator._free)
        for i in range(batch):
            cache.tables[i].append(context - (i % 3))    # lengths differ by a token or two
        if fused:
            cache.enable_fused_append()
        outs = []
        pd.set_decode_backend("cuda")
        pdc.set_programmatic_launch(True, early_pages=True)
        try:
            for step in range(3):
                cache.advance(1, batch_size=batch)
                for layer in range(layers):
                    x = feed[step, layer]
                    cache.write(layer, x[:, :, 6:7], x[:, :, 7:8])
                    outs.append(pd.paged_decode_attention(
                        x[:, :, :6], cache.k_pool[layer], cache.v_pool[layer], cache.block_tables_tensor(batch),
                        cache.seq_lens_tensor(batch), max_seq_len=cache.max_len).clone())
            cache.advance(1, batch_size=batch)           # flushes rows nobody attended (none here)
            torch.cuda.synchronize()
        finally:
            pdc.set_programmatic_launch(False)
        return outs, cache

    plain_outs, plain = run(False)
    fused_outs, fused = run(True)
    for a, b in zip(plain_outs, fused_outs):
        assert torch.equal(a, b)
    for layer in range(layers):
        assert torch.equal(plain.k_pool[layer], fused.k_pool[layer])
        assert torch.equal(plain.v_pool[layer], fused.v_pool[layer])
    assert torch.equal(plain.block_tables_tensor(batch), fused.block_tables_tensor(batch))

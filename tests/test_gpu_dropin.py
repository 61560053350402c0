"""The drop-in under the reference's own callers, on the GPU.

An importable LatentServe tree (the installed copy under `baseline/_ref`, or the
directory `LATENTSERVE_REFERENCE` names) has its kernel modules patched by
`dropin.install()`, and then ITS code drives this library:

  * `LatentServeQwen` (random-init Qwen2, head_dim 128) with its own
    `PagedKVCache`: `GQAAttention.forward`'s kernel branch
    (model/attention/gqa.py:283-344) against the reference's torch route;
  * its `Int8PagedKVCache` in deferred-finalize mode: pool bytes, scales and
    residual against the oracle's quantisers, attention against its own
    `paged_decode_reference` (cases: tests/test_phase14_int8_graph.py:139-223);
  * `model.set_sparse` (model/latentserve_qwen.py:264-286): page bounds kept by
    the reference cache through `update_bounds`, the sparse branch of
    `GQAAttention.forward` against the oracle;
  * `GraphedDecoder.step_greedy` (runtime/cuda_graph.py:307-388): replayed
    steps against eager steps (cases: tests/test_cuda_decode.py:125-171);
  * `ServingEngine` (runtime/engine.py:59-455) draining a queue of requests with
    its `PrefixCache` and its graphed decoder switched on, against the same
    engine without either.

Skipped only where no LatentServe tree (or no `transformers`) is importable.
"""

import os
import pathlib
import sys
from collections import Counter

import numpy as np
import pytest
import torch

from oracle import paged_attention_oracle as orc
from tests.gpu_util import close, device

ROOT = pathlib.Path(__file__).resolve().parents[1]
REF = os.environ.get("LATENTSERVE_REFERENCE") or str(ROOT / "baseline" / "_ref")
have_reference = os.path.isdir(os.path.join(REF, "kernels", "cuda"))
pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not have_reference, reason="no LatentServe tree to install into")]

LAYERS, Q_HEADS, KV_HEADS, HEAD_DIM, VOCAB = 2, 12, 2, 128, 128


@pytest.fixture()
def ref(monkeypatch):
    """The reference tree on sys.path with the drop-in installed; `calls` counts
    how often its code reached this library's entry points."""
    pytest.importorskip("transformers")
    sys.path.insert(0, REF)
    sys.dont_write_bytecode = True
    from latentserve_b200 import dropin

    import importlib

    names = dropin.install()
    calls = Counter()
    for mod_name, attr in [("kernels.cuda.paged_decode_cuda", "paged_decode_cuda"),
                           ("kernels.cuda.paged_sparse", "sparse_attention"),
                           ("kernels.cuda.paged_sparse", "update_bounds"),
                           ("kernels.cuda.int8_write", "decode_write")]:
        mod = importlib.import_module(mod_name)
        inner = getattr(mod, attr)

        def counted(*a, _inner=inner, _attr=attr, **k):
            calls[_attr] += 1
            return _inner(*a, **k)

        monkeypatch.setattr(mod, attr, counted)
    try:
        yield calls, names
    finally:
        monkeypatch.undo()
        dropin.uninstall()
        sys.path.remove(REF)


def _model(attn_impl="triton_paged", seed=0):
    from transformers import Qwen2Config, Qwen2ForCausalLM

    from model.latentserve_qwen import LatentServeQwen
    from model.qwen import ModelShape

    torch.manual_seed(seed)
    cfg = Qwen2Config(vocab_size=VOCAB, hidden_size=HEAD_DIM * Q_HEADS, intermediate_size=512,
                      num_hidden_layers=LAYERS, num_attention_heads=Q_HEADS,
                      num_key_value_heads=KV_HEADS, max_position_embeddings=2048)
    hf = Qwen2ForCausalLM(cfg).half().cuda().eval()
    shape = ModelShape(LAYERS, Q_HEADS, KV_HEADS, HEAD_DIM, HEAD_DIM * Q_HEADS, VOCAB, 2048, "torch.float16")
    return LatentServeQwen(hf_model=hf, tokenizer=None, shape=shape, device="cuda",
                           attn_impl=attn_impl, max_seq_len_hint=1024)


def _attention_inputs(cache, layer, batch, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(batch, KV_HEADS, Q_HEADS // KV_HEADS, HEAD_DIM, dtype=torch.float16, device="cuda",
                    generator=g)
    return q, cache.k_pool[layer], cache.v_pool[layer], cache.block_tables_tensor(batch), \
        cache.seq_lens_tensor(batch)


def test_reference_model_decodes_through_the_kernel_branch(ref):
    calls, names = ref
    from kernels.gqa import paged_decode as rpd

    assert "kernels.cuda.paged_decode_cuda.paged_decode_cuda" in names and rpd.decode_backend() == "cuda"
    prompt = torch.randint(0, VOCAB, (2, 100), generator=torch.Generator().manual_seed(1)).cuda()
    token = torch.zeros(2, 1, dtype=torch.long, device="cuda")

    def decode(attn_impl):
        m = _model(attn_impl)
        m.allocate_cache(2, 256, paged=True, block_size=16)
        m.cache.reset()
        m.prefill(prompt)
        return m, m.decode_step(token).float()

    m, got = decode("triton_paged")                    # kernel branch -> this library
    assert calls["paged_decode_cuda"] == LAYERS
    _, want = decode("sdpa")                           # the reference's gather-then-attend torch route
    torch.testing.assert_close(got, want, atol=2e-2, rtol=2e-2)
    # The attention call itself, on the reference cache's state, against its torch reference.
    q, k, v, tables, lens = _attention_inputs(m.cache, 1, 2, seed=3)
    out = rpd.paged_decode_attention(q, k, v, tables, lens, max_seq_len=m.cache.max_len)
    want = rpd.paged_decode_reference(q.float(), k, v, tables, lens, num_splits=1)
    close(out, want.cpu().numpy())
    assert calls["paged_decode_cuda"] == LAYERS + 1


def test_reference_int8_cache_deferred_finalize_bytes_and_attention(ref):
    calls, _ = ref
    from cache.int8_paged_cache import Int8PagedKVCache
    from cache.kv_cache import KVCacheSpec
    from kernels.gqa import paged_decode as rpd

    spec = KVCacheSpec(num_layers=1, num_kv_heads=KV_HEADS, head_dim=HEAD_DIM, max_batch_size=2,
                       max_seq_len=128, dtype=torch.float16, device="cuda")
    cache = Int8PagedKVCache(spec, block_size=16)
    cache.enable_deferred_finalize()
    g = torch.Generator(device="cuda").manual_seed(5)
    prompts, steps = [10, 23], 40
    fed_k = [torch.randn(KV_HEADS, p + steps, HEAD_DIM, dtype=torch.float16, device="cuda", generator=g)
             for p in prompts]
    fed_v = [torch.randn(KV_HEADS, p + steps, HEAD_DIM, dtype=torch.float16, device="cuda", generator=g)
             for p in prompts]
    for i, p in enumerate(prompts):
        cache.advance(p, slots=[i])
        cache.write(0, fed_k[i][None, :, :p], fed_v[i][None, :, :p])
    for s in range(steps):
        cache.advance(1, slots=[0, 1])
        k = torch.stack([fed_k[i][:, prompts[i] + s] for i in range(2)])[:, :, None]
        v = torch.stack([fed_v[i][:, prompts[i] + s] for i in range(2)])[:, :, None]
        cache.write(0, k, v)
    assert calls["decode_write"] == steps              # the graph-path write reached this library
    tables = cache.block_tables_tensor(2).cpu().numpy()
    for i, p in enumerate(prompts):
        L = p + steps
        fk, fv = fed_k[i].cpu().numpy(), fed_v[i].cpu().numpy()
        # Decode-step rows went through this library's quantize-on-write kernel (GPU
        # arithmetic: reciprocal multiply); prefill rows through the reference's torch
        # ops on the GPU, which is the same arithmetic.
        vq, vstep, _ = orc.quantize_v_rows(fv, reciprocal=True)
        for pos in range(L):
            blk, off = int(tables[i, pos // 16]), pos % 16
            assert np.array_equal(cache.v_pool[0][blk, off].cpu().numpy(), vq[:, pos]), (i, pos)
            assert np.array_equal(cache.v_scale_pool[0][blk, off].cpu().numpy(), vstep[:, pos])
        done = (L - 1) // 16
        for pg in range(done):
            kq, kstep, _ = orc.quantize_k_blocks(fk[:, pg * 16:(pg + 1) * 16].transpose(1, 0, 2)[None],
                                                 reciprocal=True)
            blk = int(tables[i, pg])
            assert np.array_equal(cache.k_pool[0][blk].cpu().numpy(), kq[0]), (i, pg)
            assert np.array_equal(cache.k_scale_pool[0][blk].cpu().numpy(), kstep[0])
        tail0 = done * 16
        row = int(cache.residual_rows_tensor(2)[i])
        assert np.array_equal(cache.residual(0)[row, :L - tail0].cpu().numpy(),
                              fk[:, tail0:L].transpose(1, 0, 2))
    q = torch.randn(2, KV_HEADS, 6, HEAD_DIM, dtype=torch.float16, device="cuda", generator=g)
    kw = dict(k_scale=cache.k_scale_pool[0], v_scale=cache.v_scale_pool[0], k_residual=cache.residual(0),
              res_rows=cache.residual_rows_tensor(2))
    before = calls["paged_decode_cuda"]
    got = rpd.paged_decode_attention(q, cache.k_pool[0], cache.v_pool[0], cache.block_tables_tensor(2),
                                     cache.seq_lens_tensor(2), max_seq_len=cache.max_len, **kw)
    assert calls["paged_decode_cuda"] == before + 1
    want = rpd.paged_decode_reference(q.float(), cache.k_pool[0], cache.v_pool[0],
                                      cache.block_tables_tensor(2), cache.seq_lens_tensor(2),
                                      num_splits=1, **kw)
    close(got, want.cpu().numpy())


def test_reference_set_sparse_runs_the_sparse_branch(ref):
    calls, _ = ref
    from kernels.cuda import paged_sparse as rps

    m = _model()
    m.allocate_cache(2, 1024, paged=True, block_size=16)
    m.cache.reset()
    m.set_sparse(0.25)
    prompt = torch.randint(0, VOCAB, (2, 600), generator=torch.Generator().manual_seed(2)).cuda()
    m.prefill(prompt)
    token = torch.zeros(2, 1, dtype=torch.long, device="cuda")
    logits = m.decode_step(token).float()
    assert torch.isfinite(logits).all()
    assert calls["sparse_attention"] == LAYERS and calls["update_bounds"] >= LAYERS
    # Page bounds kept by the reference cache through this library's update kernel.
    cache = m.cache
    tables, lens = cache.block_tables_tensor(2), cache.seq_lens_tensor(2)
    kmin, kmax = cache.page_bounds(0)
    for b in range(2):
        L = int(lens[b])
        for pg in range(-(-L // 16)):
            blk, rows = int(tables[b, pg]), min(16, L - pg * 16)
            assert torch.equal(kmin[blk], cache.k_pool[0][blk, :rows].amin(dim=0))
            assert torch.equal(kmax[blk], cache.k_pool[0][blk, :rows].amax(dim=0))
    # The sparse branch's call, on the cache's state, against the oracle's selection + masked softmax.
    q, k, v, tables, lens = _attention_inputs(cache, 0, 2, seed=4)
    got = rps.sparse_attention(q, k, v, tables, lens, kmin, kmax, ratio=0.25, recent=2,
                               max_seq_len=cache.max_len).clone()
    host = [x.cpu().numpy() for x in (q, k, v, tables, lens)]
    pages = -(-cache.max_len // 16)
    scores = orc.page_scores(host[0], kmin.cpu().numpy(), kmax.cpu().numpy(), host[3], host[4],
                             max_pages=tables.shape[1])
    sel = orc.select(scores, rps.budget(0.25, pages))
    close(got, orc.sparse_decode(*host, sel, ratio=0.25))
    # A full budget is dense attention: same logits as with sparsity off.
    m.set_sparse(1.0)
    m2 = _model()
    m2.allocate_cache(2, 1024, paged=True, block_size=16)
    m2.cache.reset()
    m2.prefill(prompt)
    dense = m2.decode_step(token).float()
    m.cache.reset()
    m.prefill(prompt)
    full = m.decode_step(token).float()
    torch.testing.assert_close(full, dense, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("kv_dtype", ["fp16", "int8"])
def test_reference_graphed_decoder_replays_what_eager_steps_compute(ref, kv_dtype):
    calls, _ = ref
    from runtime.cuda_graph import GraphedDecoder

    prompts = [torch.randint(0, VOCAB, (1, n), generator=torch.Generator().manual_seed(7 + n)).cuda()
               for n in (90, 37)]
    steps = 24

    def run(graphed):
        m = _model()
        m.allocate_cache(2, 256, paged=True, block_size=16, kv_dtype=kv_dtype)
        m.cache.reset()
        first = [m.prefill_slot(p, slot=i)[:, -1].argmax(dim=-1, keepdim=True) for i, p in enumerate(prompts)]
        decoder = GraphedDecoder(m, enabled=graphed, greedy=True)
        token = torch.cat(first, dim=0)
        out_tokens, out_logits = [], []
        for t in range(steps):
            pos = torch.tensor([[90 + t], [37 + t]], device="cuda")
            logits = decoder.step(token, pos, [0, 1])
            out_logits.append(logits.float().clone())
            token = logits[:, -1, :].argmax(dim=-1, keepdim=True).clone()
            out_tokens.append(token)
        return decoder, torch.cat(out_tokens, dim=1), torch.cat(out_logits, dim=1)

    eager, want_tokens, want_logits = run(False)
    before = calls["paged_decode_cuda"]
    graphed, got_tokens, got_logits = run(True)
    assert graphed.graph_steps == steps and graphed.eager_steps == 0 and graphed.captures >= 1
    assert calls["paged_decode_cuda"] > before        # recorded at capture, replayed afterwards
    # Same kernels on the same inputs: the sequences agree until a near-tie in the
    # random-init logits could flip an argmax, after which they legitimately diverge.
    agree = (got_tokens == want_tokens).all(dim=0).int().cumprod(dim=0).sum().item()
    assert agree >= 1
    torch.testing.assert_close(got_logits[:, :agree], want_logits[:, :agree], atol=3e-2, rtol=3e-2)
    top2 = want_logits[:, :agree].topk(2, dim=-1).values
    clear = (top2[..., 0] - top2[..., 1]) > 6e-2
    assert (got_tokens[:, :agree][clear] == want_tokens[:, :agree][clear]).all()
    if agree < steps:                                  # the step that diverged was a near-tie
        top2 = want_logits[:, agree].topk(2, dim=-1).values
        flipped = got_tokens[:, agree] != want_tokens[:, agree]
        assert ((top2[:, 0] - top2[:, 1])[flipped] <= 6e-2).all()


def test_reference_serving_engine_with_prefix_cache_and_graphs(ref):
    """The reference's `ServingEngine` (runtime/engine.py:59-455) — continuous batching over
    its own paged cache, its `PrefixCache` sharing full prompt blocks between requests, decode
    steps replayed by its `GraphedDecoder` — drains a queue of requests with this library
    under it, and generates what the same engine generates step by step without graphs and
    without prefix sharing."""
    calls, _ = ref
    from runtime.engine import ServingEngine
    from runtime.request import ServedRequest

    g = torch.Generator().manual_seed(3)
    shared = torch.randint(0, VOCAB, (48,), generator=g).tolist()          # three full blocks in common
    prompts = [shared + torch.randint(0, VOCAB, (n,), generator=g).tolist() for n in (21, 5, 40, 13, 30)]
    new_tokens = 12

    def serve(graphs, prefix):
        engine = ServingEngine(_model(), max_running=3, max_seq_len=256, use_cuda_graphs=graphs,
                               prefix_caching=prefix)
        for i, p in enumerate(prompts):
            engine.add_request(ServedRequest(i, list(p), max_new_tokens=new_tokens))
        done = engine.run(max_steps=4000)
        assert len(done) == len(prompts) and not engine.has_work
        return engine, {r.request_id: list(r.output_ids) for r in done}

    plain, want = serve(False, False)
    before = calls["paged_decode_cuda"]
    engine, got = serve(True, True)
    assert calls["paged_decode_cuda"] > before                 # captured (and run) through this library
    assert engine.decoder is not None and engine.decoder.graph_steps > 0
    assert engine.prefix_hit_tokens >= 48                      # later requests reused the shared blocks
    agree = total = 0
    for i in range(len(prompts)):
        assert len(got[i]) == new_tokens and len(want[i]) == new_tokens
        assert all(0 <= t < VOCAB for t in got[i])
        same = 0
        while same < new_tokens and got[i][same] == want[i][same]:
            same += 1
        agree += same
        total += new_tokens
    # Same kernels and weights; what differs is how the shared prompt blocks were prefilled
    # (once, in another batch shape), so a near-tie in the random-init logits may flip a
    # token, after which that request legitimately goes its own way.
    assert agree >= total // 2, (agree, total, got, want)

"""A whole decode step (random-init Qwen2-shaped layers) over the paged caches:
this library's append + attention kernels inside the step against the same step
with attention done by gather-then-softmax in torch (the reference's own
whole-model check is tests/test_cuda_decode.py:125-171)."""

import numpy as np
import pytest
import torch

from latentserve_b200 import cache as lc
from latentserve_b200 import decode_step as ds
from latentserve_b200 import paged_decode_cuda as pdc
from tests.gpu_util import device

pytestmark = pytest.mark.gpu
SHAPE = ds.QwenShape(num_layers=3, hidden=256, q_heads=12, kv_heads=2, head_dim=128,
                     intermediate=512, vocab=997)


def _torch_attend(model):
    """Replacement for DecodeModel.attend: gather the sequence's K/V rows out of
    the fp16 pools and do softmax attention in fp32."""

    def attend(cache, layer, q, batch, context_hint):
        tables, lens = cache.block_tables_tensor(batch), cache.seq_lens_tensor(batch)
        out = torch.zeros_like(q, dtype=torch.float32)
        for b in range(batch):
            L = int(lens[b])
            pos = torch.arange(L, device=q.device)
            slots = tables[b, pos // 16].long() * 16 + pos % 16
            k = cache.k_pool[layer].view(-1, 2, 128)[slots].float()           # [L, H, D]
            v = cache.v_pool[layer].view(-1, 2, 128)[slots].float()
            s = torch.einsum("hrd,lhd->hrl", q[b].float(), k) / np.sqrt(128.0)
            out[b] = torch.einsum("hrl,lhd->hrd", torch.softmax(s, -1), v)
        return out.to(q.dtype)

    return attend


def _drive(model, cache, prompts, steps, attend=None, graphed=False):
    """Feed each prompt token by token (decode steps only), then `steps` greedy
    steps for the whole batch; returns the logits of every batched step."""
    if attend is not None:
        model.attend = attend
    dev = model.device
    b = len(prompts)
    for i, prompt in enumerate(prompts):
        for pos, tok in enumerate(prompt):
            cache.advance(1, slots=[i])
            model.forward(cache, torch.tensor([tok], device=dev), torch.tensor([pos], device=dev), 512)
    tokens = torch.tensor([p[-1] for p in prompts], device=dev)
    logits = []
    runner = None
    for step in range(steps):
        cache.advance(1, slots=list(range(b)))
        positions = torch.tensor([n - 1 for n in cache.seq_lens], device=dev)
        if graphed:
            if runner is None:
                runner = ds.GraphedStep(model, cache, b, 512)
                runner.tokens.copy_(tokens)
                runner.positions.copy_(positions)
                runner.capture()
            runner.tokens.copy_(tokens)
            tokens = runner.step(feed_back=False).clone()
            logits.append(tokens.clone())
        else:
            out = model.forward(cache, tokens, positions, 512, return_logits=True)
            logits.append(out.float().clone())
            tokens = out.argmax(-1)
    return logits


def _fresh(kind):
    spec = lc.KVCacheSpec(num_layers=SHAPE.num_layers, num_kv_heads=2, head_dim=128, max_seq_len=512,
                          max_batch_size=3, device="cuda")
    return lc.PagedKVCache(spec, num_blocks=64) if kind == "fp16" else lc.Int8PagedKVCache(spec, num_blocks=64)


def _prompts():
    rng = np.random.default_rng(3)
    return [rng.integers(0, SHAPE.vocab, size=n).tolist() for n in (37, 5, 18)]


@pytest.mark.parametrize("pdl", [False, True])
def test_step_with_library_attention_matches_torch_attention(pdl):
    dev = device()
    pdc.set_programmatic_launch(pdl)
    try:
        model = ds.DecodeModel(SHAPE, dev, max_pos=512, seed=1, fused=False)
        got = _drive(model, _fresh("fp16"), _prompts(), steps=20)
        ref_model = ds.DecodeModel(SHAPE, dev, max_pos=512, seed=1, fused=False)
        want = _drive(ref_model, _fresh("fp16"), _prompts(), steps=20, attend=_torch_attend(ref_model))
    finally:
        pdc.set_programmatic_launch(False)
    for a, b in zip(got, want):
        assert torch.isfinite(a).all()
        assert (a - b).abs().max() <= 3e-2 + 2e-2 * b.abs().max()
    # The two runs pick the same greedy token almost everywhere (logit gaps are tiny in a random model).
    same = np.mean([(a.argmax(-1) == b.argmax(-1)).float().mean().item() for a, b in zip(got, want)])
    assert same >= 0.9


@pytest.mark.parametrize("projections", ["ls", "cublas"])
@pytest.mark.parametrize("kind", ["fp16", "int8"])
def test_fused_layer_kernels_match_the_unfused_step(kind, projections):
    """RMSNorm (+ residual), RoPE + append and SiLU * up as this library's kernels
    (stand-alone with cuBLAS projections, or folded into this library's own
    projections) against the same step with torch element-wise ops and cache.write."""
    dev = device()
    fused = _drive(ds.DecodeModel(SHAPE, dev, max_pos=512, seed=5, fused=True, projections=projections),
                   _fresh(kind), _prompts(), steps=20)
    plain = _drive(ds.DecodeModel(SHAPE, dev, max_pos=512, seed=5, fused=False), _fresh(kind), _prompts(),
                   steps=20)
    for a, b in zip(fused, plain):
        assert torch.isfinite(a).all()
        assert (a - b).abs().max() <= 3e-2 + 2e-2 * b.abs().max()


def test_streamed_output_head():
    """vocab a multiple of 32: the final norm and the output head run on the projection kernel too."""
    import dataclasses

    dev = device()
    shape = dataclasses.replace(SHAPE, vocab=1024)
    a = ds.DecodeModel(shape, dev, max_pos=512, seed=6, fused=True, projections="ls")
    b = ds.DecodeModel(shape, dev, max_pos=512, seed=6, fused=False)
    prompts = [[int(t) % 1024 for t in p] for p in _prompts()]
    for x, y in zip(_drive(a, _fresh("fp16"), prompts, steps=6), _drive(b, _fresh("fp16"), prompts, steps=6)):
        assert torch.isfinite(x).all()
        assert (x - y).abs().max() <= 3e-2 + 2e-2 * y.abs().max()


def test_graph_replay_produces_the_eager_tokens():
    dev = device()
    eager = _drive(ds.DecodeModel(SHAPE, dev, max_pos=512, seed=2), _fresh("fp16"), _prompts(), steps=24)
    graphed = _drive(ds.DecodeModel(SHAPE, dev, max_pos=512, seed=2), _fresh("fp16"), _prompts(), steps=24,
                     graphed=True)
    # The graph was captured at the first step and replayed 23 times across page boundaries.
    assert [t.argmax(-1).tolist() for t in eager] == [t.tolist() for t in graphed]


def test_int8_cache_step_stays_close_to_the_fp16_step():
    dev = device()
    fp16 = _drive(ds.DecodeModel(SHAPE, dev, max_pos=512, seed=4), _fresh("fp16"), _prompts(), steps=20)
    int8 = _drive(ds.DecodeModel(SHAPE, dev, max_pos=512, seed=4), _fresh("int8"), _prompts(), steps=20)
    # First batched step: identical inputs, only the cache precision differs.
    a, b = int8[0], fp16[0]
    assert torch.isfinite(a).all()
    assert (a - b).abs().max() <= 0.05 * b.abs().max() + 0.05

"""Regenerate the golden fixtures in this directory from the reference itself.

    PYTHONPATH=/path/to/LatentServe python tests/golden/make_golden.py

Needs an importable LatentServe tree (its repository root on PYTHONPATH); runs
on CPU. Inputs come from `latentserve_b200.synthetic` (numpy PCG64, so a seed is
the same bytes everywhere); outputs come from the reference's own functions:

    dense_*.npz    kernels.gqa.paged_decode.paged_decode_reference on fp32 queries
    int8_*.npz     cache.int8_paged_cache.Int8PagedKVCache driven through prefill and
                   deferred-finalize decode steps on CPU: pool bytes, scales, residual,
                   block tables, and paged_decode_reference over that state
    elementwise.npz  kernels.fused_elementwise.{rms_norm_ref, fused_add_rms_norm_ref, silu_and_mul_ref,
                   rope_qk_ref}
    sparse.npz     model.attention.sparse.page_bounds, kernels.cuda.paged_sparse.budget/budgets,
                   torch.topk on the scores, and the reference tests' masked-softmax attention

Each file also stores a checksum of its inputs, so a drift in the input
generator is told apart from a drift in the code under test.
"""

from __future__ import annotations

import hashlib
import pathlib
import sys

import numpy as np
import torch

HERE = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))

from latentserve_b200 import synthetic  # noqa: E402

from cache.int8_paged_cache import Int8PagedKVCache  # noqa: E402  (reference)
from cache.kv_cache import KVCacheSpec  # noqa: E402
from kernels.cuda import paged_sparse as ref_ps  # noqa: E402
from kernels.gqa import paged_decode as ref_pd  # noqa: E402
from model.attention.sparse import page_bounds as ref_page_bounds  # noqa: E402


def checksum(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def t(x):
    return torch.from_numpy(np.ascontiguousarray(x))


def dense(name, case):
    q, k, v = t(case["q"]), t(case["k_pool"]), t(case["v_pool"])
    tables, lens = t(case["block_tables"]), t(case["seq_lens"])
    out1 = ref_pd.paged_decode_reference(q.float(), k, v, tables, lens, num_splits=1)
    out3 = ref_pd.paged_decode_reference(q.float(), k, v, tables, lens, num_splits=3)
    np.savez_compressed(HERE / f"{name}.npz", out_splits1=out1.numpy(), out_splits3=out3.numpy(),
                        seq_lens=case["seq_lens"],
                        inputs_sha256=checksum(case["q"], case["k_pool"], case["v_pool"],
                                               case["block_tables"], case["seq_lens"]))


def int8_state(name, asym):
    """Prefill three sequences, then decode 21 steps in deferred-finalize mode
    (the CUDA-graph path's order of operations), all on CPU."""
    rng = np.random.default_rng(7 + int(asym))
    layers, h, d, mb, bs = 1, 2, 128, 3, 16
    spec = KVCacheSpec(num_layers=layers, num_kv_heads=h, head_dim=d, max_seq_len=160,
                       max_batch_size=mb, dtype=torch.float16, device="cpu")
    cache = Int8PagedKVCache(spec, block_size=bs, num_blocks=40, asymmetric=asym)
    prompt = [37, 80, 16]
    fed_k = [[] for _ in range(mb)]
    fed_v = [[] for _ in range(mb)]
    for i, n in enumerate(prompt):
        k = (rng.standard_normal((1, h, n, d), dtype=np.float32) * (0.3 + i)).astype(np.float16)
        v = (rng.standard_normal((1, h, n, d), dtype=np.float32) * (2.0 - 0.5 * i)).astype(np.float16)
        cache.advance(n, slots=[i])
        cache.write(0, t(k), t(v))
        fed_k[i].append(k[0])
        fed_v[i].append(v[0])
    cache.enable_deferred_finalize()
    steps = 21
    for _ in range(steps):
        k = rng.standard_normal((mb, h, 1, d), dtype=np.float32).astype(np.float16)
        v = (rng.standard_normal((mb, h, 1, d), dtype=np.float32) * 1.7).astype(np.float16)
        cache.advance(1, slots=[0, 1, 2])
        cache.write(0, t(k), t(v))
        for i in range(mb):
            fed_k[i].append(k[i])
            fed_v[i].append(v[i])
    q = rng.standard_normal((mb, h, 6, d), dtype=np.float32).astype(np.float16)
    tables = cache.block_tables_tensor(mb)
    lens = cache.seq_lens_tensor(mb)
    rows = cache.residual_rows_tensor(mb)
    kz = cache.k_zero_pool[0] if asym else None
    vz = cache.v_zero_pool[0] if asym else None
    out = ref_pd.paged_decode_reference(
        t(q).float(), cache.k_pool[0], cache.v_pool[0], tables, lens,
        k_scale=cache.k_scale_pool[0], v_scale=cache.v_scale_pool[0], k_zero=kz, v_zero=vz,
        num_splits=1, k_residual=cache.residual(0), res_rows=rows)
    save = dict(
        q=q, k_pool=cache.k_pool[0].numpy(), v_pool=cache.v_pool[0].numpy(),
        k_scale=cache.k_scale_pool[0].numpy(), v_scale=cache.v_scale_pool[0].numpy(),
        k_residual=cache.residual(0).numpy(), res_rows=rows.numpy(),
        block_tables=tables.numpy(), seq_lens=lens.numpy(), out=out.numpy(),
        prompt=np.asarray(prompt), steps=np.asarray(steps))
    if asym:
        save.update(k_zero=kz.numpy(), v_zero=vz.numpy())
    for i in range(mb):
        save[f"fed_k{i}"] = np.concatenate(fed_k[i], axis=1)       # [H, L, D]
        save[f"fed_v{i}"] = np.concatenate(fed_v[i], axis=1)
    np.savez_compressed(HERE / f"{name}.npz", **save)


def sparse():
    lens = [700, 333]
    case = synthetic.dense_case(lens, seed=11, page_offset_std=0.5)
    q, k, v = t(case["q"]), t(case["k_pool"]), t(case["v_pool"])
    tables, seq = t(case["block_tables"]), t(case["seq_lens"])
    bounds = {}
    for b, L in enumerate(lens):
        np_ = -(-L // 16)
        rows = torch.stack([k[int(tables[b, p // 16]), p % 16] for p in range(np_ * 16)], dim=1)
        ref = ref_page_bounds(q[b:b + 1].float(), rows[None].float(), 16).amax(dim=2)[0]   # [H, P]
        bounds[f"bounds{b}"] = ref.numpy()
    ratios = np.asarray([0.125, 0.25, 0.375, 0.5, 1.0], dtype=np.float64)
    probe_lens = torch.tensor([1, 15, 16, 17, 333, 700, 4096, 32768, 32767], dtype=torch.int32)
    per_seq = np.stack([ref_ps.budgets(probe_lens, float(r)).numpy() for r in ratios])
    per_call = np.asarray([[ref_ps.budget(float(r), p) for p in (1, 3, 21, 44, 2048)] for r in ratios])
    # The reference tests' own masked-softmax attention over fixed page picks.
    picks = [[0, 3, 7, 12, 20, 43], [0, 2, 5, 9, 30, 40]]
    out = torch.zeros(q.shape, dtype=torch.float32)
    for b, L in enumerate(lens):
        K = torch.stack([k[int(tables[b, p // 16]), p % 16] for p in range(L)], dim=1).float()
        V = torch.stack([v[int(tables[b, p // 16]), p % 16] for p in range(L)], dim=1).float()
        for h in range(q.shape[1]):
            keep = torch.zeros(L, dtype=torch.bool)
            for p in picks[b]:
                if p < -(-L // 16):
                    keep[p * 16:min(L, (p + 1) * 16)] = True
            s = (q[b, h].float() @ K[h].T) / np.sqrt(q.shape[-1])
            s = s.masked_fill(~keep[None, :], float("-inf"))
            out[b, h] = torch.softmax(s, -1) @ V[h]
    np.savez_compressed(
        HERE / "sparse.npz", seq_lens=np.asarray(lens), ratios=ratios,
        probe_lens=probe_lens.numpy(), budgets=per_seq, budget=per_call,
        picks=np.asarray(picks), attend_picks=out.numpy(),
        inputs_sha256=checksum(case["q"], case["k_pool"], case["v_pool"], case["block_tables"]),
        **bounds)


def elementwise():
    """The per-layer ops around attention, from the reference's torch forms
    (kernels/fused_elementwise.py:75-107): RMSNorm (+ residual), SiLU * up, RoPE."""
    from kernels import fused_elementwise as ref_fe

    rng = np.random.default_rng(21)
    x = (rng.standard_normal((7, 1536)) * 3).astype(np.float16)
    r = (rng.standard_normal((7, 1536)) * 2).astype(np.float16)
    w = (1 + 0.1 * rng.standard_normal(1536)).astype(np.float16)
    y = ref_fe.rms_norm_ref(t(x), t(w), 1e-6)
    y2, s2 = ref_fe.fused_add_rms_norm_ref(t(x), t(r), t(w), 1e-6)
    gu = (rng.standard_normal((5, 2 * 896)) * 2).astype(np.float16)
    act = ref_fe.silu_and_mul_ref(t(gu))
    q = rng.standard_normal((3, 1, 12 * 128)).astype(np.float16)
    k = rng.standard_normal((3, 1, 2 * 128)).astype(np.float16)
    ang = rng.uniform(0, 6.28, (3, 1, 1, 64)).astype(np.float32)
    ang = np.concatenate([ang, ang], -1)
    cos, sin = np.cos(ang).astype(np.float16), np.sin(ang).astype(np.float16)
    qo, ko = ref_fe.rope_qk_ref(t(q), t(k), t(cos), t(sin), 12, 2, 128)
    np.savez_compressed(HERE / "elementwise.npz", x=x, r=r, w=w, rms=y.numpy(), add_rms=y2.numpy(),
                        add_rms_sum=s2.numpy(), gu=gu, silu_mul=act.numpy(), q=q, k=k, cos=cos, sin=sin,
                        rope_q=qo.numpy(), rope_k=ko.numpy())


def main():
    torch.manual_seed(0)
    dense("dense_ragged", synthetic.dense_case([1024, 300, 61, 17, 1], seed=0))
    dense("dense_config1", synthetic.config1(seed=0))
    dense("dense_edges", synthetic.dense_case([15, 16, 17, 31, 32, 33, 1], seed=3))
    int8_state("int8_sym", asym=False)
    int8_state("int8_asym", asym=True)
    sparse()
    elementwise()
    for f in sorted(HERE.glob("*.npz")):
        print(f.name, f.stat().st_size)


if __name__ == "__main__":
    main()

"""Seeded synthetic workloads for the decode-attention path.

The reference's own benchmarks and kernel tests run on synthetic inputs —
N(0,1) K/V in a block pool, shuffled block tables, random queries
(benchmarks/runners/phase12_diag.py:91-124, tests/test_cuda_decode.py:69-79) —
and so does everything here. Inputs are drawn with numpy's PCG64 so that a
seed means the same bytes on every machine; the large benchmark pools are
drawn on the device instead (`dense_pools_on_device`).
"""

from __future__ import annotations

import numpy as np

PAGE = 16


def dense_case(lens, n_rep=6, h=2, d=128, seed=0, pool_blocks=None, q_scale=1.0, spare=3,
               page_offset_std=0.0):
    """A ragged decode batch over fp16 pools, as numpy arrays.

    Block tables are disjoint slices of one permutation of the pool, at the
    width of the longest sequence. `page_offset_std` adds a per-(block, head)
    mean offset to K so that page scores are well separated (the sparse cases).
    """
    rng = np.random.default_rng(seed)
    lens = [int(x) for x in lens]
    pages = max(1, (max(lens) + PAGE - 1) // PAGE)
    nb = pool_blocks if pool_blocks is not None else len(lens) * pages + spare
    if nb < len(lens) * pages:
        raise ValueError("pool too small for disjoint block tables")
    k = rng.standard_normal((nb, PAGE, h, d), dtype=np.float32)
    if page_offset_std:
        k += rng.standard_normal((nb, 1, h, d), dtype=np.float32) * np.float32(page_offset_std)
    v = rng.standard_normal((nb, PAGE, h, d), dtype=np.float32)
    tables = rng.permutation(nb)[: len(lens) * pages].reshape(len(lens), pages).astype(np.int32)
    q = rng.standard_normal((len(lens), h, n_rep, d), dtype=np.float32) * np.float32(q_scale)
    return {"q": q.astype(np.float16), "k_pool": k.astype(np.float16), "v_pool": v.astype(np.float16),
            "block_tables": tables, "seq_lens": np.asarray(lens, dtype=np.int32)}


def config1(seed=0):
    """Batch 4, 12 query / 2 KV heads, head_dim 128, page 16, lengths uniform
    in [512, 2048], pool of 1024 blocks, Q scaled by 1/sqrt(128)."""
    rng = np.random.default_rng(seed)
    lens = rng.integers(512, 2049, size=4)
    return dense_case(lens, seed=seed + 1, pool_blocks=1024, q_scale=1.0 / np.sqrt(128.0))


def to_torch(case: dict, device):
    import torch

    return {k: torch.from_numpy(np.ascontiguousarray(v)).to(device) for k, v in case.items()}


def dense_pools_on_device(batch, context, layers, device, n_rep=6, h=2, d=128, slack=1.2, seed=0,
                          dtype=None):
    """Benchmark-sized fp16 pools drawn on the device: `layers` pairs of
    [num_blocks, 16, h, d] N(0,1) pools with num_blocks = ceil(slack * needed),
    one shuffled block table shared by the layers, uniform `context` lengths
    (or a list of per-sequence lengths)."""
    import torch

    dtype = dtype or torch.float16
    g = torch.Generator(device=device).manual_seed(seed)
    lens = [context] * batch if isinstance(context, int) else [int(x) for x in context]
    pages = [-(-x // PAGE) for x in lens]
    width = max(pages)
    nb = int(np.ceil(slack * sum(pages)))
    perm = torch.randperm(nb, device=device, generator=g)
    tables = torch.zeros((batch, width), dtype=torch.int32, device=device)
    at = 0
    for i, n in enumerate(pages):
        tables[i, :n] = perm[at:at + n].to(torch.int32)
        at += n
    pools = []
    for _ in range(layers):
        k = torch.randn((nb, PAGE, h, d), dtype=dtype, device=device, generator=g)
        v = torch.randn((nb, PAGE, h, d), dtype=dtype, device=device, generator=g)
        pools.append((k, v))
    q = torch.randn((layers, batch, h, n_rep, d), dtype=dtype, device=device, generator=g)
    seq = torch.tensor(lens, dtype=torch.int32, device=device)
    return {"q": q, "pools": pools, "block_tables": tables, "seq_lens": seq, "num_blocks": nb}


def kv_bytes_fp16(lens, h=2, d=128) -> int:
    """Algorithmic bytes one layer call reads: every valid K and V row once."""
    return int(sum(int(x) for x in lens)) * h * d * 2 * 2


def kv_bytes_int8(lens, h=2, d=128) -> int:
    """INT8 layout: int8 K and V rows, an fp32 V scale per (token, head), an
    fp32 K scale per (page, head, channel)."""
    total = 0
    for x in lens:
        x = int(x)
        total += x * h * (d + d + 4) + (-(-x // PAGE)) * h * d * 4
    return total


def int8_pools_on_device(lens, layers, device, h=2, d=128, n_rep=6, slack=1.2, seed=0):
    """INT8 pools for a ragged batch, produced the way a serving cache produces
    them: N(0,1) fp16 K/V pushed through this library's quantize-on-write kernel
    (V, per token) and page-finalize kernel (K, per completed page); each
    sequence's last page of K stays exact in an fp16 residual row."""
    import torch

    from latentserve_b200 import int8_write as iw

    g = torch.Generator(device=device).manual_seed(seed)
    lens = [int(x) for x in lens]
    batch = len(lens)
    pages = [-(-x // PAGE) for x in lens]
    width = max(pages)
    nb = int(np.ceil(slack * sum(pages)))
    perm = torch.randperm(nb, device=device, generator=g)
    tables = torch.zeros((batch, width), dtype=torch.int32, device=device)
    at = 0
    for i, n in enumerate(pages):
        tables[i, :n] = perm[at:at + n].to(torch.int32)
        at += n
    consts = dict(eps=1e-8, qmax=127.0, levels=255.0, offset=128.0)
    out = []
    chunk = 2048                                     # blocks quantised per kernel call
    for _ in range(layers):
        k_pool = torch.zeros((nb, PAGE, h, d), dtype=torch.int8, device=device)
        v_pool = torch.zeros_like(k_pool)
        k_scale = torch.ones((nb, h, d), dtype=torch.float32, device=device)
        v_scale = torch.ones((nb, PAGE, h), dtype=torch.float32, device=device)
        residual = torch.randn((batch, PAGE, h, d), dtype=torch.float16, device=device, generator=g)
        scratch_res = torch.empty((chunk * PAGE, h, d), dtype=torch.float16, device=device)
        for lo in range(0, nb, chunk):
            n = min(chunk, nb - lo)
            ids = torch.arange(lo, lo + n, device=device)
            data = torch.randn((n, PAGE, h, d), dtype=torch.float16, device=device, generator=g)
            iw.finalize_blocks(data, torch.arange(n, device=device), ids, k_pool, k_scale, None, **consts)
            vals = torch.randn((n * PAGE, h, 1, d), dtype=torch.float16, device=device, generator=g)
            slots = torch.arange(lo * PAGE, (lo + n) * PAGE, device=device)
            iw.decode_write(vals, vals, slots, torch.arange(n * PAGE, device=device),
                            v_pool.view(-1, h, d), v_scale.view(-1, h), None, scratch_res,
                            asym=False, **consts)
        out.append(dict(k_pool=k_pool, v_pool=v_pool, k_scale=k_scale, v_scale=v_scale,
                        k_residual=residual))
    q = torch.randn((layers, batch, h, n_rep, d), dtype=torch.float16, device=device, generator=g)
    return {"q": q, "layers": out, "block_tables": tables,
            "seq_lens": torch.tensor(lens, dtype=torch.int32, device=device),
            "res_rows": torch.arange(batch, dtype=torch.int32, device=device), "num_blocks": nb}


def sparse_pools_on_device(batch, context, layers, device, h=2, d=128, n_rep=6, slack=1.2, seed=0,
                           offset_std=0.5):
    """fp16 pools whose K carries a per-(page, head) mean offset, so page scores
    are well separated, plus the per-page K bounds the indexer reads."""
    import torch

    w = dense_pools_on_device(batch, context, layers, device, n_rep, h, d, slack, seed)
    g = torch.Generator(device=device).manual_seed(seed + 1)
    bounds = []
    for k, _ in w["pools"]:
        off = torch.randn((k.shape[0], 1, h, d), dtype=torch.float16, device=device, generator=g)
        k.add_(off * offset_std)
        bounds.append((k.amin(dim=1), k.amax(dim=1)))
    w["bounds"] = bounds
    return w

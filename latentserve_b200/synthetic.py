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

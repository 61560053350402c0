"""Host-side logic that needs no device: block bookkeeping, budgets, the
eligibility rules, and the loud failures of the GPU-only entry points."""

import pytest
import torch

from latentserve_b200 import cache as lc
from latentserve_b200 import paged_decode as pd
from latentserve_b200 import paged_decode_cuda as pdc
from latentserve_b200 import paged_sparse as ps


def test_allocator_hands_out_reference_counted_blocks():
    a = lc.BlockAllocator(8, 16)
    got = a.allocate(3)
    assert len(set(got)) == 3 and a.num_free == 5 and a.num_used == 3
    a.incref(got[:1])
    a.free(got)
    assert a.num_free == 7 and a.ref_count(got[0]) == 1      # still shared
    a.free(got[:1])
    assert a.num_free == 8
    with pytest.raises(ValueError):
        a.free(got[:1])
    with pytest.raises(lc.OutOfBlocks):
        a.allocate(9)


def test_block_table_grows_by_pages_and_bumps_its_version():
    a = lc.BlockAllocator(8, 16)
    t = lc.BlockTable(a)
    t.append(15)
    v = t.version
    assert len(t.blocks) == 1
    t.append(1)
    assert len(t.blocks) == 1 and t.version == v                # same page: unchanged
    t.append(1)
    assert len(t.blocks) == 2 and t.version == v + 1
    assert t.slot(16) == t.blocks[1] * 16
    with pytest.raises(IndexError):
        t.slot(17)
    t.free()
    assert a.num_free == 8 and t.length == 0


def test_slot_reuse_gets_its_own_blocks():
    """A freed slot reused by a sequence with the same page count must not be
    taken for unchanged: the version moves on free()."""
    a = lc.BlockAllocator(8, 16)
    t = lc.BlockTable(a)
    t.append(20)
    before = (tuple(t.blocks), t.version)
    t.free()
    t.append(20)
    assert t.version != before[1]


def test_budget_rules():
    assert ps.budget(0.25, 2048) == 512 and ps.budget(1.0, 77) == 77
    assert ps.budget(0.01, 10) == 3                              # sink + 2 recent at least
    lens = torch.tensor([4096, 700, 17, 1], dtype=torch.int32)
    assert ps.budgets(lens, 0.375).tolist() == [96, 17, 2, 1]


def test_cpu_tensors_are_refused_not_rerouted():
    q = torch.zeros(1, 2, 6, 128, dtype=torch.float16)
    k = torch.zeros(4, 16, 2, 128, dtype=torch.float16)
    tables = torch.zeros(1, 4, dtype=torch.int32)
    lens = torch.ones(1, dtype=torch.int32)
    assert not pdc.eligible(q, k)
    with pytest.raises(RuntimeError, match="no CPU path"):
        pd.paged_decode_attention(q, k, k, tables, lens)
    with pytest.raises(RuntimeError, match="no CPU path"):
        pdc.paged_decode_cuda(q, k, k, tables, lens, 16)
    with pytest.raises(RuntimeError, match="no reference"):
        pd.paged_decode_attention(q, k, k, tables, lens, force_reference=True)
    with pytest.raises(RuntimeError, match="CUDA device"):
        lc.PagedKVCache(lc.KVCacheSpec(1, 2, 128, 64, 2, device="cpu"))


def test_only_the_cuda_backend_exists():
    pd.set_decode_backend("cuda")
    assert pd.decode_backend() == "cuda"
    with pytest.raises(ValueError):
        pd.set_decode_backend("triton")

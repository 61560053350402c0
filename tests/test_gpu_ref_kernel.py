"""The reference's own CUDA kernels, compiled for sm_100a by oracle/build_ref.py,
driven by oracle/ref_kernels.py: checked here against the numpy oracle and
against this library, so that the time bench.py reports for "the reference's
kernel on this box" is the time of a correct run."""

import numpy as np
import pytest
import torch

from latentserve_b200 import paged_decode_cuda as pdc
from latentserve_b200 import synthetic
from oracle import paged_attention_oracle as orc
from oracle import ref_kernels
from tests.gpu_util import close, on_device

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(not ref_kernels.available("paged_decode_fp16"),
                    reason="oracle/_ref/paged_decode_fp16.cubin not built (needs a LatentServe checkout)")
def test_reference_fp16_kernel_agrees_with_the_oracle_and_with_this_library():
    case = synthetic.dense_case([1024, 300, 61, 17, 1], seed=0)
    want = orc.paged_decode(case["q"], case["k_pool"], case["v_pool"], case["block_tables"],
                            case["seq_lens"])
    t = on_device(case)
    ref = ref_kernels.RefDecode(t["q"], t["k_pool"], t["v_pool"], t["block_tables"], t["seq_lens"], 1024)
    ref.launch()
    got_ref = ref.combine()
    close(got_ref, want)
    ours = pdc.paged_decode_cuda(t["q"], t["k_pool"], t["v_pool"], t["block_tables"], t["seq_lens"], 1024)
    assert (ours.float() - got_ref.float()).abs().max() <= 4e-3


@pytest.mark.skipif(not ref_kernels.available("paged_decode_int8"),
                    reason="oracle/_ref/paged_decode_int8.cubin not built (needs a LatentServe checkout)")
def test_reference_int8_kernel_agrees_with_the_oracle(golden_dir):
    g = np.load(golden_dir / "int8_sym.npz")
    dev = torch.device("cuda")
    t = {k: torch.from_numpy(np.ascontiguousarray(g[k])).to(dev)
         for k in ("q", "k_pool", "v_pool", "k_scale", "v_scale", "k_residual", "res_rows", "block_tables",
                   "seq_lens")}
    ref = ref_kernels.RefDecode(t["q"], t["k_pool"], t["v_pool"], t["block_tables"], t["seq_lens"],
                                int(g["seq_lens"].max()), k_scale=t["k_scale"], v_scale=t["v_scale"],
                                k_residual=t["k_residual"], res_rows=t["res_rows"])
    ref.launch()
    close(ref.combine(), g["out"])


@pytest.mark.skipif(not ref_kernels.available("paged_sparse_fp16"),
                    reason="oracle/_ref/paged_sparse_fp16.cubin not built (needs a LatentServe checkout)")
def test_reference_sparse_trio_agrees_with_the_oracle_and_with_this_library():
    from latentserve_b200 import paged_sparse as ps

    case = synthetic.dense_case([2000, 1111, 300], seed=5, page_offset_std=0.5)
    t = on_device(case)
    kmin, kmax = t["k_pool"].amin(dim=1), t["k_pool"].amax(dim=1)      # every page here is full or last
    for b, L in enumerate([2000, 1111, 300]):                          # last pages: written rows only
        if L % 16:
            blk = int(t["block_tables"][b, L // 16])
            kmin[blk] = t["k_pool"][blk, :L % 16].amin(dim=0)
            kmax[blk] = t["k_pool"][blk, :L % 16].amax(dim=0)
    ref = ref_kernels.RefSparse(t["q"], t["k_pool"], t["v_pool"], t["block_tables"], t["seq_lens"], kmin, kmax,
                                ratio=0.5, max_seq_len=2000)
    ref.launch()
    got_ref = ref.combine()
    scores = orc.page_scores(case["q"], kmin.cpu().numpy(), kmax.cpu().numpy(), case["block_tables"],
                             case["seq_lens"])
    assert np.array_equal(ref.scores.cpu().numpy(), scores)            # the same fp32 evaluation order
    sel = orc.select(scores, ref.k)
    want = orc.sparse_decode(case["q"], case["k_pool"], case["v_pool"], case["block_tables"],
                             case["seq_lens"], sel, ratio=0.5)
    close(got_ref, want)
    ours = ps.sparse_attention(t["q"], t["k_pool"], t["v_pool"], t["block_tables"], t["seq_lens"], kmin, kmax,
                               ratio=0.5, max_seq_len=2000)
    assert (ours.float() - got_ref.float()).abs().max() <= 4e-3

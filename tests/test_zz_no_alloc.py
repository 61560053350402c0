"""The allocation-free decode entry point, called through the C ABI.

`ls_paged_decode_fp16_noalloc` exists for callers that have nowhere to get
scratch memory from — an FFI host without a device allocator, or a server that
gave all device memory to its KV pools at start-up — so this test hands it
nothing but inputs and an output and checks the result against the ordinary
entry point, which takes its scratch from the caller. Two calls in a row with
different batch shapes make sure that what the first call leaves in the shared
built-in array does not leak into the second.

Collected last on purpose (the name sorts after every other test file): a run
that stops at the first failure has by then exercised everything else.
"""

import numpy as np
import pytest
import torch

from latentserve_b200 import _lib
from latentserve_b200 import paged_decode_cuda as pdc
from latentserve_b200 import synthetic
from oracle import paged_attention_oracle as orc
from tests.gpu_util import ATOL, RTOL, close, device, on_device

pytestmark = pytest.mark.gpu


def _noalloc(t, chunks):
    q, k, v = t["q"], t["k_pool"], t["v_pool"]
    b, h, r, d = q.shape
    out = torch.full((b, h, r, d), float("nan"), dtype=torch.float16, device=q.device)
    rc = _lib.lib().ls_paged_decode_fp16_noalloc(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), t["block_tables"].data_ptr(),
        t["seq_lens"].data_ptr(), out.data_ptr(), b, h, r, d, k.shape[1],
        t["block_tables"].stride(0), k.shape[0], chunks, pdc.MIN_CHUNK_PAGES,
        q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
        out.stride(0), out.stride(1), out.stride(2), 1.0 / np.sqrt(d),
        _lib.current_stream(q.device))
    return rc, out


def test_two_calls_in_a_row_match_the_ordinary_entry_point():
    dev = device()
    cases = [synthetic.dense_case([4000, 900, 33, 0, 17], seed=41),     # 5 sequences, several segments
             synthetic.dense_case([2500, 64], seed=42)]                 # then a smaller batch
    for case in cases:
        t = on_device(case)
        chunks = pdc.choose_chunks(dev, t["q"].shape[1], None, t["q"].shape[0])
        want = pdc.paged_decode_cuda(t["q"], t["k_pool"], t["v_pool"], t["block_tables"],
                                     t["seq_lens"], 4096).clone()
        rc, got = _noalloc(t, chunks)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.isfinite(got).all()
        assert torch.allclose(got.float(), want.float(), atol=ATOL, rtol=RTOL)
        # and both against the CPU oracle, like every other decode test
        close(got, orc.paged_decode(case["q"], case["k_pool"], case["v_pool"], case["block_tables"],
                                    case["seq_lens"]))


def test_shapes_past_the_fixed_scratch_are_refused():
    t = on_device(synthetic.dense_case([64, 64], seed=43))
    rc, _ = _noalloc(t, 2000)                      # (2 + 2000) * 2 rows > 1024
    assert rc == -8
    with pytest.raises(ValueError, match="fixed scratch"):
        _lib.check(rc, "noalloc")
    big = on_device(synthetic.dense_case([16] * 65, seed=44))
    rc, _ = _noalloc(big, 8)                       # 65 sequences > 64
    assert rc == -8


def test_a_block_id_outside_the_pool_is_skipped_not_read():
    """The kernel checks every block id against the pool size on the device and
    skips a page whose id is out of range, so a corrupt table cannot make this
    entry point read outside the pool. The flag that records the skip lives in the
    built-in array, which this entry point gives no way to read: the call still
    returns 0 and the output is finite, computed without that page."""
    case = synthetic.dense_case([64, 64], seed=45)
    t = on_device(case)
    t["block_tables"][1, 2] = 10_000_000
    rc, got = _noalloc(t, pdc.choose_chunks(device(), 2, None, 2))
    torch.cuda.synchronize()
    assert rc == 0 and torch.isfinite(got).all()
    # Sequence 0 is untouched by the bad entry; sequence 1 equals attention without page 2.
    want = orc.paged_decode(case["q"], case["k_pool"], case["v_pool"], case["block_tables"], case["seq_lens"])
    close(got[0:1], want[0:1])
    sel = np.array([[[0, 1, 3], [0, 1, 3]]] * 2, dtype=np.int32)
    without = orc.sparse_decode(case["q"], case["k_pool"], case["v_pool"], case["block_tables"],
                                case["seq_lens"], sel)
    close(got[1:2], without[1:2])

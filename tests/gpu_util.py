"""Helpers shared by the GPU parity tests."""

import numpy as np
import torch

from latentserve_b200 import synthetic

# Tolerance of the fp16 attention output against the fp32 oracle.
ATOL, RTOL = 2e-3, 1e-2


def device():
    if not torch.cuda.is_available():
        raise RuntimeError("this test was selected with -m gpu but no CUDA device is visible")
    return torch.device("cuda", 0)


def on_device(case):
    return synthetic.to_torch(case, device())


def close(got: torch.Tensor, want: np.ndarray, atol=ATOL, rtol=RTOL):
    got = got.detach().float().cpu().numpy()
    assert np.isfinite(got).all(), "non-finite values in the kernel output"
    err = np.abs(got - want)
    bound = atol + rtol * np.abs(want)
    assert (err <= bound).all(), f"max abs err {err.max():.3e}, worst excess {(err - bound).max():.3e}"

"""Loader for the C-ABI library (`_C/libls_b200.so`) and its ctypes prototypes.

The library is the product: there is no PyTorch, Triton or CPU stand-in behind
these calls. If it is missing or fails to load, `lib()` raises — callers do not
catch that and carry on. Build it with `python -m latentserve_b200.build`.

Status codes (`include/latentserve_b200.h`) become the exceptions the
reference raises for the same mistakes: layout violations are `ValueError`
(kernels/cuda/paged_decode_cuda.py:214-217), CUDA launch errors `RuntimeError`.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_int64, c_void_p

import torch

from latentserve_b200 import build as _build

_LIB = None

STATUS = {
    -1: "null pointer for a required tensor",
    -2: "bad shape or count",
    -3: "unsupported stride",
    -4: "pointer or stride not aligned for vector access",
    -5: "size past what the kernel supports",
    -6: "unsupported configuration (needs head_dim 128, page 16, <= 8 query rows per KV head)",
    -7: "scratch buffer too small",
    -8: "shape past the fixed scratch of the allocation-free entry point "
        "(needs batch <= 64 and (batch + num_chunks) * kv_heads <= 1024)",
}

P, I, L, F = c_void_p, c_int, c_int64, c_float

_PROTOTYPES = {
    "ls_decode_slots": [I, I],
    "ls_paged_decode_fp16": [P, P, P, P, P, P, P, P, P, P] + [I] * 10 + [L] * 9 + [F, P],
    "ls_paged_decode_append_fp16": [P] * 12 + [I] * 10 + [L] * 13 + [F, P],
    "ls_paged_sparse_fp16": [P, P, P, P, P, P, F, I, P, P, P, P, P] + [I] * 11 + [L] * 11 + [F, P],
    "ls_paged_decode_int8": [P] * 16 + [I] * 11 + [L] * 17 + [F, P],
    "ls_paged_sparse_int8": [P, F, I, I, L, L] + [P] * 16 + [I] * 11 + [L] * 17 + [F, P],
    "ls_paged_decode_fp16_noalloc": [P, P, P, P, P, P] + [I] * 9 + [L] * 9 + [F, P],
    "ls_combine": [P, P, P, P, P, I, I, I, L, L, L, P],
    "ls_kv_append_fp16": [P, P, P, P, P, P, P, I, I, I, I] + [L] * 9 + [P],
    "ls_int8_decode_write": [P, P, P, P, P, P, P, P, I, I, I] + [L] * 6 + [I] + [F] * 6 + [P],
    "ls_int8_finalize_blocks": [P, P, P, P, P, P, I, I, I, I] + [L] * 10 + [I] + [F] * 6 + [P],
    "ls_int8_finalize_layers": [P, P, P, P, P, P, I, I, I, I, I] + [L] * 13 + [I] + [F] * 6 + [P],
    "ls_int8_finalize_pending": [P, P, P, P, P, P, P, I, I, I, I, I] + [L] * 13 + [I] + [F] * 6 + [P],
    "ls_page_index": [P, P, P, P, P, P] + [I] * 9 + [L] * 7 + [P],
    "ls_page_index_heads": [P, P, P, P, P, P] + [I] * 8 + [L] * 8 + [P],
    "ls_page_index_select": [P] * 7 + [I] * 10 + [F, I] + [L] * 9 + [P],
    "ls_select_pages": [P, P, P, I, I, I, I, F, I, L, L, L, L, P],
    "ls_topk_pages": [P, P, I, I, I, I, L, L, L, L, P],
    "ls_rms_norm": [P, P, P, P, P, I, I, F, L, L, L, L, P],
    "ls_silu_mul": [P, P, I, I, L, L, P],
    "ls_rope_append_fp16": [P] * 10 + [I] * 5 + [L] * 9 + [P],
    "ls_skinny_gemm": [P] * 5 + [I] + [P] * 7 + [I] * 5 + [F] + [L] * 6 + [P],
    "ls_rope_append_int8": [P] * 13 + [I] * 4 + [L] * 8 + [I] + [F] * 6 + [P],
    "ls_qkv_rope_append_fp16": [P] * 3 + [I] + [P] * 13 + [I] * 8 + [F] + [L] * 10 + [P],
}


def exported_symbols() -> list[str]:
    return sorted(_PROTOTYPES)


def lib() -> ctypes.CDLL:
    """The loaded library, building it first if the sources are newer."""
    global _LIB
    if _LIB is None:
        # LATENTSERVE_B200_LIB names a prebuilt library to load instead (tuning builds).
        path = os.environ.get("LATENTSERVE_B200_LIB") or _build.build()
        handle = ctypes.CDLL(str(path))
        for name, argtypes in _PROTOTYPES.items():
            fn = getattr(handle, name)          # AttributeError = a symbol the header promises is gone
            fn.argtypes = argtypes
            fn.restype = c_int
        _LIB = handle
    return _LIB


def check(status: int, what: str) -> None:
    if status == 0:
        return
    if status < 0:
        raise ValueError(f"{what}: {STATUS.get(status, f'status {status}')}")
    raise RuntimeError(f"{what}: CUDA error {status} at launch")


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def current_stream(device) -> int:
    """Raw handle of torch's current stream on `device`."""
    index = device.index if isinstance(device, torch.device) else torch.device(device).index
    return raw_stream(torch.cuda.current_device() if index is None else index)


def raw_stream(device_index: int) -> int:
    """Raw handle of torch's current stream on device `device_index`, which must be
    the current device: the library launches on whatever device is current, so a
    stream of another device would fail at launch with an opaque CUDA error (and the
    allocation-free entry point would take the wrong device's built-in array)."""
    current = torch.cuda.current_device()
    if device_index != current:
        raise RuntimeError(f"tensors live on cuda:{device_index} but the current device is cuda:{current}; "
                           f"call inside `with torch.cuda.device({device_index}):`")
    return torch._C._cuda_getCurrentRawStream(device_index)

"""B200-native (sm_100a) paged decode attention for LatentServe.

The package holds one hot path and nothing else:

    paged_decode        entry point / backend switch      (reference: kernels/gqa/paged_decode.py)
    paged_decode_cuda   dense fp16 + INT8 decode           (reference: kernels/cuda/paged_decode_cuda.py)
    paged_sparse        page scores, top-k, sparse decode  (reference: kernels/cuda/paged_sparse.py)
    int8_write          quantize-on-write, page finalize   (reference: kernels/cuda/int8_write.py)
    kv_write            fp16 append + page bounds          (reference: cache/paged_cache.py write path)
    cache               paged caches over those kernels    (reference: cache/*.py)
    dropin              installs the above into an importable reference tree
    csrc/, _C/          the CUDA sources and the built C-ABI library

Importing the package does not load the library; the first kernel call does,
and raises if it is missing.
"""

__version__ = "0.1.0"

"""dyninfer_b200 — B200 (sm_100a) `cuda` target for dyninfer's direct quantized decoder path.

The compute lives in libdyninfer_cuda.so (hand-written CUDA behind a C ABI, see
include/dyninfer_cuda.h); this package is the host-side mirror of the reference's
runtime interface for that path plus the checkpoint/byte-range plumbing.
"""
from ._lib import DynInferError  # noqa: F401

__all__ = ["DynInferError"]

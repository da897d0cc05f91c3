"""ctypes binding of libdyninfer_cuda.so — the reference-side FFI stub, in Python.

Every prototype here matches include/dyninfer_cuda.h. Loading fails loudly when the
library has not been built: there is no Python or CPU substitute for it.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# DYNINFER_CUDA_LIB names another build of the library (e.g. one compiled with different kernel options)
LIB_PATH = os.environ.get("DYNINFER_CUDA_LIB") or os.path.join(HERE, "libdyninfer_cuda.so")

ENC = {"plain.f32": 0, "plain.f16": 1, "plain.bf16": 2, "gguf.q4_0": 3, "gguf.q4_1": 4,
       "gguf.q8_0": 5, "gguf.q6_k": 6, "mlx.affine.u4": 7, "gguf.q4_k": 8, "gguf.q5_k": 9, "gguf.iq4_xs": 10}
ENC_NAME = {v: k for k, v in ENC.items()}


class DynInferError(RuntimeError):
    """A failed native call; the message is the library's thread-local last error."""


class Weight(C.Structure):
    _fields_ = [("encoding", C.c_int32), ("aux_type", C.c_int32), ("group", C.c_int32),
                ("reserved", C.c_int32), ("rows", C.c_int64), ("cols", C.c_int64),
                ("data", C.c_void_p), ("scales", C.c_void_p), ("biases", C.c_void_p)]


class ParameterFile(C.Structure):
    _fields_ = [("path", C.c_char_p)]


class FileParam(C.Structure):
    _fields_ = [("key", C.c_char_p), ("source_file_index", C.c_size_t),
                ("offset", C.c_uint64), ("length", C.c_uint64)]


class AllocatorStatistics(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("host_bytes_peak", "host_bytes_allocated",
                                          "host_bytes_freed", "device_bytes_peak",
                                          "device_bytes_allocated", "device_bytes_freed")]


_P = C.c_void_p
_I64 = C.c_int64
PROTOTYPES = {
    "dyninfer_cuda_abi_version": (C.c_int, []),
    "dyninfer_cuda_last_error": (C.c_char_p, []),
    "dyninfer_cuda_device_count": (C.c_int, [C.POINTER(C.c_int)]),
    "dyninfer_cuda_check_device_error": (C.c_int, []),
    "dyninfer_cuda_row_bytes": (C.c_uint64, [C.c_int, _I64]),
    "dyninfer_cuda_dequant": (C.c_int, [C.POINTER(Weight), _P, _P]),
    "dyninfer_cuda_embedding_gather": (C.c_int, [C.POINTER(Weight), _P, _I64, _P, _P]),
    "dyninfer_cuda_linear": (C.c_int, [C.POINTER(Weight), _P, C.c_int, _I64, _P, _P]),
    "dyninfer_cuda_rms_norm": (C.c_int, [_P, _P, C.c_int, _I64, _I64, C.c_float, _P, _P]),
    "dyninfer_cuda_rope": (C.c_int, [_P, _I64, _I64, _I64, _I64, C.c_float, _P]),
    "dyninfer_cuda_silu_mul": (C.c_int, [_P, _P, _I64, _P, _P]),
    "dyninfer_cuda_attention": (C.c_int, [_P, _P, _P, C.c_int, _I64, _I64, _I64, _I64, _I64, _I64, _P, _P]),
    "dyninfer_cuda_argmax_scratch_bytes": (C.c_size_t, [_I64]),
    "dyninfer_cuda_argmax": (C.c_int, [_P, _I64, _P, _P, _P]),
    "dyninfer_cuda_argmax_static_max_n": (_I64, []),
    "dyninfer_cuda_argmax_static": (C.c_int, [_P, _I64, _P, _P]),
    "dyninfer_cuda_session_create_with_file_params": (
        C.c_int, [C.c_char_p, C.c_char_p, C.POINTER(ParameterFile), C.c_size_t,
                  C.POINTER(FileParam), C.c_size_t, C.POINTER(_P)]),
    "dyninfer_cuda_session_destroy": (None, [_P]),
    "dyninfer_cuda_free": (None, [_P]),
    "dyninfer_cuda_session_configure_paged_kv": (C.c_int, [_P] + [C.c_size_t] * 7),
    "dyninfer_cuda_session_ensure_kv_pages": (C.c_int, [_P, C.c_size_t]),
    "dyninfer_cuda_session_invoke_paged_chunk": (
        C.c_int, [_P, C.POINTER(_I64), C.c_size_t, _I64, _I64, C.POINTER(C.POINTER(C.c_float)),
                  C.POINTER(C.c_size_t), C.POINTER(_I64), C.c_int]),
    "dyninfer_cuda_session_invoke_paged_chunk_slot": (
        C.c_int, [_P, C.POINTER(_I64), C.c_size_t, _I64, _I64, _I64, C.POINTER(C.POINTER(C.c_float)),
                  C.POINTER(C.c_size_t), C.POINTER(_I64), C.c_int]),
    "dyninfer_cuda_session_decode_batch": (
        C.c_int, [_P, C.POINTER(_I64), C.POINTER(_I64), C.POINTER(_I64), C.c_size_t, C.POINTER(_I64),
                  C.POINTER(C.POINTER(C.c_float)), C.c_int]),
    "dyninfer_cuda_tp_unique_id_bytes": (C.c_size_t, []),
    "dyninfer_cuda_tp_unique_id": (C.c_int, [C.c_char_p, C.c_size_t]),
    "dyninfer_cuda_session_tp_init": (C.c_int, [_P, C.c_char_p, C.c_size_t]),
    "dyninfer_cuda_tp_peer_handle_bytes": (C.c_size_t, []),
    "dyninfer_cuda_session_tp_peer_handle": (C.c_int, [_P, C.c_char_p, C.c_size_t]),
    "dyninfer_cuda_session_tp_peer_attach": (C.c_int, [_P, C.c_char_p, C.c_size_t]),
    "dyninfer_cuda_tp_exchange_wait_probe": (C.c_int, [C.c_int, _I64, _I64]),
    "dyninfer_cuda_session_reset_paged_kv": (C.c_int, [_P]),
    "dyninfer_cuda_session_kv_page_count": (C.c_size_t, [_P]),
    "dyninfer_cuda_session_kv_allocated_bytes": (C.c_size_t, [_P]),
    "dyninfer_cuda_session_allocator_statistics": (C.c_int, [_P, C.POINTER(AllocatorStatistics)]),
    "dyninfer_cuda_session_weight_bytes": (C.c_uint64, [_P]),
    "dyninfer_cuda_session_decode_weight_bytes": (C.c_uint64, [_P]),
    "dyninfer_cuda_session_decode_loop": (C.c_int, [_P, _I64, _I64, C.c_size_t, C.POINTER(_I64),
                                                    C.POINTER(C.c_float)]),
    "dyninfer_cuda_session_launch_count": (C.c_uint64, [_P]),
    "dyninfer_cuda_session_uses_persistent_kernel": (C.c_int, [_P]),
    "dyninfer_cuda_session_decode_trace": (C.c_int, [_P, C.POINTER(C.c_uint64), C.c_size_t, C.POINTER(C.c_size_t)]),
    "dyninfer_cuda_session_timer": (C.c_int, [_P, C.c_int, C.POINTER(C.c_float)]),
    "dyninfer_cuda_session_decode_phase_profile": (C.c_int, [_P, C.POINTER(C.c_double), C.c_size_t]),
}

_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise DynInferError(
                f"{LIB_PATH} is missing: build it with `python -m dyninfer_b200.build` "
                "(nvcc, sm_100a). There is no fallback implementation.")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def last_error() -> str:
    return (lib().dyninfer_cuda_last_error() or b"").decode("utf-8", "replace")


def check(rc: int):
    if rc != 0:
        raise DynInferError(last_error())

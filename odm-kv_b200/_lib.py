"""ctypes binding of ``libodmkv_b200.so`` (the C ABI declared in ``include/odmkv_b200.h``).

There is no fallback: if the shared object is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_double, c_float, c_int, c_int32, c_int64, c_longlong, c_size_t, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libodmkv_b200.so")

NUM_QLEVELS = 4
NUM_CLASSES = 6
SEG_ALIGN = 16
TILE = 128
HEAD_DIM = 128
MAX_LEVELS = 8
MAX_CHUNKS = 12
QLEVEL_BITS = (2, 3, 4, 8)
CLASS_BITS = (0, 2, 3, 4, 8, 16)
CODE_BYTES = (32, 48, 64, 128)
REF_CODE_BYTES = (32, 64, 64, 128)

DTYPE_F16, DTYPE_BF16, DTYPE_F32 = 0, 1, 2


class Chunk(ctypes.Structure):
    """Mirror of ``odmkv_chunk``."""

    _fields_ = [
        ("k_codes", c_void_p * NUM_QLEVELS),
        ("v_codes", c_void_p * NUM_QLEVELS),
        ("k_norm", c_void_p * NUM_QLEVELS),
        ("v_norm", c_void_p * NUM_QLEVELS),
        ("pos", c_void_p * NUM_QLEVELS),
        ("exact_k", c_void_p),
        ("exact_v", c_void_p),
        ("exact_pos", c_void_p),
        ("evicted_pos", c_void_p),
        ("seg_start", c_void_p),
        ("seg_count", c_void_p),
        ("cap", c_int32 * NUM_CLASSES),
        ("B", c_int32),
        ("H", c_int32),
        ("T", c_int32),
        ("t_offset", c_int32),
    ]


class AllocReport(ctypes.Structure):
    """Mirror of ``odmkv_alloc_report``."""

    _fields_ = [
        ("lam", c_double),
        ("gap_before", c_double),
        ("counts", c_longlong * MAX_LEVELS),
        ("n_active", c_int),
        ("evaluations", c_int),
        ("moved", c_int),
        ("ties_lambda", c_int),
        ("ties_cut", c_int),
        ("done", c_int),
    ]


_PROTOTYPES = {
    "odmkv_abi_version": (c_int, []),
    "odmkv_status_string": (c_char_p, [c_int]),
    "odmkv_score_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "odmkv_score_status_offset": (c_size_t, [c_int, c_int, c_int, c_int, c_int]),
    "odmkv_score_prefill": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                    c_void_p, c_void_p, c_size_t, c_void_p]),
    "odmkv_score_with_attn": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p, c_void_p]),
    "odmkv_alloc_workspace_bytes": (c_size_t, [c_int, c_int]),
    "odmkv_allocate_bits": (c_int, [c_void_p, c_void_p, c_int, c_int, POINTER(c_int), POINTER(c_double), c_int, c_double,
                                    c_int, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "odmkv_alloc_exchange_len": (c_size_t, []),
    "odmkv_alloc_begin": (c_int, [c_void_p, c_void_p, c_int, c_int, c_longlong, POINTER(c_int), POINTER(c_double), c_int,
                                  c_double, c_int, c_void_p, c_size_t, c_void_p, c_void_p]),
    "odmkv_alloc_eval": (c_int, [c_void_p, c_void_p, c_void_p]),
    "odmkv_alloc_update": (c_int, [c_void_p, c_void_p, c_void_p]),
    "odmkv_alloc_num_rounds": (c_int, [c_int]),
    "odmkv_alloc_finish": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p]),
    "odmkv_pack_plan_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "odmkv_pack_plan": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "odmkv_quantize_workspace_bytes": (c_size_t, [POINTER(c_int32)]),
    "odmkv_quantize_pack": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, POINTER(Chunk),
                                    c_void_p, c_void_p, c_size_t, c_void_p]),
    "odmkv_encode_pack": (c_int, [c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p]),
    "odmkv_dequant_chunk": (c_int, [POINTER(Chunk), c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                    c_int, c_void_p]),
    "odmkv_export_bank": (c_int, [POINTER(Chunk), c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "odmkv_export_positions": (c_int, [POINTER(Chunk), c_int, c_void_p, c_void_p, c_void_p]),
    "odmkv_compact_chunks": (c_int, [POINTER(Chunk), c_int, POINTER(Chunk), c_void_p, c_int, c_void_p, c_size_t, c_void_p]),
    "odmkv_decode_attn_mma": (c_int, [c_void_p, c_int, POINTER(Chunk), c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p,
                                      c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_int, c_void_p, c_int,
                                      c_void_p, c_size_t, POINTER(c_float), c_void_p]),
    "odmkv_decode_attn_mma_devtail": (c_int, [c_void_p, c_int, POINTER(Chunk), c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                              c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_int,
                                              c_void_p, c_int, c_void_p, c_size_t, POINTER(c_float), c_void_p]),
    "odmkv_decode_attn_noalloc_scratch_bytes": (c_size_t, []),
    "odmkv_decode_attn_noalloc": (c_int, [c_void_p, c_int, POINTER(Chunk), c_int, c_int, c_void_p, c_void_p, c_int, c_int,
                                          c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_int, c_void_p,
                                          c_int, POINTER(c_float), c_void_p]),
    "odmkv_quantize_status": (c_int, []),
    "odmkv_window_stats_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "odmkv_window_stats_status_offset": (c_size_t, [c_int, c_int, c_int, c_int]),
    "odmkv_window_stats_last_path": (c_int, []),
    "odmkv_window_stats_force_thread_copies": (None, [c_int]),
    "odmkv_window_attn_stats": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p,
                                        c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "odmkv_timing_enable": (None, [c_int]),
    "odmkv_timing_read": (c_int, [c_char_p, POINTER(c_double), POINTER(c_longlong)]),
    "odmkv_decode_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "odmkv_decode_default_splits": (c_int, [c_int, c_int, c_longlong]),
    "odmkv_decode_attn": (c_int, [c_void_p, c_int, POINTER(Chunk), c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p,
                                  c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_int, c_void_p, c_int,
                                  c_void_p, c_size_t, c_void_p]),
}

_OPTIONAL: dict = {}

_lib = None


class OdmkvError(RuntimeError):
    pass


def exported_symbols() -> list[str]:
    """Every symbol the public header declares (used by the load test)."""
    return sorted(_PROTOTYPES)


def lib() -> ctypes.CDLL:
    """Load the CUDA library; fail loudly when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise OdmkvError(
                f"{LIB_PATH} is missing: build it with `python odm-kv_b200/build.py` (needs nvcc). "
                "There is no CPU or PyTorch fallback for this library's kernels.")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        for name, (res, args) in _OPTIONAL.items():
            if hasattr(handle, name):
                fn = getattr(handle, name)
                fn.restype = res
                fn.argtypes = args
        if handle.odmkv_abi_version() != 1:
            raise OdmkvError("libodmkv_b200.so has an unexpected ABI version")
        _lib = handle
    return _lib


def check(rc: int, what: str) -> None:
    """Map a status code to an exception: shape errors are ValueError as in the reference's
    ``_validate_shapes`` (kvquant/tq_adaptive_backend.py:320-336), everything else RuntimeError."""
    if rc == 0:
        return
    msg = lib().odmkv_status_string(rc).decode()
    if rc in (-1, -2, -4):
        raise ValueError(f"{what}: {msg} (status {rc})")
    raise OdmkvError(f"{what}: {msg} (status {rc})")


def dtype_code(dtype) -> int:
    import torch

    if dtype == torch.float16:
        return DTYPE_F16
    if dtype == torch.bfloat16:
        return DTYPE_BF16
    if dtype == torch.float32:
        return DTYPE_F32
    raise ValueError(f"unsupported cache dtype {dtype}")


def ptr(t) -> c_void_p:
    """Device pointer of a torch tensor (None -> NULL)."""
    return c_void_p(0) if t is None else c_void_p(t.data_ptr())


def stream_ptr(device=None) -> c_void_p:
    import torch

    return c_void_p(torch.cuda.current_stream(device).cuda_stream)


def require_cuda(t, name: str) -> None:
    if not t.is_cuda:
        raise OdmkvError(f"{name} must live on a CUDA device: this library has no CPU path")

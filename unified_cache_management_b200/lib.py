"""ctypes binding of ``libucmr_b200.so`` (declarations: ``include/ucmr.h``)."""
from __future__ import annotations

import ctypes as C
import os

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
_LIB_NAME = "libucmr_b200.so"

UCMR_OK = 0
UCMR_ERR_BAD_ARG = -1
UCMR_ERR_UNSUPPORTED = -2
UCMR_ERR_LAUNCH = -3
UCMR_ERR_DEVICE = -4
UCMR_ERR_WORKSPACE = -5

UCMR_DEV_BAD_BLOCK_ID = 1
UCMR_DEV_WAIT_TIMEOUT = 2

REDUCE_MIN = 0
REDUCE_SUM = 1

MAX_MUST_SELECT = 16
WORKSPACE_HEADER_BYTES = 256


class UcmrError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, status: int, what: str, detail: str = ""):
        self.status = status
        super().__init__(f"{what}: status {status} ({detail})" if detail else f"{what}: status {status}")


def library_path() -> str:
    return os.environ.get("UCMR_LIBRARY", os.path.join(_PKG_DIR, _LIB_NAME))


_vp, _i, _i64, _sz, _f = C.c_void_p, C.c_int, C.c_int64, C.c_size_t, C.c_float

# name -> (restype, argtypes); one entry per function declared in include/ucmr.h
SIGNATURES = {
    "ucmr_version": (_i, []),
    "ucmr_status_string": (C.c_char_p, [_i]),
    "ucmr_last_cuda_error": (C.c_char_p, []),
    "ucmr_trace_read": (_i, [_i, _vp]),
    "ucmr_hash_encode": (_i, [_vp, _i64, _i64, _vp, _i, _i, _vp, _vp, _vp]),
    "ucmr_hash_encode_query": (_i, [_vp, _i64, _i, _i64, _i64, _i, _vp, _i, _i, _vp, _vp, _vp]),
    "ucmr_hash_encode_and_cache": (_i, [_vp, _i64, _i, _i64, _i64, _vp, _i, _i, _vp, _i, _vp, _i64, _i, _vp, _vp]),
    "ucmr_hash_encode_blocks": (_i, [_vp, _i64, _i, _i, _i64, _i64, _i64, _vp, _vp, _i64, _vp, _i, _i, _vp, _i64, _vp, _vp]),
    "ucmr_hash_encode_and_cache_at": (_i, [_vp, _i64, _i, _i64, _i64, _vp, _i, _i, _vp, _i, _vp, _i64, _i, _i, _i, _vp, _vp]),
    "ucmr_hash_encode_blocks_at": (_i, [_vp, _i64, _i, _i, _i64, _i64, _i64, _vp, _vp, _i64, _vp, _i, _i, _vp, _i64, _i, _i,
                                        _vp, _vp]),
    "ucmr_hash_encode_decode_step": (_i, [_vp, _i64, _i, _i64, _i64, _i, _vp, _vp, _i64, _i, _i64, _i64, _vp, _i, _vp, _i64,
                                          _i, _vp, _i, _i, _vp, _vp]),
    "ucmr_hamming_topk_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "ucmr_workspace_init": (_i, [_vp, _sz, _vp]),
    "ucmr_workspace_status": (_i, [_vp, C.POINTER(C.c_int), _vp]),
    "ucmr_hamming_topk": (_i, [_vp, _i64, _i, _i, _i, _vp, _i, _vp, _i, _i64, _vp, _i, _i, _vp, _vp, _i, _i,
                               C.POINTER(C.c_int32), _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "ucmr_static_workspace_capacity": (_sz, []),
    "ucmr_hamming_topk_static": (_i, [_vp, _i64, _i, _i, _i, _vp, _i, _vp, _i, _i64, _vp, _i, _i, _vp, _vp, _i, _i,
                                      C.POINTER(C.c_int32), _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "ucmr_block_scores": (_i, [_vp, _i64, _i, _i, _i, _vp, _i, _vp, _i, _i64, _vp, _i, _i, _i, _vp, _vp, _vp]),
    "ucmr_hamming_score": (_i, [_vp, _i64, _i, _i, _i, _vp, _i, _vp, _i, _i64, _vp, _i, _i, _i, _i, _vp, _vp]),
    "ucmr_update_seq_lens": (_i, [_vp, _i, _i, _i, _vp, _vp]),
    "ucmr_topk_candidates": (_i, [_vp, _i64, _i, _i, _i, _vp, _i, _vp, _i, _i64, _vp, _vp, _i, _i, _i, _f, _i, _i,
                                  C.POINTER(C.c_int32), _i, _i, _i, _vp, _vp, _vp, _sz, _vp]),
    "ucmr_merge_topk": (_i, [_vp, _vp, _i64, _i, _i, _i, _i, _i, _vp, _vp, _vp]),
    "ucmr_block_repr_mean": (_i, [_vp, _i64, _i, _i, _i64, _i64, _vp, _i64, _i, _vp, _vp, _vp]),
    "ucmr_dot_topk_workspace_bytes": (_sz, [_i, _i]),
    "ucmr_dot_topk": (_i, [_vp, _i64, _i, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _sz, _vp]),
    "ucmr_softmax_topk_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "ucmr_softmax_topk": (_i, [_vp, _i, _i, _i, _i, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _sz, _vp]),
    "ucmr_topk_candidates_p2p": (_i, [_vp, _i64, _i, _i, _i, _vp, _i, _vp, _i, _i64, _vp, _vp, _i, _i, _i, _f, _i, _i,
                                      C.POINTER(C.c_int32), _i, _i, _i, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                                      C.POINTER(C.c_void_p), _i, _i, _vp, _sz, _vp]),
    "ucmr_merge_topk_wait": (_i, [_vp, _vp, _i64, _i, _i, _i, _i, _i, _vp, _vp, _vp, _i, _vp, _vp]),
    "ucmr_topk_candidates_p2p_step": (_i, [_vp, _i64, _i, _i, _i, _vp, _i, _vp, _i, _i64, _vp, _vp, _i, _i, _i, _f, _i, _i,
                                           C.POINTER(C.c_int32), _i, _i, _i, C.POINTER(C.c_void_p),
                                           C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), _i, _vp, _vp, _sz, _vp]),
    "ucmr_merge_topk_wait_step": (_i, [_vp, _vp, _i64, _i64, _i, _i, _i, _i, _i, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp]),
    "ucmr_copy_blocks": (_i, [_vp, _vp, _vp, _vp, _i64, _i64, _vp, _vp]),
    "ucmr_gather_kv": (_i, [_vp, _vp, _i64, _i64, _vp, _i, _i, _i, _i, _i, _i64, _vp, _vp, _vp, _vp]),
}

_lib = None


def load_library():
    """Loads the CUDA library; raises if it has not been built (there is no fallback path)."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not os.path.exists(path):
        raise ImportError(
            f"{path} not found: build it with `python -m unified_cache_management_b200.build` "
            "(the retrieval ops have no CPU or PyTorch fallback)")
    lib = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = header and library disagree
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status: int, what: str) -> None:
    if status == UCMR_OK:
        return
    lib = load_library()
    detail = lib.ucmr_status_string(status).decode()
    if status == UCMR_ERR_LAUNCH:
        detail += ": " + lib.ucmr_last_cuda_error().decode()
    if status in (UCMR_ERR_BAD_ARG, UCMR_ERR_UNSUPPORTED):
        raise ValueError(f"{what}: {detail}")
    raise UcmrError(status, what, detail)

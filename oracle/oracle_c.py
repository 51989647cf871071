"""ctypes front-end of ``oracle_c.c`` (TEST INFRASTRUCTURE ONLY).

Mirrors the numpy oracle's signatures closely enough for the tests to
cross-check the two, and gives the benchmark a multi-threaded CPU arm.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import build_oracle

_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(build_oracle.build_oracle_c())
        _lib.orc_num_threads.restype = C.c_int
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def num_threads() -> int:
    return int(lib().orc_num_threads())


def use_all_cores() -> int:
    """Sizes the OpenMP team to the cores this process may run on; returns the team size."""
    import os
    lib().orc_set_num_threads(len(os.sched_getaffinity(0)))
    return num_threads()


def hash_encode(x_bf16: np.ndarray, r_bf16: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x_bf16, dtype=np.uint16)
    r = np.ascontiguousarray(r_bf16, dtype=np.uint16)
    in_dim, bits = r.shape
    rows = x.size // in_dim
    out = np.empty(x.shape[:-1] + (bits // 32,), dtype=np.uint32)
    rc = lib().orc_hash_encode(_p(x), C.c_int64(rows), C.c_int64(in_dim), _p(r), C.c_int(in_dim),
                               C.c_int(bits), _p(out))
    assert rc == 0, rc
    return out


def block_scores(codes, q_codes, block_table, seq_lens, mode, reduce_kvhead=False) -> np.ndarray:
    codes = np.ascontiguousarray(codes, dtype=np.uint32)
    q = np.ascontiguousarray(q_codes, dtype=np.uint32)
    bt = np.ascontiguousarray(block_table, dtype=np.int32)
    sl = np.ascontiguousarray(seq_lens, dtype=np.int32)
    nb, bs, hkv, w = codes.shape
    b, hq, _ = q.shape
    hout = 1 if reduce_kvhead else hkv
    out = np.empty((b, hout, bt.shape[1]), dtype=np.int32)
    rc = lib().orc_block_scores(_p(codes), C.c_int64(nb), bs, hkv, w, _p(q), hq, _p(bt), bt.shape[1],
                                _p(sl), b, int(mode), int(bool(reduce_kvhead)), _p(out))
    assert rc == 0, rc
    return out


def select(scores, block_table, seq_lens, block_size, k, must_select=(), sink_tokens=0,
           recent_tokens=0, k_per_request=None, request_mask=None):
    s = np.ascontiguousarray(scores, dtype=np.int32)
    bt = np.ascontiguousarray(block_table, dtype=np.int32)
    sl = np.ascontiguousarray(seq_lens, dtype=np.int32)
    b, hout, mb = s.shape
    must = np.ascontiguousarray(must_select, dtype=np.int32)
    kpr = None if k_per_request is None else np.ascontiguousarray(k_per_request, dtype=np.int32)
    msk = None if request_mask is None else np.ascontiguousarray(request_mask, dtype=np.uint8)
    logical = np.empty((b, hout, k), dtype=np.int32)
    physical = np.empty((b, hout, k), dtype=np.int32)
    sel = np.empty((b, hout, k), dtype=np.int32)
    vc = np.empty(b, dtype=np.int32)
    ns = np.empty(b, dtype=np.int32)
    rc = lib().orc_select(_p(s), b, hout, mb, _p(bt), _p(sl), int(block_size), int(k), _p(kpr), _p(msk),
                          _p(must), int(must.size), int(sink_tokens), int(recent_tokens),
                          _p(logical), _p(physical), _p(sel), _p(vc), _p(ns))
    assert rc == 0, rc
    return dict(logical=logical, physical=physical, scores=sel, valid_count=vc, new_seq_lens=ns)


def hamming_topk(codes, q_codes, block_table, seq_lens, k, mode, reduce_kvhead=False, **kw):
    s = block_scores(codes, q_codes, block_table, seq_lens, mode, reduce_kvhead)
    out = select(s, block_table, seq_lens, codes.shape[1], k, **kw)
    out["block_scores"] = s
    return out


def gather_kv(pool: np.ndarray, physical: np.ndarray) -> np.ndarray:
    pool = np.ascontiguousarray(pool)
    nb, bs, hkv, d = pool.shape
    phys = np.ascontiguousarray(physical, dtype=np.int32)
    per_head = phys.ndim == 3
    b, k = phys.shape[0], phys.shape[-1]
    out = np.empty((b, k * bs, hkv, d), dtype=pool.dtype)
    rc = lib().orc_gather_kv(_p(pool), C.c_int64(nb), bs, hkv, C.c_int64(d * pool.itemsize), _p(phys),
                             b, k, int(per_head), _p(out))
    assert rc == 0, rc
    return out

"""Tensor-level wrappers over the C ABI (``include/ucmr.h``).

Every function takes CUDA tensors, passes raw pointers plus the current torch stream to
``libucmr_b200.so`` and returns without synchronising.  torch is only used to own memory; there
is no PyTorch or CPU implementation behind these functions.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from . import lib as _l

REDUCE_MIN = _l.REDUCE_MIN
REDUCE_SUM = _l.REDUCE_SUM
_REDUCE_NAMES = {"min": REDUCE_MIN, "max": REDUCE_MIN, "sum": REDUCE_SUM, "mean": REDUCE_SUM}


def reduce_mode(mode) -> int:
    """'min' (the reference: closest token; its config spells it 'max' similarity), 'sum'/'mean'."""
    if isinstance(mode, str):
        if mode not in _REDUCE_NAMES:
            raise ValueError(f"reduce mode should be one of {sorted(_REDUCE_NAMES)}, got {mode!r}")
        return _REDUCE_NAMES[mode]
    if mode not in (REDUCE_MIN, REDUCE_SUM):
        raise ValueError(f"bad reduce mode {mode!r}")
    return int(mode)


FLAG_INPUTS_STABLE = 0x100  # UCMR_FLAG_INPUTS_STABLE
FLAG_CACHE_APPEND_ONLY = 0x200  # UCMR_FLAG_CACHE_APPEND_ONLY


def _mode(reduce, inputs_stable: bool, cache_append_only: bool = False) -> int:
    """reduce mode with the caller's promises about kernels that may still be in flight on the stream:
    inputs_stable - none of them writes seq_lens / block_table (the scan sets itself up while they drain);
    cache_append_only (with inputs_stable) - of the code blocks scanned they write at most each request's last
    block, as a decode step's key encode does (the scan starts copying its first blocks meanwhile)."""
    if cache_append_only and not inputs_stable:
        raise ValueError("cache_append_only needs inputs_stable")
    return reduce_mode(reduce) | (FLAG_INPUTS_STABLE if inputs_stable else 0) | \
        (FLAG_CACHE_APPEND_ONLY if cache_append_only else 0)


def _stream(t: torch.Tensor) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> C.c_void_p:
    return C.c_void_p(0 if t is None else t.data_ptr())


def _need_cuda(name: str, t: torch.Tensor, dtype=None, contiguous=True) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if dtype is not None and t.dtype not in (dtype if isinstance(dtype, tuple) else (dtype,)):
        raise ValueError(f"{name} must have dtype {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def _need_cuda_or_pinned(name: str, t: torch.Tensor, dtype=None, contiguous=True) -> None:
    """Small per-step operands may also live in page-locked host memory: under unified addressing the
    kernels read (or write) it across the bus themselves, which saves a separate copy."""
    if isinstance(t, torch.Tensor) and not t.is_cuda and t.is_pinned():
        if dtype is not None and t.dtype not in (dtype if isinstance(dtype, tuple) else (dtype,)):
            raise ValueError(f"{name} must have dtype {dtype}, got {t.dtype}")
        if contiguous and not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
        return
    _need_cuda(name, t, dtype, contiguous)


def as_words(t: torch.Tensor) -> torch.Tensor:
    """Reinterpret a packed-code tensor (uint8 / bf16 / int32 ...) as int32 words, last dim = W."""
    if t.dtype == torch.int32:
        return t
    if (t.shape[-1] * t.element_size()) % 4 != 0:
        raise ValueError("packed codes must be a whole number of 32-bit words per row")
    return t.view(torch.int32)


# ----------------------------------------------------------------------------------------------
# (1) encode
# ----------------------------------------------------------------------------------------------
def _check_r(r: torch.Tensor, in_dim: int) -> int:
    _need_cuda("hash weights", r, torch.bfloat16)
    if r.dim() != 2 or r.shape[0] != in_dim:
        raise ValueError(f"hash weights must be [{in_dim}, hash_bits], got {tuple(r.shape)}")
    return int(r.shape[1])


def hash_encode(x: torch.Tensor, r: torch.Tensor, out: Optional[torch.Tensor] = None,
                status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x bf16 [..., in_dim] -> int32 codes [..., hash_bits/32]."""
    _need_cuda("x", x, torch.bfloat16, contiguous=False)
    in_dim = x.shape[-1]
    bits = _check_r(r, in_dim)
    x2 = x.reshape(-1, in_dim)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    rows = x2.shape[0]
    w = bits // 32
    if out is None:
        out = torch.empty(x.shape[:-1] + (w,), dtype=torch.int32, device=x.device)
    else:
        _need_cuda("out", out, torch.int32)
        if out.numel() != rows * w:
            raise ValueError("out has the wrong size")
    lib = _l.load_library()
    _l.check(lib.ucmr_hash_encode(_ptr(x2), rows, x2.stride(0) if rows > 1 else in_dim, _ptr(r), in_dim, bits,
                                  _ptr(out), _ptr(status), _stream(x)), "ucmr_hash_encode")
    return out


def hash_encode_query(q: torch.Tensor, r: torch.Tensor, group_mean: int = 1,
                      out: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q bf16 [T, Hq, in_dim] -> int32 [T, Hq/group_mean, W]; group_mean>1 averages head groups first."""
    _need_cuda("q", q, torch.bfloat16, contiguous=False)
    if q.dim() != 3 or q.stride(2) != 1:
        raise ValueError("q must be [T, Hq, in_dim] with a unit inner stride")
    t, hq, in_dim = q.shape
    bits = _check_r(r, in_dim)
    if group_mean <= 0 or hq % group_mean != 0:
        raise ValueError("group_mean must divide the number of query heads")
    w = bits // 32
    if out is None:
        out = torch.empty((t, hq // group_mean, w), dtype=torch.int32, device=q.device)
    else:
        _need_cuda("out", out, torch.int32)
    lib = _l.load_library()
    _l.check(lib.ucmr_hash_encode_query(_ptr(q), t, hq, q.stride(0), q.stride(1), group_mean, _ptr(r), in_dim, bits,
                                        _ptr(out), _ptr(status), _stream(q)), "ucmr_hash_encode_query")
    return out


def hash_encode_and_cache(x: torch.Tensor, slot_mapping: torch.Tensor, cache: torch.Tensor, r: torch.Tensor,
                          status: Optional[torch.Tensor] = None, word_offset: Optional[int] = None) -> torch.Tensor:
    """Encode x bf16 [T, H, in_dim] and scatter token t's codes to slot ``slot_mapping[t]`` of the paged
    cache [NB, BS, H, W] (int32 words, or any dtype that views to them).  With ``word_offset`` the cache rows
    may be wider than one code (W >= word_offset + hash_bits/32) and the code lands at that word."""
    _need_cuda("x", x, torch.bfloat16, contiguous=False)
    if x.dim() != 3 or x.stride(2) != 1:
        raise ValueError(f"x must be [T,H,K] with a unit inner stride, got {tuple(x.shape)}")
    _need_cuda("slot_mapping", slot_mapping, (torch.int64, torch.int32))
    if slot_mapping.dim() != 1 or slot_mapping.shape[0] != x.shape[0]:
        raise ValueError(f"slot_mapping length {tuple(slot_mapping.shape)} != T {x.shape[0]}")
    _need_cuda("cache", cache)
    cw = as_words(cache)
    t, h, in_dim = x.shape
    bits = _check_r(r, in_dim)
    lib = _l.load_library()
    if word_offset is not None:
        if cw.dim() != 4 or cw.shape[2] != h or word_offset < 0 or word_offset + bits // 32 > cw.shape[3]:
            raise ValueError(f"cache shape {tuple(cw.shape)} cannot hold {bits // 32} words at word {word_offset}")
        _l.check(lib.ucmr_hash_encode_and_cache_at(_ptr(x), t, h, x.stride(0), x.stride(1), _ptr(r), in_dim, bits,
                                                   _ptr(slot_mapping), int(slot_mapping.dtype == torch.int64), _ptr(cw),
                                                   cw.shape[0], cw.shape[1], cw.shape[3], int(word_offset), _ptr(status),
                                                   _stream(x)), "ucmr_hash_encode_and_cache_at")
        return cache
    if cw.dim() != 4 or cw.shape[2] != h or cw.shape[3] != bits // 32:
        raise ValueError(f"cache shape {tuple(cw.shape)} does not match [NB, BS, {h}, {bits // 32}]")
    _l.check(lib.ucmr_hash_encode_and_cache(_ptr(x), t, h, x.stride(0), x.stride(1), _ptr(r), in_dim, bits,
                                            _ptr(slot_mapping), int(slot_mapping.dtype == torch.int64), _ptr(cw),
                                            cw.shape[0], cw.shape[1], _ptr(status), _stream(x)),
             "ucmr_hash_encode_and_cache")
    return cache


def hash_encode_blocks(k_cache: torch.Tensor, block_ids: torch.Tensor, cache: torch.Tensor, r: torch.Tensor,
                       block_tokens: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None,
                       word_offset: Optional[int] = None) -> torch.Tensor:
    """Re-hash key blocks in place of the paged K cache: for every listed block id, encode its first
    ``block_tokens[i]`` tokens (all of them when None) of k_cache bf16 [NB, BS, H, in_dim] into the same block of the
    code cache [NB_codes, BS, H, W].  No gathered copy of the keys is made."""
    _need_cuda("k_cache", k_cache, torch.bfloat16, contiguous=False)
    if k_cache.dim() != 4 or k_cache.stride(3) != 1:
        raise ValueError(f"k_cache must be [NB,BS,H,K] with a unit inner stride, got {tuple(k_cache.shape)}")
    _need_cuda("block_ids", block_ids, torch.int32)
    if block_ids.dim() != 1:
        raise ValueError("block_ids must be one-dimensional")
    if block_tokens is not None:
        _need_cuda("block_tokens", block_tokens, torch.int32)
        if block_tokens.shape != block_ids.shape:
            raise ValueError("block_tokens must have one entry per listed block")
    _need_cuda("cache", cache)
    cw = as_words(cache)
    nb, bs, h, in_dim = k_cache.shape
    bits = _check_r(r, in_dim)
    lib = _l.load_library()
    if word_offset is not None:  # rows wider than one code, see hash_encode_and_cache
        if (cw.dim() != 4 or cw.shape[1] != bs or cw.shape[2] != h or word_offset < 0
                or word_offset + bits // 32 > cw.shape[3]):
            raise ValueError(f"cache shape {tuple(cw.shape)} cannot hold {bits // 32} words at word {word_offset}")
        _l.check(lib.ucmr_hash_encode_blocks_at(_ptr(k_cache), nb, bs, h, k_cache.stride(0), k_cache.stride(1),
                                                k_cache.stride(2), _ptr(block_ids), _ptr(block_tokens),
                                                block_ids.numel(), _ptr(r), in_dim, bits, _ptr(cw), cw.shape[0],
                                                cw.shape[3], int(word_offset), _ptr(status), _stream(k_cache)),
                 "ucmr_hash_encode_blocks_at")
        return cache
    if cw.dim() != 4 or cw.shape[1] != bs or cw.shape[2] != h or cw.shape[3] != bits // 32:
        raise ValueError(f"cache shape {tuple(cw.shape)} does not match [*, {bs}, {h}, {bits // 32}]")
    _l.check(lib.ucmr_hash_encode_blocks(_ptr(k_cache), nb, bs, h, k_cache.stride(0), k_cache.stride(1),
                                         k_cache.stride(2), _ptr(block_ids), _ptr(block_tokens), block_ids.numel(),
                                         _ptr(r), in_dim, bits, _ptr(cw), cw.shape[0], _ptr(status), _stream(k_cache)),
             "ucmr_hash_encode_blocks")
    return cache


def hash_encode_decode_step(q: torch.Tensor, k_new: torch.Tensor, slot_mapping: torch.Tensor, cache: torch.Tensor,
                            r: torch.Tensor, group_mean: int = 1, q_codes_out: Optional[torch.Tensor] = None,
                            status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One launch for a decode step's two encodes: q [T,Hq,D] -> codes [T,Hq/group_mean,W] (returned) and
    k_new [T,Hkv,D] -> slot ``slot_mapping[t]`` of the paged cache."""
    _need_cuda_or_pinned("q", q, torch.bfloat16, contiguous=False)
    _need_cuda_or_pinned("k_new", k_new, torch.bfloat16, contiguous=False)
    if q.dim() != 3 or k_new.dim() != 3 or q.stride(2) != 1 or k_new.stride(2) != 1:
        raise ValueError("q and k_new must be [T, H, in_dim] with a unit inner stride")
    _need_cuda("slot_mapping", slot_mapping, (torch.int64, torch.int32))
    if slot_mapping.dim() != 1 or slot_mapping.shape[0] != k_new.shape[0]:
        raise ValueError("slot_mapping must have one entry per new key token")
    _need_cuda("cache", cache)
    cw = as_words(cache)
    tq, hq, in_dim = q.shape
    tk, hk, _ = k_new.shape
    bits = _check_r(r, in_dim)
    if k_new.shape[2] != in_dim or cw.dim() != 4 or cw.shape[2] != hk or cw.shape[3] != bits // 32:
        raise ValueError("k_new / cache shapes do not match")
    if group_mean <= 0 or hq % group_mean != 0:
        raise ValueError("group_mean must divide the number of query heads")
    if q_codes_out is None:
        q_codes_out = torch.empty((tq, hq // group_mean, bits // 32), dtype=torch.int32, device=cache.device)
    lib = _l.load_library()
    _l.check(lib.ucmr_hash_encode_decode_step(
        _ptr(q), tq, hq, q.stride(0), q.stride(1), group_mean, _ptr(q_codes_out), _ptr(k_new), tk, hk, k_new.stride(0),
        k_new.stride(1), _ptr(slot_mapping), int(slot_mapping.dtype == torch.int64), _ptr(cw), cw.shape[0], cw.shape[1],
        _ptr(r), in_dim, bits, _ptr(status), _stream(cache)), "ucmr_hash_encode_decode_step")
    return q_codes_out


# ----------------------------------------------------------------------------------------------
# (2)+(3) scan + top-k
# ----------------------------------------------------------------------------------------------
def workspace_bytes(batch: int, num_kv_heads: int, max_blocks: int, reduce_kvhead: bool = False) -> int:
    return int(_l.load_library().ucmr_hamming_topk_workspace_bytes(batch, num_kv_heads, max_blocks,
                                                                   int(bool(reduce_kvhead))))


TRACE_UNITS = {"encode": 0, "scan": 1, "select": 2}  # UCMR_TRACE_ENCODE / _SCAN / _SELECT
TRACE_SLOTS = 32                                      # UCMR_TRACE_SLOTS


def trace_read(unit: str):
    """Device-timer stamps (ns) left by the last launch of one decode-step kernel; needs the library built with
    ``python -m unified_cache_management_b200.build --trace`` (any other build raises: unsupported).  Slot
    meanings: ucmr.h, ucmr_trace_read."""
    buf = (C.c_ulonglong * TRACE_SLOTS)()
    _l.check(_l.load_library().ucmr_trace_read(TRACE_UNITS[unit], C.cast(buf, C.c_void_p)), "ucmr_trace_read")
    return list(buf)


def new_workspace(batch: int, num_kv_heads: int, max_blocks: int, device, reduce_kvhead: bool = False) -> torch.Tensor:
    """Allocates and clears a workspace big enough for the given shapes (either head mode)."""
    n = max(workspace_bytes(batch, num_kv_heads, max_blocks, False),
            workspace_bytes(batch, num_kv_heads, max_blocks, reduce_kvhead))
    ws = torch.empty(n, dtype=torch.uint8, device=device)
    _l.check(_l.load_library().ucmr_workspace_init(_ptr(ws), n, _stream(ws)), "ucmr_workspace_init")
    return ws


def workspace_status(ws: torch.Tensor) -> int:
    """Reads the sticky device status word (synchronises the current stream)."""
    host = C.c_int(0)
    rc = _l.load_library().ucmr_workspace_status(_ptr(ws), C.byref(host), _stream(ws))
    if rc not in (_l.UCMR_OK, _l.UCMR_ERR_DEVICE):
        _l.check(rc, "ucmr_workspace_status")
    return int(host.value)


@dataclass
class Retrieval:
    physical: torch.Tensor       # int32 [B, Hout, k]  block-table entries of the chosen blocks
    logical: torch.Tensor        # int32 [B, Hout, k]  ascending logical block index (-1 = padding)
    scores: Optional[torch.Tensor]  # int32 [B, Hout, k]  raw block scores (-1 = padding)
    valid_count: torch.Tensor    # int32 [B]
    new_seq_lens: torch.Tensor   # int32 [B]


def _check_out(out: "Retrieval", b: int, hout: int, k: int, device) -> None:
    """Every non-None member of ``out`` must be what the kernel writes: int32, contiguous, on the codes' device,
    [B, Hout, k] for the id / score arrays and [B] for the two per-request arrays.  ``physical`` alone may be
    page-locked host memory.  The kernel writes B*Hout*k entries whatever the tensor's size, so a buffer shaped for
    another k or head mode is refused here."""
    for name, t, shape, host_ok in (("physical", out.physical, (b, hout, k), True),
                                    ("logical", out.logical, (b, hout, k), False),
                                    ("scores", out.scores, (b, hout, k), False),
                                    ("valid_count", out.valid_count, (b,), False),
                                    ("new_seq_lens", out.new_seq_lens, (b,), False)):
        if t is None:
            if name == "physical":
                raise ValueError("out.physical is required")
            continue
        (_need_cuda_or_pinned if host_ok else _need_cuda)(f"out.{name}", t, torch.int32)
        if tuple(t.shape) != shape:
            raise ValueError(f"out.{name} must have shape {shape}, got {tuple(t.shape)}")
        if t.is_cuda and t.device != device:
            raise ValueError(f"out.{name} is on {t.device}, the codes are on {device}")


def _scan_args(codes, q_codes, block_table, seq_lens):
    _need_cuda("codes", codes)
    codes = as_words(codes)
    _need_cuda("q_codes", q_codes)
    q_codes = as_words(q_codes)
    if codes.dim() != 4:
        raise ValueError("codes must be [NB, BS, Hkv, W]")
    if q_codes.dim() != 3 or q_codes.shape[2] != codes.shape[3]:
        raise ValueError("q_codes must be [B, Hq, W] with the cache's W")
    _need_cuda("block_table", block_table, torch.int32, contiguous=False)
    if block_table.dim() != 2 or block_table.stride(1) != 1:
        raise ValueError("block_table must be [B, max_blocks] with a unit inner stride")
    _need_cuda("seq_lens", seq_lens, torch.int32)
    b = q_codes.shape[0]
    if block_table.shape[0] != b:
        raise RuntimeError("batch size mismatch between query_code and block_table")
    if seq_lens.shape[0] < b:
        raise ValueError("seq_lens shorter than the batch")
    if q_codes.shape[1] % codes.shape[2] != 0:
        raise ValueError("number of query heads must be a multiple of the kv heads")
    bt_stride = block_table.stride(0) if b > 1 else max(block_table.stride(0), block_table.shape[1])
    return codes, q_codes, bt_stride


def _must_array(must_select: Sequence[int]):
    must = list(must_select or ())
    if len(must) > _l.MAX_MUST_SELECT:
        raise ValueError(f"at most {_l.MAX_MUST_SELECT} must_select entries")
    arr = (C.c_int32 * max(1, len(must)))(*must)
    return arr, len(must)


def hamming_topk(codes: torch.Tensor, q_codes: torch.Tensor, block_table: torch.Tensor, seq_lens: torch.Tensor,
                 k: int, *, reduce="sum", reduce_kvhead: bool = False, must_select: Sequence[int] = (),
                 sink_tokens: int = 0, recent_tokens: int = 0, k_per_request: Optional[torch.Tensor] = None,
                 request_mask: Optional[torch.Tensor] = None, workspace: Optional[torch.Tensor] = None,
                 out: Optional[Retrieval] = None, want_scores: bool = True, inputs_stable: bool = False,
                 cache_append_only: bool = False) -> Retrieval:
    """Scan + exact top-k in two launches.  See ``ucmr_hamming_topk`` in include/ucmr.h."""
    codes, q_codes, bt_stride = _scan_args(codes, q_codes, block_table, seq_lens)
    nb, bs, hkv, w = codes.shape
    b, hq, _ = q_codes.shape
    mb = block_table.shape[1]
    if k < 0 or k > mb:
        raise ValueError(f"k={k} outside [0, max_blocks={mb}]")
    hout = 1 if reduce_kvhead else hkv
    dev = codes.device
    if workspace is None:
        workspace = new_workspace(b, hkv, mb, dev, reduce_kvhead)
    if k_per_request is not None:
        _need_cuda("k_per_request", k_per_request, torch.int32)
    if request_mask is not None:
        _need_cuda("request_mask", request_mask, (torch.uint8, torch.bool))
    if out is None:
        out = Retrieval(
            physical=torch.empty((b, hout, k), dtype=torch.int32, device=dev),
            logical=torch.empty((b, hout, k), dtype=torch.int32, device=dev),
            scores=torch.empty((b, hout, k), dtype=torch.int32, device=dev) if want_scores else None,
            valid_count=torch.empty((b,), dtype=torch.int32, device=dev),
            new_seq_lens=torch.empty((b,), dtype=torch.int32, device=dev))
    if b == 0:
        return out
    _check_out(out, b, hout, k, dev)
    must, n_must = _must_array(must_select)
    lib = _l.load_library()
    _l.check(lib.ucmr_hamming_topk(
        _ptr(codes), nb, bs, hkv, w, _ptr(q_codes), hq, _ptr(block_table), mb, bt_stride, _ptr(seq_lens), b, k,
        _ptr(k_per_request), _ptr(request_mask), _mode(reduce, inputs_stable, cache_append_only),
        int(bool(reduce_kvhead)), must, n_must,
        int(sink_tokens), int(recent_tokens), _ptr(out.physical), _ptr(out.logical), _ptr(out.scores),
        _ptr(out.valid_count), _ptr(out.new_seq_lens), _ptr(workspace), workspace.numel(), _stream(codes)),
        "ucmr_hamming_topk")
    return out


def hamming_topk_static(codes: torch.Tensor, q_codes: torch.Tensor, block_table: torch.Tensor, seq_lens: torch.Tensor,
                        k: int, *, out: Retrieval, reduce="sum", reduce_kvhead: bool = False,
                        must_select: Sequence[int] = (), sink_tokens: int = 0, recent_tokens: int = 0,
                        k_per_request: Optional[torch.Tensor] = None,
                        request_mask: Optional[torch.Tensor] = None) -> Retrieval:
    """``hamming_topk`` for callers that cannot allocate device memory: the scores between the two kernels
    live in a fixed 4 MiB array inside the library, and the caller passes every output buffer (``out``),
    so nothing here allocates.  Calls that may overlap on the GPU share that array and must be serialised;
    shapes needing more than the array are refused (``UcmrError`` with the workspace status)."""
    codes, q_codes, bt_stride = _scan_args(codes, q_codes, block_table, seq_lens)
    nb, bs, hkv, w = codes.shape
    b, hq, _ = q_codes.shape
    mb = block_table.shape[1]
    if k < 0 or k > mb:
        raise ValueError(f"k={k} outside [0, max_blocks={mb}]")
    if b == 0:
        return out
    _check_out(out, b, 1 if reduce_kvhead else hkv, k, codes.device)
    must, n_must = _must_array(must_select)
    lib = _l.load_library()
    _l.check(lib.ucmr_hamming_topk_static(
        _ptr(codes), nb, bs, hkv, w, _ptr(q_codes), hq, _ptr(block_table), mb, bt_stride, _ptr(seq_lens), b, k,
        _ptr(k_per_request), _ptr(request_mask), reduce_mode(reduce), int(bool(reduce_kvhead)), must, n_must,
        int(sink_tokens), int(recent_tokens), _ptr(out.physical), _ptr(out.logical), _ptr(out.scores),
        _ptr(out.valid_count), _ptr(out.new_seq_lens), _stream(codes)), "ucmr_hamming_topk_static")
    return out


def block_scores(codes, q_codes, block_table, seq_lens, *, reduce="sum", reduce_kvhead=False,
                 out: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None,
                 inputs_stable: bool = False, cache_append_only: bool = False) -> torch.Tensor:
    """int32 [B, Hout, max_blocks] block scores (-1 past each request's length)."""
    codes, q_codes, bt_stride = _scan_args(codes, q_codes, block_table, seq_lens)
    nb, bs, hkv, w = codes.shape
    b, hq, _ = q_codes.shape
    mb = block_table.shape[1]
    hout = 1 if reduce_kvhead else hkv
    if out is None:
        out = torch.empty((b, hout, mb), dtype=torch.int32, device=codes.device)
    lib = _l.load_library()
    _l.check(lib.ucmr_block_scores(_ptr(codes), nb, bs, hkv, w, _ptr(q_codes), hq, _ptr(block_table), mb, bt_stride,
                                   _ptr(seq_lens), b, _mode(reduce, inputs_stable, cache_append_only),
                                   int(bool(reduce_kvhead)), _ptr(out),
                                   _ptr(status), _stream(codes)), "ucmr_block_scores")
    return out


def hamming_score(key_codes, query_code, block_table, seq_len, max_seq_len: int, sink: int, recent: int,
                  reduce_kvhead: bool) -> torch.Tensor:
    """Signature of the reference op ``hamming.hamming_score`` (block mode): per-token fp16 scores
    [B, 1 or Hkv, max_seq_len].  query_code is [B, 1, Hq, W]."""
    if block_table is None:
        raise ValueError("only the paged (block_table) form is provided")
    q = as_words(query_code)
    if q.dim() == 4:
        q = q.reshape(q.shape[0], q.shape[2], q.shape[3])
    codes, q, bt_stride = _scan_args(key_codes, q, block_table, seq_len)
    nb, bs, hkv, w = codes.shape
    b, hq, _ = q.shape
    mb = block_table.shape[1]
    if max_seq_len != mb * bs:
        raise ValueError("max_seq_len must equal block_size * block_table.shape[1]")
    out = torch.empty((b, 1 if reduce_kvhead else hkv, max_seq_len), dtype=torch.float16, device=codes.device)
    lib = _l.load_library()
    _l.check(lib.ucmr_hamming_score(_ptr(codes), nb, bs, hkv, w, _ptr(q), hq, _ptr(block_table), mb, bt_stride,
                                    _ptr(seq_len), b, int(sink), int(recent), int(bool(reduce_kvhead)), _ptr(out),
                                    _stream(codes)), "ucmr_hamming_score")
    return out


def update_seq_lens(seq_lens: torch.Tensor, topk_token: int, block_size: int) -> torch.Tensor:
    _need_cuda("seq_lens", seq_lens, torch.int32)
    out = torch.empty_like(seq_lens)
    _l.check(_l.load_library().ucmr_update_seq_lens(_ptr(seq_lens), seq_lens.numel(), int(topk_token),
                                                    int(block_size), _ptr(out), _stream(seq_lens)),
             "ucmr_update_seq_lens")
    return out


# ----------------------------------------------------------------------------------------------
# sequence-sharded retrieval
# ----------------------------------------------------------------------------------------------
def topk_candidates(codes, q_codes, block_table, seq_lens_local, seq_lens_global, k: int, block_id_offset: int,
                    score_scale: float, *, reduce="sum", reduce_kvhead=False, must_select=(), sink_tokens=0,
                    recent_tokens=0, workspace=None, out_scores=None, out_ids=None, inputs_stable: bool = False,
                    cache_append_only: bool = False):
    """Local top-k of one sequence shard as (float32 score, int32 global block id) records [B,Hout,k]."""
    codes, q_codes, bt_stride = _scan_args(codes, q_codes, block_table, seq_lens_local)
    _need_cuda("seq_lens_global", seq_lens_global, torch.int32)
    nb, bs, hkv, w = codes.shape
    b, hq, _ = q_codes.shape
    mb = block_table.shape[1]
    if k < 0 or k > mb:
        raise ValueError(f"k={k} outside [0, max_blocks={mb}]")
    hout = 1 if reduce_kvhead else hkv
    dev = codes.device
    if workspace is None:
        workspace = new_workspace(b, hkv, mb, dev, reduce_kvhead)
    if out_scores is None:
        out_scores = torch.empty((b, hout, k), dtype=torch.float32, device=dev)
    if out_ids is None:
        out_ids = torch.empty((b, hout, k), dtype=torch.int32, device=dev)
    must, n_must = _must_array(must_select)
    lib = _l.load_library()
    _l.check(lib.ucmr_topk_candidates(
        _ptr(codes), nb, bs, hkv, w, _ptr(q_codes), hq, _ptr(block_table), mb, bt_stride, _ptr(seq_lens_local),
        _ptr(seq_lens_global), b, k, int(block_id_offset), float(score_scale),
        _mode(reduce, inputs_stable, cache_append_only),
        int(bool(reduce_kvhead)), must, n_must, int(sink_tokens), int(recent_tokens), _ptr(out_scores),
        _ptr(out_ids), _ptr(workspace), workspace.numel(), _stream(codes)), "ucmr_topk_candidates")
    return out_scores, out_ids


def topk_candidates_p2p(codes, q_codes, block_table, seq_lens_local, seq_lens_global, k: int, block_id_offset: int,
                        score_scale: float, peer_scores_ptrs: Sequence[int], peer_ids_ptrs: Sequence[int],
                        peer_flag_ptrs: Sequence[int], seq: int, *, reduce="sum", reduce_kvhead=False, must_select=(),
                        sink_tokens=0, recent_tokens=0, workspace=None, inputs_stable: bool = False,
                        cache_append_only: bool = False) -> None:
    """``topk_candidates`` whose records go straight into every rank's gather buffer over peer memory: the three
    pointer lists hold, per rank r, the device address of THIS rank's [B,Hout,k] slice of rank r's score / id
    buffers and of this rank's flag word on rank r; ``seq`` is published to the flags when the launch is done."""
    codes, q_codes, bt_stride = _scan_args(codes, q_codes, block_table, seq_lens_local)
    _need_cuda("seq_lens_global", seq_lens_global, torch.int32)
    nb, bs, hkv, w = codes.shape
    b, hq, _ = q_codes.shape
    mb = block_table.shape[1]
    if k <= 0 or k > mb:
        raise ValueError(f"k={k} outside [1, max_blocks={mb}]")
    n = len(peer_scores_ptrs)
    if n == 0 or n != len(peer_ids_ptrs) or n != len(peer_flag_ptrs):
        raise ValueError("the three pointer lists must have one entry per rank")
    if workspace is None:
        workspace = new_workspace(b, hkv, mb, codes.device, reduce_kvhead)
    arr = C.c_void_p * n
    must, n_must = _must_array(must_select)
    _l.check(_l.load_library().ucmr_topk_candidates_p2p(
        _ptr(codes), nb, bs, hkv, w, _ptr(q_codes), hq, _ptr(block_table), mb, bt_stride, _ptr(seq_lens_local),
        _ptr(seq_lens_global), b, k, int(block_id_offset), float(score_scale),
        _mode(reduce, inputs_stable, cache_append_only),
        int(bool(reduce_kvhead)), must, n_must, int(sink_tokens), int(recent_tokens),
        arr(*[int(p) for p in peer_scores_ptrs]), arr(*[int(p) for p in peer_ids_ptrs]),
        arr(*[int(p) for p in peer_flag_ptrs]), n, int(seq), _ptr(workspace), workspace.numel(), _stream(codes)),
        "ucmr_topk_candidates_p2p")


def merge_topk_wait(cand_scores: torch.Tensor, cand_ids: torch.Tensor, k: int, flags: torch.Tensor, seq: int,
                    status: Optional[torch.Tensor] = None, out_scores=None, out_ids=None):
    """``merge_topk`` that first waits until ``flags[r] == seq`` for every rank (the records were written by the
    other GPUs' ``topk_candidates_p2p``).  cand_* dense [R, B, Hout, kl]."""
    _need_cuda("cand_scores", cand_scores, torch.float32)
    _need_cuda("cand_ids", cand_ids, torch.int32)
    _need_cuda("flags", flags, torch.int32)
    r, b, h, kl = cand_scores.shape
    if flags.numel() < r:
        raise ValueError("one flag per rank is needed")
    dev = cand_scores.device
    if out_scores is None:
        out_scores = torch.empty((b, h, k), dtype=torch.float32, device=dev)
    if out_ids is None:
        out_ids = torch.empty((b, h, k), dtype=torch.int32, device=dev)
    _l.check(_l.load_library().ucmr_merge_topk_wait(_ptr(cand_scores), _ptr(cand_ids), b * h * kl, r, b, h, kl, int(k),
                                                    _ptr(out_scores), _ptr(out_ids), _ptr(flags), int(seq),
                                                    _ptr(status), _stream(cand_scores)), "ucmr_merge_topk_wait")
    return out_scores, out_ids


def topk_candidates_p2p_step(codes, q_codes, block_table, seq_lens_local, seq_lens_global, k: int, block_id_offset: int,
                             score_scale: float, peer_scores_ptrs: Sequence[int], peer_ids_ptrs: Sequence[int],
                             peer_flag_ptrs: Sequence[int], step_word: torch.Tensor, *, reduce="sum",
                             reduce_kvhead=False, must_select=(), sink_tokens=0, recent_tokens=0, workspace=None,
                             inputs_stable: bool = False, cache_append_only: bool = False) -> None:
    """``topk_candidates_p2p`` whose step number is read on the device from ``step_word`` (int32, one element, this
    rank's memory): safe to capture in a CUDA graph and replay.  The pointer lists hold the ranks' pointers of buffer
    parity 0 followed by those of parity 1."""
    codes, q_codes, bt_stride = _scan_args(codes, q_codes, block_table, seq_lens_local)
    _need_cuda("seq_lens_global", seq_lens_global, torch.int32)
    _need_cuda("step_word", step_word, torch.int32)
    nb, bs, hkv, w = codes.shape
    b, hq, _ = q_codes.shape
    mb = block_table.shape[1]
    if k <= 0 or k > mb:
        raise ValueError(f"k={k} outside [1, max_blocks={mb}]")
    n2 = len(peer_scores_ptrs)
    if n2 == 0 or n2 % 2 or n2 != len(peer_ids_ptrs) or n2 != len(peer_flag_ptrs):
        raise ValueError("the three pointer lists must have two entries (one per buffer parity) per rank")
    if workspace is None:
        workspace = new_workspace(b, hkv, mb, codes.device, reduce_kvhead)
    arr = C.c_void_p * n2
    must, n_must = _must_array(must_select)
    _l.check(_l.load_library().ucmr_topk_candidates_p2p_step(
        _ptr(codes), nb, bs, hkv, w, _ptr(q_codes), hq, _ptr(block_table), mb, bt_stride, _ptr(seq_lens_local),
        _ptr(seq_lens_global), b, k, int(block_id_offset), float(score_scale),
        _mode(reduce, inputs_stable, cache_append_only),
        int(bool(reduce_kvhead)), must, n_must, int(sink_tokens), int(recent_tokens),
        arr(*[int(p) for p in peer_scores_ptrs]), arr(*[int(p) for p in peer_ids_ptrs]),
        arr(*[int(p) for p in peer_flag_ptrs]), n2 // 2, _ptr(step_word), _ptr(workspace), workspace.numel(),
        _stream(codes)), "ucmr_topk_candidates_p2p_step")


def merge_topk_wait_step(cand_scores: torch.Tensor, cand_ids: torch.Tensor, k: int, flags: torch.Tensor,
                         parity_stride: int, flags_parity_stride: int, step_state: torch.Tensor,
                         status: Optional[torch.Tensor] = None, out_scores=None, out_ids=None):
    """``merge_topk_wait`` for the replay-safe exchange: ``cand_*`` [R, B, Hout, kl] and ``flags`` are the views of
    buffer parity 0, parity 1 lies ``parity_stride`` elements / ``flags_parity_stride`` words further;
    ``step_state`` is int32 [2] = (step word, arrival counter), zero before the first step."""
    _need_cuda("cand_scores", cand_scores, torch.float32)
    _need_cuda("cand_ids", cand_ids, torch.int32)
    _need_cuda("flags", flags, torch.int32)
    _need_cuda("step_state", step_state, torch.int32)
    if step_state.numel() < 2:
        raise ValueError("step_state needs two words")
    r, b, h, kl = cand_scores.shape
    if flags.numel() < r:
        raise ValueError("one flag per rank is needed")
    dev = cand_scores.device
    if out_scores is None:
        out_scores = torch.empty((b, h, k), dtype=torch.float32, device=dev)
    if out_ids is None:
        out_ids = torch.empty((b, h, k), dtype=torch.int32, device=dev)
    _l.check(_l.load_library().ucmr_merge_topk_wait_step(
        _ptr(cand_scores), _ptr(cand_ids), int(parity_stride), b * h * kl, r, b, h, kl, int(k), _ptr(out_scores),
        _ptr(out_ids), _ptr(flags), int(flags_parity_stride), C.c_void_p(step_state.data_ptr()),
        C.c_void_p(step_state.data_ptr() + 4), _ptr(status), _stream(cand_scores)), "ucmr_merge_topk_wait_step")
    return out_scores, out_ids


def merge_topk(cand_scores: torch.Tensor, cand_ids: torch.Tensor, k: int, out_scores=None, out_ids=None):
    """cand_* [R, B, Hout, kl] (ascending shard order) -> global top-k [B, Hout, k], ascending id.
    The two tensors may be strided views of one gathered buffer as long as each shard's [B,Hout,kl]
    slab is dense and both use the same shard stride."""
    for name, t, dt in (("cand_scores", cand_scores, torch.float32), ("cand_ids", cand_ids, torch.int32)):
        _need_cuda(name, t, dt, contiguous=False)
        if t.dim() != 4 or not t[0].is_contiguous():
            raise ValueError(f"{name} must be [R, B, Hout, kl] with dense per-shard slabs")
    if cand_scores.shape != cand_ids.shape:
        raise ValueError("candidates must be [R, B, Hout, kl]")
    r, b, h, kl = cand_scores.shape
    stride = cand_scores.stride(0) if r > 1 else b * h * kl
    if r > 1 and cand_ids.stride(0) != stride:
        raise ValueError("scores and ids must use the same shard stride")
    dev = cand_scores.device
    if out_scores is None:
        out_scores = torch.empty((b, h, k), dtype=torch.float32, device=dev)
    if out_ids is None:
        out_ids = torch.empty((b, h, k), dtype=torch.int32, device=dev)
    _l.check(_l.load_library().ucmr_merge_topk(_ptr(cand_scores), _ptr(cand_ids), stride, r, b, h, kl, int(k),
                                               _ptr(out_scores), _ptr(out_ids), _stream(cand_scores)),
             "ucmr_merge_topk")
    return out_scores, out_ids


# ----------------------------------------------------------------------------------------------
# (4) paged-KV gather
# ----------------------------------------------------------------------------------------------
def gather_kv(k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor], sel: torch.Tensor,
              out_k: Optional[torch.Tensor] = None, out_v: Optional[torch.Tensor] = None,
              status: Optional[torch.Tensor] = None):
    """pools [NB, BS, Hkv, D]; sel int32 [B, k] (whole blocks) or [B, Hkv, k] (per kv head).
    Returns (out_k, out_v), each [B, k*BS, Hkv, D] (None for a pool that was not given)."""
    pool = k_pool if k_pool is not None else v_pool
    if pool is None:
        raise ValueError("give at least one pool")
    for name, t in (("k_pool", k_pool), ("v_pool", v_pool)):
        if t is not None:
            _need_cuda(name, t)
            if t.shape != pool.shape or t.dtype != pool.dtype:
                raise ValueError("pools must agree in shape and dtype")
    _need_cuda("sel", sel, torch.int32)
    if pool.dim() != 4 or sel.dim() not in (2, 3):
        raise ValueError("pool must be [NB,BS,Hkv,D]; sel [B,k] or [B,Hkv,k]")
    nb, bs, hkv, d = pool.shape
    per_head = sel.dim() == 3
    if per_head and sel.shape[1] != hkv:
        raise ValueError("per-head sel must be [B, Hkv, k]")
    b, k = sel.shape[0], sel.shape[-1]
    shape = (b, k * bs, hkv, d)
    if k_pool is not None and out_k is None:
        out_k = torch.empty(shape, dtype=pool.dtype, device=pool.device)
    if v_pool is not None and out_v is None:
        out_v = torch.empty(shape, dtype=pool.dtype, device=pool.device)
    for name, t in (("out_k", out_k), ("out_v", out_v)):
        if t is not None:
            _need_cuda(name, t, pool.dtype)
            if t.numel() != b * k * bs * hkv * d:
                raise ValueError(f"{name} has the wrong size")
    row_bytes = d * pool.element_size()
    _l.check(_l.load_library().ucmr_gather_kv(_ptr(k_pool), _ptr(v_pool), nb, bs * hkv * row_bytes, _ptr(sel), b, k,
                                              int(per_head), bs, hkv, row_bytes, _ptr(out_k), _ptr(out_v),
                                              _ptr(status), _stream(pool)), "ucmr_gather_kv")
    return out_k, out_v


def copy_blocks(size: int, num: int, *, src_ptrs: Optional[torch.Tensor] = None, src: Optional[torch.Tensor] = None,
                dst_ptrs: Optional[torch.Tensor] = None, dst: Optional[torch.Tensor] = None,
                status: Optional[torch.Tensor] = None) -> None:
    """``num`` blocks of ``size`` bytes through the copy engine: from the addresses in ``src_ptrs`` (int64 CUDA tensor
    of device pointers) or from the contiguous tensor ``src``, to the addresses in ``dst_ptrs`` or the contiguous
    ``dst``.  The three forms of the reference's CudaSMCopyAsync."""
    if (src_ptrs is None) == (src is None) or (dst_ptrs is None) == (dst is None):
        raise ValueError("give exactly one of src_ptrs / src and one of dst_ptrs / dst")
    ref = src_ptrs if src_ptrs is not None else src
    for name, t in (("src_ptrs", src_ptrs), ("dst_ptrs", dst_ptrs)):
        if t is not None:
            _need_cuda(name, t, torch.int64)
            if t.numel() < num:
                raise ValueError(f"{name} holds fewer than {num} pointers")
    for name, t in (("src", src), ("dst", dst)):
        if t is not None:
            _need_cuda(name, t)
            if t.numel() * t.element_size() < size * num:
                raise ValueError(f"{name} is smaller than {num} blocks of {size} bytes")
    _l.check(_l.load_library().ucmr_copy_blocks(_ptr(src_ptrs), _ptr(src), _ptr(dst_ptrs), _ptr(dst), int(size),
                                                int(num), _ptr(status), _stream(ref)), "ucmr_copy_blocks")


# ----------------------------------------------------------------------------------------------
# float block retrieval (ESA / KVStar style)
# ----------------------------------------------------------------------------------------------
def block_repr_mean(k_cache: torch.Tensor, block_ids: torch.Tensor, merge: Optional[int] = None,
                    out: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Mean key of each listed block over groups of ``merge`` tokens (default: the whole block).
    k_cache bf16 [NB, BS, H, D] -> [n, BS/merge, H, D] bf16."""
    _need_cuda("k_cache", k_cache, torch.bfloat16, contiguous=False)
    if k_cache.dim() != 4 or k_cache.stride(3) != 1 or k_cache.stride(2) != k_cache.shape[3]:
        raise ValueError("k_cache must be [NB, BS, H, D] with contiguous token rows")
    _need_cuda("block_ids", block_ids, torch.int32)
    nb, bs, h, d = k_cache.shape
    merge = bs if merge is None else int(merge)
    if merge <= 0 or bs % merge != 0:
        raise ValueError(f"merge={merge} must divide the block size {bs}")
    n = block_ids.numel()
    if out is None:
        out = torch.empty((n, bs // merge, h, d), dtype=torch.bfloat16, device=k_cache.device)
    else:
        _need_cuda("out", out, torch.bfloat16)
    _l.check(_l.load_library().ucmr_block_repr_mean(_ptr(k_cache), nb, bs, h * d, k_cache.stride(0), k_cache.stride(1),
                                                    _ptr(block_ids), n, merge, _ptr(out), _ptr(status),
                                                    _stream(k_cache)), "ucmr_block_repr_mean")
    return out


def dot_topk(repr_pool: torch.Tensor, q: torch.Tensor, indexes: torch.Tensor, k: int,
             workspace: Optional[torch.Tensor] = None):
    """Per request the k candidates of ``indexes[b]`` (-1 padded) with the largest inner product with q[b].
    repr_pool bf16 [N, dim], q bf16 [B, dim] -> (scores float32 [B, k], ids int32 [B, k]), in candidate order."""
    _need_cuda("repr_pool", repr_pool, torch.bfloat16)
    _need_cuda("q", q, torch.bfloat16)
    _need_cuda("indexes", indexes, torch.int32)
    rp = repr_pool.reshape(repr_pool.shape[0], -1)
    qq = q.reshape(q.shape[0], -1)
    if qq.shape[1] != rp.shape[1] or indexes.dim() != 2 or indexes.shape[0] != qq.shape[0]:
        raise ValueError("q must be [B, dim] with the pool's dim and indexes [B, n]")
    b, n = indexes.shape
    lib = _l.load_library()
    need = lib.ucmr_dot_topk_workspace_bytes(b, n)
    if workspace is None:
        workspace = torch.empty(max(need, 1), dtype=torch.uint8, device=rp.device)
    scores = torch.empty((b, k), dtype=torch.float32, device=rp.device)
    ids = torch.empty((b, k), dtype=torch.int32, device=rp.device)
    if b == 0 or k == 0:
        return scores, ids
    _l.check(lib.ucmr_dot_topk(_ptr(rp), rp.shape[0], rp.shape[1], _ptr(qq), _ptr(indexes), b, n, int(k), _ptr(scores),
                               _ptr(ids), _ptr(workspace), workspace.numel(), _stream(rp)), "ucmr_dot_topk")
    return scores, ids


def softmax_topk(repr_blocks: torch.Tensor, q: torch.Tensor, k: int, workspace: Optional[torch.Tensor] = None):
    """KVStar block scores of one request: repr_blocks bf16 [n_blocks, M, Hkv, D], q bf16 [X, Hq, D] ->
    (block_scores float32 [n_blocks], top scores float32 [k], top block ids int32 [k] in ascending block order)."""
    _need_cuda("repr_blocks", repr_blocks, torch.bfloat16)
    _need_cuda("q", q, torch.bfloat16)
    if repr_blocks.dim() != 4 or q.dim() != 3 or q.shape[2] != repr_blocks.shape[3]:
        raise ValueError("repr_blocks must be [n_blocks, M, Hkv, D] and q [X, Hq, D]")
    n, m, hkv, d = repr_blocks.shape
    x, hq, _ = q.shape
    if hq % hkv != 0:
        raise ValueError("query heads must be a multiple of kv heads")
    lib = _l.load_library()
    need = lib.ucmr_softmax_topk_workspace_bytes(x, hq, n, m)
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=q.device)
    block_scores = torch.empty((n,), dtype=torch.float32, device=q.device)
    scores = torch.empty((k,), dtype=torch.float32, device=q.device)
    ids = torch.empty((k,), dtype=torch.int32, device=q.device)
    _l.check(lib.ucmr_softmax_topk(_ptr(repr_blocks), n, m, hkv, d, _ptr(q), x, hq, int(k), _ptr(block_scores),
                                   _ptr(scores), _ptr(ids), _ptr(workspace), workspace.numel(), _stream(q)),
             "ucmr_softmax_topk")
    return block_scores, scores, ids

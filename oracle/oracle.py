"""CPU oracle for the hash-code top-k block retrieval path (TEST INFRASTRUCTURE ONLY).

This module is a numpy restatement of the reference algorithm.  It exists to
check the CUDA kernels; nothing in the shipped package imports it.  Only the
test-suite, the smoke check and the CPU-baseline leg of the benchmark may call
it.

Parity status: the reference ships no golden vectors for this path (its op
scripts assert nothing).  The restatement is pinned instead against (a) outputs
of the reference's own Python functions run on CPU (fixtures under
``tests/golden``, produced by ``tests/golden/make_golden.py``) and (b) the
reference's C++ retrieval backend compiled from its own source
(recipe: ``oracle/build_oracle.py``).

Reference lines followed (paths inside the reference project):

* encode ............ ucm/sparse/gsa_on_device/hash_encoder.py:359-370
                      (``x @ code`` -> ``> 0`` -> LSB-first pack, bit masks :445-448)
* token distance .... ucm/sparse/gsa_on_device/csrc/cuda/ham_dist/paged_ham_dist_mla.cu:148-182
* sink/recent/inf ... paged_ham_dist_mla.cu:194-197,213-214
* block min ......... ucm/sparse/gsa_on_device/hamming_topk.py:45-47 and
                      ucm/sparse/gsa_on_device/csrc/cuda/hash_retrieval/cpy/hash_retrieval_backend.cpp:361-389
* top-k + sort + block-table gather  hamming_topk.py:49-54 (with a total
                      ``(score, id)`` order added; the reference's tie order is unspecified)
* seq_lens .......... hamming_topk.py:7-12
* query grouping .... ucm/sparse/gsa_on_device/gsa_on_device.py:396-412
* KV gather ......... gsa_on_device.py:579-580 (``kv[block_ids]``)

Conventions: bf16 tensors travel as ``uint16`` bit patterns; codes are
``uint32`` words where bit ``b`` of word ``w`` is projection column ``32*w+b``
(the little-endian view of the reference's LSB-first bytes).
"""
from __future__ import annotations

import numpy as np

REDUCE_MIN = 0
REDUCE_SUM = 1

KEY_FORCED = 0
KEY_INVALID = 0xFFFFFFFF
SCORE_INVALID = -1


# --------------------------------------------------------------------------
# bf16 helpers
# --------------------------------------------------------------------------
def bf16_bits_to_f32(u16: np.ndarray) -> np.ndarray:
    """Exact widening of bf16 bit patterns to float32."""
    u16 = np.ascontiguousarray(u16, dtype=np.uint16)
    return (u16.astype(np.uint32) << np.uint32(16)).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bf16 bit patterns (NaN kept quiet)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    lsb = (u >> np.uint32(16)) & np.uint32(1)
    rounded = (u + np.uint32(0x7FFF) + lsb) >> np.uint32(16)
    out = rounded.astype(np.uint16)
    nan = np.isnan(x)
    if nan.any():
        out = np.where(nan, np.uint16(0x7FC0), out)
    return out


# --------------------------------------------------------------------------
# (1) hash encode
# --------------------------------------------------------------------------
def pack_bits_u32(bits: np.ndarray) -> np.ndarray:
    """[..., nbits] bool -> [..., nbits/32] uint32, bit b of word w = column 32w+b.

    hash_encoder.py:362-369 packs 8 columns per byte with weights 1,2,...,128;
    viewing 4 such bytes as one little-endian word gives this layout.
    """
    bits = np.asarray(bits, dtype=bool)
    nbits = bits.shape[-1]
    assert nbits % 32 == 0
    b = bits.reshape(bits.shape[:-1] + (nbits // 32, 32)).astype(np.uint32)
    weights = (np.uint32(1) << np.arange(32, dtype=np.uint32))
    return (b * weights).sum(axis=-1, dtype=np.uint32)


def unpack_bits_u32(codes: np.ndarray) -> np.ndarray:
    codes = np.asarray(codes, dtype=np.uint32)
    sh = np.arange(32, dtype=np.uint32)
    bits = (codes[..., None] >> sh) & np.uint32(1)
    return bits.reshape(codes.shape[:-1] + (codes.shape[-1] * 32,)).astype(bool)


def hash_project(x_bf16: np.ndarray, r_bf16: np.ndarray):
    """Projection of bf16 rows by the bf16 matrix R[in_dim, hash_bits].

    Returns (P32, P64): float32-accumulated and float64-accumulated products of
    the exact bf16 values.  P64 only classifies near-zero bits.
    """
    x = bf16_bits_to_f32(x_bf16)
    r = bf16_bits_to_f32(r_bf16)
    p32 = x.reshape(-1, x.shape[-1]) @ r
    p64 = x.reshape(-1, x.shape[-1]).astype(np.float64) @ r.astype(np.float64)
    return p32.reshape(x.shape[:-1] + (r.shape[1],)), p64.reshape(x.shape[:-1] + (r.shape[1],))


def hash_encode(x_bf16: np.ndarray, r_bf16: np.ndarray):
    """hash_encoder.py:359-370.  Returns (codes uint32 [..., bits/32], P64)."""
    p32, p64 = hash_project(x_bf16, r_bf16)
    return pack_bits_u32(p32 > 0), p64


def group_mean_bf16(q_bf16: np.ndarray, num_kv_heads: int) -> np.ndarray:
    """gsa_on_device.py:400-406: ``query.view(T,Hkv,G,D).mean(2)`` in bf16.

    torch accumulates the mean of a bf16 tensor in float32 and rounds the
    result to bf16 once.
    """
    t, hq, d = q_bf16.shape
    g = hq // num_kv_heads
    x = bf16_bits_to_f32(q_bf16).reshape(t, num_kv_heads, g, d)
    acc = np.zeros((t, num_kv_heads, d), dtype=np.float32)
    for i in range(g):
        acc = acc + x[:, :, i, :]
    return f32_to_bf16_bits(acc / np.float32(g))


def count_code_mismatches(dev_codes: np.ndarray, p64: np.ndarray, tol: float = 1e-3):
    """Compare device codes with sign(P64).  Returns (hard, soft).

    ``hard`` = differing bits whose |projection| >= tol (must be zero);
    ``soft`` = differing bits below tol (allowed, reported).
    """
    want = p64 > 0
    got = unpack_bits_u32(dev_codes).reshape(want.shape)
    diff = want != got
    soft = diff & (np.abs(p64) < tol)
    hard = diff & ~soft
    return int(hard.sum()), int(soft.sum())


# --------------------------------------------------------------------------
# (2) Hamming scan
# --------------------------------------------------------------------------
def token_distances(codes, q_codes, block_table, seq_lens):
    """d[b,h,p] = sum_{g<G} sum_w popcount(codes[phys,row,h,w] ^ q[b,h*G+g,w]).

    codes [NB,BS,Hkv,W] uint32, q_codes [B,Hq,W] uint32, block_table
    [B,max_blocks] int32, seq_lens [B].  Positions >= seq_len hold -1.
    paged_ham_dist_mla.cu:148-182 with the declared ``[NB,BS,Hkv,W]`` layout.
    """
    codes = np.asarray(codes, dtype=np.uint32)
    q_codes = np.asarray(q_codes, dtype=np.uint32)
    nb_pool, bs, hkv, w = codes.shape
    b, hq, _ = q_codes.shape
    g = hq // hkv
    max_blocks = block_table.shape[1]
    out = np.full((b, hkv, max_blocks * bs), -1, dtype=np.int64)
    for bi in range(b):
        sl = int(seq_lens[bi])
        nblk = (sl + bs - 1) // bs
        if nblk == 0:
            continue
        phys = np.asarray(block_table[bi, :nblk], dtype=np.int64)
        k = codes[phys]                                   # [nblk,BS,Hkv,W]
        q = q_codes[bi].reshape(hkv, g, w)                # [Hkv,G,W]
        x = k[:, :, :, None, :] ^ q[None, None, :, :, :]  # [nblk,BS,Hkv,G,W]
        d = np.bitwise_count(x).sum(axis=(-1, -2), dtype=np.int64)  # [nblk,BS,Hkv]
        d = d.reshape(nblk * bs, hkv).T                   # [Hkv, nblk*BS]
        out[bi, :, :sl] = d[:, :sl]
    return out


def block_scores(codes, q_codes, block_table, seq_lens, mode, reduce_kvhead=False):
    """S[b,h,j] over the valid tokens of logical block j; SCORE_INVALID for j >= nb.

    mode REDUCE_MIN: min over tokens (hamming_topk.py:45-47); REDUCE_SUM: sum
    over tokens.  reduce_kvhead combines heads with the same operator
    (paged_ham_dist_mla.cu:200-211 takes the min over kv heads).
    Returns int64 [B,Hout,max_blocks].
    """
    d = token_distances(codes, q_codes, block_table, seq_lens)
    b, hkv, max_seq = d.shape
    bs = codes.shape[1]
    max_blocks = block_table.shape[1]
    d = d.reshape(b, hkv, max_blocks, bs)
    valid = d >= 0
    if mode == REDUCE_SUM:
        s = np.where(valid, d, 0).sum(axis=-1)
    else:
        s = np.where(valid, d, np.iinfo(np.int64).max).min(axis=-1)
    has = valid.any(axis=-1)
    if reduce_kvhead:
        s = s.sum(axis=1, keepdims=True) if mode == REDUCE_SUM else s.min(axis=1, keepdims=True)
        has = has.any(axis=1, keepdims=True)
    return np.where(has, s, SCORE_INVALID)


def hamming_score_fp16(codes, q_codes, block_table, seq_lens, sink, recent, reduce_kvhead):
    """Per-token fp16 output of the reference op ``hamming_score``.

    paged_ham_dist_mla.cu:189-247 with the declared key layout: positions below
    ``sink`` or inside ``[seq_len-recent, seq_len)`` -> 0, positions >= seq_len
    -> +inf, otherwise the G-way distance (min over kv heads when
    reduce_kvhead).  Shape [B, 1 or Hkv, max_blocks*BS] float16.
    """
    d = token_distances(codes, q_codes, block_table, seq_lens)
    b, hkv, max_seq = d.shape
    pos = np.arange(max_seq)[None, None, :]
    sl = np.asarray(seq_lens, dtype=np.int64)[:, None, None]
    if reduce_kvhead:
        big = np.iinfo(np.int64).max
        d = np.where(d >= 0, d, big).min(axis=1, keepdims=True)
    out = d.astype(np.float32)
    forced = (pos < sink) | ((pos >= sl - recent) & (pos < sl))
    out = np.where(forced, 0.0, out)
    out = np.where(pos >= sl, np.inf, out)
    return out.astype(np.float16)


# --------------------------------------------------------------------------
# (3) forced blocks + exact top-k
# --------------------------------------------------------------------------
def forced_blocks(seq_len, block_size, max_blocks, must_select=(), sink_tokens=0, recent_tokens=0):
    """Boolean [max_blocks]: blocks that are always selected.

    ``must_select``: non-negative = index from the start, negative = from the
    request's block count (gsa_on_device_config.py:72-73).  ``sink_tokens`` /
    ``recent_tokens``: every block overlapping ``[0,sink)`` or
    ``[seq_len-recent, seq_len)`` (the token ranges paged_ham_dist_mla.cu:194-196
    zeroes).
    """
    nb = (int(seq_len) + block_size - 1) // block_size
    f = np.zeros(max_blocks, dtype=bool)
    for m in must_select:
        j = m if m >= 0 else nb + m
        if 0 <= j < nb:
            f[j] = True
    j = np.arange(max_blocks)
    lo = j * block_size
    hi = np.minimum(lo + block_size, int(seq_len))
    in_range = j < nb
    if sink_tokens > 0:
        f |= in_range & (lo < sink_tokens)
    if recent_tokens > 0:
        f |= in_range & (hi > int(seq_len) - recent_tokens)
    return f


def selection_keys(scores_row, forced_row):
    """uint64 keys: forced -> 0, valid -> score+1, invalid -> 0xFFFFFFFF."""
    s = np.asarray(scores_row, dtype=np.int64)
    key = np.where(s == SCORE_INVALID, KEY_INVALID, s + 1).astype(np.uint64)
    key = np.where(forced_row & (s != SCORE_INVALID), np.uint64(KEY_FORCED), key)
    return key


def select_topk(keys, k, ids=None):
    """First k entries under the (key, id) total order, returned sorted by id.

    hamming_topk.py:49-52 (topk largest=False, then sort of the indices).
    """
    keys = np.asarray(keys, dtype=np.uint64)
    n = keys.shape[0]
    if ids is None:
        ids = np.arange(n, dtype=np.int64)
    order = np.lexsort((ids, keys))[:k]
    chosen = order[np.argsort(ids[order], kind="stable")]
    return chosen


def update_seq_lens(seq_lens, topk_token, block_size):
    """hamming_topk.py:7-12."""
    s = np.asarray(seq_lens, dtype=np.int64)
    drop = (np.clip(s - topk_token, 0, None) + block_size - 1) // block_size
    return s - drop * block_size


def hamming_topk(codes, q_codes, block_table, seq_lens, k, mode=REDUCE_SUM,
                 reduce_kvhead=False, must_select=(), sink_tokens=0, recent_tokens=0,
                 k_per_request=None, request_mask=None):
    """Full retrieval: scores -> keys -> top-k -> block-table lookup.

    Returns dict with ``logical`` / ``physical`` int32 [B,Hout,k], ``scores``
    int32 [B,Hout,k] (raw block score of each selected block, -1 for padding),
    ``valid_count`` int32 [B], ``new_seq_lens`` int32 [B], ``block_scores``
    int64 [B,Hout,max_blocks].

    Rows whose ``request_mask`` is 0 keep the head of their own block table
    (logical ids 0..k-1) and their seq_len.  With ``k_per_request`` row b uses
    ``min(k_per_request[b], k)`` and pads with logical -1 / physical 0.
    """
    bs = codes.shape[1]
    b = q_codes.shape[0]
    max_blocks = block_table.shape[1]
    assert k <= max_blocks
    s = block_scores(codes, q_codes, block_table, seq_lens, mode, reduce_kvhead)
    hout = s.shape[1]
    logical = np.full((b, hout, k), -1, dtype=np.int32)
    physical = np.zeros((b, hout, k), dtype=np.int32)
    sel_scores = np.full((b, hout, k), -1, dtype=np.int32)
    valid_count = np.zeros(b, dtype=np.int32)
    new_seq = np.asarray(seq_lens, dtype=np.int64).copy()
    for bi in range(b):
        sl = int(seq_lens[bi])
        nb = (sl + bs - 1) // bs
        kb = k if k_per_request is None else max(0, min(int(k_per_request[bi]), k))
        if request_mask is not None and not request_mask[bi]:
            ids = np.arange(kb)
            for h in range(hout):
                logical[bi, h, :kb] = ids
                physical[bi, h, :kb] = block_table[bi, :kb]
                sel_scores[bi, h, :kb] = s[bi, h, :kb]
            valid_count[bi] = min(kb, nb)
            continue
        f = forced_blocks(sl, bs, max_blocks, must_select, sink_tokens, recent_tokens)
        for h in range(hout):
            keys = selection_keys(s[bi, h], f)
            ch = select_topk(keys, kb)
            logical[bi, h, :kb] = ch
            physical[bi, h, :kb] = block_table[bi, ch]
            sel_scores[bi, h, :kb] = s[bi, h, ch]
        valid_count[bi] = min(kb, nb)
        new_seq[bi] = update_seq_lens(np.array([sl]), kb * bs, bs)[0]
    return dict(logical=logical, physical=physical, scores=sel_scores,
                valid_count=valid_count, new_seq_lens=new_seq.astype(np.int32),
                block_scores=s)


# --------------------------------------------------------------------------
# (4) paged-KV gather
# --------------------------------------------------------------------------
def gather_kv(pool, physical):
    """out[b, i*BS+t, h, :] = pool[physical[b,(h),i], t, h, :]  (gsa_on_device.py:579-580).

    pool [NB,BS,Hkv,D] (any dtype); physical [B,k] (whole blocks) or [B,Hkv,k]
    (per kv head).  Returns [B, k*BS, Hkv, D].
    """
    nb, bs, hkv, d = pool.shape
    physical = np.asarray(physical)
    if physical.ndim == 2:
        b, k = physical.shape
        return pool[physical.reshape(-1)].reshape(b, k * bs, hkv, d)
    b, h, k = physical.shape
    assert h == hkv
    out = np.empty((b, k * bs, hkv, d), dtype=pool.dtype)
    for hi in range(hkv):
        out[:, :, hi, :] = pool[physical[:, hi, :].reshape(-1), :, hi, :].reshape(b, k * bs, d)
    return out


# --------------------------------------------------------------------------
# (5) sharded candidates + merge
# --------------------------------------------------------------------------
def f32_order_key(x):
    """Monotone map float32 -> uint32 (total order of the values, -0 < +0)."""
    u = np.asarray(x, dtype=np.float32).view(np.uint32)
    neg = (u >> np.uint32(31)).astype(bool)
    return np.where(neg, ~u, u | np.uint32(0x80000000)).astype(np.uint32)


CAND_FORCED_SCORE = np.float32(-1.0)
CAND_INVALID_SCORE = np.float32(np.inf)


def topk_candidates(codes, q_codes, block_table, seq_lens_local, k, block_id_offset, score_scale,
                    forced_local, mode=REDUCE_SUM, reduce_kvhead=False):
    """Local top-k of one sequence shard as (float32 score, int32 global id) records.

    ``seq_lens_local``: tokens this shard holds per request; ``forced_local``
    bool [B,max_blocks] marks this shard's forced blocks (score -1 so that they
    survive the merge); padding records carry +inf and id -1.  Score =
    block score * score_scale (1/(BS*G) turns a sum into the mean Hamming distance).
    """
    s = block_scores(codes, q_codes, block_table, seq_lens_local, mode, reduce_kvhead)
    b, hout, max_blocks = s.shape
    sc = np.full((b, hout, k), CAND_INVALID_SCORE, dtype=np.float32)
    ids = np.full((b, hout, k), -1, dtype=np.int32)
    for bi in range(b):
        for h in range(hout):
            keys = selection_keys(s[bi, h], forced_local[bi])
            valid = s[bi, h] != SCORE_INVALID
            ch = select_topk(keys, min(k, max_blocks))
            ch = ch[valid[ch]]
            n = len(ch)
            val = (s[bi, h, ch].astype(np.float32) * np.float32(score_scale)).astype(np.float32)
            val = np.where(forced_local[bi][ch], CAND_FORCED_SCORE, val)
            sc[bi, h, :n] = val
            ids[bi, h, :n] = ch + block_id_offset
    return sc, ids


def merge_topk(cand_scores, cand_ids, k):
    """Global top-k over gathered records [R,B,H,kl] -> ids [B,H,k] sorted by id.

    Order: (score, id) ascending, padding (+inf, -1) last.  Returns
    (scores float32 [B,H,k], ids int32 [B,H,k]); unused tail = (+inf, -1).
    """
    r, b, h, kl = cand_scores.shape
    out_s = np.full((b, h, k), CAND_INVALID_SCORE, dtype=np.float32)
    out_i = np.full((b, h, k), -1, dtype=np.int32)
    for bi in range(b):
        for hi in range(h):
            s = cand_scores[:, bi, hi, :].reshape(-1)
            i = cand_ids[:, bi, hi, :].reshape(-1).astype(np.int64)
            real = i >= 0
            s, i = s[real], i[real]
            order = np.lexsort((i, f32_order_key(s)))[:k]
            order = order[np.argsort(i[order], kind="stable")]
            out_s[bi, hi, :len(order)] = s[order]
            out_i[bi, hi, :len(order)] = i[order]
    return out_s, out_i


# ----------------------------------------------------------------------------------------------
# float block retrieval (ESA / KVStar plugins)
# ----------------------------------------------------------------------------------------------
def block_repr_mean(k_bf16: np.ndarray, block_ids, merge: int = 0):
    """Mean key over groups of ``merge`` tokens of each listed block (0 = the whole block): esa.py:254-263
    (``k_cache[ids].mean(1)``) and kvstar/multistep.py:322-327 (``reshape(n, M, c, h, d).mean(dim=2)``).
    k_bf16 uint16 [NB, BS, H, D].  Returns (bf16 bits [n, BS/merge, H, D], float64 means): torch accumulates in
    float32 and rounds once; the float64 mean is kept to tell a rounding tie from an error."""
    k = bf16_bits_to_f32(np.asarray(k_bf16)).astype(np.float64)
    blk = k[np.asarray(block_ids, dtype=np.int64)]
    n, bs, h, d = blk.shape
    merge = bs if merge <= 0 else merge
    m64 = blk.reshape(n, bs // merge, merge, h, d).mean(axis=2)
    return f32_to_bf16_bits(m64.astype(np.float32)), m64


def dot_topk(repr_bf16: np.ndarray, q_bf16: np.ndarray, indexes: np.ndarray, k: int):
    """Inner-product retrieval of retrieval_backend.cpp:206-225: per request the k allowed indexes with the largest
    <q, data[idx]>.  Returns (scores float64 [B, n] for every candidate position (-inf where none), chosen candidate
    POSITIONS by descending score as a list per request)."""
    data = bf16_bits_to_f32(np.asarray(repr_bf16)).astype(np.float64)
    data = data.reshape(data.shape[0], -1)
    q = bf16_bits_to_f32(np.asarray(q_bf16)).astype(np.float64).reshape(len(q_bf16), -1)
    idx = np.asarray(indexes)
    scores = np.full(idx.shape, -np.inf)
    chosen = []
    for b in range(idx.shape[0]):
        ok = (idx[b] >= 0) & (idx[b] < data.shape[0])
        scores[b, ok] = data[idx[b, ok]] @ q[b]
        order = [p for p in np.argsort(-scores[b], kind="stable") if ok[p]][:k]
        chosen.append(order)
    return scores, chosen


def softmax_block_scores(repr_bf16: np.ndarray, q_bf16: np.ndarray) -> np.ndarray:
    """KVStar block scores (kvstar/retrieve/core/domain/retrieve_task/simd_compute_kernel.cpp:884-947):
    repr [n_blocks, M, Hkv, D], q [X, Hq, D]; per (token, query head) softmax over all n_blocks*M inner products
    with its kv head's representations, summed over rows and over each block's M.  float64."""
    r = bf16_bits_to_f32(np.asarray(repr_bf16)).astype(np.float64)
    q = bf16_bits_to_f32(np.asarray(q_bf16)).astype(np.float64)
    n, m, hkv, d = r.shape
    x, hq, _ = q.shape
    g = hq // hkv
    out = np.zeros(n)
    for xi in range(x):
        for hh in range(hq):
            logits = r[:, :, hh // g, :].reshape(n * m, d) @ q[xi, hh]
            e = np.exp(logits - logits.max())
            s = e.sum()
            if s > 1e-9:
                e = e / s
            out += e.reshape(n, m).sum(axis=1)
    return out

"""CPU tests of the oracle: numpy restatement vs C restatement, vs the golden fixtures generated
from the reference's own Python code, and vs the reference's C++ retrieval backend when its compiled
module is present."""
import os

import numpy as np
import pytest

from oracle import build_oracle
from oracle import oracle as O
from oracle import oracle_c as OC
from tests import helpers as H

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _g(name):
    return np.load(os.path.join(GOLDEN, name))


# ---------------------------------------------------------------- numpy vs C -----------------
@pytest.mark.parametrize("mode", [O.REDUCE_MIN, O.REDUCE_SUM])
@pytest.mark.parametrize("reduce_kvhead", [False, True])
@pytest.mark.parametrize("shape", [(3, 8, 4, 4, 16, 12), (2, 1, 8, 4, 32, 9), (2, 4, 1, 18, 8, 7), (1, 3, 2, 2, 8, 5)])
def test_numpy_and_c_oracles_agree(shape, mode, reduce_kvhead):
    B, Hkv, G, W, BS, mb = shape
    case = H.make_paged_case(sum(shape), B, Hkv, G, W, BS, mb)
    kw = dict(must_select=(0, -2, -1), sink_tokens=BS // 2, recent_tokens=BS + 1)
    a = O.hamming_topk(case["codes"], case["q"], case["block_table"], case["seq_lens"], min(4, mb), mode,
                       reduce_kvhead, **kw)
    c = OC.hamming_topk(case["codes"], case["q"], case["block_table"], case["seq_lens"], min(4, mb), mode,
                        reduce_kvhead, **kw)
    for key in ("logical", "physical", "scores", "valid_count", "new_seq_lens", "block_scores"):
        assert np.array_equal(np.asarray(a[key]), np.asarray(c[key])), key


def test_c_encode_matches_numpy():
    rng = np.random.default_rng(0)
    x = H.bf16_normal(rng, (300, 128))
    r = H.bf16_normal(rng, (128, 128), 1 / np.sqrt(128))
    codes, p64 = O.hash_encode(x, r)
    hard, soft = O.count_code_mismatches(OC.hash_encode(x, r), p64)
    assert hard == 0 and soft <= 2


def test_c_gather_matches_numpy():
    rng = np.random.default_rng(1)
    pool = rng.integers(0, 2**16, size=(12, 8, 2, 16), dtype=np.uint16)
    for sel in (rng.integers(0, 12, size=(3, 4)), rng.integers(0, 12, size=(3, 2, 4))):
        assert np.array_equal(O.gather_kv(pool, sel.astype(np.int32)), OC.gather_kv(pool, sel.astype(np.int32)))


# ---------------------------------------------------------------- golden fixtures ------------
def test_golden_encode():
    """Reference torch_hash_code (CPU, eager): same bits except where |projection| < 1e-3."""
    g = _g("encode.npz")
    assert g["bit_masks"].tolist() == [1, 2, 4, 8, 16, 32, 64, 128]       # LSB-first packing
    codes, p64 = O.hash_encode(g["x_bf16"], g["r_bf16"])
    for key in ("codes_u8_f32", "codes_u8_bf16"):
        ref_words = np.ascontiguousarray(g[key]).view("<u4")              # 4 bytes -> one little-endian word
        hard, soft = O.count_code_mismatches(ref_words, p64)
        assert hard == 0, key
        assert soft <= 2, key
    assert np.array_equal(codes, np.ascontiguousarray(g["codes_u8_f32"]).view("<u4"))


def test_golden_encode_query_group_mean():
    g = _g("encode_query.npz")
    qm = O.group_mean_bf16(g["q_bf16"], 8)
    assert np.array_equal(qm, g["qmean_bf16"])                             # bf16 mean, bit-exact
    codes, p64 = O.hash_encode(qm, _g("encode.npz")["r_bf16"])
    hard, soft = O.count_code_mismatches(np.ascontiguousarray(g["codes_u8"]).view("<u4"), p64)
    assert hard == 0 and soft <= 1


def test_golden_distances():
    """Reference formulation: unpack to +-1, einsum, distance = (bits - similarity)/2."""
    g = _g("distances.npz")
    codes = np.ascontiguousarray(g["key_u8"]).view("<u4")
    q = np.ascontiguousarray(g["q_u8"]).view("<u4")
    d = O.token_distances(codes, q, g["block_table"], g["seq_lens"])
    assert np.array_equal(d, g["dist"].astype(np.int64))


def test_golden_update_seq_lens():
    g = _g("update_seq_lens.npz")
    for (topk, bs), want in zip(g["params"], g["out"]):
        assert np.array_equal(O.update_seq_lens(g["seq_lens"], int(topk), int(bs)), want)


def test_golden_topk_tail():
    """Reference cuda_hamming_topk tail (torch.min / topk / sort / gather) on per-token scores.

    The reference's tie order is unspecified, so: block scores must match exactly, every block
    strictly below the k-th score must be selected by both, and every selected block must be at or
    below it.
    """
    g = _g("topk_tail.npz")
    topk_token, sink, recent, BS = (int(v) for v in g["params"])
    codes = np.ascontiguousarray(g["key_u8"]).view("<u4")
    q = np.ascontiguousarray(g["q_u8"]).view("<u4")
    bt, seq = g["block_table"], g["seq_lens"]
    k = topk_token // BS
    out = O.hamming_topk(codes, q, bt, seq, k, O.REDUCE_MIN, True, sink_tokens=sink, recent_tokens=recent)
    ref_scores = g["block_scores_f16"].astype(np.float32)                  # [B, max_blocks], forced = 0, past end = inf
    B, mb = ref_scores.shape
    for b in range(B):
        forced = O.forced_blocks(seq[b], BS, mb, (), sink, recent)
        s = out["block_scores"][b, 0].astype(np.float32)
        mine = np.where(s < 0, np.inf, np.where(forced, 0.0, s))
        assert np.array_equal(mine, ref_scores[b])
        kth = np.sort(ref_scores[b])[k - 1]
        # map the reference's physical ids back to logical positions
        nb = int((seq[b] + BS - 1) // BS)
        phys_to_log = {int(bt[b, j]): j for j in range(nb)}
        ref_log = {phys_to_log[int(p)] for p in g["selected_physical"][b] if int(p) in phys_to_log}
        my_log = set(int(j) for j in out["logical"][b, 0])
        must = {j for j in range(mb) if ref_scores[b, j] < kth}
        assert must <= ref_log and must <= my_log
        assert all(ref_scores[b, j] <= kth for j in ref_log | my_log)
        assert len(ref_log) == len(my_log) == k


def test_declared_layout_vs_reference_kernel_indexing():
    """The reference kernel indexes a block as [Hkv][BS][W] although the cache is written as
    [BS][Hkv][W]; the two agree for one kv head.  The oracle follows the written layout."""
    rng = np.random.default_rng(3)
    BS, W = 8, 4
    codes1 = H.rand_codes(rng, (2, BS, 1, W))
    as_kernel = codes1.reshape(2, 1, BS, W).transpose(0, 2, 1, 3)          # [NB][Hkv][BS][W] read back as [NB,BS,Hkv,W]
    assert np.array_equal(codes1, as_kernel)
    codes2 = H.rand_codes(rng, (2, BS, 2, W))
    as_kernel2 = codes2.reshape(2, 2, BS, W).transpose(0, 2, 1, 3)
    assert not np.array_equal(codes2, as_kernel2)


# ---------------------------------------------------------------- compiled reference backend --
def test_reference_cpp_backend_min_scores():
    """hash_retrieval_backend.cpp compiled from the reference checkout: min over tokens of the
    popcount distance, ascending partial sort.  Scores must equal the oracle's k smallest."""
    build_oracle.build_ref()
    ref = build_oracle.load_ref()
    if ref is None:
        pytest.skip("reference backend not built (no reference checkout on this machine)")
    rng = np.random.default_rng(5)
    NB, BS, dim, B, n, k = 64, 16, 32, 3, 40, 7
    data = rng.integers(0, 256, size=(NB, BS, dim), dtype=np.uint8)
    query = rng.integers(0, 256, size=(B, dim), dtype=np.uint8)
    idx = np.stack([rng.permutation(NB)[:n] for _ in range(B)]).astype(np.int32)
    idx[1, 30:] = -1                                                      # padded index list
    backend = ref.HashRetrievalWorkerBackend(data, {0: [0]})
    rid = backend.submit(query, k, idx)
    backend.wait(rid)
    res = backend.get_result(rid)
    del backend
    codes = data.reshape(NB, BS, 1, dim).view("<u4")                      # one "head" of dim*8 bits
    q = query.reshape(B, 1, dim).view("<u4")
    for b in range(B):
        allowed = idx[b][idx[b] >= 0]
        bt = allowed[None, :].astype(np.int32)
        s = O.block_scores(codes, q[b:b + 1], bt, np.array([len(allowed) * BS]), O.REDUCE_MIN)[0, 0]
        assert np.array_equal(np.sort(s)[:k], res["scores"][b])
        pos = {int(p): i for i, p in enumerate(allowed)}
        assert all(s[pos[int(p)]] == sc for p, sc in zip(res["indices"][b], res["scores"][b]))


def run_esa_backend(mod, pool_f32, q_f32, indexes, k):
    """submit / wait / get_result round trips through the reference's RetrievalWorkerBackend, one request at a
    time: its get_result copies as many entries for every request as the FIRST request produced
    (retrieval_backend.cpp:133-141), which reads past the end of shorter result lists in a ragged batch."""
    backend = mod.RetrievalWorkerBackend(np.ascontiguousarray(pool_f32, dtype=np.float32), {0: [0]})
    out = {"indices": [], "scores": []}
    for b in range(len(q_f32)):
        rid = backend.submit(np.ascontiguousarray(q_f32[b:b + 1], dtype=np.float32), int(k),
                             np.ascontiguousarray(indexes[b:b + 1], dtype=np.int32))
        backend.wait(rid)
        res = backend.get_result(rid)
        out["indices"].append(np.asarray(res["indices"])[0].copy())
        out["scores"].append(np.asarray(res["scores"])[0].copy())
    del backend
    return out


def test_reference_esa_backend_dot_topk():
    """ucm/sparse/esa/retrieval/cpy/retrieval_backend.cpp compiled unmodified (its <numaif.h> include is met by a
    stand-in header where libnuma is missing): inner products and the k best per request.  The oracle's float64
    scores must match its float32 scalar loop to 1e-5 and pick the same candidates in the same order."""
    build_oracle.build_ref_esa()
    mod = build_oracle.load_ref_esa()
    if mod is None:
        pytest.skip("ESA backend not built (no reference checkout on this machine)")
    rng = np.random.default_rng(21)
    N, dim, B, n, k = 400, 256, 4, 120, 9
    pool = H.bf16_normal(rng, (N, dim))
    q = H.bf16_normal(rng, (B, dim))
    indexes = np.full((B, n), -1, dtype=np.int32)
    for b, cnt in enumerate([120, 60, 9, 3]):
        indexes[b, :cnt] = rng.permutation(N)[:cnt]
    res = run_esa_backend(mod, O.bf16_bits_to_f32(pool), O.bf16_bits_to_f32(q), indexes, k)
    scores, chosen = O.dot_topk(pool, q, indexes, k)
    for b in range(B):
        got_idx = [int(i) for i in res["indices"][b]]
        want_idx = [int(indexes[b][p]) for p in chosen[b]]
        assert got_idx == want_idx            # continuous random scores: no ties, so the order is determined
        assert np.allclose(np.asarray(res["scores"][b], dtype=np.float64), scores[b][chosen[b]], rtol=1e-5, atol=1e-5)


def test_golden_float_retrieval():
    """Block representations as torch computes them in the ESA / KVStar plugins, and the inner-product top-k."""
    g = np.load(os.path.join(GOLDEN, "float_retrieval.npz"))
    r, _ = O.block_repr_mean(g["k_cache"], g["block_ids"])
    assert np.array_equal(r[:, 0], g["repr_esa"])
    r, _ = O.block_repr_mean(g["k_cache"], g["block_ids"], int(g["merge"]))
    assert np.array_equal(r, g["repr_kvstar"])
    scores, chosen = O.dot_topk(g["pool"], g["q"], g["indexes"], int(g["k"]))
    fin = np.isfinite(g["scores"])
    assert np.array_equal(fin, np.isfinite(scores))
    assert np.allclose(scores[fin], g["scores"][fin], rtol=1e-5, atol=1e-5)
    for b, pos in enumerate(chosen):
        want = [int(i) for i in g["top_ids"][b] if i >= 0]
        assert [int(g["indexes"][b][p]) for p in pos] == want

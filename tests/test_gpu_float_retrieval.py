"""GPU parity: float block retrieval (block representations, inner-product top-k) vs the oracle and the golden
fixture made with torch.  Tolerance: representations are bf16 roundings of float32 means - an element may differ by
one bf16 step where the exact mean sits at a rounding boundary; scores are float32 sums in another order than the
reference's scalar loop - relative 1e-5."""
import os

import numpy as np
import pytest

from oracle import oracle as O
from tests import helpers as H

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _bits(t):
    import torch
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def _check_repr(got_bits, want_bits, m64):
    diff = got_bits != want_bits
    if diff.any():
        got, want = O.bf16_bits_to_f32(got_bits), O.bf16_bits_to_f32(want_bits)
        step = np.abs(want) * 2.0 ** -7 + 1e-30          # one bf16 step at that magnitude (upper bound)
        assert (np.abs(got - want)[diff] <= step[diff]).all()
        # ... and only where the exact mean lies half-way between two bf16 values to float32 accuracy
        mid = (got.astype(np.float64) + want.astype(np.float64)) / 2
        assert (np.abs(m64 - mid)[diff] <= np.abs(m64[diff]) * 2.0 ** -20 + 1e-30).all()
        assert diff.mean() < 1e-3


def test_block_repr_matches_torch_golden(cuda_device):
    import torch
    from unified_cache_management_b200 import ops
    g = np.load(os.path.join(GOLDEN, "float_retrieval.npz"))
    kc = H.bf16_to_dev(g["k_cache"], cuda_device)
    ids = torch.from_numpy(g["block_ids"]).to(cuda_device)
    r = ops.block_repr_mean(kc, ids)
    torch.cuda.synchronize()
    assert np.array_equal(_bits(r)[:, 0], g["repr_esa"])
    r = ops.block_repr_mean(kc, ids, merge=int(g["merge"]))
    torch.cuda.synchronize()
    assert np.array_equal(_bits(r), g["repr_kvstar"])


@pytest.mark.parametrize("BS,Hh,D,merge,strided", [(128, 8, 128, None, False), (128, 8, 128, 8, True), (16, 2, 64, 4, False)])
def test_block_repr_random(cuda_device, BS, Hh, D, merge, strided):
    import torch
    from unified_cache_management_b200 import ops
    rng = np.random.default_rng(BS + D)
    NB = 50
    kv = H.bf16_normal(rng, (NB, 2, BS, Hh, D)) if strided else H.bf16_normal(rng, (NB, BS, Hh, D))
    kd = H.bf16_to_dev(kv, cuda_device)
    kd = kd[:, 0] if strided else kd
    kh = kv[:, 0] if strided else kv
    ids = np.array([3, 49, 0, 17, 17, 8, 21], dtype=np.int32)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    r = ops.block_repr_mean(kd, torch.from_numpy(ids).to(cuda_device), merge=merge, status=status)
    torch.cuda.synchronize()
    want, m64 = O.block_repr_mean(kh, ids, merge or 0)
    _check_repr(_bits(r), want, m64)
    assert int(status.item()) == 0
    bad = torch.tensor([1, NB, 2], dtype=torch.int32, device=cuda_device)
    ops.block_repr_mean(kd, bad, merge=merge, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) & 1


def _check_topk(scores_dev, ids_dev, oracle_scores, indexes, k):
    B = indexes.shape[0]
    for b in range(B):
        cand = [(p, int(i)) for p, i in enumerate(indexes[b]) if i >= 0]
        kk = min(k, len(cand))
        got_ids = [int(i) for i in ids_dev[b] if i >= 0]
        assert len(got_ids) == kk and (ids_dev[b, kk:] == -1).all() and np.isneginf(scores_dev[b, kk:]).all()
        # chosen candidates come in the order of the index list
        pos_of = {}
        for p, i in cand:
            pos_of.setdefault(i, p)
        pos = [pos_of[i] for i in got_ids]
        assert pos == sorted(pos)
        sc = oracle_scores[b]
        assert np.allclose(scores_dev[b, :kk], sc[pos], rtol=1e-5, atol=1e-4)
        best = np.sort(sc[[p for p, _ in cand]])[::-1][:kk]
        assert np.allclose(np.sort(sc[pos])[::-1], best, rtol=1e-5, atol=1e-4)   # same scores up to near-ties


def test_dot_topk_matches_golden(cuda_device):
    import torch
    from unified_cache_management_b200 import ops
    g = np.load(os.path.join(GOLDEN, "float_retrieval.npz"))
    k = int(g["k"])
    s, i = ops.dot_topk(H.bf16_to_dev(g["pool"], cuda_device), H.bf16_to_dev(g["q"], cuda_device),
                        torch.from_numpy(g["indexes"]).to(cuda_device), k)
    torch.cuda.synchronize()
    i = i.cpu().numpy()
    for b in range(i.shape[0]):
        assert sorted(int(x) for x in i[b] if x >= 0) == sorted(int(x) for x in g["top_ids"][b] if x >= 0)
    _check_topk(s.cpu().numpy(), i, g["scores"].astype(np.float64), g["indexes"], k)


def test_dot_topk_random(cuda_device):
    import torch
    from unified_cache_management_b200 import ops
    rng = np.random.default_rng(12)
    N, dim, B, n, k = 5000, 1024, 5, 3000, 200
    pool = H.bf16_normal(rng, (N, dim))
    q = H.bf16_normal(rng, (B, dim))
    indexes = np.full((B, n), -1, dtype=np.int32)
    for b, cnt in enumerate([3000, 1500, 200, 150, 1]):
        indexes[b, :cnt] = rng.permutation(N)[:cnt]
    indexes[0, 5] = N + 7          # out of range: not a candidate
    s, i = ops.dot_topk(H.bf16_to_dev(pool, cuda_device), H.bf16_to_dev(q, cuda_device),
                        torch.from_numpy(indexes).to(cuda_device), k)
    torch.cuda.synchronize()
    clean = indexes.copy()
    clean[0, 5] = -1
    sc, _ = O.dot_topk(pool, q, clean, k)
    _check_topk(s.cpu().numpy(), i.cpu().numpy(), sc, clean, k)


def test_dot_topk_matches_reference_esa_backend(cuda_device):
    """ucmr_dot_topk against the reference's own RetrievalWorkerBackend (retrieval_backend.cpp:206-225, compiled
    unmodified by oracle/build_oracle.py): same chosen candidates, scores within 1e-5 relative of its float32 loop."""
    import torch
    from oracle import build_oracle
    from tests.test_oracle import run_esa_backend
    from unified_cache_management_b200 import ops
    mod = build_oracle.load_ref_esa()
    if mod is None:
        pytest.skip("ESA backend of the reference not built on this machine")
    rng = np.random.default_rng(33)
    N, dim, B, n, k = 3000, 1024, 6, 2000, 64
    pool = H.bf16_normal(rng, (N, dim))
    q = H.bf16_normal(rng, (B, dim))
    indexes = np.full((B, n), -1, dtype=np.int32)
    for b, cnt in enumerate([2000, 1000, 500, 64, 10, 1]):
        indexes[b, :cnt] = rng.permutation(N)[:cnt]
    res = run_esa_backend(mod, O.bf16_bits_to_f32(pool), O.bf16_bits_to_f32(q), indexes, k)
    s, i = ops.dot_topk(H.bf16_to_dev(pool, cuda_device), H.bf16_to_dev(q, cuda_device),
                        torch.from_numpy(indexes).to(cuda_device), k)
    torch.cuda.synchronize()
    s, i = s.cpu().numpy(), i.cpu().numpy()
    for b in range(B):
        ref_ids = [int(x) for x in res["indices"][b]]
        ref_scores = {int(x): float(v) for x, v in zip(res["indices"][b], res["scores"][b])}
        mine = [int(x) for x in i[b] if x >= 0]
        assert sorted(mine) == sorted(ref_ids)
        for pos, idx in enumerate(i[b]):
            if idx >= 0:
                assert abs(float(s[b, pos]) - ref_scores[int(idx)]) <= 1e-5 * abs(ref_scores[int(idx)]) + 1e-4


@pytest.mark.parametrize("n,M,Hkv,G,D,X", [(300, 4, 2, 4, 128, 1), (64, 1, 8, 4, 128, 3), (1000, 16, 1, 2, 64, 2)])
def test_softmax_block_scores_and_topk(cuda_device, n, M, Hkv, G, D, X):
    import torch
    from unified_cache_management_b200 import ops
    rng = np.random.default_rng(n + M)
    rep = H.bf16_normal(rng, (n, M, Hkv, D), scale=0.3)
    q = H.bf16_normal(rng, (X, Hkv * G, D))
    k = min(20, n)
    bs, s, i = ops.softmax_topk(H.bf16_to_dev(rep, cuda_device), H.bf16_to_dev(q, cuda_device), k)
    torch.cuda.synchronize()
    want = O.softmax_block_scores(rep, q)
    got = bs.cpu().numpy()
    assert np.allclose(got, want, rtol=2e-4, atol=1e-6)
    ids = i.cpu().numpy()
    assert (np.diff(ids) > 0).all() and np.allclose(s.cpu().numpy(), got[ids])
    assert np.allclose(np.sort(want[ids])[::-1], np.sort(want)[::-1][:k], rtol=2e-4, atol=1e-6)

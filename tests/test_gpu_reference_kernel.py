"""GPU parity against the reference project's own CUDA kernel, compiled unmodified for this GPU.

``oracle/build_oracle.py --cuda-ref`` builds ``HammingScoreContiCUDA``
(ucm/sparse/gsa_on_device/csrc/cuda/ham_dist/paged_ham_dist_mla.cu:332-443) into ``oracle/_ref/hamming_cuda``.
These tests are skipped when that module was never built.

The reference kernel indexes a block as [Hkv][BS][W] (paged_ham_dist_mla.cu:168-170) although the cache is written
as [BS][Hkv][W] (hash_encoder.py:346-355); for more than one kv head the tests hand it a copy of the codes
permuted into its indexing, so both sides score the same (token, head) codes.
"""
import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref_cuda():
    from oracle import build_oracle
    mod = build_oracle.load_ref_cuda()
    if mod is None:
        pytest.skip("reference CUDA extension not built (python oracle/build_oracle.py --cuda-ref)")
    return mod


def _case(dev, seed, B, Hkv, G, W, BS, mb, seq):
    import torch
    case = H.make_paged_case(seed, B, Hkv, G, W, BS, mb, seq_lens=np.asarray(seq, dtype=np.int32))
    codes = H.to_dev_i32(case["codes"], dev)
    # the reference's view of the same codes: [NB][Hkv][BS][W] bytes under a [NB,BS,Hkv,W] shape
    codes_ref = codes.permute(0, 2, 1, 3).contiguous().view(codes.shape) if Hkv > 1 else codes
    q = H.to_dev_i32(case["q"], dev).view(B, 1, Hkv * G, W)
    bt = H.to_dev_i32(case["block_table"], dev)
    sl = torch.from_numpy(case["seq_lens"]).to(dev)
    return codes, codes_ref, q, bt, sl


@pytest.mark.parametrize("Hkv,G,W,reduce_kvhead", [(1, 8, 4, False), (1, 4, 18, False), (8, 4, 4, False),
                                                    (8, 4, 4, True), (2, 4, 8, True), (4, 1, 4, True)])
def test_per_token_scores_equal_reference_kernel(cuda_device, ref_cuda, Hkv, G, W, reduce_kvhead):
    import torch
    from unified_cache_management_b200 import ops
    B, BS, mb = 3, 128, 12
    seq = [mb * BS, 5 * BS + 77, 300]
    codes, codes_ref, q, bt, sl = _case(cuda_device, 31 + Hkv + W, B, Hkv, G, W, BS, mb, seq)
    sink, recent = 128, 200
    want = ref_cuda.hamming_score(codes_ref, q, bt, sl, mb * BS, sink, recent, reduce_kvhead)
    got = ops.hamming_score(codes, q, bt, sl, mb * BS, sink, recent, reduce_kvhead)
    torch.cuda.synchronize()
    assert want.shape == got.shape and want.dtype == got.dtype
    # bit-exact fp16, +inf past the request's end included.  (The reference adds the per-word counts in fp16,
    # which is exact while a token's sum stays <= 2048 - true for every shape here.)
    assert torch.equal(want.view(torch.int16), got.view(torch.int16))


@pytest.mark.parametrize("Hkv,G,W,is_mla", [(1, 8, 4, True), (8, 4, 4, False), (8, 1, 4, False)])
def test_selection_matches_reference_pipeline(cuda_device, ref_cuda, Hkv, G, W, is_mla):
    """hamming_score -> block min -> topk -> sort -> block-table gather (hamming_topk.py:33-54) against the
    fused retrieval.  torch.topk leaves the order of equal scores open, so the comparison is on the selected
    blocks' scores (a multiset) and on every block that is strictly better than the k-th."""
    import torch
    from unified_cache_management_b200 import hamming_topk as HT
    B, BS, mb, k = 4, 128, 40, 8
    seq = [mb * BS, 33 * BS + 5, 20 * BS, 9 * BS + 127]
    codes, codes_ref, q, bt, sl = _case(cuda_device, 57 + Hkv, B, Hkv, G, W, BS, mb, seq)
    sink, recent = 128, 256
    reduce_kvhead = (not is_mla) and Hkv > 1
    per_token = ref_cuda.hamming_score(codes_ref, q, bt, sl, mb * BS, sink, recent, reduce_kvhead)
    block = per_token.view(B, mb, BS).min(dim=-1)[0].float()
    ind = torch.sort(torch.topk(block, k=k, dim=-1, largest=False)[1], dim=-1)[0]
    want_phys = torch.gather(bt, -1, ind)
    got_phys = HT.cuda_hamming_topk(q, codes, bt, sl, k * BS, sink, recent, is_mla)
    torch.cuda.synchronize()
    assert got_phys.shape == want_phys.shape
    block, bt_c = block.cpu().numpy(), bt.cpu().numpy()
    for b in range(B):
        nb = (seq[b] + BS - 1) // BS
        phys_to_logical = {int(bt_c[b, j]): j for j in range(nb)}
        got_logical = [phys_to_logical[int(p)] for p in got_phys[b].cpu().tolist()]
        assert got_logical == sorted(got_logical) and len(set(got_logical)) == k
        want_scores = np.sort(block[b, ind[b].cpu().numpy()])
        got_scores = np.sort(block[b, got_logical])
        assert np.array_equal(want_scores, got_scores)
        kth = want_scores[-1]
        assert set(np.nonzero(block[b, :nb] < kth)[0].tolist()) <= set(got_logical)

"""Golden fixture for the float block-retrieval kernels, made with the torch statements the reference plugins run.

    python tests/golden/make_golden_float.py

* block representations: ``k_cache[vllm_block_ids].mean(1)`` (ucm/sparse/esa/esa.py:254-263, non-MLA branch) and
  ``k_cache.reshape(n, M, c, h, d).mean(dim=2)`` (ucm/sparse/kvstar/multistep.py:322-327), evaluated by torch on CPU
  in bf16 exactly as the plugins call them;
* retrieval: the reference's worker (ucm/sparse/esa/retrieval/cpy/retrieval_backend.cpp:206-225) cannot be compiled
  in the build container (it needs libnuma's ``numaif.h``), so its loop is restated here with float32 numpy: score =
  sum_d q[d] * data[idx, d] over the request's allowed indexes, the top-k by descending score.  The fixture stores the
  scores of every candidate so that a test can compare selections up to float rounding.
"""
import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    g = torch.Generator().manual_seed(7)
    NB, BS, H, D = 10, 16, 2, 32
    k_cache = torch.randn((NB, BS, H, D), generator=g).to(torch.bfloat16)
    ids = torch.tensor([7, 0, 3, 9, 4, 1], dtype=torch.int64)
    repr_esa = k_cache[ids].mean(1)                                          # [n, H, D] bf16
    blk = k_cache[ids]
    n, S, h, d = blk.shape
    c = 4
    repr_kvstar = blk.reshape(n, S // c, c, h, d).mean(dim=2)                # [n, M, H, D] bf16
    pool = k_cache.mean(1).reshape(NB, H * D)                                # representation of every block
    B, k = 3, 4
    q = torch.randn((B, H * D), generator=g).to(torch.bfloat16)
    indexes = np.full((B, 8), -1, dtype=np.int32)
    indexes[0, :8] = [9, 2, 5, 0, 7, 1, 3, 8]
    indexes[1, :5] = [4, 6, 2, 9, 1]
    indexes[2, :3] = [8, 3, 0]                                               # fewer candidates than k
    data = pool.float().numpy()
    qf = q.float().numpy()
    scores = np.full(indexes.shape, -np.inf, dtype=np.float32)
    top_ids = np.full((B, k), -1, dtype=np.int32)
    for b in range(B):
        allowed = [int(i) for i in indexes[b] if i >= 0]
        for pos, idx in enumerate(allowed):
            s = np.float32(0.0)
            for dd in range(data.shape[1]):
                s = np.float32(s + qf[b, dd] * data[idx, dd])
            scores[b, pos] = s
        order = sorted(range(len(allowed)), key=lambda p: -scores[b, p])[:k]
        top_ids[b, :len(order)] = [allowed[p] for p in order]
    u16 = lambda t: t.contiguous().view(torch.int16).numpy().view(np.uint16)
    np.savez_compressed(os.path.join(HERE, "float_retrieval.npz"), k_cache=u16(k_cache), block_ids=ids.numpy().astype(np.int32),
                        repr_esa=u16(repr_esa), repr_kvstar=u16(repr_kvstar), merge=np.int32(c), pool=u16(pool), q=u16(q),
                        indexes=indexes, scores=scores, top_ids=top_ids, k=np.int32(k))
    print("wrote float_retrieval.npz")


if __name__ == "__main__":
    main()

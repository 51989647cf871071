"""Generates the golden fixtures in this directory from the REFERENCE project's own Python code.

Run in a checkout where the reference tree is available:

    python tests/golden/make_golden.py [/path/to/reference]

It imports (never copies) these reference modules and runs them on CPU with seeded inputs:

* ``ucm/sparse/gsa_on_device/hash_encoder.py``: ``torch_hash_code`` (eager form of the CPU encode,
  :359-370), ``HashEncoder._unpack_hash`` (:664-724) and the bit masks (:445-448);
* ``ucm/sparse/gsa_on_device/hamming_topk.py``: ``update_seq_lens`` (:7-12) and
  ``cuda_hamming_topk`` (:15-54), whose CUDA op is replaced by a stand-in that returns per-token
  scores computed with the reference's own +-1/einsum formulation
  (``csrc/cuda/hash_retrieval/hash_retrieval_worker.py:102-119``: similarity = <unpack(q), unpack(k)>,
  distance = (bits - similarity)/2) and the sink/recent/inf rule of ``paged_ham_dist_mla.cu:194-197``.

The fixtures are small ``.npz`` files; the tests compare the oracle (and through it the CUDA
kernels) with them.  Nothing in the test-suite needs the reference tree at run time.
"""
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("UCM_REFERENCE_ROOT")
if not REF:
    raise SystemExit("usage: make_golden.py <reference checkout>   (or set UCM_REFERENCE_ROOT)")


def _load(name, rel):
    spec = importlib.util.spec_from_file_location(name, os.path.join(REF, rel))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main():
    import logging
    stub = types.ModuleType("ucm.logger")
    stub.init_logger = lambda name: logging.getLogger(name)
    sys.modules.setdefault("ucm", types.ModuleType("ucm"))
    sys.modules["ucm.logger"] = stub
    he = _load("ref_hash_encoder", "ucm/sparse/gsa_on_device/hash_encoder.py")
    ht = _load("ref_hamming_topk", "ucm/sparse/gsa_on_device/hamming_topk.py")
    eager_hash = getattr(he.torch_hash_code, "_torchdynamo_orig_callable", he.torch_hash_code)

    # ---- 1. encode ---------------------------------------------------------------------------
    g = torch.Generator().manual_seed(1)
    R = (torch.randn(128, 128, generator=g) / 128 ** 0.5).to(torch.bfloat16)
    X = torch.randn(192, 128, generator=g).to(torch.bfloat16)
    enc = he.HashEncoder(128, 128, torch.float32, torch.device("cpu"))
    enc.set_hash_weight(R.float())
    codes_f32 = eager_hash(X.float(), enc.hash_weights, enc.bit_masks)            # uint8 [192,16]
    codes_bf16 = eager_hash(X, R, enc.bit_masks)                                   # bf16 matmul variant
    np.savez_compressed(os.path.join(HERE, "encode.npz"),
                        x_bf16=X.view(torch.int16).numpy().view(np.uint16),
                        r_bf16=R.view(torch.int16).numpy().view(np.uint16),
                        codes_u8_f32=codes_f32.numpy(), codes_u8_bf16=codes_bf16.numpy(),
                        bit_masks=enc.bit_masks.numpy())

    # query path of the plugin: mean over the group in bf16, then encode (gsa_on_device.py:400-412)
    Q = torch.randn(6, 32, 128, generator=g).to(torch.bfloat16)
    qm = Q.view(6, 8, 4, 128).mean(2)
    q_codes = eager_hash(qm.float().reshape(-1, 128), enc.hash_weights, enc.bit_masks)
    np.savez_compressed(os.path.join(HERE, "encode_query.npz"),
                        q_bf16=Q.view(torch.int16).numpy().view(np.uint16),
                        qmean_bf16=qm.contiguous().view(torch.int16).numpy().view(np.uint16),
                        codes_u8=q_codes.numpy().reshape(6, 8, 16))

    # ---- 2. distances by the reference's +-1 / einsum formulation -------------------------------
    g = torch.Generator().manual_seed(2)
    NB, BS, Hkv, G, nbytes = 24, 16, 4, 2, 16
    key_u8 = torch.randint(0, 256, (NB, BS, Hkv, nbytes), generator=g, dtype=torch.uint8)
    B, mb = 3, 7
    q_u8 = torch.randint(0, 256, (B, Hkv * G, nbytes), generator=g, dtype=torch.uint8)
    perm = torch.randperm(NB, generator=g)
    bt = torch.zeros(B, mb, dtype=torch.int32)
    seq = torch.tensor([mb * BS, 3 * BS + 5, 1 * BS + 1], dtype=torch.int32)
    off = 0
    for b in range(B):
        n = (int(seq[b]) + BS - 1) // BS
        bt[b, :n] = perm[off:off + n].to(torch.int32)
        off += n
    uk = enc._unpack_hash(key_u8).float()           # [NB,BS,Hkv,128]  +-1
    uq = enc._unpack_hash(q_u8).float()             # [B,Hq,128]
    bits = nbytes * 8
    # per request: gather the request's blocks, similarity per (token, kv head, group member)
    dist = torch.full((B, Hkv, mb * BS), -1, dtype=torch.int32)
    for b in range(B):
        kk = uk[bt[b].long()].reshape(mb * BS, Hkv, bits)                     # logical token order
        sim = torch.einsum("thd,hgd->thg", kk, uq[b].view(Hkv, G, bits))      # [tokens,Hkv,G]
        d = ((bits - sim) / 2).sum(-1).to(torch.int32).T                      # [Hkv,tokens]
        dist[b, :, :int(seq[b])] = d[:, :int(seq[b])]
    np.savez_compressed(os.path.join(HERE, "distances.npz"), key_u8=key_u8.numpy(), q_u8=q_u8.numpy(),
                        block_table=bt.numpy(), seq_lens=seq.numpy(), dist=dist.numpy(),
                        meta=np.array([NB, BS, Hkv, G, nbytes, B, mb]))

    # ---- 3. update_seq_lens --------------------------------------------------------------------
    s = torch.tensor([0, 1, 127, 128, 129, 2047, 2048, 2049, 4096, 5000, 131072, 131073], dtype=torch.int32)
    rows = []
    for topk, bs in ((2048, 128), (2048, 16), (512, 64), (128, 128)):
        rows.append(ht.update_seq_lens(s, topk, bs).numpy())
    np.savez_compressed(os.path.join(HERE, "update_seq_lens.npz"), seq_lens=s.numpy(), out=np.stack(rows),
                        params=np.array([(2048, 128), (2048, 16), (512, 64), (128, 128)]))

    # ---- 4. cuda_hamming_topk with the CUDA op replaced by the formulation of (2) ----------------
    class _FakeHamming:
        @staticmethod
        def hamming_score(k_hash, q_hash, block_table, seq_lens, max_seqlen, sink, recent, reduce_kvhead):
            kb = k_hash.view(torch.uint8)       # [NB,BS,Hkv,nbytes]
            qb = q_hash.view(torch.uint8)       # [B,1,Hq,nbytes]
            nb_, bs_, hkv_, nby = kb.shape
            b_, _, hq_, _ = qb.shape
            g_ = hq_ // hkv_
            bits_ = nby * 8
            e = he.HashEncoder(bits_, bits_, torch.float32, torch.device("cpu"))
            uk_ = e._unpack_hash(kb.contiguous()).float()
            uq_ = e._unpack_hash(qb.contiguous()).float()
            out = torch.empty(b_, 1 if reduce_kvhead else hkv_, max_seqlen, dtype=torch.float16)
            pos = torch.arange(max_seqlen)
            for b in range(b_):
                kk = uk_[block_table[b].long()].reshape(max_seqlen, hkv_, bits_)
                sim = torch.einsum("thd,hgd->thg", kk, uq_[b, 0].view(hkv_, g_, bits_))
                d = ((bits_ - sim) / 2).sum(-1).T                     # [Hkv, tokens]
                if reduce_kvhead:
                    d = d.min(0, keepdim=True).values
                sl = int(seq_lens[b])
                d = torch.where((pos < sink) | ((pos >= sl - recent) & (pos < sl)), torch.zeros(()), d)
                d = torch.where(pos >= sl, torch.full((), float("inf")), d)
                out[b] = d.to(torch.float16)
            return out

    ht.hamming = _FakeHamming
    g = torch.Generator().manual_seed(3)
    NB, BS, Hkv, nbytes, B, mb = 80, 16, 2, 16, 3, 24
    key_u8 = torch.randint(0, 256, (NB, BS, Hkv, nbytes), generator=g, dtype=torch.uint8)
    q_u8 = torch.randint(0, 256, (B, Hkv, nbytes), generator=g, dtype=torch.uint8)   # one code per kv head
    perm = torch.randperm(NB, generator=g)
    seq = torch.tensor([mb * BS, 20 * BS + 3, 13 * BS], dtype=torch.int32)
    bt = torch.zeros(B, mb, dtype=torch.int32)
    off = 0
    for b in range(B):
        n = (int(seq[b]) + BS - 1) // BS
        bt[b, :n] = perm[off:off + n].to(torch.int32)
        off += n
    topk_token, sink, recent = 8 * BS, BS, 4 * BS
    sel = ht.cuda_hamming_topk(q_u8.unsqueeze(1).view(torch.bfloat16), key_u8.view(torch.bfloat16), bt, seq,
                               topk_token, sink, recent, False)
    score = _FakeHamming.hamming_score(key_u8, q_u8.unsqueeze(1), bt, seq, mb * BS, sink, recent, True)
    blk = torch.min(score.view(B, mb, BS), dim=-1)[0]
    np.savez_compressed(os.path.join(HERE, "topk_tail.npz"), key_u8=key_u8.numpy(), q_u8=q_u8.numpy(),
                        block_table=bt.numpy(), seq_lens=seq.numpy(), selected_physical=sel.numpy(),
                        block_scores_f16=blk.numpy(), params=np.array([topk_token, sink, recent, BS]))
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))


if __name__ == "__main__":
    main()

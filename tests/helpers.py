"""Seeded synthetic inputs shared by the tests (shapes follow the benchmark configs)."""
from __future__ import annotations

import numpy as np


def rand_codes(rng, shape):
    return rng.integers(0, 2**32, size=shape, dtype=np.uint32)


def make_paged_case(seed, B, Hkv, G, W, BS, max_blocks, seq_lens=None, pool_extra=7, identity=False):
    """Returns dict of numpy arrays: codes [NB,BS,Hkv,W], q [B,Hq,W], block_table [B,max_blocks], seq_lens [B].

    Each request owns distinct physical blocks drawn from one permutation of the pool; unused
    block-table entries are 0 (the padding value vLLM uses).
    """
    rng = np.random.default_rng(seed)
    if seq_lens is None:
        seq_lens = rng.integers(1, max_blocks * BS + 1, size=B)
    seq_lens = np.asarray(seq_lens, dtype=np.int32)
    nblk = (seq_lens + BS - 1) // BS
    NB = int(nblk.sum()) + pool_extra
    perm = np.arange(NB) if identity else rng.permutation(NB)
    bt = np.zeros((B, max_blocks), dtype=np.int32)
    off = 0
    for b in range(B):
        bt[b, :nblk[b]] = perm[off:off + nblk[b]]
        off += nblk[b]
    codes = rand_codes(rng, (NB, BS, Hkv, W))
    q = rand_codes(rng, (B, Hkv * G, W))
    return dict(codes=codes, q=q, block_table=bt, seq_lens=seq_lens, NB=NB)


def bf16_normal(rng, shape, scale=1.0):
    """N(0,1)*scale rounded to bf16, returned as uint16 bit patterns."""
    from oracle import oracle as O
    return O.f32_to_bf16_bits((rng.standard_normal(shape) * scale).astype(np.float32))


def to_dev_i32(a, device):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int32) if a.dtype == np.uint32 else np.ascontiguousarray(a)).to(device)


def bf16_to_dev(u16, device):
    import torch
    return torch.from_numpy(np.ascontiguousarray(u16).view(np.int16)).to(device).view(torch.bfloat16)


def dev_to_u32(t):
    return t.detach().cpu().numpy().view(np.uint32)

"""The reference's ``hamming_topk`` module interface on top of the sm_100a kernels.

Mirrors ``ucm/sparse/gsa_on_device/hamming_topk.py``: ``update_seq_lens`` (:7-12),
``cuda_hamming_topk`` (:15-54, same arguments, same asserts, returns the [B, k] physical block ids in
ascending logical order) and ``fake_hamming_topk`` (:57-76).  The per-token score tensor of the
reference is never materialised: scan + block-min + top-k + sort + block-table lookup run as two
launches inside ``ops.hamming_topk``.  Ties, which ``torch.topk`` leaves unspecified, go to the
lower block id.
"""
from __future__ import annotations

import torch

from . import ops


def update_seq_lens(seq_lens, topk_token, block_size):
    if isinstance(seq_lens, torch.Tensor) and seq_lens.is_cuda and seq_lens.dtype == torch.int32 \
            and seq_lens.is_contiguous():
        return ops.update_seq_lens(seq_lens, topk_token, block_size)
    # host-side bookkeeping (scheduler role) keeps the reference's arithmetic
    drop_block_num = ((seq_lens - topk_token).clip(min=0) + block_size - 1) // block_size
    return seq_lens - drop_block_num * block_size


def cuda_hamming_topk(q_hash, k_hash, block_table, seq_lens, topk_token, sink_token, recent_token, is_mla,
                      workspace=None):
    q_words = ops.as_words(q_hash)
    k_words = ops.as_words(k_hash)
    block_size = k_words.shape[1]
    assert topk_token % block_size == 0
    assert recent_token > 0 and topk_token > (sink_token + recent_token)
    if q_words.dim() == 4:  # [B, 1, Hq, W] as the plugin passes it
        q_words = q_words.reshape(q_words.shape[0], q_words.shape[2], q_words.shape[3])
    reduce_kvhead = (not is_mla) and (k_words.size(2) > 1)
    if not reduce_kvhead and k_words.size(2) != 1:
        raise ValueError("per-kv-head selection is not what this entry returns; call ops.hamming_topk")
    out = ops.hamming_topk(k_words, q_words, block_table, seq_lens, topk_token // block_size, reduce="min",
                           reduce_kvhead=reduce_kvhead, sink_tokens=sink_token, recent_tokens=recent_token,
                           workspace=workspace, want_scores=False)
    return out.physical[:, 0, :]


def fake_hamming_topk(q_hash, k_hash, block_table, seq_lens, topk_token, sink_token, recent_token):
    k_words = ops.as_words(k_hash)
    block_size = k_words.shape[1]
    assert topk_token % block_size == 0
    assert recent_token > 0 and topk_token > (sink_token + recent_token)
    return block_table[:, : topk_token // block_size]

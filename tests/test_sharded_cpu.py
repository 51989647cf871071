"""World-size-2 gloo test of the sequence-sharded retrieval plumbing on CPU ranks.

The compute functions are replaced by the oracle (the CUDA kernels have no CPU form); what is tested
is the shard plan, the single all-gather of packed records and that the merged result equals the
unsharded retrieval on every rank.
"""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle as O
        from tests import helpers as H
        from unified_cache_management_b200 import sharded
        B, Hkv, G, W, BS, nblk, k = 2, 2, 2, 4, 8, 16, 5
        seq = np.array([nblk * BS, nblk * BS - 2 * BS - 3], dtype=np.int32)
        case = H.make_paged_case(7, B, Hkv, G, W, BS, nblk, seq_lens=seq)
        must = (0, -2, -1)
        per = nblk // world

        def cand(codes, q, bt, sl_local, sl_global, kl, off, scale, **kw):
            forced = np.stack([O.forced_blocks(int(sl_global[b]), BS, nblk, kw["must_select"])[off:off + per]
                               for b in range(B)])
            s, i = O.topk_candidates(codes, q.numpy().view(np.uint32), bt.numpy(), sl_local.numpy(), kl, off, scale,
                                     forced, O.REDUCE_SUM, kw["reduce_kvhead"])
            return torch.from_numpy(s), torch.from_numpy(i)

        def merge(cs, ci, kk):
            s, i = O.merge_topk(cs.numpy(), ci.numpy(), kk)
            return torch.from_numpy(s), torch.from_numpy(i)

        bt_local = torch.from_numpy(np.ascontiguousarray(case["block_table"][:, rank * per:(rank + 1) * per]))
        q = torch.from_numpy(case["q"].view(np.int32))
        s, ids = sharded.sharded_hamming_topk(case["codes"], q, bt_local, torch.from_numpy(seq), k, BS, nblk,
                                              1.0 / (BS * G), must_select=must, candidates_fn=cand, merge_fn=merge)
        full = O.hamming_topk(case["codes"], case["q"], case["block_table"], seq, k, O.REDUCE_SUM, False,
                              must_select=must)
        ok = np.array_equal(ids.numpy(), full["logical"])
        plan = sharded.shard_plan(torch.from_numpy(seq), BS, nblk, world, rank)
        ok = ok and plan.block_offset == rank * per and int(plan.seq_lens_local.sum()) == int(
            np.clip(seq - rank * per * BS, 0, per * BS).sum())
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_sharded_retrieval_two_cpu_ranks():
    world = 2
    port = 29500 + os.getpid() % 2000
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        assert dict(ret) == {0: True, 1: True}


def test_shard_plan_rejects_uneven_split():
    from unified_cache_management_b200 import sharded
    with pytest.raises(ValueError):
        sharded.shard_plan(torch.tensor([100], dtype=torch.int32), 8, 15, 2, 0)

"""Two-GPU test of the sequence-sharded retrieval over NCCL (skipped with fewer than two devices).

Each rank scans its half of the logical blocks with the CUDA kernels, the (score, id) records travel with one
`all_gather_into_tensor`, and the merged global top-k must equal the unsharded oracle on both ranks.
"""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dev = torch.device(f"cuda:{rank}")
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from oracle import oracle as O
        from tests import helpers as H
        from unified_cache_management_b200 import ops as ops_mod
        from unified_cache_management_b200 import sharded
        B, Hkv, G, W, BS, nblk, k = 2, 8, 4, 8, 64, 256, 24
        seq = np.array([nblk * BS, nblk * BS - 5 * BS - 7], dtype=np.int32)
        case = H.make_paged_case(17, B, Hkv, G, W, BS, nblk, seq_lens=seq)
        must = (0, -2, -1)
        per = nblk // world
        bt_local = H.to_dev_i32(np.ascontiguousarray(case["block_table"][:, rank * per:(rank + 1) * per]), dev)
        s, ids = sharded.sharded_hamming_topk(H.to_dev_i32(case["codes"], dev), H.to_dev_i32(case["q"], dev), bt_local,
                                              H.to_dev_i32(seq, dev), k, BS, nblk, 1.0 / (BS * G), must_select=must)
        torch.cuda.synchronize()
        full = O.hamming_topk(case["codes"], case["q"], case["block_table"], seq, k, O.REDUCE_SUM, False,
                              must_select=must)
        ok = bool(np.array_equal(ids.cpu().numpy(), full["logical"]))
        # the same through peer memory: records stored into every rank's buffer over NVLink, no collective
        ex = sharded.PeerExchange(B, Hkv, min(k, per), dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        for _ in range(3):   # three steps: both buffer parities and a reuse
            s2, ids2 = sharded.sharded_hamming_topk_p2p(H.to_dev_i32(case["codes"], dev), H.to_dev_i32(case["q"], dev),
                                                        bt_local, H.to_dev_i32(seq, dev), k, BS, nblk, 1.0 / (BS * G),
                                                        ex, must_select=must, status=status)
            torch.cuda.synchronize()
            ok = ok and bool(np.array_equal(ids2.cpu().numpy(), full["logical"])) and int(status.item()) == 0
            ok = ok and bool(torch.equal(s2, s))
        # the same step captured once in a CUDA graph and replayed: the step number is counted on the device, so
        # every replay publishes / waits for a new number (a by-value number would be frozen by the capture)
        codes_d, q_d, seq_d = H.to_dev_i32(case["codes"], dev), H.to_dev_i32(case["q"], dev), H.to_dev_i32(seq, dev)
        ws = ops_mod.new_workspace(B, Hkv, per, dev)
        plan = sharded.shard_plan(seq_d, BS, nblk, world, rank)
        o_s = torch.empty((B, Hkv, k), dtype=torch.float32, device=dev)
        o_i = torch.empty((B, Hkv, k), dtype=torch.int32, device=dev)
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        torch.cuda.synchronize()
        dist.barrier()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                sharded.sharded_hamming_topk_p2p(codes_d, q_d, bt_local, seq_d, k, BS, nblk, 1.0 / (BS * G), ex,
                                                 must_select=must, status=status, workspace=ws, plan=plan,
                                                 out_scores=o_s, out_ids=o_i)
        torch.cuda.synchronize()
        dist.barrier()
        for rep in range(4):
            o_i.fill_(-5)
            graph.replay()
            torch.cuda.synchronize()
            ok = ok and bool(np.array_equal(o_i.cpu().numpy(), full["logical"])) and int(status.item()) == 0
        ok = ok and ex.state.cpu().tolist() == [3 + 4, 0]
        ret[rank] = ok
    finally:
        dist.destroy_process_group()


def test_sharded_retrieval_two_gpus(cuda_device):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    port = 29600 + os.getpid() % 2000
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        assert dict(ret) == {0: True, 1: True}

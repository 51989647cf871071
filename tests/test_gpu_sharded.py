"""GPU parity: sequence-sharded retrieval (local candidates + merge) on one device.

The shards are processed one after the other on the same GPU and their records concatenated the way
an all-gather would deliver them; the merged result must equal the unsharded top-k.
"""
import numpy as np
import pytest

from oracle import oracle as O
from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("R", [2, 8])
@pytest.mark.parametrize("reduce_kvhead", [False, True])
def test_sharded_equals_unsharded(cuda_device, R, reduce_kvhead):
    import torch
    from unified_cache_management_b200 import ops
    dev = cuda_device
    B, Hkv, G, W, BS = 2, 8, 4, 8, 64
    nblk = 64 * R
    k = 24
    seq = np.array([nblk * BS, nblk * BS - 3 * BS - 5], dtype=np.int32)   # second request is ragged
    case = H.make_paged_case(40 + R, B, Hkv, G, W, BS, nblk, seq_lens=seq)
    must = (0, -2, -1)
    scale = 1.0 / (BS * G)
    codes, q = H.to_dev_i32(case["codes"], dev), H.to_dev_i32(case["q"], dev)
    seq_g = H.to_dev_i32(seq, dev)
    per = nblk // R
    cs, ci = [], []
    for r in range(R):
        bt_local = np.ascontiguousarray(case["block_table"][:, r * per:(r + 1) * per])
        seq_local = np.clip(seq - r * per * BS, 0, per * BS).astype(np.int32)
        s, i = ops.topk_candidates(codes, q, H.to_dev_i32(bt_local, dev), H.to_dev_i32(seq_local, dev), seq_g, k,
                                   r * per, scale, reduce="sum", reduce_kvhead=reduce_kvhead, must_select=must)
        # oracle for the shard
        forced = np.stack([O.forced_blocks(seq[b], BS, nblk, must)[r * per:(r + 1) * per] for b in range(B)])
        ws, wi = O.topk_candidates(case["codes"], case["q"], bt_local, seq_local, k, r * per, scale, forced,
                                   O.REDUCE_SUM, reduce_kvhead)
        torch.cuda.synchronize()
        assert np.array_equal(i.cpu().numpy(), wi)
        assert np.array_equal(s.cpu().numpy().view(np.uint32), ws.view(np.uint32))
        cs.append(s)
        ci.append(i)
    ms, mi = ops.merge_topk(torch.stack(cs), torch.stack(ci), k)
    torch.cuda.synchronize()
    full = O.hamming_topk(case["codes"], case["q"], case["block_table"], seq, k, O.REDUCE_SUM, reduce_kvhead,
                          must_select=must)
    assert np.array_equal(mi.cpu().numpy(), full["logical"])
    ws, wi = O.merge_topk(np.stack([c.cpu().numpy() for c in cs]), np.stack([c.cpu().numpy() for c in ci]), k)
    assert np.array_equal(mi.cpu().numpy(), wi)
    assert np.array_equal(ms.cpu().numpy().view(np.uint32), ws.view(np.uint32))


def test_merge_with_short_shards(cuda_device):
    """Shards that hold fewer than k blocks pad with (+inf, -1); padding never wins over a real record."""
    import torch
    from unified_cache_management_b200 import ops
    rng = np.random.default_rng(5)
    R, B, Hh, kl, k = 4, 2, 3, 16, 20
    sc = rng.integers(0, 50, size=(R, B, Hh, kl)).astype(np.float32) / 8
    ids = np.sort(rng.permutation(1000)[:R * kl]).reshape(R, 1, 1, kl).repeat(B, 1).repeat(Hh, 2).astype(np.int32)
    sc[1, :, :, 5:] = np.inf
    ids = ids.copy()
    ids[1, :, :, 5:] = -1
    sc[3, 0] = np.inf
    ids[3, 0] = -1
    ms, mi = ops.merge_topk(torch.from_numpy(sc).to(cuda_device), torch.from_numpy(ids).to(cuda_device), k)
    torch.cuda.synchronize()
    ws, wi = O.merge_topk(sc, ids, k)
    assert np.array_equal(mi.cpu().numpy(), wi)
    assert np.array_equal(ms.cpu().numpy().view(np.uint32), ws.view(np.uint32))


def test_long_shards_cluster_candidates(cuda_device):
    """Shards of 4500 blocks each: the candidate selection runs split over thread-block clusters."""
    import torch
    from unified_cache_management_b200 import ops
    dev = cuda_device
    B, Hkv, G, W, BS, R, per, k = 2, 2, 2, 4, 16, 2, 4500, 256
    nblk = R * per
    seq = np.array([nblk * BS, nblk * BS - 700 * BS - 9], dtype=np.int32)
    case = H.make_paged_case(91, B, Hkv, G, W, BS, nblk, seq_lens=seq)
    must = (0, 1, -1)
    scale = 1.0 / (BS * G)
    codes, q = H.to_dev_i32(case["codes"], dev), H.to_dev_i32(case["q"], dev)
    cs, ci = [], []
    for r in range(R):
        bt_local = np.ascontiguousarray(case["block_table"][:, r * per:(r + 1) * per])
        seq_local = np.clip(seq - r * per * BS, 0, per * BS).astype(np.int32)
        s, i = ops.topk_candidates(codes, q, H.to_dev_i32(bt_local, dev), H.to_dev_i32(seq_local, dev),
                                   H.to_dev_i32(seq, dev), k, r * per, scale, reduce="sum", must_select=must)
        forced = np.stack([O.forced_blocks(seq[b], BS, nblk, must)[r * per:(r + 1) * per] for b in range(B)])
        ws, wi = O.topk_candidates(case["codes"], case["q"], bt_local, seq_local, k, r * per, scale, forced,
                                   O.REDUCE_SUM, False)
        torch.cuda.synchronize()
        assert np.array_equal(i.cpu().numpy(), wi)
        assert np.array_equal(s.cpu().numpy().view(np.uint32), ws.view(np.uint32))
        cs.append(s)
        ci.append(i)
    ms, mi = ops.merge_topk(torch.stack(cs), torch.stack(ci), k)
    torch.cuda.synchronize()
    full = O.hamming_topk(case["codes"], case["q"], case["block_table"], seq, k, O.REDUCE_SUM, False, must_select=must)
    assert np.array_equal(mi.cpu().numpy(), full["logical"])


@pytest.mark.parametrize("R,blocks_per_rank", [(2, 48), (4, 48), (8, 12)])
def test_peer_memory_exchange_emulated_on_one_gpu(cuda_device, R, blocks_per_rank):
    """The collective-free exchange with the ranks emulated one after the other on one GPU: every rank's
    selection writes its records into all R gather buffers and publishes the step number, then every rank's
    merge (launched after all selections, so nothing waits for a later launch) must equal the unsharded top-k.
    Two steps, to exercise the alternating buffers."""
    import torch
    from unified_cache_management_b200 import ops
    dev = cuda_device
    B, Hkv, G, W, BS, k = 2, 4, 2, 4, 32, 20
    nblk = blocks_per_rank * R
    per = nblk // R
    kl = min(k, per)              # a rank holding fewer than k blocks sends all of them
    slab = B * Hkv * kl
    bufs_s = [[torch.zeros((R, B, Hkv, kl), dtype=torch.float32, device=dev) for _ in range(R)] for _ in range(2)]
    bufs_i = [[torch.zeros((R, B, Hkv, kl), dtype=torch.int32, device=dev) for _ in range(R)] for _ in range(2)]
    flags = [[torch.zeros((R,), dtype=torch.int32, device=dev) for _ in range(R)] for _ in range(2)]
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    for step in (1, 2, 3):
        par = step & 1
        seq = np.array([nblk * BS - step, nblk * BS - 9 * BS - 3], dtype=np.int32)
        case = H.make_paged_case(300 + step, B, Hkv, G, W, BS, nblk, seq_lens=seq)
        codes, q = H.to_dev_i32(case["codes"], dev), H.to_dev_i32(case["q"], dev)
        seq_g = H.to_dev_i32(seq, dev)
        must = (0, -1)
        for r in range(R):
            bt_local = H.to_dev_i32(np.ascontiguousarray(case["block_table"][:, r * per:(r + 1) * per]), dev)
            seq_local = H.to_dev_i32(np.clip(seq - r * per * BS, 0, per * BS).astype(np.int32), dev)
            ps = [bufs_s[par][d].data_ptr() + 4 * r * slab for d in range(R)]
            pi = [bufs_i[par][d].data_ptr() + 4 * r * slab for d in range(R)]
            pf = [flags[par][d].data_ptr() + 4 * r for d in range(R)]
            ops.topk_candidates_p2p(codes, q, bt_local, seq_local, seq_g, kl, r * per, 1.0 / (BS * G), ps, pi, pf, step,
                                    must_select=must)
        full = O.hamming_topk(case["codes"], case["q"], case["block_table"], seq, k, O.REDUCE_SUM, False,
                              must_select=must)
        for d in range(R):
            ms, mi = ops.merge_topk_wait(bufs_s[par][d], bufs_i[par][d], k, flags[par][d], step, status=status)
            torch.cuda.synchronize()
            assert flags[par][d].cpu().tolist() == [step] * R
            assert np.array_equal(mi.cpu().numpy(), full["logical"])
        assert int(status.item()) == 0


@pytest.mark.parametrize("R", [2, 8])
def test_peer_exchange_step_word_survives_graph_replay(cuda_device, R):
    """The replay-safe exchange (step number counted in a device word) with the ranks emulated on one GPU: all
    selections, then all merges, captured ONCE in a CUDA graph and replayed with new query codes each time.  A
    by-value step number would be frozen by the capture; here every replay publishes and waits for the next number
    and alternates the buffer parity by itself."""
    import torch
    from unified_cache_management_b200 import ops
    dev = cuda_device
    B, Hkv, G, W, BS, k, per = 2, 4, 2, 4, 32, 20, 24
    nblk = per * R
    kl = min(k, per)
    slab = B * Hkv * kl
    words = 2 * R * slab + 64                                   # one parity: scores | ids | flags (padded)
    bufs = [torch.zeros(2 * words, dtype=torch.int32, device=dev) for _ in range(R)]   # rank d's exchange buffer
    states = [torch.zeros(2, dtype=torch.int32, device=dev) for _ in range(R)]
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    seq = np.array([nblk * BS - 1, nblk * BS - 9 * BS - 3], dtype=np.int32)
    case = H.make_paged_case(500 + R, B, Hkv, G, W, BS, nblk, seq_lens=seq)
    codes = H.to_dev_i32(case["codes"], dev)
    q = H.to_dev_i32(case["q"], dev)
    seq_g = H.to_dev_i32(seq, dev)
    must = (0, -1)
    bt_local = [H.to_dev_i32(np.ascontiguousarray(case["block_table"][:, r * per:(r + 1) * per]), dev) for r in range(R)]
    seq_local = [H.to_dev_i32(np.clip(seq - r * per * BS, 0, per * BS).astype(np.int32), dev) for r in range(R)]
    wss = [ops.new_workspace(B, Hkv, per, dev) for _ in range(R)]
    outs = [(torch.empty((B, Hkv, k), dtype=torch.float32, device=dev),
             torch.empty((B, Hkv, k), dtype=torch.int32, device=dev)) for _ in range(R)]

    def all_ranks_one_step():
        for r in range(R):
            ps, pi, pf = [], [], []
            for par in (0, 1):
                base = par * words
                ps += [bufs[d].data_ptr() + 4 * (base + r * slab) for d in range(R)]
                pi += [bufs[d].data_ptr() + 4 * (base + R * slab + r * slab) for d in range(R)]
                pf += [bufs[d].data_ptr() + 4 * (base + 2 * R * slab + r) for d in range(R)]
            ops.topk_candidates_p2p_step(codes, q, bt_local[r], seq_local[r], seq_g, kl, r * per, 1.0 / (BS * G),
                                         ps, pi, pf, states[r][0:1], must_select=must, workspace=wss[r])
        for d in range(R):
            sc = bufs[d][0:R * slab].view(torch.float32).view(R, B, Hkv, kl)
            ids = bufs[d][R * slab:2 * R * slab].view(R, B, Hkv, kl)
            flags = bufs[d][2 * R * slab:2 * R * slab + R]
            ops.merge_topk_wait_step(sc, ids, k, flags, words, words, states[d], status=status,
                                     out_scores=outs[d][0], out_ids=outs[d][1])

    all_ranks_one_step()                                         # warm-up outside the capture: step 1
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            all_ranks_one_step()
    torch.cuda.synchronize()
    rng = np.random.default_rng(9)
    for step in (2, 3, 4):
        qh = H.rand_codes(rng, case["q"].shape)
        q.copy_(H.to_dev_i32(qh, dev))
        graph.replay()
        torch.cuda.synchronize()
        full = O.hamming_topk(case["codes"], qh, case["block_table"], seq, k, O.REDUCE_SUM, False, must_select=must)
        for d in range(R):
            assert states[d].cpu().tolist() == [step, 0]
            par = step & 1
            flags = bufs[d][par * words + 2 * R * slab: par * words + 2 * R * slab + R]
            assert flags.cpu().tolist() == [step] * R
            assert np.array_equal(outs[d][1].cpu().numpy(), full["logical"])
    assert int(status.item()) == 0


def test_merge_wait_gives_up_when_a_rank_never_delivers(cuda_device):
    """A flag that nothing sets: the wait runs out after its time limit, the status word says so, the output stays
    padding and the context remains usable."""
    import torch
    from unified_cache_management_b200 import ops
    dev = cuda_device
    R, B, Hh, k = 2, 1, 1, 4
    s = torch.zeros((R, B, Hh, k), dtype=torch.float32, device=dev)
    i = torch.zeros((R, B, Hh, k), dtype=torch.int32, device=dev)
    flags = torch.tensor([5, 0], dtype=torch.int32, device=dev)      # rank 1 never publishes step 5
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    ms, mi = ops.merge_topk_wait(s, i, k, flags, 5, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) & 2
    assert (mi.cpu().numpy() == -1).all() and np.isinf(ms.cpu().numpy()).all()
    flags[1] = 5
    status.zero_()
    ms, mi = ops.merge_topk_wait(s, i, k, flags, 5, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and (mi.cpu().numpy() >= 0).all()

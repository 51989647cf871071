"""GPU parity at the benchmark configurations' stated sizes (configs 1-4), through the C ABI, against the CPU oracle.

Every test builds the configuration's inputs on the device from a seed, copies what the oracle needs to the host,
runs the oracle's C restatement (all host threads) and compares bit for bit: block scores, selected ids, new sequence
lengths, gathered bytes.  Hash codes follow the configuration's rule: a device bit may differ from the sign of the
float64 projection only where |projection| < 1e-3; such bits are counted and printed, any other difference fails.
"""
import numpy as np
import pytest

from oracle import oracle as O
from oracle import oracle_c as OC
from tests import helpers as H
from tests.test_gpu_scan_topk import _cmp

pytestmark = pytest.mark.gpu
MUST = (0, -2, -1)


def _u16(t):
    import torch
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def _u32(t):
    return t.contiguous().cpu().numpy().view(np.uint32)


def _rand_codes(shape, dev, gen):
    import torch
    return torch.randint(-2**31, 2**31 - 1, shape, dtype=torch.int32, device=dev, generator=gen)


def _free_gib(dev):
    import torch
    return torch.cuda.mem_get_info(dev)[0] / 2**30


def _encode_flips(dev_codes, keys_u16, r_u16, rng, sample=2048):
    """(hard, soft, differing bits vs the float32 C port) for one batch of rows.  The C port accumulates in float32
    like the kernel, so the two differ in a bit only where the projection is at rounding-noise level; every row with
    a differing word, and a random sample of all rows, is classified against the float64 projection."""
    rows = keys_u16.reshape(-1, keys_u16.shape[-1])
    got = dev_codes.reshape(rows.shape[0], -1)
    port = OC.hash_encode(rows, r_u16).reshape(got.shape)
    differing = np.nonzero((got != port).any(axis=1))[0]
    pick = np.union1d(differing, rng.choice(rows.shape[0], size=min(sample, rows.shape[0]), replace=False))
    _, p64 = O.hash_encode(rows[pick], r_u16)
    hard, soft = O.count_code_mismatches(got[pick], p64)
    return hard, soft, int(np.bitwise_count(got[differing] ^ port[differing]).sum())


def _new_out(B, Hout, k, dev, scores=True):
    import torch
    from unified_cache_management_b200 import ops
    z = lambda *s: torch.full(s, -7, dtype=torch.int32, device=dev)
    return ops.Retrieval(physical=z(B, Hout, k), logical=z(B, Hout, k), scores=z(B, Hout, k) if scores else None,
                         valid_count=z(B), new_seq_lens=z(B))


def test_config1_llama3_8b_decode16_full_size(cuda_device, capsys):
    """Config 1: 16 requests x 131072 tokens, 8 kv heads, 32 query heads, bf16 keys ~N(0,1) encoded with the shared
    bf16 projection (seed 1) into the paged code cache, then the decode step exactly as the benchmark issues it:
    one encode launch for the queries and the new key rows, then scan + top-k on a persistent workspace with the
    inputs-stable flag, three steps back to back (16384 work items: the scan's dynamic tail and early set-up run)."""
    import torch
    from unified_cache_management_b200 import ops
    dev = cuda_device
    B, seq, Hkv, Hq, D, BS, k = 16, 131072, 8, 32, 128, 128, 16
    W, mb = D // 32, seq // BS
    NB = B * mb + 8
    if _free_gib(dev) < 8:
        pytest.skip("needs 8 GiB of free device memory")
    OC.use_all_cores()
    rng = np.random.default_rng(1)
    g = torch.Generator(device=dev)
    g.manual_seed(1)
    R = (torch.randn((D, D), device=dev, generator=g) / D ** 0.5).to(torch.bfloat16)
    r_host = _u16(R)
    bt = torch.randperm(NB, device=dev, generator=g)[:B * mb].to(torch.int32).view(B, mb).contiguous()
    seq_lens = torch.full((B,), seq, dtype=torch.int32, device=dev)
    cache = torch.zeros((NB, BS, Hkv, W), dtype=torch.int32, device=dev)
    pos = torch.arange(seq, device=dev)
    hard = soft = vs_port = 0
    for b in range(B):
        g.manual_seed(1000 + b)
        keys = torch.randn((seq, Hkv, D), device=dev, generator=g, dtype=torch.float32).to(torch.bfloat16)
        slots = bt[b].to(torch.int64)[pos // BS] * BS + (pos % BS)
        ops.hash_encode_and_cache(keys, slots, cache, R)
        got = _u32(cache[bt[b].to(torch.int64)])                     # [mb, BS, Hkv, W] in logical order
        h, s, d = _encode_flips(got, _u16(keys), r_host, rng)
        hard, soft, vs_port = hard + h, soft + s, vs_port + d
        del keys
    assert hard == 0, f"{hard} code bits differ where |projection| >= 1e-3"

    # the decode step's inputs: queries and one new key row per request, written to each request's last slot
    g.manual_seed(77)
    q = torch.randn((B, Hq, D), device=dev, generator=g, dtype=torch.float32).to(torch.bfloat16)
    k_new = torch.randn((B, Hkv, D), device=dev, generator=g, dtype=torch.float32).to(torch.bfloat16)
    last_slot = (bt[:, mb - 1].to(torch.int64) * BS + (BS - 1)).contiguous()
    q_codes = torch.empty((B, Hq, W), dtype=torch.int32, device=dev)
    ws = ops.new_workspace(B, Hkv, mb, dev)
    outs = [_new_out(B, Hkv, k, dev) for _ in range(3)]
    for o in outs:   # no synchronisation between the steps
        ops.hash_encode_decode_step(q, k_new, last_slot, cache, R, q_codes_out=q_codes)
        ops.hamming_topk(cache, q_codes, bt, seq_lens, k, reduce="sum", must_select=MUST, workspace=ws, out=o,
                         inputs_stable=True)
    torch.cuda.synchronize()
    assert ops.workspace_status(ws) == 0
    _, pq = O.hash_encode(_u16(q), r_host)
    hq, sq = O.count_code_mismatches(_u32(q_codes), pq)
    _, pk = O.hash_encode(_u16(k_new), r_host)
    new_rows = _u32(cache.view(NB * BS, Hkv, W)[last_slot])
    hk, sk = O.count_code_mismatches(new_rows, pk)
    assert hq == 0 and hk == 0
    codes_host = _u32(cache)
    ref = OC.hamming_topk(codes_host, _u32(q_codes), bt.cpu().numpy(), seq_lens.cpu().numpy(), k, O.REDUCE_SUM, False,
                          must_select=MUST)
    for o in outs:
        _cmp(o, ref)
    lg = outs[0].logical.cpu().numpy()
    assert (lg[..., 0] == 0).all() and (lg[..., -2] == mb - 2).all() and (lg[..., -1] == mb - 1).all()
    # the scan alone, as the benchmark's roofline leg launches it
    scores = ops.block_scores(cache, q_codes, bt, seq_lens, reduce="sum", inputs_stable=True)
    torch.cuda.synchronize()
    assert np.array_equal(scores.cpu().numpy(), ref["block_scores"])
    with capsys.disabled():
        print(f"\n[config 1] {B * seq * Hkv} key rows encoded: {hard} hard / {soft} near-zero sign flips among the rows "
              f"checked against float64, {vs_port} bits differ from the float32 CPU port; queries {sq}, new keys {sk} "
              f"near-zero flips; 3 steps x {B * mb} blocks bit-exact")


def test_config2_paged_gather_b64_full_size(cuda_device, capsys):
    """Config 2: ragged batch of 64 (8192..131072 tokens, multiples of 128) over a 200000-block pool, block table = one
    random permutation of the physical ids, selection over all kv heads (k = 32), then the K/V gather of the selected
    blocks into [64, 32*128, 8, 128].  The K/V pools span all 200000 blocks (52 GB each) so that the byte offsets are
    the real ones; only the blocks the selection refers to are filled and compared."""
    import torch
    from unified_cache_management_b200 import ops
    dev = cuda_device
    B, Hkv, Hq, D, BS, k, NB = 64, 8, 32, 128, 128, 32, 200000
    W = D // 32
    block_elems = BS * Hkv * D
    if _free_gib(dev) < 125:
        pytest.skip("needs 125 GiB of free device memory for the 200000-block K and V pools")
    OC.use_all_cores()
    gs = torch.Generator().manual_seed(2)
    seq = (torch.randint(8192 // BS, 131072 // BS + 1, (B,), generator=gs) * BS).to(torch.int32)
    nblk = (seq // BS).tolist()
    mb = 131072 // BS
    perm = torch.randperm(NB, generator=gs)[: sum(nblk)].to(torch.int32)
    bt = torch.zeros((B, mb), dtype=torch.int32)
    off = 0
    for b in range(B):
        bt[b, : nblk[b]] = perm[off: off + nblk[b]]
        off += nblk[b]
    g = torch.Generator(device=dev)
    g.manual_seed(2)
    codes = _rand_codes((NB, BS, Hkv, W), dev, g)
    q = _rand_codes((B, Hq, W), dev, g)
    bt_d, seq_d = bt.to(dev), seq.to(dev)
    ws = ops.new_workspace(B, Hkv, mb, dev, True)
    out = _new_out(B, 1, k, dev)
    ops.hamming_topk(codes, q, bt_d, seq_d, k, reduce="sum", reduce_kvhead=True, must_select=MUST, workspace=ws,
                     out=out, inputs_stable=True)
    torch.cuda.synchronize()
    assert ops.workspace_status(ws) == 0
    ref = OC.hamming_topk(_u32(codes), _u32(q), bt.numpy(), seq.numpy(), k, O.REDUCE_SUM, True, must_select=MUST)
    _cmp(out, ref)
    del codes
    torch.cuda.empty_cache()

    sel = out.physical.view(B, k)
    kp = torch.empty((NB, BS, Hkv, D), dtype=torch.bfloat16, device=dev)
    vp = torch.empty((NB, BS, Hkv, D), dtype=torch.bfloat16, device=dev)
    ids = torch.unique(sel.to(torch.int64))
    g.manual_seed(22)
    fill_k = torch.randint(-2**15, 2**15 - 1, (ids.numel(), block_elems), dtype=torch.int16, device=dev, generator=g)
    fill_v = torch.randint(-2**15, 2**15 - 1, (ids.numel(), block_elems), dtype=torch.int16, device=dev, generator=g)
    kp.view(torch.int16).view(NB, block_elems)[ids] = fill_k
    vp.view(torch.int16).view(NB, block_elems)[ids] = fill_v
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    ok, ov = ops.gather_kv(kp, vp, sel.contiguous(), status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    # expected bytes: row (b, i) of the output is the fill of physical block ref[b, i]
    where = torch.searchsorted(ids, torch.from_numpy(ref["physical"].reshape(B, k).astype(np.int64)).to(dev))
    for b in range(B):   # one request at a time: 64 MiB per pool per request
        want_k = fill_k[where[b]].view(k * BS, Hkv, D)
        want_v = fill_v[where[b]].view(k * BS, Hkv, D)
        assert torch.equal(ok[b].view(torch.int16), want_k), f"K bytes of request {b} differ"
        assert torch.equal(ov[b].view(torch.int16), want_v), f"V bytes of request {b} differ"
    # and the same bytes through the CPU oracle's gather for the first and the last request
    for b in (0, B - 1):
        pool_small = fill_k.cpu().numpy().view(np.uint16).reshape(-1, BS, Hkv, D)
        want = OC.gather_kv(pool_small, where[b:b + 1].cpu().numpy().astype(np.int32))
        assert np.array_equal(_u16(ok[b:b + 1]), want)
    with capsys.disabled():
        print(f"\n[config 2] {int(seq.sum())} tokens scanned over a {NB}-block pool, {B}x{k} blocks selected and "
              f"{2 * B * k * block_elems * 2 / 2**30:.2f} GiB gathered: bit-exact")
    del kp, vp, ok, ov
    torch.cuda.empty_cache()


@pytest.mark.parametrize("tp", [2, 4, 8])
def test_config3_llama3_70b_tp_rank_shapes_full_size(cuda_device, tp, capsys):
    """Config 3: the per-rank problem of a tensor-parallel split by kv head (no collective): batch 8 x 262144 tokens
    (2048 blocks), 8/tp kv heads and 64/tp query heads per rank, k = 32 per kv head.  At tp = 8 the codes come from
    bf16 keys through the encode kernel (one kv head per token row), otherwise from Bernoulli bits."""
    import torch
    from unified_cache_management_b200 import ops
    dev = cuda_device
    B, seq, D, BS, k = 8, 262144, 128, 128, 32
    Hkv, Hq = 8 // tp, 64 // tp
    W, mb = D // 32, seq // BS
    NB = B * mb
    OC.use_all_cores()
    g = torch.Generator(device=dev)
    g.manual_seed(30 + tp)
    bt = torch.randperm(NB, device=dev, generator=g).to(torch.int32).view(B, mb).contiguous()
    seq_lens = torch.full((B,), seq, dtype=torch.int32, device=dev)
    note = "Bernoulli code bits"
    if tp == 8:
        rng = np.random.default_rng(3)
        g.manual_seed(1)
        R = (torch.randn((D, D), device=dev, generator=g) / D ** 0.5).to(torch.bfloat16)
        codes = torch.zeros((NB, BS, Hkv, W), dtype=torch.int32, device=dev)
        pos = torch.arange(seq, device=dev)
        hard = soft = 0
        for b in range(B):
            keys = torch.randn((seq, Hkv, D), device=dev, generator=g, dtype=torch.float32).to(torch.bfloat16)
            slots = bt[b].to(torch.int64)[pos // BS] * BS + (pos % BS)
            ops.hash_encode_and_cache(keys, slots, codes, R)
            h, s, _ = _encode_flips(_u32(codes[bt[b].to(torch.int64)]), _u16(keys), _u16(R), rng)
            hard, soft = hard + h, soft + s
        assert hard == 0
        qf = torch.randn((B, Hq, D), device=dev, generator=g, dtype=torch.float32).to(torch.bfloat16)
        q = ops.hash_encode_query(qf, R)
        note = f"codes from bf16 keys, {soft} near-zero sign flips"
    else:
        codes = _rand_codes((NB, BS, Hkv, W), dev, g)
        q = _rand_codes((B, Hq, W), dev, g)
    ws = ops.new_workspace(B, Hkv, mb, dev)
    outs = [_new_out(B, Hkv, k, dev) for _ in range(2)]
    for o in outs:
        ops.hamming_topk(codes, q, bt, seq_lens, k, reduce="sum", must_select=MUST, workspace=ws, out=o,
                         inputs_stable=True)
    torch.cuda.synchronize()
    assert ops.workspace_status(ws) == 0
    ref = OC.hamming_topk(_u32(codes), _u32(q), bt.cpu().numpy(), seq_lens.cpu().numpy(), k, O.REDUCE_SUM, False,
                          must_select=MUST)
    for o in outs:
        _cmp(o, ref)
    with capsys.disabled():
        print(f"\n[config 3, tp={tp}] {B * seq} tokens x {Hkv} kv head(s): bit-exact ({note})")


def test_config4_million_token_sharded_full_size(cuda_device, capsys):
    """Config 4: 2 requests x 4194304 tokens, 256-bit codes, block 64 (65536 blocks per request), k = 256 per kv head.
    (a) eight shards of 8192 blocks, each through the candidate selection, their records merged as an all-gather
    would deliver them: ids and scores must equal the unsharded oracle; (b) the unsharded problem itself, whose 65536-
    block rows go through the selection split over thread-block clusters."""
    import torch
    from unified_cache_management_b200 import ops
    dev = cuda_device
    B, seq, Hkv, Hq, BS, k, W, R = 2, 4194304, 8, 32, 64, 256, 8, 8
    nblk = seq // BS
    per = nblk // R
    NB = B * nblk
    if _free_gib(dev) < 6:
        pytest.skip("needs 6 GiB of free device memory")
    OC.use_all_cores()
    g = torch.Generator(device=dev)
    g.manual_seed(4)
    codes = _rand_codes((NB, BS, Hkv, W), dev, g)
    q = _rand_codes((B, Hq, W), dev, g)
    bt = torch.randperm(NB, device=dev, generator=g).to(torch.int32).view(B, nblk).contiguous()
    seq_g = torch.full((B,), seq, dtype=torch.int32, device=dev)
    scale = 1.0 / (BS * (Hq // Hkv))
    ref = OC.hamming_topk(_u32(codes), _u32(q), bt.cpu().numpy(), seq_g.cpu().numpy(), k, O.REDUCE_SUM, False,
                          must_select=MUST)
    forced = O.forced_blocks(seq, BS, nblk, MUST)
    want_scores = np.where(forced[ref["logical"]], np.float32(-1.0), ref["scores"].astype(np.float32) * np.float32(scale))

    # (a) eight shards -> records -> merge
    ws = ops.new_workspace(B, Hkv, per, dev)
    cs = torch.empty((R, B, Hkv, k), dtype=torch.float32, device=dev)
    ci = torch.empty((R, B, Hkv, k), dtype=torch.int32, device=dev)
    seq_local = torch.full((B,), per * BS, dtype=torch.int32, device=dev)
    for r in range(R):
        bt_local = bt[:, r * per:(r + 1) * per].contiguous()
        ops.topk_candidates(codes, q, bt_local, seq_local, seq_g, k, r * per, scale, reduce="sum", must_select=MUST,
                            workspace=ws, out_scores=cs[r], out_ids=ci[r], inputs_stable=True)
    ms, mi = ops.merge_topk(cs, ci, k)
    torch.cuda.synchronize()
    assert ops.workspace_status(ws) == 0
    assert np.array_equal(mi.cpu().numpy(), ref["logical"])
    assert np.array_equal(ms.cpu().numpy().view(np.uint32), want_scores.view(np.uint32))
    # every shard's records against the oracle's selection restricted to the shard
    s_all = ref["block_scores"]
    for r in (0, R - 1):
        sl = slice(r * per, (r + 1) * per)
        shard = OC.select(s_all[:, :, sl], bt[:, sl].cpu().numpy(), seq_local.cpu().numpy(), BS, k,
                          must_select=[j - r * per for j in np.nonzero(forced[sl])[0] + r * per])
        assert np.array_equal(ci[r].cpu().numpy(), shard["logical"] + r * per)

    # (b) unsharded: rows of 65536 blocks
    ws_full = ops.new_workspace(B, Hkv, nblk, dev)
    out = _new_out(B, Hkv, k, dev)
    ops.hamming_topk(codes, q, bt, seq_g, k, reduce="sum", must_select=MUST, workspace=ws_full, out=out,
                     inputs_stable=True)
    torch.cuda.synchronize()
    assert ops.workspace_status(ws_full) == 0
    _cmp(out, ref)
    with capsys.disabled():
        print(f"\n[config 4] {B * seq} tokens, 256-bit codes: 8 shards x {per} blocks merged == unsharded top-{k}; "
              f"65536-block rows through the cluster selection: bit-exact")

"""GPU parity: Hamming scan + exact top-k through the C ABI vs the CPU oracle (bit-exact)."""
import numpy as np
import pytest

from oracle import oracle as O
from oracle import oracle_c as OC
from tests import helpers as H

pytestmark = pytest.mark.gpu

MODES = {"min": O.REDUCE_MIN, "sum": O.REDUCE_SUM}


def _run_dev(case, dev, k, **kw):
    import torch
    from unified_cache_management_b200 import ops
    out = ops.hamming_topk(H.to_dev_i32(case["codes"], dev), H.to_dev_i32(case["q"], dev),
                           H.to_dev_i32(case["block_table"], dev), H.to_dev_i32(case["seq_lens"], dev), k, **kw)
    torch.cuda.synchronize()
    return out


def _cmp(out, ref):
    for name in ("logical", "physical", "scores", "valid_count", "new_seq_lens"):
        got = getattr(out, name).cpu().numpy()
        want = np.asarray(ref[name])
        assert np.array_equal(got, want), f"{name} differs"


@pytest.mark.parametrize("mode", ["min", "sum"])
@pytest.mark.parametrize("reduce_kvhead", [False, True])
@pytest.mark.parametrize("shape", [
    # (B, Hkv, G, W, BS, max_blocks)
    (3, 8, 4, 4, 128, 12),   # the Llama-3-8B layer shape
    (2, 1, 4, 4, 128, 40),   # one kv head per device (TP=8): several blocks per CTA
    (2, 2, 8, 4, 128, 17),   # Llama-3-70B at TP=4
    (2, 8, 4, 8, 64, 20),    # 256-bit codes, block 64
    (2, 4, 1, 4, 16, 33),    # plugin path: one code per kv head, vLLM block 16
    (3, 8, 4, 4, 16, 70),    # 8 kv heads, block 16: eight 2 KiB blocks per stage, scanned one after the other
    (2, 8, 1, 4, 16, 70),    # the same with one code per kv head (min mode: four blocks per stage, lane groups)
    (2, 8, 4, 4, 32, 45),    # block 32: four blocks per stage
    (2, 8, 2, 8, 16, 37),    # 256-bit codes, block 16: two passes per block, four blocks per stage
    (2, 4, 2, 8, 16, 50),    # 4 kv heads x 256-bit codes, block 16: a head spans two 16-byte pieces of the row
    (2, 4, 4, 8, 32, 21),    # the same with block 32 and groups of 4
    (2, 8, 8, 4, 32, 30),    # block 32, groups of 8
    (1, 8, 2, 4, 16, 130),   # block 16, groups of 2, a long ragged row
    (2, 8, 1, 16, 32, 9),    # 512-bit codes
    (1, 2, 3, 4, 128, 6),    # G outside {1,2,4,8}: query codes in shared memory
    (2, 1, 16, 18, 64, 7),   # 576-bit MLA codes, W=18: token-row path of the staged kernel
    (3, 1, 64, 18, 64, 9),   # MLA, 64 query codes per request (128 heads, reduction 2)
    (2, 1, 128, 18, 128, 5), # MLA, 128 query codes, block 128
    (2, 1, 5, 18, 16, 21),   # MLA, odd group size, block 16 (several blocks per stage)
    (2, 3, 2, 4, 128, 5),    # non power-of-two kv heads: generic kernel
])
def test_topk_matches_oracle(cuda_device, shape, mode, reduce_kvhead):
    B, Hkv, G, W, BS, mb = shape
    case = H.make_paged_case(hash(shape) % 1000, B, Hkv, G, W, BS, mb)
    k = min(5, mb)
    kw = dict(must_select=(0, -2, -1))
    out = _run_dev(case, cuda_device, k, reduce=mode, reduce_kvhead=reduce_kvhead, **kw)
    ref = O.hamming_topk(case["codes"], case["q"], case["block_table"], case["seq_lens"], k, MODES[mode],
                         reduce_kvhead, **kw)
    _cmp(out, ref)


def test_block_scores_match_oracle(cuda_device):
    import torch
    from unified_cache_management_b200 import ops
    dev = cuda_device
    for mode in ("min", "sum"):
        for red in (False, True):
            case = H.make_paged_case(5, 4, 8, 4, 4, 128, 9)
            s = ops.block_scores(H.to_dev_i32(case["codes"], dev), H.to_dev_i32(case["q"], dev),
                                 H.to_dev_i32(case["block_table"], dev), H.to_dev_i32(case["seq_lens"], dev),
                                 reduce=mode, reduce_kvhead=red)
            torch.cuda.synchronize()
            want = O.block_scores(case["codes"], case["q"], case["block_table"], case["seq_lens"], MODES[mode], red)
            assert np.array_equal(s.cpu().numpy(), want)


def test_sink_recent_and_ragged(cuda_device):
    """Plugin-style forcing by token ranges; seq_lens not multiples of the block; k above the valid blocks."""
    B, Hkv, G, W, BS, mb = 5, 8, 1, 4, 16, 24
    case = H.make_paged_case(11, B, Hkv, G, W, BS, mb, seq_lens=[1, 17, 100, 383, 384])
    k = 8
    kw = dict(sink_tokens=BS, recent_tokens=4 * BS)
    out = _run_dev(case, cuda_device, k, reduce="min", reduce_kvhead=True, **kw)
    ref = O.hamming_topk(case["codes"], case["q"], case["block_table"], case["seq_lens"], k, O.REDUCE_MIN, True, **kw)
    _cmp(out, ref)
    # fewer valid blocks than k: the tail points at block-table padding, valid_count says how many are real
    assert out.valid_count.cpu().tolist() == [1, 2, 7, 8, 8]


def test_ties_break_by_lower_id(cuda_device):
    """All keys equal: the selection must be the first k ids; duplicated scores split at the boundary."""
    B, Hkv, G, W, BS, mb = 2, 2, 1, 4, 16, 50
    case = H.make_paged_case(3, B, Hkv, G, W, BS, mb, seq_lens=[mb * BS, mb * BS])
    case["codes"][:] = 0x12345678   # every token identical -> every block score identical
    out = _run_dev(case, cuda_device, 7, reduce="sum")
    assert np.array_equal(out.logical.cpu().numpy(), np.broadcast_to(np.arange(7, dtype=np.int32), (B, Hkv, 7)))
    ref = O.hamming_topk(case["codes"], case["q"], case["block_table"], case["seq_lens"], 7, O.REDUCE_SUM)
    _cmp(out, ref)
    # two score values only: the boundary falls inside a run of equal scores
    case["codes"][case["block_table"][0, 10:30]] = 0x0F0F0F0F
    out = _run_dev(case, cuda_device, 25, reduce="sum")
    ref = O.hamming_topk(case["codes"], case["q"], case["block_table"], case["seq_lens"], 25, O.REDUCE_SUM)
    _cmp(out, ref)


def test_k_per_request_and_mask(cuda_device):
    import torch
    B, Hkv, G, W, BS, mb = 4, 4, 2, 4, 32, 16
    case = H.make_paged_case(21, B, Hkv, G, W, BS, mb, seq_lens=[512, 300, 64, 512])
    kpr = np.array([6, 2, 6, 0], dtype=np.int32)
    mask = np.array([1, 1, 0, 1], dtype=np.uint8)
    dev = cuda_device
    out = _run_dev(case, dev, 6, reduce="min", must_select=(0, -1),
                   k_per_request=torch.from_numpy(kpr).to(dev), request_mask=torch.from_numpy(mask).to(dev))
    ref = O.hamming_topk(case["codes"], case["q"], case["block_table"], case["seq_lens"], 6, O.REDUCE_MIN, False,
                         must_select=(0, -1), k_per_request=kpr, request_mask=mask)
    _cmp(out, ref)


def test_strided_block_table_and_empty_batch(cuda_device):
    import torch
    from unified_cache_management_b200 import ops
    dev = cuda_device
    case = H.make_paged_case(8, 3, 8, 4, 4, 128, 10)
    wide = np.zeros((3, 37), dtype=np.int32)
    wide[:, :10] = case["block_table"]
    bt = torch.from_numpy(wide).to(dev)[:, :10]          # row stride 37
    out = ops.hamming_topk(H.to_dev_i32(case["codes"], dev), H.to_dev_i32(case["q"], dev), bt,
                           H.to_dev_i32(case["seq_lens"], dev), 4, reduce="sum", must_select=(0, -2, -1))
    ref = O.hamming_topk(case["codes"], case["q"], case["block_table"], case["seq_lens"], 4, O.REDUCE_SUM,
                         must_select=(0, -2, -1))
    torch.cuda.synchronize()
    _cmp(out, ref)
    empty = ops.hamming_topk(H.to_dev_i32(case["codes"], dev), torch.empty((0, 32, 4), dtype=torch.int32, device=dev),
                             torch.empty((0, 10), dtype=torch.int32, device=dev),
                             torch.empty((0,), dtype=torch.int32, device=dev), 4)
    assert empty.physical.shape == (0, 8, 4)


def test_bad_block_id_is_flagged_not_read(cuda_device):
    import torch
    from unified_cache_management_b200 import ops
    dev = cuda_device
    case = H.make_paged_case(9, 2, 8, 4, 4, 128, 6, seq_lens=[768, 768])
    case["block_table"][1, 2] = case["NB"] + 1000   # outside the pool
    ws = ops.new_workspace(2, 8, 6, dev)
    out = ops.hamming_topk(H.to_dev_i32(case["codes"], dev), H.to_dev_i32(case["q"], dev),
                           H.to_dev_i32(case["block_table"], dev), H.to_dev_i32(case["seq_lens"], dev), 3,
                           workspace=ws)
    assert ops.workspace_status(ws) & 1
    assert 2 not in out.logical[1].cpu().numpy()     # the bad block scores as invalid


def test_argument_errors(cuda_device):
    import torch
    from unified_cache_management_b200 import ops
    dev = cuda_device
    case = H.make_paged_case(1, 2, 8, 4, 4, 128, 6)
    c, q, bt, sl = (H.to_dev_i32(case[n], dev) for n in ("codes", "q", "block_table", "seq_lens"))
    with pytest.raises(ValueError):
        ops.hamming_topk(c, q, bt, sl, 7)                      # k > max_blocks
    with pytest.raises(RuntimeError):
        ops.hamming_topk(c, q, bt[:1], sl, 2)                  # batch mismatch (reference: TORCH_CHECK)
    with pytest.raises(ValueError):
        ops.hamming_topk(c, q[:, :30], bt, sl, 2)              # heads not a multiple
    with pytest.raises(ValueError):
        ops.hamming_topk(c, q, bt, sl, 2, reduce="median")


def test_hamming_score_per_token(cuda_device):
    """The old op's fp16 per-token output (sink/recent -> 0, past the end -> inf)."""
    import torch
    from unified_cache_management_b200 import ops
    dev = cuda_device
    B, Hkv, G, W, BS, mb = 3, 4, 2, 4, 16, 12
    case = H.make_paged_case(31, B, Hkv, G, W, BS, mb)
    for red in (True, False):
        got = ops.hamming_score(H.to_dev_i32(case["codes"], dev), H.to_dev_i32(case["q"], dev).unsqueeze(1),
                                H.to_dev_i32(case["block_table"], dev), H.to_dev_i32(case["seq_lens"], dev),
                                mb * BS, BS, 2 * BS, red)
        torch.cuda.synchronize()
        want = O.hamming_score_fp16(case["codes"], case["q"], case["block_table"], case["seq_lens"], BS, 2 * BS, red)
        assert np.array_equal(got.cpu().numpy().view(np.uint16), want.view(np.uint16))


def test_config0_full_size(cuda_device):
    """Benchmark config 0 at full size: 32768 tokens, 8 kv heads, 32 query heads, 128-bit codes, k=64."""
    rng = np.random.default_rng(0)
    B, Hkv, G, W, BS, mb = 1, 8, 4, 4, 128, 256
    case = H.make_paged_case(0, B, Hkv, G, W, BS, mb, seq_lens=[32768])
    for red in (False, True):
        out = _run_dev(case, cuda_device, 64, reduce="sum", reduce_kvhead=red, must_select=(0, -2, -1))
        ref = OC.hamming_topk(case["codes"], case["q"], case["block_table"], case["seq_lens"], 64, O.REDUCE_SUM, red,
                              must_select=(0, -2, -1))
        _cmp(out, ref)
        lg = out.logical.cpu().numpy()
        assert (lg[..., 0] == 0).all() and (lg[..., -1] == 255).all() and (lg[..., -2] == 254).all()
        assert (np.diff(lg, axis=-1) > 0).all()


def test_large_row_select(cuda_device):
    """65536 blocks per request (the million-token shape): keys do not all fit in shared memory."""
    B, Hkv, G, W, BS, mb = 1, 1, 1, 4, 2, 65536
    case = H.make_paged_case(4, B, Hkv, G, W, BS, mb, seq_lens=[mb * BS], identity=True)
    out = _run_dev(case, cuda_device, 256, reduce="sum", must_select=(0, -2, -1))
    ref = OC.hamming_topk(case["codes"], case["q"], case["block_table"], case["seq_lens"], 256, O.REDUCE_SUM, False,
                          must_select=(0, -2, -1))
    _cmp(out, ref)


@pytest.mark.parametrize("mode", ["min", "sum"])
@pytest.mark.parametrize("reduce_kvhead", [False, True])
def test_few_long_rows_cluster_select(cuda_device, mode, reduce_kvhead):
    """Few rows of thousands of blocks: the selection splits each row over a thread-block cluster.  Small codes
    give many equal scores, so ties cross the slice boundaries; lengths are ragged and sink / recent windows set."""
    B, Hkv, G, W, BS, mb = 2, 2, 1, 4, 16, 3000
    seq = [mb * BS - 5, 1000 * BS + 3]
    case = H.make_paged_case(77, B, Hkv, G, W, BS, mb, seq_lens=seq)
    kw = dict(must_select=(0, 7, -3), sink_tokens=40, recent_tokens=100)
    for k in (1, 100, 1500):
        out = _run_dev(case, cuda_device, k, reduce=mode, reduce_kvhead=reduce_kvhead, **kw)
        ref = OC.hamming_topk(case["codes"], case["q"], case["block_table"], case["seq_lens"], k, MODES[mode],
                              reduce_kvhead, **kw)
        _cmp(out, ref)


def test_cluster_select_k_per_request_and_mask(cuda_device):
    import torch
    B, Hkv, G, W, BS, mb = 3, 1, 2, 4, 16, 2100
    case = H.make_paged_case(78, B, Hkv, G, W, BS, mb, seq_lens=[mb * BS, 50 * BS, 1300 * BS + 1])
    kpr = np.array([600, 64, 0], dtype=np.int32)
    mask = np.array([1, 1, 0], dtype=np.uint8)
    out = _run_dev(case, cuda_device, 600, reduce="sum", k_per_request=torch.from_numpy(kpr).to(cuda_device),
                   request_mask=torch.from_numpy(mask).to(cuda_device))
    ref = OC.hamming_topk(case["codes"], case["q"], case["block_table"], case["seq_lens"], 600, O.REDUCE_SUM, False,
                          k_per_request=kpr, request_mask=mask)
    _cmp(out, ref)


def test_many_long_rows_uncached_keys(cuda_device):
    """More rows than a cluster split is used for, each longer than the shared-memory key cache."""
    B, Hkv, G, W, BS, mb = 84, 1, 1, 4, 2, 41500
    case = H.make_paged_case(79, B, Hkv, G, W, BS, mb, identity=True)
    out = _run_dev(case, cuda_device, 300, reduce="sum", must_select=(0, -1))
    ref = OC.hamming_topk(case["codes"], case["q"], case["block_table"], case["seq_lens"], 300, O.REDUCE_SUM, False,
                          must_select=(0, -1))
    _cmp(out, ref)


def test_inputs_stable_flag_changes_nothing_but_the_schedule(cuda_device):
    """UCMR_FLAG_INPUTS_STABLE only moves the scan's dependency wait: same results, back to back launches included;
    unknown flag bits are refused."""
    import torch
    from unified_cache_management_b200 import lib, ops
    B, Hkv, G, W, BS, mb = 4, 8, 4, 4, 128, 300
    case = H.make_paged_case(5, B, Hkv, G, W, BS, mb)
    dev = cuda_device
    args = [H.to_dev_i32(case[n], dev) for n in ("codes", "q", "block_table", "seq_lens")]
    ws = ops.new_workspace(B, Hkv, mb, dev)
    ref = O.hamming_topk(case["codes"], case["q"], case["block_table"], case["seq_lens"], 9, O.REDUCE_SUM, False,
                         must_select=(0, -1))
    for _ in range(3):   # consecutive launches overlap their set-up with the predecessor's drain
        out = ops.hamming_topk(*args, 9, reduce="sum", must_select=(0, -1), workspace=ws, inputs_stable=True)
    torch.cuda.synchronize()
    _cmp(out, ref)
    s0 = ops.block_scores(*args, reduce="min")
    s1 = ops.block_scores(*args, reduce="min", inputs_stable=True)
    torch.cuda.synchronize()
    assert torch.equal(s0, s1)
    with pytest.raises(ValueError):
        codes, q, bt, sl = args
        rc = lib.load_library().ucmr_block_scores(codes.data_ptr(), codes.shape[0], BS, Hkv, W, q.data_ptr(), Hkv * G,
                                                  bt.data_ptr(), mb, mb, sl.data_ptr(), B, 1 | 0x400, 0, s0.data_ptr(),
                                                  None, None)
        lib.check(rc, "ucmr_block_scores")


@pytest.mark.parametrize("mode", ["min", "sum"])
@pytest.mark.parametrize("BS,mb", [(128, 40), (16, 260), (64, 3)])
def test_cache_append_only_scan_sees_the_new_token(cuda_device, mode, BS, mb):
    """UCMR_FLAG_CACHE_APPEND_ONLY lets the scan copy blocks before the decode-step encode in front of it has finished,
    except a request's last block.  Each step first poisons the slot of the newest token, then encodes a key equal to
    the query (distance 0) into it and scans: the last block's score must come from the fresh code, stream-ordered
    and as a replayed graph."""
    import torch
    from unified_cache_management_b200 import ops
    dev = cuda_device
    B, Hkv, W, D = 5, 2, 4, 128
    g = torch.Generator(device=dev)
    g.manual_seed(77)
    NB = B * mb
    cache = torch.randint(-2**31, 2**31 - 1, (NB, BS, Hkv, W), dtype=torch.int32, device=dev, generator=g)
    bt = torch.randperm(NB, device=dev, generator=g).to(torch.int32).view(B, mb).contiguous()
    seq = torch.tensor([mb * BS, mb * BS - BS // 2, (mb - 1) * BS + 1, 5, max(1, mb // 2) * BS], dtype=torch.int32)
    sl = seq.to(dev)
    last = seq.to(torch.int64) - 1
    slots = (bt.cpu()[torch.arange(B), last // BS].to(torch.int64) * BS + last % BS).to(dev)
    R = (torch.randn((D, 32 * W), device=dev, generator=g) / D ** 0.5).to(torch.bfloat16)
    k = min(4, mb)
    ws = ops.new_workspace(B, Hkv, mb, dev)
    qc = torch.empty((B, Hkv, W), dtype=torch.int32, device=dev)
    out = ops.hamming_topk(cache, torch.zeros_like(qc), bt, sl, k, reduce=mode, workspace=ws)
    flat = cache.view(NB * BS, Hkv, W)

    def step(x):
        ops.hash_encode_decode_step(x, x, slots, cache, R, q_codes_out=qc)
        ops.hamming_topk(cache, qc, bt, sl, k, reduce=mode, workspace=ws, out=out, inputs_stable=True,
                         cache_append_only=True)

    def check(x):
        torch.cuda.synchronize()
        assert torch.equal(flat[slots], qc), "the new keys' codes equal the query codes"
        ref = O.hamming_topk(cache.cpu().numpy().view(np.uint32), qc.cpu().numpy().view(np.uint32), bt.cpu().numpy(),
                             seq.numpy(), k, MODES[mode], False)
        _cmp(out, ref)
        if mode == "min":   # the block with the new token has a token at distance 0
            assert (out.scores.cpu().numpy() == 0).any(axis=2).all()

    xs = [torch.randn((B, Hkv, D), device=dev, generator=g).to(torch.bfloat16) for _ in range(4)]
    for x in xs:
        flat[slots] = -1
        step(x)
        check(x)
    x_static = xs[0].clone()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step(x_static)
    for x in xs[1:]:
        x_static.copy_(x)
        flat[slots] = -1
        graph.replay()
        check(x)


def test_selection_inside_the_scan_ragged_batch_repeated(cuda_device):
    """A ragged batch with empty, one-block and full requests, per-request k and a request mask, run
    three times on one workspace: the counters must come back to zero every time.  (Also run with the selection
    folded into the scan kernel, see test_selection_folded_into_the_scan.)"""
    import torch
    from unified_cache_management_b200 import ops
    dev = cuda_device
    B, Hkv, G, W, BS, mb = 37, 8, 4, 4, 128, 96
    rng = np.random.default_rng(11)
    seq = rng.integers(1, mb * BS + 1, size=B).astype(np.int32)
    seq[3], seq[7], seq[20], seq[36] = 0, 1, mb * BS, BS          # empty, one token, full, one block
    case = H.make_paged_case(123, B, Hkv, G, W, BS, mb, seq_lens=seq)
    kpr = rng.integers(0, 12, size=B).astype(np.int32)
    mask = (rng.random(B) > 0.2).astype(np.uint8)
    k = 10
    codes, q = H.to_dev_i32(case["codes"], dev), H.to_dev_i32(case["q"], dev)
    bt, sl = H.to_dev_i32(case["block_table"], dev), H.to_dev_i32(seq, dev)
    ws = ops.new_workspace(B, Hkv, mb, dev, True)
    for mode in ("sum", "min"):
        for red in (False, True):
            kw = dict(must_select=(0, -1), sink_tokens=100, recent_tokens=300)
            ref = OC.hamming_topk(case["codes"], case["q"], case["block_table"], seq, k, MODES[mode], red,
                                  k_per_request=kpr, request_mask=mask, **kw)
            for _ in range(3):
                out = ops.hamming_topk(codes, q, bt, sl, k, reduce=mode, reduce_kvhead=red, workspace=ws,
                                       k_per_request=H.to_dev_i32(kpr, dev),
                                       request_mask=torch.from_numpy(mask).to(dev), **kw)
                torch.cuda.synchronize()
                _cmp(out, ref)
            assert ops.workspace_status(ws) == 0
            head = ws[:ops._l.WORKSPACE_HEADER_BYTES].view(torch.int32).cpu().numpy().copy()
            head[36] = 0    # the "all blocks scored" word counts launches
            assert not head.any(), "a counter of the workspace header was left non-zero"


def test_selection_inside_the_scan_2048_blocks(cuda_device):
    """2048 blocks per row (64 keys per lane of the selecting warp) and k = 32, with ties (small codes)."""
    B, Hkv, G, W, BS, mb = 3, 2, 1, 4, 16, 2048
    seq = [mb * BS, mb * BS - 7, 1500 * BS + 3]
    case = H.make_paged_case(55, B, Hkv, G, W, BS, mb, seq_lens=seq)
    for mode in ("sum", "min"):
        for k in (1, 32, 700, 2048):
            out = _run_dev(case, cuda_device, k, reduce=mode, must_select=(0, -2, -1))
            ref = OC.hamming_topk(case["codes"], case["q"], case["block_table"], case["seq_lens"], k, MODES[mode], False,
                                  must_select=(0, -2, -1))
            _cmp(out, ref)


def test_rejected_call_leaves_the_workspace_usable(cuda_device):
    """A call that is refused (k larger than the block table) must not disturb the counters of the workspace: the next
    call on it still matches the oracle."""
    import torch
    from unified_cache_management_b200 import ops
    dev = cuda_device
    B, Hkv, G, W, BS, mb = 4, 8, 4, 4, 128, 300
    case = H.make_paged_case(5, B, Hkv, G, W, BS, mb, seq_lens=[mb * BS] * B)
    codes, q = H.to_dev_i32(case["codes"], dev), H.to_dev_i32(case["q"], dev)
    bt, sl = H.to_dev_i32(case["block_table"], dev), H.to_dev_i32(case["seq_lens"], dev)
    ws = ops.new_workspace(B, Hkv, mb, dev)
    good = ops.hamming_topk(codes, q, bt, sl, 8, reduce="sum", workspace=ws)
    with pytest.raises(ValueError):
        ops.hamming_topk(codes, q, bt, sl, mb + 1, reduce="sum", workspace=ws)
    with pytest.raises(ValueError):
        ops.hamming_topk(codes, q, bt, sl, 8, reduce="sum", workspace=ws, must_select=tuple(range(17)))
    again = ops.hamming_topk(codes, q, bt, sl, 8, reduce="sum", workspace=ws)
    torch.cuda.synchronize()
    ref = OC.hamming_topk(case["codes"], case["q"], case["block_table"], case["seq_lens"], 8, O.REDUCE_SUM, False)
    _cmp(good, ref)
    _cmp(again, ref)


def test_selection_folded_into_the_scan(cuda_device):
    """UCMR_FUSED_SELECT=1 makes the staged scan select the rows itself (rows of at most 2048 blocks).  The switch is
    read once per process, so the cases run in a child process: the ragged repeated batch, the 2048-block rows, the
    full-size config 0 and a few shapes of the oracle sweep, all through that path."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = r"""
import sys, torch
sys.path.insert(0, %r)
from tests import test_gpu_scan_topk as T
dev = torch.device("cuda:0")
T.test_selection_inside_the_scan_ragged_batch_repeated(dev)
T.test_selection_inside_the_scan_2048_blocks(dev)
T.test_config0_full_size(dev)
T.test_rejected_call_leaves_the_workspace_usable(dev)
for shape in [(3, 8, 4, 4, 128, 12), (2, 1, 4, 4, 128, 40), (2, 4, 1, 4, 16, 33), (3, 1, 64, 18, 64, 9), (2, 3, 2, 4, 128, 5)]:
    for mode in ("min", "sum"):
        for red in (False, True):
            T.test_topk_matches_oracle(dev, shape, mode, red)
print("fused ok")
""" % root
    env = dict(os.environ, UCMR_FUSED_SELECT="1")
    res = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=900)
    assert res.returncode == 0 and "fused ok" in res.stdout, res.stdout[-2000:] + res.stderr[-4000:]


@pytest.mark.parametrize("BS,mb,G", [(64, 2400, 16), (16, 12000, 5), (128, 1300, 64), (32, 5000, 2)])
def test_token_row_codes_many_ring_rounds(cuda_device, BS, mb, G):
    """576-bit token-row codes (MLA) with enough blocks that every CTA of the producer / consumer kernel goes round
    its ring of stages several times; ragged lengths, both block reduces."""
    B = 4
    seq = [mb * BS, mb * BS - 7, (mb // 2) * BS + 1, mb * BS - BS]
    case = H.make_paged_case(600 + BS, B, 1, G, 18, BS, mb, seq_lens=seq)
    for mode in ("min", "sum"):
        out = _run_dev(case, cuda_device, 32, reduce=mode, must_select=(0, -2, -1))
        ref = OC.hamming_topk(case["codes"], case["q"], case["block_table"], case["seq_lens"], 32, MODES[mode], False,
                              must_select=(0, -2, -1))
        _cmp(out, ref)

"""GPU parity: paged-KV gather vs numpy indexing (byte-exact)."""
import numpy as np
import pytest

from oracle import oracle as O
from oracle import oracle_c as OC
from tests import helpers as H

pytestmark = pytest.mark.gpu


def _pools(rng, NB, BS, Hkv, D):
    k = rng.integers(0, 2**16, size=(NB, BS, Hkv, D), dtype=np.uint16)
    v = rng.integers(0, 2**16, size=(NB, BS, Hkv, D), dtype=np.uint16)
    return k, v


@pytest.mark.parametrize("shape", [(50, 128, 8, 128, 4, 6), (30, 16, 8, 128, 3, 5), (20, 64, 2, 64, 2, 7),
                                   (9, 16, 1, 8, 1, 3)])
@pytest.mark.parametrize("per_head", [False, True])
def test_gather_matches_indexing(cuda_device, shape, per_head):
    import torch
    from unified_cache_management_b200 import ops
    NB, BS, Hkv, D, B, k = shape
    rng = np.random.default_rng(NB + BS)
    kp, vp = _pools(rng, NB, BS, Hkv, D)
    sel = rng.integers(0, NB, size=(B, Hkv, k) if per_head else (B, k)).astype(np.int32)
    kd, vd = H.bf16_to_dev(kp, cuda_device), H.bf16_to_dev(vp, cuda_device)
    ok, ov = ops.gather_kv(kd, vd, torch.from_numpy(sel).to(cuda_device))
    torch.cuda.synchronize()
    assert np.array_equal(ok.view(torch.int16).cpu().numpy().view(np.uint16), O.gather_kv(kp, sel))
    assert np.array_equal(ov.view(torch.int16).cpu().numpy().view(np.uint16), O.gather_kv(vp, sel))
    # one pool only
    ok2, none = ops.gather_kv(kd, None, torch.from_numpy(sel).to(cuda_device))
    torch.cuda.synchronize()
    assert none is None and torch.equal(ok2.view(torch.int16), ok.view(torch.int16))


def test_gather_many_blocks(cuda_device):
    """More chunks than one wave of CTAs x ring stages: exercises stage reuse and barrier phases."""
    import torch
    from unified_cache_management_b200 import ops
    NB, BS, Hkv, D, B, k = 600, 128, 8, 128, 16, 32   # 512 selected blocks x 256 KiB x 2 pools
    rng = np.random.default_rng(2)
    kp, vp = _pools(rng, NB, BS, Hkv, D)
    sel = np.stack([rng.permutation(NB)[:k] for _ in range(B)]).astype(np.int32)
    ok, ov = ops.gather_kv(H.bf16_to_dev(kp, cuda_device), H.bf16_to_dev(vp, cuda_device),
                           torch.from_numpy(sel).to(cuda_device))
    torch.cuda.synchronize()
    assert np.array_equal(ok.view(torch.int16).cpu().numpy().view(np.uint16), OC.gather_kv(kp, sel))
    assert np.array_equal(ov.view(torch.int16).cpu().numpy().view(np.uint16), OC.gather_kv(vp, sel))


def test_gather_bad_id_skipped_and_flagged(cuda_device):
    import torch
    from unified_cache_management_b200 import ops
    NB, BS, Hkv, D = 10, 16, 2, 64
    rng = np.random.default_rng(3)
    kp, _ = _pools(rng, NB, BS, Hkv, D)
    for per_head in (False, True):
        sel = np.array([[1, NB + 3, 2]], dtype=np.int32)
        if per_head:
            sel = np.repeat(sel[:, None, :], Hkv, axis=1)
        status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
        out = torch.full((1, 3 * BS, Hkv, D), 0x55AA, dtype=torch.int16, device=cuda_device).view(torch.bfloat16)
        ops.gather_kv(H.bf16_to_dev(kp, cuda_device), None, torch.from_numpy(sel).to(cuda_device), out_k=out,
                      status=status)
        torch.cuda.synchronize()
        got = out.view(torch.int16).cpu().numpy().view(np.uint16)
        assert status.item() & 1
        assert np.array_equal(got[0, :BS], kp[1]) and np.array_equal(got[0, 2 * BS:], kp[2])
        assert (got[0, BS:2 * BS] == 0x55AA).all()      # the slot of the bad id is left alone


def test_retrieve_then_gather_round_trip(cuda_device):
    """End of the decode-step chain: the gathered K rows are the rows of the blocks the top-k picked."""
    import torch
    from unified_cache_management_b200 import ops
    dev = cuda_device
    B, Hkv, G, W, BS, mb, k = 3, 8, 4, 4, 128, 20, 6
    case = H.make_paged_case(77, B, Hkv, G, W, BS, mb)
    rng = np.random.default_rng(78)
    kp, vp = _pools(rng, case["NB"], BS, Hkv, 128)
    out = ops.hamming_topk(H.to_dev_i32(case["codes"], dev), H.to_dev_i32(case["q"], dev),
                           H.to_dev_i32(case["block_table"], dev), H.to_dev_i32(case["seq_lens"], dev), k,
                           reduce="sum", reduce_kvhead=True, must_select=(0, -2, -1))
    gk, gv = ops.gather_kv(H.bf16_to_dev(kp, dev), H.bf16_to_dev(vp, dev), out.physical[:, 0, :].contiguous())
    torch.cuda.synchronize()
    ref = O.hamming_topk(case["codes"], case["q"], case["block_table"], case["seq_lens"], k, O.REDUCE_SUM, True,
                         must_select=(0, -2, -1))
    assert np.array_equal(gk.view(torch.int16).cpu().numpy().view(np.uint16), O.gather_kv(kp, ref["physical"][:, 0]))
    assert np.array_equal(gv.view(torch.int16).cpu().numpy().view(np.uint16), O.gather_kv(vp, ref["physical"][:, 0]))


@pytest.mark.parametrize("size", [256 * 1024, 48 * 1024 + 16, 4096])
def test_copy_blocks_pointer_lists(cuda_device, size):
    """The three pointer-list copies of the reference's landing path: list -> list, list -> contiguous,
    contiguous -> list; a null and a misaligned entry are skipped and flagged."""
    import torch
    from unified_cache_management_b200 import ops
    dev = cuda_device
    g = torch.Generator(device=dev).manual_seed(size)
    num, pool_blocks = 37, 90
    pool = torch.randint(0, 256, (pool_blocks, size), dtype=torch.uint8, device=dev, generator=g)
    land = torch.zeros((pool_blocks, size), dtype=torch.uint8, device=dev)
    src_ids = torch.randperm(pool_blocks, generator=torch.Generator().manual_seed(1))[:num]
    dst_ids = torch.randperm(pool_blocks, generator=torch.Generator().manual_seed(2))[:num]
    sp = torch.tensor([pool.data_ptr() + int(i) * size for i in src_ids], dtype=torch.int64, device=dev)
    dp = torch.tensor([land.data_ptr() + int(i) * size for i in dst_ids], dtype=torch.int64, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    ops.copy_blocks(size, num, src_ptrs=sp, dst_ptrs=dp, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.equal(land[dst_ids.to(dev)], pool[src_ids.to(dev)])
    untouched = torch.ones(pool_blocks, dtype=torch.bool, device=dev)
    untouched[dst_ids.to(dev)] = False
    assert int(land[untouched].sum().item()) == 0
    flat = torch.zeros((num, size), dtype=torch.uint8, device=dev)
    ops.copy_blocks(size, num, src_ptrs=sp, dst=flat, status=status)
    torch.cuda.synchronize()
    assert torch.equal(flat, pool[src_ids.to(dev)])
    land.zero_()
    ops.copy_blocks(size, num, src=flat, dst_ptrs=dp, status=status)
    torch.cuda.synchronize()
    assert torch.equal(land[dst_ids.to(dev)], flat) and int(status.item()) == 0
    # bad entries
    land.zero_()
    sp_bad = sp.clone()
    sp_bad[3] = 0
    sp_bad[5] += 8
    ops.copy_blocks(size, num, src_ptrs=sp_bad, dst_ptrs=dp, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) & 1
    ok = torch.ones(num, dtype=torch.bool)
    ok[3] = ok[5] = False
    assert torch.equal(land[dst_ids[ok].to(dev)], pool[src_ids[ok].to(dev)])
    assert int(land[dst_ids[~ok].to(dev)].sum().item()) == 0
    with pytest.raises(ValueError):
        ops.copy_blocks(size, num, src_ptrs=sp, src=flat, dst=flat)

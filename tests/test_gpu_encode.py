"""GPU parity: hash encode (tensor-core and CUDA-core paths) vs the CPU oracle.

Tolerance (stated by the task): a code bit may differ from sign(projection) only where the
float64 projection magnitude is below 1e-3; such flips are counted and must stay rare.
"""
import numpy as np
import pytest

from oracle import oracle as O
from tests import helpers as H

pytestmark = pytest.mark.gpu

TOL = 1e-3


def _r_matrix(seed, in_dim=128, bits=128):
    rng = np.random.default_rng(seed)
    return O.f32_to_bf16_bits((rng.standard_normal((in_dim, bits)) / np.sqrt(in_dim)).astype(np.float32))


def _check(dev_codes, x_bits, r_bits, max_soft_frac=1e-3):
    want_codes, p64 = O.hash_encode(x_bits, r_bits)
    hard, soft = O.count_code_mismatches(dev_codes.reshape(want_codes.shape), p64, TOL)
    assert hard == 0, f"{hard} bits differ where |projection| >= {TOL}"
    assert soft <= max_soft_frac * p64.size + 2, f"{soft} near-zero flips"
    return soft


@pytest.mark.parametrize("rows", [1, 5, 127, 128, 129, 1000, 148 * 128 * 3 + 77])
def test_encode_rows(cuda_device, rows):
    import torch
    from unified_cache_management_b200 import ops
    rng = np.random.default_rng(rows)
    x = H.bf16_normal(rng, (rows, 128))
    r = _r_matrix(1)
    out = ops.hash_encode(H.bf16_to_dev(x, cuda_device), H.bf16_to_dev(r, cuda_device))
    torch.cuda.synchronize()
    _check(H.dev_to_u32(out), x, r)


def test_encode_bit_order_and_sign_rule(cuda_device):
    """Identity projection: bit b of word w is exactly (x[32w+b] > 0); zeros, -0 and NaN give 0."""
    import torch
    from unified_cache_management_b200 import ops
    eye = O.f32_to_bf16_bits(np.eye(128, dtype=np.float32))
    x = np.zeros((4, 128), dtype=np.float32)
    x[0, [0, 31, 32, 127]] = 1.0
    x[1, :] = -1.0
    x[2, 5] = 2.0 ** -120
    x[2, 6] = -0.0
    x[3, 7] = np.nan
    x[3, 8] = 3.0
    xb = O.f32_to_bf16_bits(x)
    out = H.dev_to_u32(ops.hash_encode(H.bf16_to_dev(xb, cuda_device), H.bf16_to_dev(eye, cuda_device)))
    torch.cuda.synchronize()
    assert out[0].tolist() == [0x80000001, 0x00000001, 0, 0x80000000]
    assert out[1].tolist() == [0, 0, 0, 0]
    assert out[2].tolist() == [1 << 5, 0, 0, 0]
    # NaN * 0 poisons the whole row's sums: every comparison is false
    assert out[3].tolist() == [0, 0, 0, 0]


def test_encode_strided_rows(cuda_device):
    """Keys sliced out of a fused qkv buffer: row stride larger than in_dim."""
    import torch
    from unified_cache_management_b200 import ops
    rng = np.random.default_rng(7)
    T, Hkv, D = 300, 8, 128
    q_size, kv_size = 32 * D, Hkv * D
    qkv = H.bf16_normal(rng, (T, q_size + 2 * kv_size))
    r = _r_matrix(1)
    qkv_d = H.bf16_to_dev(qkv, cuda_device)
    key = qkv_d[:, q_size:q_size + kv_size].view(T, Hkv, D)
    out = ops.hash_encode_query(key, H.bf16_to_dev(r, cuda_device))
    torch.cuda.synchronize()
    xk = qkv[:, q_size:q_size + kv_size].reshape(T, Hkv, D)
    _check(H.dev_to_u32(out), xk, r)


@pytest.mark.parametrize("slot_dtype", ["int64", "int32"])
@pytest.mark.parametrize("T,Hh", [(1, 8), (100, 8), (700, 4), (33, 1)])
def test_encode_and_cache(cuda_device, T, Hh, slot_dtype):
    """Fused encode + scatter into the paged cache; out-of-range slots are skipped."""
    import torch
    from unified_cache_management_b200 import ops
    rng = np.random.default_rng(T * 10 + Hh)
    NB, BS = 50, 16
    x = H.bf16_normal(rng, (T, Hh, 128))
    r = _r_matrix(1)
    slots = rng.permutation(NB * BS)[:T].astype(np.int64)
    if T > 3:
        slots[1] = -1
        slots[2] = NB * BS + 5
    cache0 = H.rand_codes(rng, (NB, BS, Hh, 4))
    cache = H.to_dev_i32(cache0, cuda_device)
    sl = torch.from_numpy(slots.astype(slot_dtype)).to(cuda_device)
    ops.hash_encode_and_cache(H.bf16_to_dev(x, cuda_device), sl, cache, H.bf16_to_dev(r, cuda_device))
    torch.cuda.synchronize()
    got = H.dev_to_u32(cache).reshape(NB * BS, Hh, 4)
    want = cache0.reshape(NB * BS, Hh, 4).copy()
    ok = (slots >= 0) & (slots < NB * BS)
    codes, p64 = O.hash_encode(x, r)
    # untouched slots keep their old contents
    untouched = np.ones(NB * BS, dtype=bool)
    untouched[slots[ok]] = False
    assert np.array_equal(got[untouched], want[untouched])
    hard, soft = O.count_code_mismatches(got[slots[ok]], p64[ok], TOL)
    assert hard == 0 and soft <= 2


@pytest.mark.parametrize("G", [1, 4, 8])
def test_encode_query_group_mean(cuda_device, G):
    """Plugin query path: mean over the G heads of a group in bf16, then encode."""
    import torch
    from unified_cache_management_b200 import ops
    rng = np.random.default_rng(G)
    T, Hkv = 16, 8
    q = H.bf16_normal(rng, (T, Hkv * G, 128))
    r = _r_matrix(1)
    out = ops.hash_encode_query(H.bf16_to_dev(q, cuda_device), H.bf16_to_dev(r, cuda_device), group_mean=G)
    torch.cuda.synchronize()
    qm = O.group_mean_bf16(q, Hkv) if G > 1 else q
    _check(H.dev_to_u32(out), qm, r)


@pytest.mark.parametrize("in_dim,bits", [(64, 64), (512, 512), (128, 256), (96, 32)])
def test_encode_other_shapes(cuda_device, in_dim, bits):
    """Shapes off the tensor-core path (e.g. the 512/64-wide MLA encoders) run on CUDA cores."""
    import torch
    from unified_cache_management_b200 import ops
    rng = np.random.default_rng(in_dim + bits)
    x = H.bf16_normal(rng, (77, in_dim))
    r = _r_matrix(2, in_dim, bits)
    out = ops.hash_encode(H.bf16_to_dev(x, cuda_device), H.bf16_to_dev(r, cuda_device))
    torch.cuda.synchronize()
    _check(H.dev_to_u32(out), x, r)


def test_tensor_core_and_cuda_core_paths_agree(cuda_device):
    """Same rows through both kernels (group_mean=1 with 3 heads cannot tile 128 -> CUDA-core path)."""
    import torch
    from unified_cache_management_b200 import ops
    rng = np.random.default_rng(99)
    x = H.bf16_normal(rng, (510, 3, 128))
    r = _r_matrix(1)
    xd, rd = H.bf16_to_dev(x, cuda_device), H.bf16_to_dev(r, cuda_device)
    a = ops.hash_encode(xd.reshape(-1, 128), rd)            # tensor cores
    b = ops.hash_encode_query(xd, rd)                       # H=3 -> CUDA cores
    torch.cuda.synchronize()
    _, p64 = O.hash_encode(x.reshape(-1, 128), r)
    diff = O.unpack_bits_u32(H.dev_to_u32(a)) != O.unpack_bits_u32(H.dev_to_u32(b).reshape(-1, 4))
    assert (np.abs(p64[diff]) < TOL).all()


@pytest.mark.parametrize("G", [1, 4])
def test_decode_step_fused_encode(cuda_device, G):
    """Queries and new key rows of one decode step in one launch (group mean on the query side)."""
    import torch
    from unified_cache_management_b200 import ops
    rng = np.random.default_rng(50 + G)
    B, Hkv, NB, BS = 16, 8, 64, 128
    q = H.bf16_normal(rng, (B, Hkv * 4, 128))
    kn = H.bf16_normal(rng, (B, Hkv, 128))
    r = _r_matrix(1)
    slots = rng.permutation(NB * BS)[:B].astype(np.int64)
    cache0 = H.rand_codes(rng, (NB, BS, Hkv, 4))
    cache = H.to_dev_i32(cache0, cuda_device)
    qc = ops.hash_encode_decode_step(H.bf16_to_dev(q, cuda_device), H.bf16_to_dev(kn, cuda_device),
                                     torch.from_numpy(slots).to(cuda_device), cache, H.bf16_to_dev(r, cuda_device),
                                     group_mean=G)
    torch.cuda.synchronize()
    qm = O.group_mean_bf16(q, Hkv * 4 // G) if G > 1 else q
    _check(H.dev_to_u32(qc), qm, r)
    got = H.dev_to_u32(cache).reshape(NB * BS, Hkv, 4)
    _, p64 = O.hash_encode(kn, r)
    hard, soft = O.count_code_mismatches(got[slots], p64, TOL)
    assert hard == 0 and soft <= 2
    untouched = np.ones(NB * BS, dtype=bool)
    untouched[slots] = False
    assert np.array_equal(got[untouched], cache0.reshape(NB * BS, Hkv, 4)[untouched])


def test_decode_step_reads_pinned_host_inputs_and_writes_pinned_result(cuda_device):
    """q / new keys in page-locked host memory and the id output in page-locked host memory give the same
    codes, cache rows and selection as device-resident operands."""
    import torch
    from unified_cache_management_b200 import ops
    dev = cuda_device
    g = torch.Generator(device=dev).manual_seed(5)
    B, Hq, Hkv, D, BS, mb, k = 6, 32, 8, 128, 128, 12, 4
    R = (torch.randn((D, 128), device=dev, generator=g) / D ** 0.5).to(torch.bfloat16)
    q = torch.randn((B, Hq, D), device=dev, generator=g).to(torch.bfloat16)
    kn = torch.randn((B, Hkv, D), device=dev, generator=g).to(torch.bfloat16)
    NB = B * mb
    cache_a = torch.randint(-2**31, 2**31 - 1, (NB, BS, Hkv, 4), dtype=torch.int32, device=dev, generator=g)
    cache_b = cache_a.clone()
    bt = torch.randperm(NB, device=dev, generator=g).to(torch.int32).view(B, mb)
    seq = torch.full((B,), mb * BS, dtype=torch.int32, device=dev)
    slots = bt[:, -1].to(torch.int64) * BS + BS - 1
    qa = ops.hash_encode_decode_step(q, kn, slots, cache_a, R)
    qb = ops.hash_encode_decode_step(q.cpu().pin_memory(), kn.cpu().pin_memory(), slots, cache_b, R)
    assert qb.is_cuda and torch.equal(qa, qb) and torch.equal(cache_a, cache_b)
    ra = ops.hamming_topk(cache_a, qa, bt, seq, k, must_select=(0, -1))
    host_ids = torch.empty((B, Hkv, k), dtype=torch.int32).pin_memory()
    rb = ops.Retrieval(physical=host_ids, logical=torch.empty_like(ra.logical), scores=None,
                       valid_count=torch.empty_like(ra.valid_count), new_seq_lens=torch.empty_like(ra.new_seq_lens))
    ops.hamming_topk(cache_b, qb, bt, seq, k, must_select=(0, -1), out=rb, want_scores=False)
    torch.cuda.synchronize()
    assert torch.equal(ra.physical.cpu(), host_ids) and torch.equal(ra.logical, rb.logical)
    with pytest.raises(ValueError):
        ops.hash_encode_decode_step(q.cpu(), kn, slots, cache_b, R)   # pageable host memory is refused


@pytest.mark.parametrize("BS,Hh,dims,strided", [
    (128, 8, (128, 128), False),  # eight tiles per block
    (16, 8, (128, 128), False),   # one tile per block (vLLM block 16)
    (16, 1, (128, 128), False),   # eight blocks per tile (one kv head per GPU)
    (16, 2, (128, 128), True),    # four blocks per tile, K sliced out of a [NB, 2, BS, H, D] cache
    (64, 4, (128, 128), True),
    (32, 2, (64, 64), False),     # other code sizes: CUDA-core kernel
    (24, 3, (128, 128), False),   # rows per block not a tile divisor: CUDA-core kernel
])
def test_rehash_blocks_in_place(cuda_device, BS, Hh, dims, strided):
    """Prefix-hit re-hash: codes of listed K-cache blocks written to the same blocks of the code cache; the
    last block of each request is partial; unlisted blocks and the tails of partial blocks keep their content;
    ids outside the cache are flagged and skipped."""
    import torch
    from unified_cache_management_b200 import ops
    dev = cuda_device
    D, bits = dims
    rng = np.random.default_rng(BS * 100 + Hh)
    NB = 40
    kv = H.bf16_normal(rng, (NB, 2, BS, Hh, D)) if strided else H.bf16_normal(rng, (NB, BS, Hh, D))
    r = _r_matrix(3, D, bits)
    kv_d = H.bf16_to_dev(kv, dev)
    k_d = kv_d[:, 0] if strided else kv_d
    k_host = kv[:, 0] if strided else kv
    ids = np.array([7, 3, 39, 0, 12, 21, 5, 30, 8, 17, 2], dtype=np.int32)
    toks = np.full(ids.shape, BS, dtype=np.int32)
    toks[4] = 1
    toks[-1] = BS - 3
    W = bits // 32
    sentinel = np.uint32(0xDEADBEEF)
    cache = torch.full((NB, BS, Hh, W), int(np.int32(sentinel.view(np.int32))), dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    ops.hash_encode_blocks(k_d, torch.from_numpy(ids).to(dev), cache, H.bf16_to_dev(r, dev),
                           block_tokens=torch.from_numpy(toks).to(dev), status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    got = H.dev_to_u32(cache)
    listed = np.zeros((NB, BS), dtype=bool)
    for i, n in zip(ids, toks):
        listed[i, :n] = True
    assert (got[~listed] == sentinel).all()
    _check(got[listed], k_host[listed], r)
    # all tokens when block_tokens is omitted; a bad id is flagged, the others still land
    cache.fill_(0)
    ids2 = np.array([4, -1, 9, NB, 1], dtype=np.int32)
    ops.hash_encode_blocks(k_d, torch.from_numpy(ids2).to(dev), cache, H.bf16_to_dev(r, dev), status=status)
    torch.cuda.synchronize()
    assert int(status.item()) & 1
    got = H.dev_to_u32(cache)
    good = [4, 9, 1]
    _check(got[good], k_host[good], r)
    rest = np.ones(NB, dtype=bool)
    rest[good] = False
    assert (got[rest] == 0).all()


@pytest.mark.parametrize("in_dim,bits", [(512, 512), (256, 384), (128, 256), (384, 128)])
def test_wide_projection_tensor_core_path(cuda_device, in_dim, bits):
    """Projections wider than 128 x 128 with enough rows take the chunked tensor-core kernel (each CTA holds a
    128-column chunk of R); rows with a stride, and a ragged last tile."""
    import torch
    from unified_cache_management_b200 import ops
    rng = np.random.default_rng(in_dim + bits)
    rows = 128 * 37 + 53
    x = H.bf16_normal(rng, (rows, in_dim + 64))
    r = _r_matrix(5, in_dim, bits)
    xd = H.bf16_to_dev(x, cuda_device)[:, :in_dim]          # row stride in_dim + 64
    out = ops.hash_encode(xd, H.bf16_to_dev(r, cuda_device))
    torch.cuda.synchronize()
    _check(H.dev_to_u32(out), x[:, :in_dim], r)


def test_mla_rows_latent_and_rope_codes_side_by_side(cuda_device):
    """512-bit and 64-bit codes written at words 0 and 16 of 18-word cache rows, through the slot mapping; enough
    tokens for the tensor-core kernel on the latent part.  Skipped slots and the other rows stay untouched."""
    import torch
    from unified_cache_management_b200 import ops
    dev = cuda_device
    rng = np.random.default_rng(99)
    T, NB, BS = 3000, 64, 64
    nope, rope = H.bf16_normal(rng, (T, 1, 512)), H.bf16_normal(rng, (T, 1, 64))
    rn, rr = _r_matrix(6, 512, 512), _r_matrix(7, 64, 64)
    slots = rng.permutation(NB * BS)[:T].astype(np.int64)
    slots[5] = -1
    slots[77] = NB * BS + 3
    cache = torch.full((NB, BS, 1, 18), 0x5A5A5A5A, dtype=torch.int32, device=dev)
    sd = torch.from_numpy(slots).to(dev)
    ops.hash_encode_and_cache(H.bf16_to_dev(nope, dev), sd, cache, H.bf16_to_dev(rn, dev), word_offset=0)
    ops.hash_encode_and_cache(H.bf16_to_dev(rope, dev), sd, cache, H.bf16_to_dev(rr, dev), word_offset=16)
    torch.cuda.synchronize()
    got = H.dev_to_u32(cache).reshape(NB * BS, 18)
    ok = (slots >= 0) & (slots < NB * BS)
    _check(got[slots[ok], :16], nope[ok, 0], rn)
    _check(got[slots[ok], 16:], rope[ok, 0], rr)
    rest = np.ones(NB * BS, dtype=bool)
    rest[slots[ok]] = False
    assert (got[rest] == 0x5A5A5A5A).all()
    with pytest.raises(ValueError):
        ops.hash_encode_and_cache(H.bf16_to_dev(rope, dev), sd, cache, H.bf16_to_dev(rr, dev), word_offset=17)

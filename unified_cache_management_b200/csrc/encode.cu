// Hash encode (sm_100a): codes = signbits(X * R), X bf16 rows, R bf16 [in_dim, hash_bits].
//
// Tensor-core path (in_dim = hash_bits = 128): persistent, warp-specialised CTA per SM.
//   warp 0   TMA producer: 128-row X tiles (two 64-column boxes, 128-byte swizzle) into a ring of
//            shared-memory stages.
//   warp 1   allocates TMEM; one thread issues eight tcgen05.mma (M=128, N=128, K=16) per tile into
//            one of two 128-column fp32 accumulators and commits to the stage's / accumulator's
//            mbarrier.
//   warps 2-5 epilogue: tcgen05.ld gives each thread one full row of the accumulator; the thread
//            packs the 128 sign bits into four words and issues a single 16-byte store (to the
//            output array, or to the row's slot in the paged code cache).
// R^T is written once per CTA into shared memory in the K-major 128-byte-swizzled layout the MMA
// descriptors expect; every CTA keeps its own copy.  X is read exactly once from HBM; the only
// other traffic is 16 bytes per row out.  All mbarrier waits are time-bounded.
//
// CUDA-core path: any in_dim / hash_bits (multiples of 32), optional group mean over G query heads
// with one rounding to bf16; used for the decode-step query codes of the plugin path and for
// shapes the tensor-core path does not cover.
//
// Stands in for triton_hash_code_kernel, fused_hash_and_cache_kernel and
// _reshape_and_cache_khash_kernel (ucm/sparse/gsa_on_device/hash_encoder.py:37-134, 263-356,
// 136-261); numerics follow torch_hash_code (:359-370): fp32 accumulate, strict "> 0".
#include <stdlib.h>

#include <cuda.h>
#include <cuda_bf16.h>

#include "common.cuh"

namespace ucmr {

// ---------------------------------------------------------------------------------------------
// tensor-core path
// ---------------------------------------------------------------------------------------------
constexpr int kEncTileM = 128;
constexpr int kEncD = 128;      // in_dim
constexpr int kEncBits = 128;   // hash_bits
constexpr int kEncStages = 5;   // X ring depth (32 KiB each)
constexpr int kEncAccs = 2;     // TMEM accumulators
constexpr int kEncThreads = 192;
constexpr int kEncHalfBytes = kEncTileM * 128;          // one 64-column box: 128 rows x 128 B
constexpr int kEncStageBytes = 2 * kEncHalfBytes;       // 32 KiB
constexpr int kEncTmemCols = kEncAccs * kEncBits;       // 256
constexpr size_t kEncSmemBytes = 1024 /*align slack*/ + 2 * kEncHalfBytes /*R^T*/ +
                                 (size_t)kEncStages * kEncStageBytes + 256 /*barriers*/;

struct EncParams {
    int64_t rows;    // T * H
    int H;           // rows per token (heads)
    int64_t n_tiles;
    uint32_t* out;   // direct: [rows, 4]; paged: cache [NB*BS, H, 4]
    const void* slot_mapping;  // null = direct
    int slot_is_int64;
    int64_t n_slots;           // NB * BS
    const __nv_bfloat16* R;    // [128, 128] row-major
    int32_t* status;           // may be null
    // Paged source (re-hash of blocks that already sit in the K cache): the tiles walk the rows of the listed
    // blocks, block i of the list being block src_blocks[i] of the source AND of the code cache.
    const int32_t* src_blocks;    // null = x is one run of consecutive tokens
    const int32_t* block_tokens;  // valid tokens per listed block, null = all BS
    int64_t n_src_blocks;
    int64_t NB_src;
    int BS;                       // tokens per block
    int rpb;                      // rows per block = BS * H (a multiple of 8; divides or is a multiple of 128)
};

__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr)
{
    // K-major, 128-byte swizzle: start address >> 4, leading byte offset 1 (unused), stride byte
    // offset 1024 >> 4 between 8-row groups, descriptor version 1, layout type 2 (SWIZZLE_128B).
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

// kind::f16 instruction descriptor: D = f32, A = B = bf16, both K-major, N = 128, M = 128.
constexpr uint32_t kEncIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((kEncBits >> 3) << 17) | ((kEncTileM >> 4) << 24);

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, int x, int y, int z,
                                            uint64_t* bar)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::
            "r"(smem_u32(smem_dst)),
        "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, int x, int y, int z, int w,
                                            uint64_t* bar)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::
            "r"(smem_u32(smem_dst)),
        "l"(map), "r"(x), "r"(y), "r"(z), "r"(w), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void tc_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ uint32_t pack_signs(const uint32_t (&r)[32])
{
    uint32_t w = 0;
#pragma unroll
    for (int i = 0; i < 32; ++i) w |= (uint32_t)(__uint_as_float(r[i]) > 0.0f) << i;
    return w;
}


// R[k][n] (row-major bf16, row stride ldr elements) -> B[n][k], K-major with the 128-byte swizzle the MMA descriptors
// expect: row n holds 64 k-values (128 bytes) per K half, and its 16-byte chunk c lives at chunk c ^ (n & 7).
// The unit of work is an 8x8 block (rows k = 8 kc .. 8 kc + 7, columns n0 + 8 nc .. + 7): eight 16-byte loads in,
// a register transpose, eight 16-byte stores out.  The two halves are separate so that a kernel may issue the loads
// early and the transposing stores late, with other memory traffic in between.
__device__ __forceinline__ void rt_block_load(uint4 (&v)[8], const __nv_bfloat16* R, int ldr, int n0, int kc, int nc)
{
#pragma unroll
    for (int r = 0; r < 8; ++r)
        v[r] = __ldg(reinterpret_cast<const uint4*>(R + (size_t)(kc * 8 + r) * ldr + n0 + nc * 8));
}

__device__ __forceinline__ void rt_block_store(uint8_t* s_b, const uint4 (&v)[8], int kc, int nc)
{
    const int half = kc >> 3, chunk = kc & 7;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t sel = (j & 1) ? 0x7632u : 0x5410u;  // low or high bf16 of each 32-bit pair
        const auto word = [&](int r) { return reinterpret_cast<const uint32_t*>(&v[r])[j >> 1]; };
        uint4 o;
        o.x = __byte_perm(word(0), word(1), sel);
        o.y = __byte_perm(word(2), word(3), sel);
        o.z = __byte_perm(word(4), word(5), sel);
        o.w = __byte_perm(word(6), word(7), sel);
        const int n = nc * 8 + j;
        const uint32_t off = (uint32_t)half * kEncHalfBytes + (uint32_t)n * 128u + ((uint32_t)(chunk ^ (n & 7)) << 4);
        *reinterpret_cast<uint4*>(s_b + off) = o;
    }
}

// Columns [n0, n0 + 128) of R[K][N] -> swizzled B, all threads of the CTA taking 8x8 blocks in turn.
__device__ __forceinline__ void build_rt_chunk_swizzled(uint8_t* s_b, const __nv_bfloat16* R, int K, int N, int n0,
                                                        int tid, int nthreads)
{
    for (int blk = tid; blk < (K / 8) * (kEncBits / 8); blk += nthreads) {
        const int kc = blk / (kEncBits / 8), nc = blk % (kEncBits / 8);
        uint4 v[8];
        rt_block_load(v, R, N, n0, kc, nc);
        rt_block_store(s_b, v, kc, nc);
    }
}

// The whole 128 x 128 matrix.
__device__ __forceinline__ void build_rt_swizzled(uint8_t* s_b, const __nv_bfloat16* R, int tid, int nthreads)
{
    build_rt_chunk_swizzled(s_b, R, kEncD, kEncBits, 0, tid, nthreads);
}

// The whole matrix by 128 threads in two steps (two 8x8 blocks per thread): loads first, stores later.
__device__ __forceinline__ void rt_load_128(uint4 (&v)[2][8], const __nv_bfloat16* R, int tid)
{
#pragma unroll
    for (int it = 0; it < 2; ++it) {
        const int blk = tid + it * 128;
        rt_block_load(v[it], R, kEncBits, 0, blk / (kEncBits / 8), blk % (kEncBits / 8));
    }
}

__device__ __forceinline__ void rt_store_128(uint8_t* s_b, const uint4 (&v)[2][8], int tid)
{
#pragma unroll
    for (int it = 0; it < 2; ++it) {
        const int blk = tid + it * 128;
        rt_block_store(s_b, v[it], blk / (kEncBits / 8), blk % (kEncBits / 8));
    }
}

__global__ void __launch_bounds__(kEncThreads, 1)
encode_tc_kernel(const __grid_constant__ CUtensorMap x_map, const EncParams p)
{
    extern __shared__ uint8_t s_raw[];
    // 1024-byte alignment: the swizzle pattern is a function of the shared-memory address bits
    uint8_t* s_base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(s_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* s_b = s_base;                                  // R^T, two K halves of [128 n][64 k]
    uint8_t* s_a = s_base + 2 * kEncHalfBytes;              // stages
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_a + (size_t)kEncStages * kEncStageBytes);
    uint64_t* full = bars;                       // [kEncStages]
    uint64_t* empty = bars + kEncStages;         // [kEncStages]
    uint64_t* acc_full = bars + 2 * kEncStages;  // [kEncAccs]
    uint64_t* acc_empty = acc_full + kEncAccs;   // [kEncAccs]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + kEncAccs);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const int64_t first = blockIdx.x, step = gridDim.x;
    const int64_t my_tiles = first < p.n_tiles ? (p.n_tiles - first + step - 1) / step : 0;
    const int tok_per_tile = kEncTileM / p.H;
    // Starts the copy of this CTA's it-th tile into its stage (which must be free).  Thread 0 only.
    auto issue_tile = [&](int64_t it) {
        const int s = (int)(it % kEncStages);
        const int64_t tile = first + it * step;
        uint8_t* dst = s_a + (size_t)s * kEncStageBytes;
        mbar_expect_tx(&full[s], kEncStageBytes);
        if (p.src_blocks == nullptr) {
            const int t0 = (int)(tile * tok_per_tile);
            tma_load_3d(dst, &x_map, 0, 0, t0, &full[s]);
            tma_load_3d(dst + kEncHalfBytes, &x_map, 64, 0, t0, &full[s]);
        } else if (p.rpb >= kEncTileM) {
            // the tile is one slice of one listed block
            const int parts = p.rpb / kEncTileM;
            const int64_t bi = tile / parts;
            int id = p.src_blocks[bi];
            if (id < 0 || id >= p.NB_src) id = 0;  // rows of a bad id are dropped by the epilogue
            const int tok0 = (int)(tile - bi * parts) * tok_per_tile;
            tma_load_4d(dst, &x_map, 0, 0, tok0, id, &full[s]);
            tma_load_4d(dst + kEncHalfBytes, &x_map, 64, 0, tok0, id, &full[s]);
        } else {
            // the tile holds several whole blocks, each a box of rpb rows
            const int sub = kEncTileM / p.rpb;
            for (int u = 0; u < sub; ++u) {
                const int64_t bi = tile * sub + u;
                int id = bi < p.n_src_blocks ? p.src_blocks[bi] : 0;
                if (id < 0 || id >= p.NB_src) id = 0;
                uint8_t* d = dst + (size_t)u * p.rpb * 128;
                tma_load_4d(d, &x_map, 0, 0, 0, id, &full[s]);
                tma_load_4d(d + kEncHalfBytes, &x_map, 64, 0, 0, id, &full[s]);
            }
        }
    };
    int64_t prefilled = 0;  // (thread 0) tiles whose copies were started before the set-up below
    if (tid == 0) {
        for (int s = 0; s < kEncStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int a = 0; a < kEncAccs; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 4); }
        fence_mbar_init();
        asm volatile("prefetch.tensormap [%0];" ::"l"(&x_map) : "memory");
        // every stage is free at the start: the first tiles travel while the CTA transposes R and allocates TMEM
        // (a few microseconds during which the copy engine would otherwise idle)
        for (; prefilled < my_tiles && prefilled < kEncStages; ++prefilled) issue_tile(prefilled);
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)kEncTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    build_rt_swizzled(s_b, p.R, tid, kEncThreads);
    fence_proxy_async();  // generic-proxy writes of R^T become visible to the MMA's async-proxy reads
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            for (int64_t it = prefilled; it < my_tiles; ++it) {
                const int s = (int)(it % kEncStages);
                const uint32_t ph = (uint32_t)((it / kEncStages) & 1);
                if (!mbar_wait(&empty[s], ph ^ 1u)) { flag_status(p.status, UCMR_DEV_WAIT_TIMEOUT); break; }
                issue_tile(it);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t b_addr = smem_u32(s_b);
            for (int64_t it = 0; it < my_tiles; ++it) {
                const int s = (int)(it % kEncStages);
                const uint32_t ph = (uint32_t)((it / kEncStages) & 1);
                const int a = (int)(it % kEncAccs);
                const uint32_t aph = (uint32_t)((it / kEncAccs) & 1);
                if (!mbar_wait(&acc_empty[a], aph ^ 1u) || !mbar_wait(&full[s], ph)) {
                    flag_status(p.status, UCMR_DEV_WAIT_TIMEOUT);
                    break;
                }
                tc_fence_after();
                const uint32_t a_addr = smem_u32(s_a + (size_t)s * kEncStageBytes);
                const uint32_t d_tmem = tmem_base + (uint32_t)(a * kEncBits);
#pragma unroll
                for (int half = 0; half < 2; ++half) {
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        const uint32_t off = (uint32_t)half * kEncHalfBytes + (uint32_t)ks * 32u;
                        tc_mma_bf16(d_tmem, make_smem_desc_sw128(a_addr + off), make_smem_desc_sw128(b_addr + off),
                                    kEncIdesc, (half | ks) ? 1u : 0u);
                    }
                }
                tc_commit(&empty[s]);     // the stage may be refilled once these MMAs have read it
                tc_commit(&acc_full[a]);  // the accumulator is complete
            }
        }
    } else {
        const int q = warp & 3;  // TMEM lane quadrant this warp may read
        for (int64_t it = 0; it < my_tiles; ++it) {
            const int a = (int)(it % kEncAccs);
            const uint32_t aph = (uint32_t)((it / kEncAccs) & 1);
            // Where this thread's row goes is looked up before waiting for the accumulator: the slot is a dependent
            // global load, and after the wait it would sit on the epilogue's critical path for every tile.
            const int64_t tile_pre = first + it * step;
            const int in_tile = q * 32 + lane;
            const int64_t tok_pre = tile_pre * tok_per_tile + in_tile / p.H;  // (a tile holds whole tokens)
            int64_t slot_pre = -1;
            if (p.src_blocks == nullptr && p.slot_mapping != nullptr && tile_pre * kEncTileM + in_tile < p.rows)
                slot_pre = p.slot_is_int64 ? static_cast<const int64_t*>(p.slot_mapping)[tok_pre]
                                           : (int64_t) static_cast<const int32_t*>(p.slot_mapping)[tok_pre];
            if (!mbar_wait(&acc_full[a], aph)) { flag_status(p.status, UCMR_DEV_WAIT_TIMEOUT); break; }
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * kEncBits);
            // the row's 128 accumulator columns in one round trip; the accumulator goes back to the MMA thread before
            // the sign bits are packed
            uint4 code;
            uint32_t r0[32], r1[32], r2[32], r3[32];
            tc_ld32(taddr + 0, r0);
            tc_ld32(taddr + 32, r1);
            tc_ld32(taddr + 64, r2);
            tc_ld32(taddr + 96, r3);
            tc_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[a]);
            code.x = pack_signs(r0);
            code.y = pack_signs(r1);
            code.z = pack_signs(r2);
            code.w = pack_signs(r3);
            const int64_t tile = first + it * step;
            const int64_t row = tile * kEncTileM + q * 32 + lane;
            if (p.src_blocks != nullptr) {
                const int64_t bi = row / p.rpb;
                if (bi < p.n_src_blocks) {
                    const int within = (int)(row - bi * p.rpb);
                    const int tok = within / p.H, h = within - tok * p.H;
                    const int id = p.src_blocks[bi];
                    const int ntok = p.block_tokens ? p.block_tokens[bi] : p.BS;
                    if (id < 0 || id >= p.NB_src) {
                        if (within == 0) flag_status(p.status, UCMR_DEV_BAD_BLOCK_ID);
                    } else if (tok < ntok) {
                        const int64_t slot = (int64_t)id * p.BS + tok;
                        if (slot < p.n_slots) *reinterpret_cast<uint4*>(p.out + (slot * p.H + h) * 4) = code;
                    }
                }
            } else if (row < p.rows) {
                if (p.slot_mapping == nullptr) {
                    *reinterpret_cast<uint4*>(p.out + row * 4) = code;
                } else {
                    const int h = in_tile % p.H;
                    const int64_t slot = slot_pre;
                    if (slot >= 0 && slot < p.n_slots)
                        *reinterpret_cast<uint4*>(p.out + (slot * p.H + h) * 4) = code;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kEncTmemCols)
                     : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
// tensor-core path for wide projections (in_dim and hash_bits multiples of 128, up to 512 x 512)
// ---------------------------------------------------------------------------------------------
// The MLA latent encoder is 512 -> 512 bits: 480 flop per byte of input, i.e. tensor-bound, and its R (512 KiB)
// does not fit in shared memory.  Each CTA keeps one 128-column chunk of R^T resident (in_dim x 128, K-major,
// swizzled: 128 KiB at in_dim 512) and streams token tiles through a ring of 128-row x 128-k stages,
// accumulating the in_dim/128 slices of a tile in TMEM; the hash_bits/128 CTAs with consecutive block ids work
// on the same token tile at about the same time, so the tile is fetched from HBM once and re-read from L2.
// Same warp roles and barriers as encode_tc_kernel.  Output rows may be wider than the code (row_words,
// word_offset): the chunk's four words go to words [word_offset + 4*chunk, +4) of the row.
constexpr int kWideStages = 3;
constexpr int kWideMaxK = 512;
constexpr size_t kWideSmemBytes = 1024 + (size_t)(kWideMaxK / 64) * kEncHalfBytes + (size_t)kWideStages * kEncStageBytes + 256;

struct WideParams {
    int64_t rows;      // tokens (one row per token)
    int64_t n_tiles;   // token tiles of 128
    int K, N;          // in_dim, hash_bits
    int n_chunks;      // N / 128
    uint32_t* out;
    int row_words, word_offset;
    const void* slot_mapping;  // null = row t of out is token t
    int slot_is_int64;
    int64_t n_slots;
    const __nv_bfloat16* R;    // [K, N] row-major
    int32_t* status;
};

__global__ void __launch_bounds__(kEncThreads, 1)
encode_wide_kernel(const __grid_constant__ CUtensorMap x_map, const WideParams p)
{
    extern __shared__ uint8_t s_raw[];
    uint8_t* s_base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(s_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* s_b = s_base;                                            // R^T chunk: K/64 blocks of [128 n][64 k]
    uint8_t* s_a = s_base + (size_t)(kWideMaxK / 64) * kEncHalfBytes; // stages: 128 rows x 128 k
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_a + (size_t)kWideStages * kEncStageBytes);
    uint64_t* full = bars;
    uint64_t* empty = bars + kWideStages;
    uint64_t* acc_full = bars + 2 * kWideStages;
    uint64_t* acc_empty = acc_full + kEncAccs;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + kEncAccs);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int chunk = blockIdx.x % p.n_chunks;
    const int k_slices = p.K / 128;

    if (tid == 0) {
        for (int s = 0; s < kWideStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int a = 0; a < kEncAccs; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 4); }
        fence_mbar_init();
        asm volatile("prefetch.tensormap [%0];" ::"l"(&x_map) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)kEncTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    build_rt_chunk_swizzled(s_b, p.R, p.K, p.N, chunk * kEncBits, tid, kEncThreads);
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int64_t first = blockIdx.x / p.n_chunks, step = gridDim.x / p.n_chunks;
    const int64_t my_tiles = first < p.n_tiles ? (p.n_tiles - first + step - 1) / step : 0;

    if (warp == 0) {
        if (lane == 0) {
            int64_t slot_it = 0;
            bool ok = true;
            for (int64_t it = 0; it < my_tiles && ok; ++it) {
                const int t0 = (int)((first + it * step) * kEncTileM);
                for (int ks = 0; ks < k_slices; ++ks, ++slot_it) {
                    const int s = (int)(slot_it % kWideStages);
                    const uint32_t ph = (uint32_t)((slot_it / kWideStages) & 1);
                    if (!mbar_wait(&empty[s], ph ^ 1u)) { flag_status(p.status, UCMR_DEV_WAIT_TIMEOUT); ok = false; break; }
                    uint8_t* dst = s_a + (size_t)s * kEncStageBytes;
                    mbar_expect_tx(&full[s], kEncStageBytes);
                    tma_load_3d(dst, &x_map, ks * 128, 0, t0, &full[s]);
                    tma_load_3d(dst + kEncHalfBytes, &x_map, ks * 128 + 64, 0, t0, &full[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t b_addr = smem_u32(s_b);
            int64_t slot_it = 0;
            bool ok = true;
            for (int64_t it = 0; it < my_tiles && ok; ++it) {
                const int a = (int)(it % kEncAccs);
                const uint32_t aph = (uint32_t)((it / kEncAccs) & 1);
                if (!mbar_wait(&acc_empty[a], aph ^ 1u)) { flag_status(p.status, UCMR_DEV_WAIT_TIMEOUT); break; }
                const uint32_t d_tmem = tmem_base + (uint32_t)(a * kEncBits);
                for (int ks = 0; ks < k_slices; ++ks, ++slot_it) {
                    const int s = (int)(slot_it % kWideStages);
                    const uint32_t ph = (uint32_t)((slot_it / kWideStages) & 1);
                    if (!mbar_wait(&full[s], ph)) { flag_status(p.status, UCMR_DEV_WAIT_TIMEOUT); ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(s_a + (size_t)s * kEncStageBytes);
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            const uint32_t a_off = (uint32_t)half * kEncHalfBytes + (uint32_t)kk * 32u;
                            const uint32_t b_off = (uint32_t)(ks * 2 + half) * kEncHalfBytes + (uint32_t)kk * 32u;
                            tc_mma_bf16(d_tmem, make_smem_desc_sw128(a_addr + a_off), make_smem_desc_sw128(b_addr + b_off),
                                        kEncIdesc, (ks | half | kk) ? 1u : 0u);
                        }
                    }
                    tc_commit(&empty[s]);
                }
                if (ok) tc_commit(&acc_full[a]);
            }
        }
    } else {
        const int q = warp & 3;
        for (int64_t it = 0; it < my_tiles; ++it) {
            const int a = (int)(it % kEncAccs);
            const uint32_t aph = (uint32_t)((it / kEncAccs) & 1);
            if (!mbar_wait(&acc_full[a], aph)) { flag_status(p.status, UCMR_DEV_WAIT_TIMEOUT); break; }
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * kEncBits);
            uint32_t code[4];
            uint32_t r[32];
            tc_ld32(taddr + 0, r);  tc_wait_ld(); code[0] = pack_signs(r);
            tc_ld32(taddr + 32, r); tc_wait_ld(); code[1] = pack_signs(r);
            tc_ld32(taddr + 64, r); tc_wait_ld(); code[2] = pack_signs(r);
            tc_ld32(taddr + 96, r); tc_wait_ld(); code[3] = pack_signs(r);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[a]);
            const int64_t row = (first + it * step) * kEncTileM + q * 32 + lane;
            if (row < p.rows) {
                int64_t dst = row;
                if (p.slot_mapping != nullptr) {
                    const int64_t slot = p.slot_is_int64 ? static_cast<const int64_t*>(p.slot_mapping)[row]
                                                         : (int64_t) static_cast<const int32_t*>(p.slot_mapping)[row];
                    dst = (slot >= 0 && slot < p.n_slots) ? slot : -1;
                }
                if (dst >= 0) {
                    uint32_t* o = p.out + dst * p.row_words + p.word_offset + chunk * 4;
                    if ((reinterpret_cast<uintptr_t>(o) & 7u) == 0) {
                        reinterpret_cast<uint2*>(o)[0] = make_uint2(code[0], code[1]);
                        reinterpret_cast<uint2*>(o)[1] = make_uint2(code[2], code[3]);
                    } else {
                        o[0] = code[0]; o[1] = code[1]; o[2] = code[2]; o[3] = code[3];
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kEncTmemCols)
                     : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
// tensor-core path for small row counts: one 128-row tile per CTA, up to two jobs per launch
// ---------------------------------------------------------------------------------------------
// A decode step encodes a few hundred rows (the batch's query heads and its new key rows).  The persistent
// kernel above would spend its time on set-up, and two launches cost more than the math.  Here every CTA
// builds its A tile with plain 16-byte loads (optionally averaging G consecutive heads with one rounding
// to bf16, which is how the plugin hashes a GQA query group), writes it swizzled next to R^T, issues the
// eight MMAs and packs the signs.  Both jobs of a step (queries -> code array, new keys -> paged cache)
// share one launch.
constexpr int kTileThreads = 128;
constexpr size_t kTileSmemBytes = 1024 + 2 * kEncHalfBytes + kEncStageBytes + 64;

struct TileJob {
    const __nv_bfloat16* x;
    int64_t T;
    int H_in, G;
    int64_t stride_t, stride_h;
    uint32_t* out;
    const void* slot_mapping;  // null = write row r of the job to out[r]
    int slot_is_int64;
    int64_t n_slots;
    int64_t tiles;  // 128-row tiles of this job
};

struct TileParams {
    TileJob job[2];
    const __nv_bfloat16* R;
    int32_t* status;
};

__global__ void __launch_bounds__(kTileThreads) encode_tile_kernel(const TileParams p)
{
    extern __shared__ uint8_t s_raw[];
    uint8_t* s_base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(s_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* s_b = s_base;
    uint8_t* s_a = s_base + 2 * kEncHalfBytes;
    uint64_t* done = reinterpret_cast<uint64_t*>(s_a + kEncStageBytes);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    grid_launch_dependents();  // a scan launched right after this kernel may set itself up meanwhile
    const bool second = (int64_t)blockIdx.x >= p.job[0].tiles;
    // (a copy picked with compile-time offsets: a run-time index into the kernel parameter would turn every field
    // access into a load through a generic address, which is slow)
    const TileJob jb = second ? p.job[1] : p.job[0];
    const int64_t tile = (int64_t)blockIdx.x - (second ? p.job[0].tiles : 0);
    const int H_out = jb.H_in / jb.G;
    const int64_t rows = jb.T * H_out;
    const int64_t row0 = tile * kEncTileM;

    if (tid == 0) { mbar_init(done, 1); fence_mbar_init(); }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)kEncBits)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // Every global load of the kernel is issued before the first dependent instruction: R (32 KiB, through L2), the
    // destination slot of the thread's output row, then the A tile (possibly across the bus from host memory);
    // the kernel then costs about one memory round trip plus the MMA.
    static_assert(kTileThreads == 128, "rt_load_128 / rt_store_128 assume 128 threads");
    uint4 vr[2][8];
    rt_load_128(vr, p.R, tid);
    int64_t my_slot = -1;
    {
        const int64_t row = row0 + tid;  // the row this thread writes in the epilogue (warp * 32 + lane = tid)
        if (jb.slot_mapping != nullptr && row < rows) {
            const int64_t tok = row / H_out;
            my_slot = jb.slot_is_int64 ? static_cast<const int64_t*>(jb.slot_mapping)[tok]
                                       : (int64_t) static_cast<const int32_t*>(jb.slot_mapping)[tok];
        }
    }
    // A tile: row r of the tile, 16-byte chunk c (8 elements) -> K half c >> 3, chunk (c & 7) ^ (r & 7).
    const int64_t t_base = row0 / H_out;
    const int h_base = (int)(row0 - t_base * H_out);
    constexpr int kChunksPerThread = kEncTileM * (kEncD / 8) / kTileThreads;  // 16
    auto src_of = [&](int r, int c) -> const __nv_bfloat16* {
        const int hh = h_base + r;
        const int64_t t = t_base + hh / H_out;
        const int ho = hh % H_out;
        return jb.x + t * jb.stride_t + (int64_t)ho * jb.G * jb.stride_h + c * 8;
    };
    auto dst_of = [&](int r, int c) -> uint4* {
        return reinterpret_cast<uint4*>(s_a + (uint32_t)(c >> 3) * kEncHalfBytes + (uint32_t)r * 128u +
                                        ((uint32_t)((c & 7) ^ (r & 7)) << 4));
    };
    if (jb.G == 1) {
        uint4 v[kChunksPerThread];
#pragma unroll
        for (int u = 0; u < kChunksPerThread; ++u) {
            const int i = tid + u * kTileThreads, r = i >> 4, c = i & 15;
            v[u] = make_uint4(0u, 0u, 0u, 0u);
            if (row0 + r < rows) v[u] = __ldg(reinterpret_cast<const uint4*>(src_of(r, c)));
        }
#pragma unroll
        for (int u = 0; u < kChunksPerThread; ++u) {
            const int i = tid + u * kTileThreads;
            *dst_of(i >> 4, i & 15) = v[u];
        }
    } else {
        constexpr int kBatch = 4;  // chunks whose G loads are in flight together
        for (int u0 = 0; u0 < kChunksPerThread; u0 += kBatch) {
            float acc[kBatch][8];
#pragma unroll
            for (int u = 0; u < kBatch; ++u)
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[u][e] = 0.f;
            for (int g0 = 0; g0 < jb.G; g0 += 4) {
                uint4 ld[kBatch][4];
#pragma unroll
                for (int u = 0; u < kBatch; ++u) {
                    const int i = tid + (u0 + u) * kTileThreads, r = i >> 4, c = i & 15;
                    const __nv_bfloat16* src = src_of(r, c);
#pragma unroll
                    for (int gg = 0; gg < 4; ++gg) {
                        ld[u][gg] = make_uint4(0u, 0u, 0u, 0u);
                        if (row0 + r < rows && g0 + gg < jb.G)
                            ld[u][gg] = __ldg(reinterpret_cast<const uint4*>(src + (int64_t)(g0 + gg) * jb.stride_h));
                    }
                }
#pragma unroll
                for (int u = 0; u < kBatch; ++u)
#pragma unroll
                    for (int gg = 0; gg < 4; ++gg) {
                        const __nv_bfloat16* ue = reinterpret_cast<const __nv_bfloat16*>(&ld[u][gg]);
#pragma unroll
                        for (int e = 0; e < 8; ++e) acc[u][e] += __bfloat162float(ue[e]);  // + 0 past G
                    }
            }
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const int i = tid + (u0 + u) * kTileThreads;
                uint4 v;
                __nv_bfloat16* ve = reinterpret_cast<__nv_bfloat16*>(&v);
#pragma unroll
                for (int e = 0; e < 8; ++e) ve[e] = __float2bfloat16_rn(acc[u][e] / (float)jb.G);
                *dst_of(i >> 4, i & 15) = v;
            }
        }
    }
    rt_store_128(s_b, vr, tid);
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (tid == 0) {
        const uint32_t a_addr = smem_u32(s_a), b_addr = smem_u32(s_b);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                const uint32_t off = (uint32_t)half * kEncHalfBytes + (uint32_t)ks * 32u;
                tc_mma_bf16(tmem_base, make_smem_desc_sw128(a_addr + off), make_smem_desc_sw128(b_addr + off), kEncIdesc,
                            (half | ks) ? 1u : 0u);
            }
        }
        tc_commit(done);
    }
    bool ok = mbar_wait(done, 0);
    if (!ok) flag_status(p.status, UCMR_DEV_WAIT_TIMEOUT);
    tc_fence_after();
    if (ok) {
        const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16);
        uint4 code;
        uint32_t r[32];
        tc_ld32(taddr + 0, r);  tc_wait_ld(); code.x = pack_signs(r);
        tc_ld32(taddr + 32, r); tc_wait_ld(); code.y = pack_signs(r);
        tc_ld32(taddr + 64, r); tc_wait_ld(); code.z = pack_signs(r);
        tc_ld32(taddr + 96, r); tc_wait_ld(); code.w = pack_signs(r);
        const int64_t row = row0 + warp * 32 + lane;
        if (row < rows) {
            if (jb.slot_mapping == nullptr) {
                *reinterpret_cast<uint4*>(jb.out + row * 4) = code;
            } else {
                const int64_t tok = row / H_out;
                const int h = (int)(row - tok * H_out);
                const int64_t slot = my_slot;
                if (slot >= 0 && slot < jb.n_slots) *reinterpret_cast<uint4*>(jb.out + (slot * H_out + h) * 4) = code;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kEncBits)
                     : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
// CUDA-core path
// ---------------------------------------------------------------------------------------------
constexpr int kSimtThreads = 128;
constexpr int kSimtRowsPerWarp = 4;
constexpr int kSimtRowsPerCta = kSimtRowsPerWarp * (kSimtThreads / 32);

struct SimtParams {
    const __nv_bfloat16* x;
    int64_t T;
    int H_in, G;  // input heads per token; G consecutive heads are averaged (1 = none)
    int64_t stride_t, stride_h;
    const __nv_bfloat16* R;
    int in_dim, bits;
    uint32_t* out;  // direct: [T*H_out, W]; paged: [n_slots, H_out, W]
    const void* slot_mapping;
    int slot_is_int64;
    int64_t n_slots;
    // paged source (see EncParams): token t of the walk is token t % BS of listed block t / BS
    const int32_t* src_blocks;
    const int32_t* block_tokens;
    int64_t stride_block, NB_src;
    int BS;
    int32_t* status;
    // Output row layout: a (token, head) row of `out` has row_words words and this job's code goes to words
    // [word_offset, word_offset + bits/32).  0 = rows of exactly bits/32 words (the plain layout).
    int row_words, word_offset;
};

// Source token and destination slot of walk position t of a paged-source job; false = skip.
__device__ __forceinline__ bool paged_token(const SimtParams& p, int64_t t, int64_t& src_off, int64_t& slot, bool& bad)
{
    const int64_t bi = t / p.BS;
    const int tok = (int)(t - bi * p.BS);
    const int id = p.src_blocks[bi];
    bad = id < 0 || id >= p.NB_src;
    if (bad) return false;
    if (tok >= (p.block_tokens ? p.block_tokens[bi] : p.BS)) return false;
    src_off = (int64_t)id * p.stride_block + (int64_t)tok * p.stride_t;
    slot = (int64_t)id * p.BS + tok;
    return true;
}

__global__ void __launch_bounds__(kSimtThreads) encode_simt_kernel(const SimtParams p)
{
    extern __shared__ float s_x[];  // [kSimtRowsPerCta][in_dim]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int H_out = p.H_in / p.G;
    const int64_t rows = p.T * H_out;
    const int64_t row0 = (int64_t)blockIdx.x * kSimtRowsPerCta;
    const int W = p.bits / 32;

    for (int i = tid; i < kSimtRowsPerCta * p.in_dim; i += kSimtThreads) {
        const int r = i / p.in_dim, k = i - r * p.in_dim;
        const int64_t row = row0 + r;
        float v = 0.f;
        if (row < rows) {
            const int64_t t = row / H_out;
            const int ho = (int)(row - t * H_out);
            int64_t src_off = t * p.stride_t, slot_unused;
            bool bad = false;
            const bool live = p.src_blocks == nullptr || paged_token(p, t, src_off, slot_unused, bad);
            const __nv_bfloat16* src = p.x + (live ? src_off : 0) + (int64_t)ho * p.G * p.stride_h + k;
            if (!live) {
                v = 0.f;
            } else if (p.G == 1) {
                v = __bfloat162float(*src);
            } else {
                float acc = 0.f;
                for (int g = 0; g < p.G; ++g) acc += __bfloat162float(src[(int64_t)g * p.stride_h]);
                v = __bfloat162float(__float2bfloat16_rn(acc / (float)p.G));
            }
        }
        s_x[i] = v;
    }
    __syncthreads();

    const float* xr = s_x + warp * kSimtRowsPerWarp * p.in_dim;
    for (int w0 = 0; w0 < W; w0 += 4) {
        float acc[kSimtRowsPerWarp][4];
#pragma unroll
        for (int r = 0; r < kSimtRowsPerWarp; ++r)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[r][c] = 0.f;
        const int wn = min(4, W - w0);
        for (int k = 0; k < p.in_dim; ++k) {
            float rv[4];
#pragma unroll
            for (int c = 0; c < 4; ++c)
                rv[c] = (c < wn) ? __bfloat162float(p.R[(size_t)k * p.bits + (w0 + c) * 32 + lane]) : 0.f;
#pragma unroll
            for (int r = 0; r < kSimtRowsPerWarp; ++r) {
                const float xv = xr[r * p.in_dim + k];
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[r][c] = fmaf(xv, rv[c], acc[r][c]);
            }
        }
#pragma unroll
        for (int r = 0; r < kSimtRowsPerWarp; ++r) {
            const int64_t row = row0 + warp * kSimtRowsPerWarp + r;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint32_t word = __ballot_sync(0xffffffffu, acc[r][c] > 0.f);
                if (lane == 0 && c < wn && row < rows) {
                    int64_t dst_row = row;
                    if (p.src_blocks != nullptr) {
                        const int64_t t = row / H_out;
                        const int ho = (int)(row - t * H_out);
                        int64_t src_off, slot;
                        bool bad = false;
                        const bool live = paged_token(p, t, src_off, slot, bad);
                        if (bad && ho == 0 && t % p.BS == 0) flag_status(p.status, UCMR_DEV_BAD_BLOCK_ID);
                        dst_row = (live && slot < p.n_slots) ? slot * H_out + ho : -1;
                    } else if (p.slot_mapping != nullptr) {
                        const int64_t t = row / H_out;
                        const int ho = (int)(row - t * H_out);
                        const int64_t slot = p.slot_is_int64 ? static_cast<const int64_t*>(p.slot_mapping)[t]
                                                             : (int64_t) static_cast<const int32_t*>(p.slot_mapping)[t];
                        dst_row = (slot >= 0 && slot < p.n_slots) ? slot * H_out + ho : -1;
                    }
                    if (dst_row >= 0) p.out[dst_row * (p.row_words > 0 ? p.row_words : W) + p.word_offset + w0 + c] = word;
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_tiled()
{
    static EncodeTiledFn fn = nullptr;  // resolving twice is harmless
    if (fn) return fn;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !ptr) {
        if (e != cudaSuccess) note_cuda_error(e);
        return nullptr;
    }
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
    return fn;
}

static bool tc_path_ok(const void* x, int64_t T, int H, int64_t stride_t, int64_t stride_h, int in_dim, int bits)
{
    if (in_dim != kEncD || bits != kEncBits) return false;
    if (H <= 0 || H > kEncTileM || kEncTileM % H != 0) return false;
    if (reinterpret_cast<uintptr_t>(x) % 16 != 0) return false;
    if (stride_t % 8 != 0 || (H > 1 && stride_h % 8 != 0)) return false;
    if (stride_h < in_dim && H > 1) return false;
    if (T <= 0 || T > 0x7FFFFFFF) return false;
    if ((uint64_t)stride_t * 2 >= (1ull << 40) || (uint64_t)stride_h * 2 >= (1ull << 40)) return false;
    return true;
}

static int launch_tc(const void* x, int64_t T, int H, int64_t stride_t, int64_t stride_h, const void* R,
                     uint32_t* out, const void* slot_mapping, int slot_is_int64, int64_t n_slots,
                     int32_t* status, cudaStream_t st)
{
    EncodeTiledFn encode = get_encode_tiled();
    if (!encode) return UCMR_ERR_LAUNCH;
    CUtensorMap map;
    const cuuint64_t dims[3] = {(cuuint64_t)kEncD, (cuuint64_t)H, (cuuint64_t)T};
    const cuuint64_t strides[2] = {(cuuint64_t)(H > 1 ? stride_h : kEncD) * 2, (cuuint64_t)stride_t * 2};
    const cuuint32_t box[3] = {64, (cuuint32_t)H, (cuuint32_t)(kEncTileM / H)};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(x), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return UCMR_ERR_LAUNCH;

    EncParams p{};
    p.rows = T * H; p.H = H;
    const int tok_per_tile = kEncTileM / H;
    p.n_tiles = (T + tok_per_tile - 1) / tok_per_tile;
    p.out = out; p.slot_mapping = slot_mapping; p.slot_is_int64 = slot_is_int64; p.n_slots = n_slots;
    p.R = static_cast<const __nv_bfloat16*>(R); p.status = status;

    {   // idempotent attribute, set on every call: a flag kept per process would leave a second device without it
        cudaError_t e = cudaFuncSetAttribute(encode_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kEncSmemBytes);
        if (e != cudaSuccess) { note_cuda_error(e); return UCMR_ERR_LAUNCH; }
    }
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int grid = (int)(p.n_tiles < sms ? p.n_tiles : sms);
    return launch_kernel(encode_tc_kernel, dim3(grid), dim3(kEncThreads), kEncSmemBytes, st, map, p);
}

// Paged-source form of launch_tc: a 4-D map {in_dim, H, BS, NB} over the K cache, one box per (block, slice).
static bool tc_blocks_path_ok(const void* x, int64_t NB, int BS, int H, int64_t stride_block, int64_t stride_t,
                              int64_t stride_h, int in_dim, int bits)
{
    if (!tc_path_ok(x, BS, H, stride_t, stride_h, in_dim, bits)) return false;
    const int64_t rpb = (int64_t)BS * H;
    if (rpb % 8 != 0 || (rpb < kEncTileM ? kEncTileM % rpb != 0 : rpb % kEncTileM != 0)) return false;
    if (stride_block % 8 != 0 || (uint64_t)stride_block * 2 >= (1ull << 40)) return false;
    if (NB <= 0 || NB > 0x7FFFFFFF || BS > 256) return false;
    return true;
}

static int launch_tc_blocks(const void* x, int64_t NB, int BS, int H, int64_t stride_block, int64_t stride_t,
                            int64_t stride_h, const int32_t* block_ids, const int32_t* block_tokens, int64_t n_blocks,
                            const void* R, uint32_t* out, int64_t n_slots, int32_t* status, cudaStream_t st)
{
    EncodeTiledFn encode = get_encode_tiled();
    if (!encode) return UCMR_ERR_LAUNCH;
    const int tok_per_tile = kEncTileM / H;
    const int box_tok = BS < tok_per_tile ? BS : tok_per_tile;
    CUtensorMap map;
    const cuuint64_t dims[4] = {(cuuint64_t)kEncD, (cuuint64_t)H, (cuuint64_t)BS, (cuuint64_t)NB};
    const cuuint64_t strides[3] = {(cuuint64_t)(H > 1 ? stride_h : kEncD) * 2, (cuuint64_t)stride_t * 2,
                                   (cuuint64_t)stride_block * 2};
    const cuuint32_t box[4] = {64, (cuuint32_t)H, (cuuint32_t)box_tok, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(x), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return UCMR_ERR_LAUNCH;

    EncParams p{};
    p.H = H; p.BS = BS; p.rpb = BS * H;
    p.rows = n_blocks * p.rpb;
    p.n_tiles = (p.rows + kEncTileM - 1) / kEncTileM;
    p.out = out; p.n_slots = n_slots;
    p.src_blocks = block_ids; p.block_tokens = block_tokens; p.n_src_blocks = n_blocks; p.NB_src = NB;
    p.R = static_cast<const __nv_bfloat16*>(R); p.status = status;
    cudaError_t e = cudaFuncSetAttribute(encode_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kEncSmemBytes);
    if (e != cudaSuccess) { note_cuda_error(e); return UCMR_ERR_LAUNCH; }
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int grid = (int)(p.n_tiles < sms ? p.n_tiles : sms);
    return launch_kernel(encode_tc_kernel, dim3(grid), dim3(kEncThreads), kEncSmemBytes, st, map, p);
}

// Wide tensor-core path: one row per token (H = 1), in_dim and hash_bits multiples of 128 up to 512, enough rows
// to fill the GPU.  out rows have row_words words (0 = hash_bits/32), the code starts at word_offset.
static bool wide_path_ok(const void* x, int64_t T, int H, int64_t stride_t, int in_dim, int bits, const void* R)
{
    if (H != 1 || in_dim % 128 != 0 || bits % 128 != 0 || in_dim > kWideMaxK || bits > 512) return false;
    if (in_dim == kEncD && bits == kEncBits) return false;  // the 128 x 128 kernels are better there
    if (reinterpret_cast<uintptr_t>(x) % 16 != 0 || reinterpret_cast<uintptr_t>(R) % 16 != 0) return false;
    if (stride_t % 8 != 0 || stride_t < in_dim || (uint64_t)stride_t * 2 >= (1ull << 40)) return false;
    if (T < 2048 || T > 0x7FFFFFFF) return false;  // small jobs: the CUDA-core kernel has no set-up cost
    return true;
}

static int launch_wide(const void* x, int64_t T, int64_t stride_t, const void* R, int in_dim, int bits, uint32_t* out,
                       int row_words, int word_offset, const void* slot_mapping, int slot_is_int64, int64_t n_slots,
                       int32_t* status, cudaStream_t st)
{
    EncodeTiledFn encode = get_encode_tiled();
    if (!encode) return UCMR_ERR_LAUNCH;
    CUtensorMap map;
    const cuuint64_t dims[3] = {(cuuint64_t)in_dim, 1, (cuuint64_t)T};
    const cuuint64_t strides[2] = {(cuuint64_t)in_dim * 2, (cuuint64_t)stride_t * 2};
    const cuuint32_t box[3] = {64, 1, (cuuint32_t)kEncTileM};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(x), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return UCMR_ERR_LAUNCH;
    WideParams p{};
    p.rows = T; p.n_tiles = (T + kEncTileM - 1) / kEncTileM;
    p.K = in_dim; p.N = bits; p.n_chunks = bits / kEncBits;
    p.out = out; p.row_words = row_words > 0 ? row_words : bits / 32; p.word_offset = word_offset;
    p.slot_mapping = slot_mapping; p.slot_is_int64 = slot_is_int64; p.n_slots = n_slots;
    p.R = static_cast<const __nv_bfloat16*>(R); p.status = status;
    cudaError_t e = cudaFuncSetAttribute(encode_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kWideSmemBytes);
    if (e != cudaSuccess) { note_cuda_error(e); return UCMR_ERR_LAUNCH; }
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int64_t groups = sms / p.n_chunks;  // CTAs of a group share a token tile
    if (groups > p.n_tiles) groups = p.n_tiles;
    if (groups < 1) return UCMR_ERR_UNSUPPORTED;
    const int grid = (int)(groups * p.n_chunks);
    return launch_kernel(encode_wide_kernel, dim3(grid), dim3(kEncThreads), kWideSmemBytes, st, map, p);
}

// Shapes the one-tile-per-CTA tensor-core kernel accepts (any head count; 16-byte aligned rows).
static bool tile_path_ok(const void* x, int64_t T, int H_in, int G, int64_t stride_t, int64_t stride_h, int in_dim,
                         int bits, const void* out, const void* R)
{
    if (in_dim != kEncD || bits != kEncBits) return false;
    if (H_in <= 0 || G <= 0 || H_in % G != 0 || T <= 0) return false;
    if (reinterpret_cast<uintptr_t>(x) % 16 != 0 || reinterpret_cast<uintptr_t>(out) % 16 != 0 ||
        reinterpret_cast<uintptr_t>(R) % 16 != 0)
        return false;
    if (stride_t % 8 != 0 || (H_in > 1 && stride_h % 8 != 0)) return false;
    return true;
}

static TileJob make_job(const void* x, int64_t T, int H_in, int G, int64_t stride_t, int64_t stride_h, uint32_t* out,
                        const void* slot_mapping, int slot_is_int64, int64_t n_slots)
{
    TileJob j{};
    j.x = static_cast<const __nv_bfloat16*>(x); j.T = T; j.H_in = H_in; j.G = G;
    j.stride_t = stride_t; j.stride_h = stride_h; j.out = out;
    j.slot_mapping = slot_mapping; j.slot_is_int64 = slot_is_int64; j.n_slots = n_slots;
    j.tiles = (T * (H_in / G) + kEncTileM - 1) / kEncTileM;
    return j;
}

static int launch_tiles(const TileJob& j0, const TileJob* j1, const void* R, int32_t* status, cudaStream_t st)
{
    TileParams p{};
    p.job[0] = j0;
    if (j1) p.job[1] = *j1; else p.job[1].tiles = 0, p.job[1].H_in = 1, p.job[1].G = 1;
    p.R = static_cast<const __nv_bfloat16*>(R); p.status = status;
    const int64_t grid = p.job[0].tiles + p.job[1].tiles;
    if (grid <= 0) return UCMR_OK;
    if (grid > 0x7FFFFFFF) return UCMR_ERR_UNSUPPORTED;
    cudaError_t e = cudaFuncSetAttribute(encode_tile_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTileSmemBytes);
    if (e != cudaSuccess) { note_cuda_error(e); return UCMR_ERR_LAUNCH; }
    return launch_kernel(encode_tile_kernel, dim3((unsigned)grid), dim3(kTileThreads), kTileSmemBytes, st, p);
}

// Row counts up to this many tiles go to the one-tile-per-CTA kernel (two waves of CTAs at most); above it the
// persistent TMA-pipelined kernel amortises its set-up.
constexpr int64_t kSmallTiles = 296;

static int launch_simt_params(const SimtParams& p, cudaStream_t st);

static int launch_simt(const void* x, int64_t T, int H_in, int G, int64_t stride_t, int64_t stride_h, const void* R,
                       int in_dim, int bits, uint32_t* out, const void* slot_mapping, int slot_is_int64,
                       int64_t n_slots, cudaStream_t st, int row_words = 0, int word_offset = 0)
{
    SimtParams p{};
    p.row_words = row_words; p.word_offset = word_offset;
    p.x = static_cast<const __nv_bfloat16*>(x); p.T = T; p.H_in = H_in; p.G = G;
    p.stride_t = stride_t; p.stride_h = stride_h;
    p.R = static_cast<const __nv_bfloat16*>(R); p.in_dim = in_dim; p.bits = bits;
    p.out = out; p.slot_mapping = slot_mapping; p.slot_is_int64 = slot_is_int64; p.n_slots = n_slots;
    return launch_simt_params(p, st);
}

static int launch_simt_params(const SimtParams& p, cudaStream_t st)
{
    const int64_t rows = p.T * (p.H_in / p.G);
    const int64_t grid = (rows + kSimtRowsPerCta - 1) / kSimtRowsPerCta;
    if (grid > 0x7FFFFFFF) return UCMR_ERR_UNSUPPORTED;
    const size_t smem = (size_t)kSimtRowsPerCta * p.in_dim * sizeof(float);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(encode_simt_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) { note_cuda_error(e); return UCMR_ERR_LAUNCH; }
    }
    encode_simt_kernel<<<(int)grid, kSimtThreads, smem, st>>>(p);
    return check_launch();
}

static int check_dims(int in_dim, int bits)
{
    if (in_dim <= 0 || bits <= 0) return UCMR_ERR_BAD_ARG;
    if (bits % 32 != 0 || in_dim > 1024 || bits > 1024) return UCMR_ERR_UNSUPPORTED;
    return UCMR_OK;
}

// UCMR_FORCE_SIMT_ENCODE=1 routes every encode through the CUDA-core kernel (debug aid).
static bool force_simt()
{
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("UCMR_FORCE_SIMT_ENCODE");
        v = (e && e[0] == '1') ? 1 : 0;
    }
    return v == 1;
}

}  // namespace ucmr

using namespace ucmr;

extern "C" int ucmr_hash_encode(const void* x, int64_t rows, int64_t row_stride, const void* R, int in_dim,
                                int hash_bits, uint32_t* codes_out, int32_t* status_word, void* stream)
{
    if (!x || !R || !codes_out || rows < 0 || row_stride < in_dim) return UCMR_ERR_BAD_ARG;
    int rc = check_dims(in_dim, hash_bits);
    if (rc != UCMR_OK) return rc;
    if (rows == 0) return UCMR_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool tile_ok = !force_simt() && tile_path_ok(x, rows, 1, 1, row_stride, in_dim, in_dim, hash_bits, codes_out, R);
    if (tile_ok && (rows + kEncTileM - 1) / kEncTileM <= kSmallTiles)
        return launch_tiles(make_job(x, rows, 1, 1, row_stride, in_dim, codes_out, nullptr, 0, 0), nullptr, R, status_word, st);
    if (!force_simt() && tc_path_ok(x, rows, 1, row_stride, in_dim, in_dim, hash_bits) &&
        reinterpret_cast<uintptr_t>(codes_out) % 16 == 0 && reinterpret_cast<uintptr_t>(R) % 16 == 0)
        return launch_tc(x, rows, 1, row_stride, in_dim, R, codes_out, nullptr, 0, 0, status_word, st);
    if (tile_ok)
        return launch_tiles(make_job(x, rows, 1, 1, row_stride, in_dim, codes_out, nullptr, 0, 0), nullptr, R, status_word, st);
    if (!force_simt() && wide_path_ok(x, rows, 1, row_stride, in_dim, hash_bits, R))
        return launch_wide(x, rows, row_stride, R, in_dim, hash_bits, codes_out, 0, 0, nullptr, 0, 0, status_word, st);
    return launch_simt(x, rows, 1, 1, row_stride, in_dim, R, in_dim, hash_bits, codes_out, nullptr, 0, 0, st);
}

extern "C" int ucmr_hash_encode_query(const void* q, int64_t T, int Hq, int64_t stride_t, int64_t stride_h,
                                      int group_mean, const void* R, int in_dim, int hash_bits,
                                      uint32_t* codes_out, int32_t* status_word, void* stream)
{
    if (!q || !R || !codes_out || T < 0 || Hq <= 0 || group_mean <= 0 || Hq % group_mean != 0) return UCMR_ERR_BAD_ARG;
    if (stride_h < in_dim || stride_t < in_dim) return UCMR_ERR_BAD_ARG;
    int rc = check_dims(in_dim, hash_bits);
    if (rc != UCMR_OK) return rc;
    if (T == 0) return UCMR_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool tile_ok = !force_simt() && tile_path_ok(q, T, Hq, group_mean, stride_t, stride_h, in_dim, hash_bits, codes_out, R);
    const int64_t tiles = (T * (Hq / group_mean) + kEncTileM - 1) / kEncTileM;
    if (tile_ok && (group_mean > 1 || tiles <= kSmallTiles))
        return launch_tiles(make_job(q, T, Hq, group_mean, stride_t, stride_h, codes_out, nullptr, 0, 0), nullptr, R, status_word, st);
    if (group_mean == 1 && !force_simt() && tc_path_ok(q, T, Hq, stride_t, stride_h, in_dim, hash_bits) &&
        reinterpret_cast<uintptr_t>(codes_out) % 16 == 0 && reinterpret_cast<uintptr_t>(R) % 16 == 0)
        return launch_tc(q, T, Hq, stride_t, stride_h, R, codes_out, nullptr, 0, 0, status_word, st);
    if (tile_ok)
        return launch_tiles(make_job(q, T, Hq, group_mean, stride_t, stride_h, codes_out, nullptr, 0, 0), nullptr, R, status_word, st);
    return launch_simt(q, T, Hq, group_mean, stride_t, stride_h, R, in_dim, hash_bits, codes_out, nullptr, 0, 0, st);
}

// row_words = 0: cache rows of exactly hash_bits/32 words.  Otherwise the code lands at words
// [word_offset, word_offset + hash_bits/32) of rows of row_words words (CUDA-core kernel only).
static int encode_and_cache_impl(const void* x, int64_t T, int H, int64_t stride_t, int64_t stride_h, const void* R,
                                 int in_dim, int hash_bits, const void* slot_mapping, int slot_is_int64,
                                 uint32_t* cache, int64_t NB, int BS, int row_words, int word_offset,
                                 int32_t* status_word, void* stream)
{
    if (!x || !R || !slot_mapping || !cache || T < 0 || H <= 0 || NB <= 0 || BS <= 0) return UCMR_ERR_BAD_ARG;
    if (stride_h < in_dim || stride_t < in_dim) return UCMR_ERR_BAD_ARG;
    int rc = check_dims(in_dim, hash_bits);
    if (rc != UCMR_OK) return rc;
    if (row_words < 0 || word_offset < 0 || (row_words > 0 && word_offset + hash_bits / 32 > row_words) ||
        (row_words == 0 && word_offset != 0))
        return UCMR_ERR_BAD_ARG;
    if (T == 0) return UCMR_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t n_slots = NB * BS;
    if (!force_simt() && wide_path_ok(x, T, H, stride_t, in_dim, hash_bits, R))
        return launch_wide(x, T, stride_t, R, in_dim, hash_bits, cache, row_words, word_offset, slot_mapping,
                           slot_is_int64 ? 1 : 0, n_slots, status_word, st);
    if (row_words > 0 && !(row_words == hash_bits / 32 && word_offset == 0))
        return launch_simt(x, T, H, 1, stride_t, stride_h, R, in_dim, hash_bits, cache, slot_mapping,
                           slot_is_int64 ? 1 : 0, n_slots, st, row_words, word_offset);
    const bool tile_ok = !force_simt() && tile_path_ok(x, T, H, 1, stride_t, stride_h, in_dim, hash_bits, cache, R);
    const bool tc_ok = !force_simt() && tc_path_ok(x, T, H, stride_t, stride_h, in_dim, hash_bits) &&
                       reinterpret_cast<uintptr_t>(cache) % 16 == 0 && reinterpret_cast<uintptr_t>(R) % 16 == 0;
    if (tile_ok && ((T * H + kEncTileM - 1) / kEncTileM <= kSmallTiles || !tc_ok))
        return launch_tiles(make_job(x, T, H, 1, stride_t, stride_h, cache, slot_mapping, slot_is_int64 ? 1 : 0, n_slots),
                            nullptr, R, status_word, st);
    if (!force_simt() && tc_path_ok(x, T, H, stride_t, stride_h, in_dim, hash_bits) &&
        reinterpret_cast<uintptr_t>(cache) % 16 == 0 && reinterpret_cast<uintptr_t>(R) % 16 == 0)
        return launch_tc(x, T, H, stride_t, stride_h, R, cache, slot_mapping, slot_is_int64 ? 1 : 0, n_slots, status_word, st);
    return launch_simt(x, T, H, 1, stride_t, stride_h, R, in_dim, hash_bits, cache, slot_mapping,
                       slot_is_int64 ? 1 : 0, n_slots, st);
}

extern "C" int ucmr_hash_encode_and_cache(const void* x, int64_t T, int H, int64_t stride_t, int64_t stride_h,
                                          const void* R, int in_dim, int hash_bits, const void* slot_mapping,
                                          int slot_is_int64, uint32_t* cache, int64_t NB, int BS,
                                          int32_t* status_word, void* stream)
{
    return encode_and_cache_impl(x, T, H, stride_t, stride_h, R, in_dim, hash_bits, slot_mapping, slot_is_int64, cache,
                                 NB, BS, 0, 0, status_word, stream);
}

extern "C" int ucmr_hash_encode_and_cache_at(const void* x, int64_t T, int H, int64_t stride_t, int64_t stride_h,
                                             const void* R, int in_dim, int hash_bits, const void* slot_mapping,
                                             int slot_is_int64, uint32_t* cache, int64_t NB, int BS, int row_words,
                                             int word_offset, int32_t* status_word, void* stream)
{
    if (row_words <= 0) return UCMR_ERR_BAD_ARG;
    return encode_and_cache_impl(x, T, H, stride_t, stride_h, R, in_dim, hash_bits, slot_mapping, slot_is_int64, cache,
                                 NB, BS, row_words, word_offset, status_word, stream);
}

static bool step_simt_enabled()
{
    static const bool v = [] {
        const char* e = getenv("UCMR_STEP_ENCODE");
        return !(e && e[0] == 't');
    }();
    return v;
}

// ---------------------------------------------------------------------------------------------
// decode step on CUDA cores: a few hundred rows, latency is everything
// ---------------------------------------------------------------------------------------------
// The two encodes of a decode step (B*Hq query rows, B*Hkv new key rows) are some 10 MFLOP: the tensor-core tile
// kernel spends its time on the set-up chain around the MMA (TMEM allocation, swizzled staging, commit / wait, four
// tcgen05.ld round trips, dealloc), not on the math, and a kernel of one warp per row is bound by that warp's
// instruction stream (128 inputs x 4 columns per lane, about a thousand instructions on one scheduler).  Here four
// warps share a row, each taking 32 of the 128 inputs: a lane fetches its warp's 32 rows of R straight into
// registers (8 bytes per row: its four columns; no staging of R in shared memory) while the row's first warp fetches
// the row itself (from device memory or, across the bus, from page-locked host memory) - a single memory round trip
// - then accumulates four columns over the warp's 32 inputs in float32 (inputs broadcast from shared memory, four per
// load).  The four partial sums meet in shared memory; the row's first warp adds them, packs the 128 sign bits with
// three shuffle steps and stores the code.
constexpr int kStepThreads = 256;
constexpr int kStepKSplit = 4;                                      // warps per row
constexpr int kStepRowsPerRound = kStepThreads / 32 / kStepKSplit;  // 2 rows at a time
constexpr int kStepKPerWarp = kEncD / kStepKSplit;                  // 32 inputs per warp
static_assert(kStepKPerWarp == 32 && kEncBits == 128, "one input per lane, four columns per lane");

// ROUNDS: row pairs a CTA works through with the same registers of R.  One round spreads a small step over as many
// SMs as it has row pairs; four rounds keep a step of several hundred rows on about half of the SMs, so that the
// scan launched behind it (whose CTAs need an SM to themselves) sets itself up on the others meanwhile.
template <int ROUNDS>
__global__ void __launch_bounds__(kStepThreads) encode_step_kernel(const TileParams p)
{
    constexpr int kRowsPerCta = kStepRowsPerRound * ROUNDS;
    __shared__ __align__(16) float s_x[ROUNDS][kStepRowsPerRound][kEncD];
    __shared__ __align__(16) float s_part[ROUNDS][kStepRowsPerRound][kStepKSplit][kEncBits];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int r_in = warp / kStepKSplit, ks = warp % kStepKSplit, k0 = ks * kStepKPerWarp;
    UCMR_STAMP(0);
    grid_launch_dependents();  // a scan launched right after this kernel may set itself up meanwhile
    grid_dependency_wait();    // q and the new keys come from the kernel before this one
    UCMR_STAMP(1);
    // rows k0 .. k0+31 of R, columns 4*lane .. 4*lane+3: 32 independent 8-byte loads per lane
    uint2 rr[kStepKPerWarp];
    {
        const uint2* src = reinterpret_cast<const uint2*>(p.R) + (int64_t)k0 * (kEncBits / 4) + lane;
#pragma unroll
        for (int i = 0; i < kStepKPerWarp; ++i) rr[i] = __ldg(src + i * (kEncBits / 4));
    }
    // job 0 rows first, then job 1
    const int H_out0 = p.job[0].H_in / p.job[0].G, H_out1 = p.job[1].x ? p.job[1].H_in / p.job[1].G : 1;
    // (the launch is limited to kStepMaxRows rows: 32-bit arithmetic, whose division costs a tenth of the 64-bit one)
    const int rows0 = (int)p.job[0].T * H_out0, rows1 = p.job[1].x ? (int)p.job[1].T * H_out1 : 0;
    // Where a row comes from and goes to.  (Fields picked with compile-time offsets: a run-time index into the
    // kernel parameter would turn every access into a load through a generic address, which is slow.)
    struct RowRef { bool live; int row, tok, ho, H_out; };
    auto locate = [&](int it, bool& second) -> RowRef {
        RowRef r;
        r.row = (int)blockIdx.x * kRowsPerCta + it * kStepRowsPerRound + r_in;
        second = r.row >= rows0;
        if (second) r.row -= rows0;
        r.H_out = second ? H_out1 : H_out0;
        r.live = r.row < (second ? rows1 : rows0);
        r.tok = r.live ? r.row / r.H_out : 0;
        r.ho = r.row - r.tok * r.H_out;
        return r;
    };
    // The rows: the first warp of a row fetches all of it, 8 bytes per lane (a 256-byte request per row and group
    // member: rows that sit in page-locked host memory cross the bus in few, wide requests), and leaves it in shared
    // memory as float32 for the row's four warps.  Addresses first, then the loads of all rounds back to back (a load
    // placed behind the previous round's branch and store would wait for that round's memory round trip).
    if (ks == 0) {
        const __nv_bfloat16* xsrc[ROUNDS];
        int64_t xstride[ROUNDS];
        int xg[ROUNDS];
        int g_max = 0;
#pragma unroll
        for (int it = 0; it < ROUNDS; ++it) {
            bool second;
            const RowRef r = locate(it, second);
            const TileJob jb = second ? p.job[1] : p.job[0];
            xg[it] = r.live ? jb.G : 0;
            xstride[it] = jb.stride_h;
            xsrc[it] = jb.x;
            if (r.live) xsrc[it] += (int64_t)r.tok * jb.stride_t + (int64_t)r.ho * jb.G * jb.stride_h + 4 * lane;
            g_max = max(g_max, xg[it]);
        }
        float xv[ROUNDS][4];
#pragma unroll
        for (int it = 0; it < ROUNDS; ++it)
#pragma unroll
            for (int i = 0; i < 4; ++i) xv[it][i] = 0.f;
        for (int g = 0; g < g_max; ++g) {
            uint2 raw[ROUNDS];
#pragma unroll
            for (int it = 0; it < ROUNDS; ++it)
                raw[it] = g < xg[it] ? __ldg(reinterpret_cast<const uint2*>(xsrc[it] + (int64_t)g * xstride[it]))
                                     : make_uint2(0u, 0u);
#pragma unroll
            for (int it = 0; it < ROUNDS; ++it) {
                xv[it][0] += __uint_as_float(raw[it].x << 16);
                xv[it][1] += __uint_as_float(raw[it].x & 0xFFFF0000u);
                xv[it][2] += __uint_as_float(raw[it].y << 16);
                xv[it][3] += __uint_as_float(raw[it].y & 0xFFFF0000u);
            }
        }
#pragma unroll
        for (int it = 0; it < ROUNDS; ++it) {
            // the group mean, rounded once to bf16 as torch's mean of a bf16 tensor is
            if (xg[it] > 1) {
#pragma unroll
                for (int i = 0; i < 4; ++i) xv[it][i] = __bfloat162float(__float2bfloat16_rn(xv[it][i] / (float)xg[it]));
            }
            reinterpret_cast<float4*>(s_x[it][r_in])[lane] = make_float4(xv[it][0], xv[it][1], xv[it][2], xv[it][3]);
        }
    }
    __syncthreads();
    UCMR_STAMP(2);
#pragma unroll
    for (int it = 0; it < ROUNDS; ++it) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};  // columns 4*lane .. 4*lane+3 over this warp's inputs
        const float4* xrow = reinterpret_cast<const float4*>(&s_x[it][r_in][k0]);
#pragma unroll
        for (int i4 = 0; i4 < kStepKPerWarp / 4; ++i4) {
            const float4 x4 = xrow[i4];
            const float xs[4] = {x4.x, x4.y, x4.z, x4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint2 r = rr[i4 * 4 + i];
                acc[0] = fmaf(xs[i], __uint_as_float(r.x << 16), acc[0]);
                acc[1] = fmaf(xs[i], __uint_as_float(r.x & 0xFFFF0000u), acc[1]);
                acc[2] = fmaf(xs[i], __uint_as_float(r.y << 16), acc[2]);
                acc[3] = fmaf(xs[i], __uint_as_float(r.y & 0xFFFF0000u), acc[3]);
            }
        }
        reinterpret_cast<float4*>(s_part[it][r_in][ks])[lane] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    }
    __syncthreads();
    // warp ks of a row pair finishes rounds ks, ks + 4, ...: adds the four partial sums, packs, stores
    for (int it = ks; it < ROUNDS; it += kStepKSplit) {
        float4 a = reinterpret_cast<const float4*>(s_part[it][r_in][0])[lane];
#pragma unroll
        for (int w = 1; w < kStepKSplit; ++w) {
            const float4 o = reinterpret_cast<const float4*>(s_part[it][r_in][w])[lane];
            a.x += o.x; a.y += o.y; a.z += o.z; a.w += o.w;
        }
        // word w of the code = columns 32w .. 32w+31 = lanes 8w .. 8w+7, four bits each
        const uint32_t nib = (uint32_t)(a.x > 0.f) | ((uint32_t)(a.y > 0.f) << 1) | ((uint32_t)(a.z > 0.f) << 2) |
                             ((uint32_t)(a.w > 0.f) << 3);
        uint32_t word = nib << (4 * (lane & 7));
        word |= __shfl_xor_sync(0xffffffffu, word, 1);
        word |= __shfl_xor_sync(0xffffffffu, word, 2);
        word |= __shfl_xor_sync(0xffffffffu, word, 4);
        // lanes 0, 8, 16, 24 hold words 0..3: gather them into lane 0
        const uint32_t w1 = __shfl_sync(0xffffffffu, word, 8), w2 = __shfl_sync(0xffffffffu, word, 16),
                       w3 = __shfl_sync(0xffffffffu, word, 24);
        bool second;
        const RowRef r = locate(it, second);
        if (r.live && lane == 0) {
            const TileJob jb = second ? p.job[1] : p.job[0];
            const uint4 code = make_uint4(word, w1, w2, w3);
            if (jb.slot_mapping == nullptr) {
                *reinterpret_cast<uint4*>(jb.out + (int64_t)r.row * 4) = code;
            } else {
                const int64_t slot = jb.slot_is_int64 ? static_cast<const int64_t*>(jb.slot_mapping)[r.tok]
                                                      : (int64_t) static_cast<const int32_t*>(jb.slot_mapping)[r.tok];
                if (slot >= 0 && slot < jb.n_slots)
                    *reinterpret_cast<uint4*>(jb.out + (slot * r.H_out + r.ho) * 4) = code;
            }
        }
    }
    UCMR_STAMP(3);
}

// Rows of a decode step up to which the CUDA-core kernel is used (beyond it the tensor-core tiles win).
constexpr int64_t kStepMaxRows = 2048;

static int launch_step(const TileJob& jq, const TileJob& jk, const void* R, int32_t* status, cudaStream_t st)
{
    TileParams p{};
    p.job[0] = jq;
    p.job[1] = jk;
    p.R = static_cast<const __nv_bfloat16*>(R);
    p.status = status;
    const int64_t rows = jq.T * (jq.H_in / jq.G) + jk.T * (jk.H_in / jk.G);
    if (rows <= 0) return UCMR_OK;
    // up to 74 row pairs (half of the SMs): one pair per CTA; more: four pairs per CTA
    constexpr int64_t kSpreadRows = 74 * kStepRowsPerRound;
    if (rows <= kSpreadRows) {
        const int64_t grid = (rows + kStepRowsPerRound - 1) / kStepRowsPerRound;
        return launch_kernel_ex(encode_step_kernel<1>, dim3((unsigned)grid), dim3(kStepThreads), 0, st, 1, true, p);
    }
    const int64_t per_cta = kStepRowsPerRound * 4;
    const int64_t grid = (rows + per_cta - 1) / per_cta;
    return launch_kernel_ex(encode_step_kernel<4>, dim3((unsigned)grid), dim3(kStepThreads), 0, st, 1, true, p);
}

extern "C" int ucmr_hash_encode_decode_step(const void* q, int64_t Tq, int Hq, int64_t q_stride_t, int64_t q_stride_h,
                                            int group_mean, uint32_t* q_codes_out, const void* k, int64_t Tk, int Hk,
                                            int64_t k_stride_t, int64_t k_stride_h, const void* slot_mapping,
                                            int slot_is_int64, uint32_t* cache, int64_t NB, int BS, const void* R,
                                            int in_dim, int hash_bits, int32_t* status_word, void* stream)
{
    if (!q || !k || !R || !q_codes_out || !slot_mapping || !cache) return UCMR_ERR_BAD_ARG;
    if (Tq < 0 || Tk < 0 || Hq <= 0 || Hk <= 0 || group_mean <= 0 || Hq % group_mean != 0 || NB <= 0 || BS <= 0)
        return UCMR_ERR_BAD_ARG;
    int rc = check_dims(in_dim, hash_bits);
    if (rc != UCMR_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool fused = !force_simt() && Tq > 0 && Tk > 0 &&
                       tile_path_ok(q, Tq, Hq, group_mean, q_stride_t, q_stride_h, in_dim, hash_bits, q_codes_out, R) &&
                       tile_path_ok(k, Tk, Hk, 1, k_stride_t, k_stride_h, in_dim, hash_bits, cache, R);
    if (fused) {
        const TileJob jq = make_job(q, Tq, Hq, group_mean, q_stride_t, q_stride_h, q_codes_out, nullptr, 0, 0);
        const TileJob jk = make_job(k, Tk, Hk, 1, k_stride_t, k_stride_h, cache, slot_mapping, slot_is_int64 ? 1 : 0, NB * BS);
        // few rows: the CUDA-core kernel (shorter dependency chain); UCMR_STEP_ENCODE=tile keeps the tensor-core tiles
        if (Tq * (Hq / group_mean) + Tk * Hk <= kStepMaxRows && step_simt_enabled() && q_stride_h % 4 == 0 &&
            k_stride_h % 4 == 0 && q_stride_t % 4 == 0 && k_stride_t % 4 == 0)
            return launch_step(jq, jk, R, status_word, st);
        return launch_tiles(jq, &jk, R, status_word, st);
    }
    rc = ucmr_hash_encode_and_cache(k, Tk, Hk, k_stride_t, k_stride_h, R, in_dim, hash_bits, slot_mapping, slot_is_int64,
                                    cache, NB, BS, status_word, stream);
    if (rc != UCMR_OK) return rc;
    return ucmr_hash_encode_query(q, Tq, Hq, q_stride_t, q_stride_h, group_mean, R, in_dim, hash_bits, q_codes_out,
                                  status_word, stream);
}

static int encode_blocks_impl(const void* k_cache, int64_t NB, int BS, int H, int64_t stride_block, int64_t stride_t,
                              int64_t stride_h, const int32_t* block_ids, const int32_t* block_tokens, int64_t n_blocks,
                              const void* R, int in_dim, int hash_bits, uint32_t* cache, int64_t NB_codes, int row_words,
                              int word_offset, int32_t* status_word, void* stream)
{
    if (!k_cache || !R || !cache || NB <= 0 || BS <= 0 || H <= 0 || NB_codes <= 0 || n_blocks < 0) return UCMR_ERR_BAD_ARG;
    if (row_words < 0 || word_offset < 0 || (row_words > 0 && word_offset + hash_bits / 32 > row_words) ||
        (row_words == 0 && word_offset != 0))
        return UCMR_ERR_BAD_ARG;
    const bool plain_rows = row_words == 0 || (row_words == hash_bits / 32 && word_offset == 0);
    if (n_blocks > 0 && !block_ids) return UCMR_ERR_BAD_ARG;
    if (stride_h < in_dim || stride_t < in_dim || stride_block < stride_t) return UCMR_ERR_BAD_ARG;
    int rc = check_dims(in_dim, hash_bits);
    if (rc != UCMR_OK) return rc;
    if (n_blocks == 0) return UCMR_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t n_slots = NB_codes * BS;
    if (plain_rows && !force_simt() && tc_blocks_path_ok(k_cache, NB, BS, H, stride_block, stride_t, stride_h, in_dim, hash_bits) &&
        reinterpret_cast<uintptr_t>(cache) % 16 == 0 && reinterpret_cast<uintptr_t>(R) % 16 == 0)
        return launch_tc_blocks(k_cache, NB, BS, H, stride_block, stride_t, stride_h, block_ids, block_tokens, n_blocks,
                                R, cache, n_slots, status_word, st);
    SimtParams p{};
    p.x = static_cast<const __nv_bfloat16*>(k_cache); p.T = n_blocks * BS; p.H_in = H; p.G = 1;
    p.stride_t = stride_t; p.stride_h = stride_h;
    p.R = static_cast<const __nv_bfloat16*>(R); p.in_dim = in_dim; p.bits = hash_bits;
    p.out = cache; p.n_slots = n_slots;
    p.src_blocks = block_ids; p.block_tokens = block_tokens; p.stride_block = stride_block; p.NB_src = NB; p.BS = BS;
    p.status = status_word;
    p.row_words = plain_rows ? 0 : row_words; p.word_offset = plain_rows ? 0 : word_offset;
    return launch_simt_params(p, st);
}

extern "C" int ucmr_hash_encode_blocks(const void* k_cache, int64_t NB, int BS, int H, int64_t stride_block,
                                       int64_t stride_t, int64_t stride_h, const int32_t* block_ids,
                                       const int32_t* block_tokens, int64_t n_blocks, const void* R, int in_dim,
                                       int hash_bits, uint32_t* cache, int64_t NB_codes, int32_t* status_word,
                                       void* stream)
{
    return encode_blocks_impl(k_cache, NB, BS, H, stride_block, stride_t, stride_h, block_ids, block_tokens, n_blocks, R,
                              in_dim, hash_bits, cache, NB_codes, 0, 0, status_word, stream);
}

extern "C" int ucmr_hash_encode_blocks_at(const void* k_cache, int64_t NB, int BS, int H, int64_t stride_block,
                                          int64_t stride_t, int64_t stride_h, const int32_t* block_ids,
                                          const int32_t* block_tokens, int64_t n_blocks, const void* R, int in_dim,
                                          int hash_bits, uint32_t* cache, int64_t NB_codes, int row_words,
                                          int word_offset, int32_t* status_word, void* stream)
{
    if (row_words <= 0) return UCMR_ERR_BAD_ARG;
    return encode_blocks_impl(k_cache, NB, BS, H, stride_block, stride_t, stride_h, block_ids, block_tokens, n_blocks, R,
                              in_dim, hash_bits, cache, NB_codes, row_words, word_offset, status_word, stream);
}

#ifdef UCMR_TRACE
namespace ucmr { UCMR_TRACE_READER(trace_read_encode) }
#endif

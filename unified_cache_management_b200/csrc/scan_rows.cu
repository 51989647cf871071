// Hamming scan of token-row codes (sm_100a): one kv head, 18 words per token (MLA: a 512-bit code of the latent
// vector and a 64-bit code of the rope part side by side), up to 255 query codes per request.
//
//   sum_g popc(k ^ q_g) only depends, bit position by bit position, on the key bit and on c = how many of the G query
//   codes have the bit set: the position contributes  k ? G - c : c.  A small kernel turns every request's query codes
//   into bit-sliced planes once (cnt[p] = bit p of c - vmin, alt[p] = bit p of G - c - vmin, vmin = the smallest
//   contribution anywhere in the row, so that only bits(max - min) planes are needed: query heads agree on most bits
//   far less often than never or always).  The scan then computes, per token,
//       d = 576 * vmin + sum_p 2^p popc( k ? alt[p] : cnt[p] ),
//   one logic instruction per plane and word plus a carry-save popcount over the 18 words: about log2(G) popcount sums
//   per token instead of G.  The planes are read straight from global memory (a few hundred bytes per request, the same
//   address in every lane: they stay in L1).
//
//   Data movement: two producer warps and fourteen consumer warps per SM around 28 shared-memory stages of 64 token
//   rows (4.5 KiB; one block of 64 tokens, or several smaller ones).  Every stage has its own producer lane: it
//   resolves the stage's next work item ahead of time (request, blocks, block-table entries) and, whenever a
//   non-blocking test finds the stage's "empty" barrier complete, starts the bulk copies.  A consumer copies its stage into registers (two tokens per
//   lane), releases the stage at once and only then does the arithmetic - so nearly all of the ring is in flight all
//   the time, which the one-stage-per-warp kernel in scan_ring.cu cannot do for rows (a stage there holds more tokens
//   than fit in registers and stays occupied during most of the arithmetic).
//
// Output: int32 [B, 1, max_blocks] block scores (min or sum over the block's tokens), bit-identical to scan_ring.cu's
// token-row path, which remains for callers without scratch memory and for other block sizes.
//
// Stands in for HammingScoreContiKernel + torch.min of the reference on its MLA shapes
// (ucm/sparse/gsa_on_device/csrc/cuda/ham_dist/paged_ham_dist_mla.cu:111-248, hamming_topk.py:45-47).
#include <limits.h>

#include "common.cuh"

namespace ucmr {

constexpr int kRowW = 18;             // words per token row
constexpr int kRowWPad = 20;          // plane rows are padded to whole 16-byte loads
constexpr int kRowPlanes = 8;         // counts up to 255
constexpr int kRowsWarps = 16;        // 2 producers + 14 consumers
constexpr int kRowsThreads = 32 * kRowsWarps;
constexpr int kRowsProducers = 2;
constexpr int kRowsConsumers = kRowsWarps - kRowsProducers;
constexpr int kRowsMaxStages = 32;
constexpr int kRowsRingBytes = 150 * 1024;
constexpr int kRowsMaxBatch = 1024;

// Per request: header {planes in use, 576 * vmin, 0, 0}, then cnt[8][20] and alt[8][20] words.
constexpr int kRowPlaneWords = 4 + 2 * kRowPlanes * kRowWPad;

size_t rows_scratch_bytes(int B) { return ((size_t)B * kRowPlaneWords * 4 + 255) / 256 * 256; }

// ---- planes of one request's query codes ---------------------------------------------------------------------
__global__ void __launch_bounds__(32) rows_planes_kernel(const uint32_t* __restrict__ q, int G, uint32_t* __restrict__ planes)
{
    grid_launch_dependents();
    grid_dependency_wait();  // the query codes come from the kernel before this one
    const int b = blockIdx.x, lane = threadIdx.x;
    uint32_t c[kRowPlanes], a[kRowPlanes];
#pragma unroll
    for (int p = 0; p < kRowPlanes; ++p) c[p] = 0u;
    if (lane < kRowW) {
        const uint32_t* qb = q + (int64_t)b * G * kRowW + lane;
        for (int g0 = 0; g0 < G; g0 += 8) {
            uint32_t wv[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) wv[u] = (g0 + u < G) ? __ldg(qb + (int64_t)(g0 + u) * kRowW) : 0u;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                uint32_t carry = wv[u];
#pragma unroll
                for (int p = 0; p < kRowPlanes; ++p) {  // bit-sliced increment
                    const uint32_t t = c[p] & carry;
                    c[p] ^= carry;
                    carry = t;
                }
            }
        }
    }
    {   // alt = G - c, bit-sliced
        uint32_t borrow = 0u;
#pragma unroll
        for (int p = 0; p < kRowPlanes; ++p) {
            const uint32_t gb = ((G >> p) & 1) ? 0xFFFFFFFFu : 0u;
            a[p] = gb ^ c[p] ^ borrow;
            borrow = (~gb & (c[p] | borrow)) | (c[p] & borrow);
        }
    }
    // smallest and largest contribution over all bit positions and both key values
    int vmin = INT_MAX, vmax = 0;
    if (lane < kRowW) {
        for (int bit = 0; bit < 32; ++bit) {
            int cv = 0, av = 0;
#pragma unroll
            for (int p = 0; p < kRowPlanes; ++p) {
                cv |= (int)((c[p] >> bit) & 1u) << p;
                av |= (int)((a[p] >> bit) & 1u) << p;
            }
            vmin = min(vmin, min(cv, av));
            vmax = max(vmax, max(cv, av));
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        vmin = min(vmin, __shfl_xor_sync(0xffffffffu, vmin, off));
        vmax = max(vmax, __shfl_xor_sync(0xffffffffu, vmax, off));
    }
    // subtract vmin from both (bit-sliced subtraction of a constant)
    auto sub_const = [&](uint32_t (&v)[kRowPlanes]) {
        uint32_t borrow = 0u;
#pragma unroll
        for (int p = 0; p < kRowPlanes; ++p) {
            const uint32_t kb = ((vmin >> p) & 1) ? 0xFFFFFFFFu : 0u;
            const uint32_t x = v[p];
            v[p] = x ^ kb ^ borrow;
            borrow = (~x & (kb | borrow)) | (kb & borrow);
        }
    };
    sub_const(c);
    sub_const(a);
    uint32_t* out = planes + (int64_t)b * kRowPlaneWords;
    if (lane == 0) {
        out[0] = (uint32_t)(32 - __clz(vmax - vmin));  // planes in use (0 when every position contributes the same)
        out[1] = (uint32_t)(vmin * 32 * kRowW);
        out[2] = 0u;
        out[3] = 0u;
    }
    if (lane < kRowWPad) {
#pragma unroll
        for (int p = 0; p < kRowPlanes; ++p) {
            out[4 + p * kRowWPad + lane] = lane < kRowW ? c[p] : 0u;
            out[4 + (kRowPlanes + p) * kRowWPad + lane] = lane < kRowW ? a[p] : 0u;
        }
    }
}

// ---- the scan ------------------------------------------------------------------------------------------------
struct RowsParams {
    const char* codes;
    int64_t NB;
    int BS, max_blocks, B;
    const uint32_t* planes;
    const int32_t* bt;
    int64_t bt_stride;
    const int32_t* seq_lens;
    int32_t* out;
    int32_t* status;
    int bps;          // blocks per work item (= per stage)
    int block_bytes;  // BS * 72
    int stage_bytes;  // bps * block_bytes
    int n_stages;
    int iters;        // 64-row steps per stage (2 for blocks of 128 tokens)
};

struct __align__(16) RowsMeta {
    int b, j0, seq;
    uint32_t valid_mask;
};

__device__ __forceinline__ void csa3(uint32_t& h, uint32_t& l, uint32_t a, uint32_t b, uint32_t c)
{
    const uint32_t u = a ^ b;
    h = (a & b) | (u & c);
    l = u ^ c;
}

// Sum of the popcounts of 18 words.  The logic pipe (which also runs the 18 mux instructions per plane) and the
// popcount unit are separate: twelve words are compressed with carry-save adders, the other six are counted directly,
// so that neither pipe carries the whole load.  The adders form a tree (four independent 3:2 steps first), not a chain:
// with three or four warps per scheduler the kernel lives on instruction-level parallelism.
__device__ __forceinline__ void half_add(uint32_t& h, uint32_t& l, uint32_t a, uint32_t b)
{
    h = a & b;
    l = a ^ b;
}
__device__ __forceinline__ int popc18(const uint32_t (&v)[kRowW])
{
    uint32_t s0, s1, s2, s3, c0, c1, c2, c3;
    csa3(c0, s0, v[0], v[1], v[2]);
    csa3(c1, s1, v[3], v[4], v[5]);
    csa3(c2, s2, v[6], v[7], v[8]);
    csa3(c3, s3, v[9], v[10], v[11]);
    uint32_t sa, ca, ones, cb;
    csa3(ca, sa, s0, s1, s2);
    half_add(cb, ones, sa, s3);
    // weight 2: c0 c1 c2 c3 ca cb
    uint32_t t0, t1, d0, d1, twos, d2;
    csa3(d0, t0, c0, c1, c2);
    csa3(d1, t1, c3, ca, cb);
    half_add(d2, twos, t0, t1);
    // weight 4: d0 d1 d2
    uint32_t eights, fours;
    csa3(eights, fours, d0, d1, d2);
    const int compressed = (__popc(ones) + 2 * __popc(twos)) + (4 * __popc(fours) + 8 * __popc(eights));
    const int direct = (__popc(v[12]) + __popc(v[13]) + __popc(v[14])) + (__popc(v[15]) + __popc(v[16]) + __popc(v[17]));
    return compressed + direct;
}

template <bool MIN>
__global__ void __launch_bounds__(kRowsThreads, 1) scan_rows_kernel(const RowsParams p)
{
    extern __shared__ __align__(128) uint8_t s_ring[];
    __shared__ __align__(8) uint64_t s_full[kRowsMaxStages];
    __shared__ __align__(8) uint64_t s_empty[kRowsMaxStages];
    __shared__ RowsMeta s_meta[kRowsMaxStages];
    __shared__ int s_cum[kRowsMaxBatch + 1];
    __shared__ int s_seq[kRowsMaxBatch];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    grid_launch_dependents();
    if (tid == 0) {
        for (int s = 0; s < kRowsMaxStages; ++s) { mbar_init(&s_full[s], 1); mbar_init(&s_empty[s], 1); }
        fence_mbar_init();
    }
    grid_dependency_wait();  // sequence lengths, block table, planes and codes may come from earlier kernels
    if (warp == 0) {  // work items per request, prefix sum
        int run = 0;
        for (int b0 = 0; b0 < p.B; b0 += 32) {
            const int b = b0 + lane;
            int n = 0;
            if (b < p.B) {
                const int sl = p.seq_lens[b];
                s_seq[b] = sl;
                const int nb = min(p.max_blocks, (sl + p.BS - 1) / p.BS);
                n = (max(nb, 0) + p.bps - 1) / p.bps;
            }
            int incl = n;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int o = __shfl_up_sync(0xffffffffu, incl, off);
                if (lane >= off) incl += o;
            }
            if (b < p.B) s_cum[b] = run + incl - n;
            run += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) s_cum[p.B] = run;
    }
    __syncthreads();
    const int total = s_cum[p.B];
    // scores of blocks past each request's length
    for (int64_t i = (int64_t)blockIdx.x * kRowsThreads + tid; i < (int64_t)p.B * p.max_blocks;
         i += (int64_t)gridDim.x * kRowsThreads) {
        const int b = (int)(i / p.max_blocks), j = (int)(i - (int64_t)b * p.max_blocks);
        if (j >= (s_seq[b] + p.BS - 1) / p.BS) p.out[i] = -1;
    }
    // Use u of the ring (u = 0, 1, ...) is stage u % n_stages in round u / n_stages and carries the CTA's u-th work
    // item, flat index blockIdx.x + u * gridDim.x (items are dealt to the CTAs round robin).
    const int my_items = (int)blockIdx.x < total ? (total - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;

    if (warp < kRowsProducers) {
        // ---- producers: lane l of producer w feeds stage 2 l + w ----
        // Every lane runs its own little state machine: the next work item of its stage is resolved ahead of time
        // (request, blocks, block-table entries), and on every turn of the warp's loop the lane tests its stage's
        // "empty" barrier without blocking; when the stage is free it starts the copies and resolves the item after.
        // No lane ever waits inside the loop, so stages are refilled as they are handed back, in whatever order.
        const int my_stage = kRowsProducers * lane + warp;
        const bool mine = my_stage < p.n_stages;
        uint8_t* const stage = s_ring + (size_t)(mine ? my_stage : 0) * p.stage_bytes;
        int u = my_stage, round = 0;
        int b = 0, j0 = 0, seq = 0;
        int phys[8];
        uint32_t mask = 0u;
        auto resolve = [&]() {
            mask = 0u;
#pragma unroll
            for (int i = 0; i < 8; ++i) phys[i] = -1;
            if (!mine || u >= my_items) return;
            const int flat = (int)blockIdx.x + u * (int)gridDim.x;
            int lo = 0, hi = p.B - 1;  // last b with s_cum[b] <= flat
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (s_cum[mid] <= flat) lo = mid; else hi = mid - 1;
            }
            b = lo; j0 = (flat - s_cum[lo]) * p.bps; seq = s_seq[lo];
            const int nb = min(p.max_blocks, (seq + p.BS - 1) / p.BS);
            // the loads are only started here; their values are first looked at when the item is issued, a ring
            // round later, so their latency is not on the producer's path
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (i < p.bps && j0 + i < nb) { phys[i] = p.bt[(int64_t)b * p.bt_stride + j0 + i]; mask |= 1u << i; }
        };
        resolve();
        unsigned long long t0 = 0;
        uint32_t idle = 0;
        bool dead = false;
        for (;;) {
            const bool want = mine && u < my_items && !dead;
            const bool ready = want && (round == 0 || mbar_test_wait(&s_empty[my_stage], (uint32_t)((round - 1) & 1)));
            if (!__any_sync(0xffffffffu, want)) break;
            if (!__any_sync(0xffffffffu, ready)) {
                // nothing to refill right now: leave the issue slots to the consumers for a moment
                __nanosleep(200);
            }
            if (!want) continue;
            if (ready) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {  // entries outside the pool are flagged and left out
                    if (((mask >> i) & 1u) && (phys[i] < 0 || phys[i] >= p.NB)) {
                        flag_status(p.status, UCMR_DEV_BAD_BLOCK_ID);
                        mask &= ~(1u << i);
                    }
                }
                s_meta[my_stage] = RowsMeta{b, j0, seq, mask};
                mbar_expect_tx(&s_full[my_stage], (uint32_t)(__popc(mask) * p.block_bytes));  // (release: the meta is visible)
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if ((mask >> i) & 1u)
                        bulk_g2s(stage + i * p.block_bytes, p.codes + (int64_t)phys[i] * p.block_bytes,
                                 (uint32_t)p.block_bytes, &s_full[my_stage]);
                u += p.n_stages;
                ++round;
                idle = 0;
                t0 = 0;
                resolve();
            } else if ((++idle & 255u) == 0u) {  // bounded: a consumer that stopped never hands the stage back
                const unsigned long long now = global_timer_ns();
                if (t0 == 0) t0 = now;
                else if (now - t0 > kWaitLimitNs) { flag_status(p.status, UCMR_DEV_WAIT_TIMEOUT); dead = true; }
            }
        }
        return;
    }

    // ---- consumers ----
    // Stage s always goes to consumer s % 14 (the number of stages is a multiple of 14), which takes its stages round
    // after round: every barrier has a single waiter that sees each of its phases in order.  (With stages handed to
    // whichever consumer comes next, a fast consumer could wait for a stage two rounds ahead of a slow one, and a
    // parity wait cannot tell those two phases apart.)
    const int ci = warp - kRowsProducers;
    const int seg = min(p.BS, 32);           // lanes that share a block within a 32-row half step
    const int per_consumer = p.n_stages / kRowsConsumers;
    bool stop = false;
    for (int round = 0; !stop; ++round) {
      if (round * p.n_stages + ci >= my_items) break;
      for (int sidx = 0; sidx < per_consumer; ++sidx) {
        const int st = ci + sidx * kRowsConsumers;
        const int u = round * p.n_stages + st;
        if (u >= my_items) break;
        if (!mbar_wait(&s_full[st], (uint32_t)(round & 1))) { flag_status(p.status, UCMR_DEV_WAIT_TIMEOUT); stop = true; break; }
        const RowsMeta m = s_meta[st];
        const uint32_t* sb = reinterpret_cast<const uint32_t*>(s_ring + (size_t)st * p.stage_bytes);
        const uint32_t* pl = p.planes + (int64_t)m.b * kRowPlaneWords;
        const uint4 hdr = __ldg(reinterpret_cast<const uint4*>(pl));
        const int np = (int)hdr.x, base = (int)hdr.y;
        int agg = MIN ? INT_MAX : 0;  // running result of a block longer than one step
        for (int it = 0; it < p.iters; ++it) {
            uint32_t k[2][kRowW];
            bool ok[2];
            int blk[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int tt = it * 64 + 32 * h + lane;  // row of the stage
                // BS is 8, 16, 32, 64 or 128 (checked on the host): shifts instead of divisions
                const int sh = 31 - __clz(p.BS);
                blk[h] = tt >> sh;
                const int within = tt & (p.BS - 1);
                const bool have = blk[h] < p.bps && ((m.valid_mask >> blk[h]) & 1u);
                const int ntok = have ? min(p.BS, m.seq - (m.j0 + blk[h]) * p.BS) : 0;
                ok[h] = within < ntok;
                if (ok[h]) {
                    const uint2* rp = reinterpret_cast<const uint2*>(sb + (size_t)tt * kRowW);
#pragma unroll
                    for (int i = 0; i < kRowW / 2; ++i) { const uint2 v = rp[i]; k[h][2 * i] = v.x; k[h][2 * i + 1] = v.y; }
                } else {
#pragma unroll
                    for (int i = 0; i < kRowW; ++i) k[h][i] = 0u;
                }
            }
            if (it == p.iters - 1) {  // the stage's last rows are in registers: hand it back before the arithmetic
                __syncwarp();
                if (lane == 0) mbar_arrive(&s_empty[st]);
            }
            int d0 = base, d1 = base;
            for (int q = 0; q < np; ++q) {
                const uint4* cp = reinterpret_cast<const uint4*>(pl + 4 + q * kRowWPad);
                const uint4* ap = reinterpret_cast<const uint4*>(pl + 4 + (kRowPlanes + q) * kRowWPad);
                uint32_t v0[kRowW], v1[kRowW];
#pragma unroll
                for (int i4 = 0; i4 < kRowWPad / 4; ++i4) {
                    const uint4 c4 = __ldg(cp + i4), a4 = __ldg(ap + i4);
                    const uint32_t cw[4] = {c4.x, c4.y, c4.z, c4.w}, aw[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int i = i4 * 4 + e;
                        if (i < kRowW) {
                            v0[i] = (k[0][i] & aw[e]) | (~k[0][i] & cw[e]);
                            v1[i] = (k[1][i] & aw[e]) | (~k[1][i] & cw[e]);
                        }
                    }
                }
                d0 += popc18(v0) << q;
                d1 += popc18(v1) << q;
            }
            // block reduce
            int v0 = ok[0] ? d0 : (MIN ? INT_MAX : 0), v1 = ok[1] ? d1 : (MIN ? INT_MAX : 0);
            if (p.BS >= 64) {
                // both rows of the lane belong to the same block
                int v = MIN ? min(v0, v1) : v0 + v1;
                agg = MIN ? min(agg, v) : agg + v;
                if (((it + 1) * 64) % p.BS == 0) {  // the block ends with this step
                    int r = agg;
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1) {
                        const int o = __shfl_xor_sync(0xffffffffu, r, off);
                        r = MIN ? min(r, o) : r + o;
                    }
                    const int bk = (it * 64) / p.BS, j = m.j0 + bk;
                    if (lane == 0 && j < p.max_blocks) p.out[(int64_t)m.b * p.max_blocks + j] = ((m.valid_mask >> bk) & 1u) ? r : -1;
                    agg = MIN ? INT_MAX : 0;
                }
            } else {
                for (int off = 1; off < seg; off <<= 1) {
                    const int o0 = __shfl_xor_sync(0xffffffffu, v0, off), o1 = __shfl_xor_sync(0xffffffffu, v1, off);
                    v0 = MIN ? min(v0, o0) : v0 + o0;
                    v1 = MIN ? min(v1, o1) : v1 + o1;
                }
                if ((lane & (seg - 1)) == 0) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int j = m.j0 + blk[h];
                        if (blk[h] < p.bps && j < p.max_blocks)
                            p.out[(int64_t)m.b * p.max_blocks + j] = ((m.valid_mask >> blk[h]) & 1u) ? (h ? v1 : v0) : -1;
                    }
                }
            }
        }
      }
    }
}

// UCMR_ROWS_KERNEL=0 (read once per process) keeps token-row codes on the one-stage-per-warp kernel.
static bool rows_kernel_enabled()
{
    static const bool v = [] {
        const char* env = getenv("UCMR_ROWS_KERNEL");
        return !(env && env[0] == '0');
    }();
    return v;
}

// Returns UCMR_OK after launching both kernels, or UCMR_ERR_UNSUPPORTED when the shape is not covered (the caller
// then uses the other scan kernels).  `scratch` holds rows_scratch_bytes(B) bytes.
int run_scan_rows(const uint32_t* codes, int64_t NB, int BS, int Hkv, int W, const uint32_t* q, int Hq,
                  const int32_t* bt, int max_blocks, int64_t bt_stride, const int32_t* seq_lens, int B,
                  int reduce_mode, int reduce_kvhead, int32_t* out, int32_t* status, void* scratch, cudaStream_t st)
{
    (void)reduce_kvhead;  // one kv head: nothing to reduce
    reduce_mode &= 0xFF;
    if (!rows_kernel_enabled() || scratch == nullptr) return UCMR_ERR_UNSUPPORTED;
    if (Hkv != 1 || W != kRowW) return UCMR_ERR_UNSUPPORTED;
    if (BS != 8 && BS != 16 && BS != 32 && BS != 64 && BS != 128) return UCMR_ERR_UNSUPPORTED;
    const int G = Hq;
    if (G < 1 || G > 255 || B > kRowsMaxBatch) return UCMR_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(codes) % 16 != 0 || reinterpret_cast<uintptr_t>(scratch) % 16 != 0) return UCMR_ERR_UNSUPPORTED;
    RowsParams p{};
    p.codes = reinterpret_cast<const char*>(codes);
    p.NB = NB; p.BS = BS; p.max_blocks = max_blocks; p.B = B;
    p.planes = static_cast<const uint32_t*>(scratch);
    p.bt = bt; p.bt_stride = bt_stride; p.seq_lens = seq_lens; p.out = out; p.status = status;
    p.block_bytes = BS * kRowW * 4;
    p.bps = BS >= 64 ? 1 : 64 / BS;
    p.iters = BS >= 64 ? BS / 64 : 1;
    p.stage_bytes = p.bps * p.block_bytes;
    p.n_stages = kRowsRingBytes / p.stage_bytes;
    if (p.n_stages > kRowsMaxStages) p.n_stages = kRowsMaxStages;
    p.n_stages = p.n_stages / kRowsConsumers * kRowsConsumers;  // whole stages per consumer (see the kernel)
    if (p.n_stages < kRowsConsumers) return UCMR_ERR_UNSUPPORTED;
    const size_t smem = (size_t)p.n_stages * p.stage_bytes;

    int rc = launch_kernel_ex(rows_planes_kernel, dim3(B), dim3(32), 0, st, 1, true, q, G, static_cast<uint32_t*>(scratch));
    if (rc != UCMR_OK) return rc;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t max_items = (int64_t)B * ((max_blocks + p.bps - 1) / p.bps);
    const int grid = (int)(max_items < sms ? (max_items > 0 ? max_items : 1) : sms);
    void (*kernel)(const RowsParams) = reduce_mode == UCMR_REDUCE_MIN ? scan_rows_kernel<true> : scan_rows_kernel<false>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { note_cuda_error(e); return UCMR_ERR_LAUNCH; }
    return launch_kernel_ex(kernel, dim3(grid), dim3(kRowsThreads), smem, st, 1, true, p);
}

}  // namespace ucmr

// Hamming scan, staged variant (sm_100a): one persistent CTA per SM streams paged code blocks through
// shared memory with the TMA engine; twelve warps each own one 16 KiB stage.
//
//   Every warp runs the same loop over its share of the work items (an item = one code block, or a
//   few small ones): wait for its stage's mbarrier, copy the block from shared memory into registers,
//   start the TMA load of its NEXT item into the now free stage, then do the arithmetic on the
//   registers while that load is in flight.  There is no producer warp and no "stage empty" barrier:
//   the warp that frees a stage is the one that refills it, so the issue latency (resolve request and
//   block-table entry, arm the barrier, launch the copy: several hundred cycles) is spread over twelve
//   instruction streams and overlaps their math.  Up to 12 x 16 KiB are in flight per SM (sum mode uses ten of the
//   stages, see run_scan_ring).  Each
//   barrier has a single waiter that sees every phase in order, so a parity wait is never ambiguous.
//   Work split: the first 7/8 (3/4 in long scans) of the items statically (CTA c, warp w), the rest claimed one by one from an
//   atomic counter so that all SMs finish together; claim and block-table load run one item ahead of use.
//
//     sum mode: the distance sum over a block only depends on how many of its tokens have each code
//       bit set.  A lane owns one 32-bit column (kv head, word) of the block and folds all its tokens
//       into bit-sliced vertical counters with carry-save adders (about 2.4 LOP3 per code word, no
//       per-token popcount); the block score is then
//           sum_g sum_i (q_g[i] ? n - c[i] : c[i]) = n * popc(q) + sum_p 2^p * (G*popc(P_p) - 2*sum_g popc(P_p & q_g)),
//       i.e. (1+G) popcounts per counter plane instead of G per token.  This keeps the kernel
//       bandwidth-bound: the per-token popcount form is limited by the SM's POPC rate (16/clk) once
//       G >= 4.
//     min mode: per-token distances are needed, so a lane owns a 16-byte piece of each token
//       (XOR per query head, then one carry-save popcount sum over the 4*G words) and keeps the running minimum.
//     token-row mode (one kv head, 18 words per token: MLA codes, up to 255 query codes): a lane owns a token;
//       the per-token sum over the query codes comes from bit-sliced per-bit counts of the query codes
//       (1 + log2 G popcount sums per token instead of G), either mode of block reduce.
//
// Output: int32 [B, Hout, max_blocks] block scores, bit-identical to the register kernel in scan.cu,
// which remains the path for shapes this one does not cover.
//
// Stands in for HammingScoreContiKernel + torch.min of the reference
// (ucm/sparse/gsa_on_device/csrc/cuda/ham_dist/paged_ham_dist_mla.cu:111-248,
//  ucm/sparse/gsa_on_device/hamming_topk.py:45-47).
#include <limits.h>
#include <stdlib.h>

#include "common.cuh"

namespace ucmr {

constexpr int kRingWarps = 12;  // each warp owns one stage of the ring
constexpr int kRingThreads = 32 * kRingWarps;
constexpr int kRingBytes = 192 * 1024;
constexpr int kRingMaxBatch = 1024;  // requests per launch (prefix table in shared memory)
constexpr int kRingMaxBps = 8;       // blocks per stage
constexpr int kRingMaxG = 16;

// Selection folded into the scan (ucmr_hamming_topk with rows of at most kFuseMaxBlocks blocks; parameters: FusedSel).
// A warp that has run out of work items arrives at a CTA counter, the CTA's last warp at a grid counter; once every CTA
// has arrived all block scores are in memory, and the warps - waiting for that moment with a bounded poll - take the
// (request, kv head) rows one by one from a ticket counter and select them, one warp per row.  The warp that makes
// the final arrival never waits and keeps taking tickets until none is left, so the result does not depend on the
// others showing up: a warp whose wait ran out simply leaves.  Compared with a second kernel this saves a launch and
// spreads the rows over all SMs while they are still resident.
// A row is selected by one warp: keys in registers, the k-th smallest (key, block) pair found by bisection on its
// packed 32-bit form, then an ordered compaction by ballots.
struct RingParams {
    const char* codes;
    int64_t NB;
    int BS, Hkv, W, G, Hq;
    const uint32_t* q;
    const int32_t* bt;
    int max_blocks;
    int64_t bt_stride;
    const int32_t* seq_lens;
    int B;
    int reduce_kvhead;
    int32_t* out;
    int32_t* status;
    int32_t* sched;    // optional zero-initialised work counter (dynamic item claiming); null = static split
    int RW;            // words per token row = Hkv * W
    int bps;           // blocks per stage
    int block_bytes;   // BS * RW * 4
    int block_stride;  // = block_bytes (blocks of a stage sit back to back)
    int stage_bytes;   // bps * block_stride
    int n_active;      // warps (= stages) in use: min(kRingWarps, ring bytes / stage bytes)
    int early_setup;   // UCMR_FLAG_INPUTS_STABLE: sequence lengths and block table may be read before the dependency wait
    int early_loads;   // UCMR_FLAG_CACHE_APPEND_ONLY: code blocks other than a request's last one may be loaded before it too
    int small_blocks;  // sum mode, rows of 32 words, blocks of 16 or 32 tokens: lane <-> 16-byte piece of the row (see kernel)
    FusedSel sel;
};

struct __align__(16) StageMeta {
    int b, j0, seq;
    uint32_t valid_mask;  // bit k: block j0+k was loaded
};

// 3 -> 2 carry-save adder on bit-sliced values: (h, l) = a + b + c.
__device__ __forceinline__ void csa(uint32_t& h, uint32_t& l, uint32_t a, uint32_t b, uint32_t c)
{
    const uint32_t u = a ^ b;
    h = (a & b) | (u & c);
    l = u ^ c;
}

// sum_i popc(v[i]) with carry-save adders (Harley-Seal): N words of weight 1 become one word of weight 1 and
// N/2 words of weight 2, recursively, so only about log2(N) + 1 popcounts are issued.  POPC runs at a
// quarter of the rate of the logic instructions, which is what bounds the per-token distance forms.
template <int N>
__device__ __forceinline__ int hs_popc(const uint32_t (&v)[N])
{
    if constexpr (N == 1) {
        return __popc(v[0]);
    } else if constexpr (N == 2) {
        return __popc(v[0]) + __popc(v[1]);
    } else {
        constexpr int K = N / 2;  // words of weight 2 produced
        uint32_t carry[K];
        uint32_t ones = v[0];
#pragma unroll
        for (int i = 0; i < (N - 1) / 2; ++i) csa(carry[i], ones, ones, v[1 + 2 * i], v[2 + 2 * i]);
        if constexpr (N % 2 == 0) {  // one word left: half adder
            carry[K - 1] = ones & v[N - 1];
            ones ^= v[N - 1];
        }
        return __popc(ones) + 2 * hs_popc<K>(carry);
    }
}

// A lane buffers CH tokens of its column in registers per chunk: 128, or 64 / 32 / 16 for blocks of at most that
// many tokens (the carry-save work of a chunk is proportional to CH).  The vertical counters of a chunk then need log2(CH) + 1 planes.
__host__ __device__ constexpr int planes_of(int ch) { return ch == 128 ? 8 : ch == 64 ? 7 : ch == 32 ? 6 : 5; }

// Folds 16 words into planes 0..3 (carry-save) and returns the carry of weight 16.
__device__ __forceinline__ uint32_t fold16(uint32_t& ones, uint32_t& twos, uint32_t& fours, uint32_t& eights,
                                           const uint32_t* x)
{
    uint32_t t2a, t2b, t4a, t4b, t8a, t8b, t16;
    csa(t2a, ones, ones, x[0], x[1]);
    csa(t2b, ones, ones, x[2], x[3]);
    csa(t4a, twos, twos, t2a, t2b);
    csa(t2a, ones, ones, x[4], x[5]);
    csa(t2b, ones, ones, x[6], x[7]);
    csa(t4b, twos, twos, t2a, t2b);
    csa(t8a, fours, fours, t4a, t4b);
    csa(t2a, ones, ones, x[8], x[9]);
    csa(t2b, ones, ones, x[10], x[11]);
    csa(t4a, twos, twos, t2a, t2b);
    csa(t2a, ones, ones, x[12], x[13]);
    csa(t2b, ones, ones, x[14], x[15]);
    csa(t4b, twos, twos, t2a, t2b);
    csa(t8b, fours, fours, t4a, t4b);
    csa(t16, eights, eights, t8a, t8b);
    return t16;
}

// Bit-sliced ripple add of two counters of NP planes; the result has NP + 1 planes.
template <int NP>
__device__ __forceinline__ void add_planes(const uint32_t (&a)[NP], const uint32_t (&b)[NP], uint32_t (&out)[NP + 1])
{
    uint32_t carry = 0u;
#pragma unroll
    for (int p = 0; p < NP; ++p) {
        uint32_t h, l;
        csa(h, l, a[p], b[p], carry);
        out[p] = l;
        carry = h;
    }
    out[NP] = carry;
}

// Counts, for every bit position, how many of the CH buffered words have the bit set: bit-sliced
// planes (plane p holds bit p of the 32 counters).  Independent carry-save chains of 32 words each
// (instruction-level parallelism: a single chain is one long dependency), then bit-sliced adds.
template <int CH>
__device__ __forceinline__ void fold_chunk(const uint32_t (&x)[CH], uint32_t (&pl)[planes_of(CH)])
{
    static_assert(CH == 128 || CH == 64 || CH == 32 || CH == 16, "chunk size");
    if constexpr (CH == 16) {
        uint32_t p0 = 0, p1 = 0, p2 = 0, p3 = 0;
        const uint32_t c0 = fold16(p0, p1, p2, p3, &x[0]);
        pl[0] = p0; pl[1] = p1; pl[2] = p2; pl[3] = p3; pl[4] = c0;
    } else {
        uint32_t q6[CH / 32][6];
#pragma unroll
        for (int c = 0; c < CH / 32; ++c) {
            uint32_t p0 = 0, p1 = 0, p2 = 0, p3 = 0;
            const uint32_t c0 = fold16(p0, p1, p2, p3, &x[c * 32]);
            const uint32_t c1 = fold16(p0, p1, p2, p3, &x[c * 32 + 16]);
            q6[c][0] = p0; q6[c][1] = p1; q6[c][2] = p2; q6[c][3] = p3;
            q6[c][4] = c0 ^ c1;
            q6[c][5] = c0 & c1;
        }
        if constexpr (CH == 128) {
            uint32_t h7a[7], h7b[7];
            add_planes<6>(q6[0], q6[1], h7a);
            add_planes<6>(q6[2], q6[3], h7b);
            add_planes<7>(h7a, h7b, pl);
        } else if constexpr (CH == 64) {
            add_planes<6>(q6[0], q6[1], pl);
        } else {
#pragma unroll
            for (int i = 0; i < 6; ++i) pl[i] = q6[0][i];
        }
    }
}

// Groups of 4 or more query heads (compile-time G): sum_g popc(P & q_g) only depends, bit position by bit position, on
// how many of the G query words have the bit set.  With that count kept bit-sliced (plane t = bit t of the count,
// values 0..G need log2(G) + 1 planes) the sum is sum_t 2^t popc(P & C_t): 1 + planes popcounts per counter plane
// instead of 1 + G (5 instead of 9 for G = 8).  The popcount unit, at a quarter of the logic rate, is what a wide
// group is bound by.
__host__ __device__ constexpr int count_planes(int g) { return g >= 16 ? 5 : g >= 8 ? 4 : g >= 4 ? 3 : g >= 2 ? 2 : 1; }
__host__ __device__ constexpr bool counts_sliced(int g_t) { return g_t >= 4; }

// In place: qw[0..G) (the query words of one column) -> qw[0..count_planes(G)) (planes of their per-bit count).
template <int G_T>
__device__ __forceinline__ void slice_query_counts(uint32_t* qw)
{
    if constexpr (counts_sliced(G_T)) {
        constexpr int NQ = count_planes(G_T);
        uint32_t c[NQ];
#pragma unroll
        for (int t = 0; t < NQ; ++t) c[t] = 0u;
#pragma unroll
        for (int g = 0; g < G_T; ++g) {  // bit-sliced increment by query word g
            uint32_t carry = qw[g];
#pragma unroll
            for (int t = 0; t < NQ; ++t) {
                const uint32_t both = c[t] & carry;
                c[t] ^= carry;
                carry = both;
            }
        }
#pragma unroll
        for (int t = 0; t < NQ; ++t) qw[t] = c[t];
    }
}

// sum_g sum_tokens popc(word ^ q[g]) of one buffered chunk of n tokens (unused slots hold 0).  qw: the G query words
// of the column, or (counts_sliced(G_T)) the planes slice_query_counts made of them.
template <int G_T, int CH>
__device__ __forceinline__ int chunk_score(const uint32_t (&x)[CH], int n, int g_rt, const uint32_t* qw)
{
    const int G = G_T > 0 ? G_T : g_rt;
    constexpr int GMAX = G_T > 0 ? G_T : kRingMaxG;
    constexpr int kPlanes = planes_of(CH);
    uint32_t pl[kPlanes];
    fold_chunk<CH>(x, pl);
    if constexpr (counts_sliced(G_T)) {
        constexpr int NQ = count_planes(G_T);
        int qpop = 0;
#pragma unroll
        for (int t = 0; t < NQ; ++t) qpop += __popc(qw[t]) << t;
        int acc = n * qpop;
#pragma unroll
        for (int i = 0; i < kPlanes; ++i) {
            int d = G_T * __popc(pl[i]);
#pragma unroll
            for (int t = 0; t < NQ; ++t) d -= __popc(pl[i] & qw[t]) << (t + 1);
            acc += d * (1 << i);
        }
        return acc;
    }
    int qpop = 0;
#pragma unroll
    for (int g = 0; g < GMAX; ++g)
        if (g < G) qpop += __popc(qw[g]);
    int acc = n * qpop;
#pragma unroll
    for (int i = 0; i < kPlanes; ++i) {
        int d = G * __popc(pl[i]);
#pragma unroll
        for (int g = 0; g < GMAX; ++g)
            if (g < G) d -= 2 * __popc(pl[i] & qw[g]);
        acc += d * (1 << i);
    }
    return acc;
}

// Copies tokens [t0, t0+CH) of the lane's 32-bit column (row stride RW words) from the stage into
// registers; slots at or past ntok read as 0.  `rot` > 0 (several blocks per stage, one per lane
// group): block k starts its walk k tokens later, wrapping inside [0, bs), because the blocks sit on
// 128-byte boundaries and the same token of every block would otherwise hit the same banks.
template <int RW_T, int CH>
__device__ __forceinline__ void load_chunk(uint32_t (&x)[CH], const uint32_t* colp, int t0, int ntok, int rw_rt,
                                           int rot, int bs, bool full_narrow)
{
    const int RW = RW_T > 0 ? RW_T : rw_rt;
    constexpr bool kMaybeNarrow = (RW_T == 0 || RW_T < 32);
    if (kMaybeNarrow && RW < 32) {
        if (full_narrow) {
            // every block of the stage is full and exactly one chunk long: the rotated walk only wraps in
            // its last kRingMaxBps slots (rot < kRingMaxBps), the rest are plain strided loads
            const uint32_t* cp = colp + rot * RW;
#pragma unroll
            for (int i = 0; i < CH; ++i) {
                if (i < CH - kRingMaxBps) x[i] = cp[i * RW];
                else x[i] = (i + rot >= CH) ? cp[(i - CH) * RW] : cp[i * RW];
            }
            return;
        }
#pragma unroll
        for (int i = 0; i < CH; ++i) {
            int tt = t0 + i + rot;
            if (tt >= bs) tt -= bs;
            x[i] = (t0 + i < bs && tt < ntok) ? colp[tt * RW] : 0u;
        }
    } else if (t0 + CH <= ntok) {
        const uint32_t* cp = colp + (size_t)t0 * RW;
#pragma unroll
        for (int i = 0; i < CH; ++i) x[i] = cp[i * RW];
    } else {
        const uint32_t* cp = colp + (size_t)t0 * RW;
#pragma unroll
        for (int i = 0; i < CH; ++i) x[i] = (t0 + i < ntok) ? cp[i * RW] : 0u;
    }
}

// Exact top-k of one (request, kv head) row by ONE warp, same results as select_kernel in topk.cu: the first `kb`
// blocks under (key, block index), key = 0 for forced blocks, score + 1 for valid ones, all ones past the request's
// length; written in ascending block order, then padding.  Lane l holds blocks l, l + 32, ... as packed words
// (key << idx_bits | block), which are distinct, so the chosen set is {word <= T} for the kb-th smallest word T.  For
// kb <= 64 a bound on T from the lanes' two smallest words leaves a handful of candidates that are ranked exactly;
// otherwise T is found by bisection on the count of words <= T.  NK = register slots per lane.
// The scores were written by other SMs: read through L2 (the caller has fenced after seeing the scan complete).
// `f` points at the CTA's shared-memory copy of the selection parameters (reading them through a generic pointer
// into the kernel's parameter space is far slower).
constexpr int kSelListLen = 128;  // chosen blocks a warp lists in shared memory before writing them out

template <int NK>
__device__ __noinline__ void warp_select_row(const FusedSel* fp, const int32_t* scores, const int32_t* bt,
                                             int64_t bt_stride, int n, int BS, int b, int h, int seq, int* list)
{
    const FusedSel& f = *fp;
    const int lane = threadIdx.x & 31;
    const int nb = max(0, min(n, (seq + BS - 1) / BS));
    int kb = f.k;
    if (f.k_per_request) kb = max(0, min(f.k_per_request[b], f.k));
    const bool masked = f.mask != nullptr && f.mask[b] == 0;
    const int row = b * f.Hout + h;
    const int64_t obase = (int64_t)row * f.k;
    const int32_t* srow = scores + (int64_t)row * n;
    const int32_t* btrow = bt + (int64_t)b * bt_stride;
    if (h == 0 && lane == 0) {
        if (f.out_valid) f.out_valid[b] = min(kb, nb);
        if (f.out_newseq) {
            int ns = seq;
            if (!masked) {
                const int over = max(seq - kb * BS, 0);
                ns = seq - (over + BS - 1) / BS * BS;
            }
            f.out_newseq[b] = ns;
        }
    }
    if (masked) {  // not retrieved: the head of the request's own block table
        for (int i = lane; i < f.k; i += 32) {
            const bool pass = i < kb;
            f.out_phys[obase + i] = pass ? btrow[i] : 0;
            if (f.out_logical) f.out_logical[obase + i] = pass ? i : -1;
            if (f.out_scores) f.out_scores[obase + i] = (pass && i < nb) ? __ldcg(srow + i) : -1;
        }
        return;
    }
    const int take = min(kb, n);
    const uint32_t key_invalid = (1u << f.key_bits) - 1u;
    // forced blocks: the sink and recent windows are two ranges; the listed blocks are patched in afterwards
    const int n_sink = f.forced.sink > 0 ? (f.forced.sink + BS - 1) / BS : 0;
    const int first_recent = f.forced.recent > 0 ? max(0, (seq - f.forced.recent) / BS) : nb;
    uint32_t pk[NK];
    {
        int sc[NK];
#pragma unroll
        for (int i = 0; i < NK; ++i) {
            const int j = i * 32 + lane;
            sc[i] = j < nb ? __ldcg(srow + j) : -1;
        }
#pragma unroll
        for (int i = 0; i < NK; ++i) {
            const int j = i * 32 + lane;
            uint32_t key = key_invalid;
            if (j < nb && sc[i] >= 0) key = (j < n_sink || j >= first_recent) ? 0u : (uint32_t)sc[i] + 1u;
            pk[i] = j < n ? ((key << f.idx_bits) | (uint32_t)j) : 0xFFFFFFFFu;
        }
    }
    for (int m = 0; m < f.forced.n_must; ++m) {  // (uniform loop) listed blocks: key 0 unless past the end / bad id
        const int t = f.forced.must[m] >= 0 ? f.forced.must[m] : nb + f.forced.must[m];
        if (t < 0 || t >= nb) continue;
        const int slot = t >> 5, owner = t & 31;
#pragma unroll
        for (int i = 0; i < NK; ++i)
            if (i == slot && lane == owner && (pk[i] >> f.idx_bits) != key_invalid) pk[i] = (uint32_t)t;
    }
    auto write_out = [&](int pos, int j) {
        f.out_phys[obase + pos] = btrow[j];
        if (f.out_logical) f.out_logical[obase + pos] = j;
        if (f.out_scores) f.out_scores[obase + pos] = j < nb ? max(__ldcg(srow + j), -1) : -1;
    };
    const uint32_t lt_mask = (1u << lane) - 1u;
    const uint32_t idx_mask = (1u << f.idx_bits) - 1u;
    uint32_t lo = 0u, hi = (key_invalid << f.idx_bits) | (uint32_t)(n - 1);
    bool done = take <= 0;
    if (!done && take <= 64) {
        // Few blocks wanted (the usual case).  The `take` smallest of the 64 values {two smallest words of every
        // lane} are `take` distinct words of the row, so the largest of them, T0, bounds the take-th smallest word
        // of the whole row from above; the words <= T0 are then few, and the exact choice is made among them.
        uint32_t m1 = 0xFFFFFFFFu, m2 = 0xFFFFFFFFu;
#pragma unroll
        for (int i = 0; i < NK; ++i) {
            m2 = min(m2, max(m1, pk[i]));
            m1 = min(m1, pk[i]);
        }
        int r1 = 0, r2 = 0;  // how many of the 64 values are below m1 / m2
#pragma unroll 8
        for (int src = 0; src < 32; ++src) {
            const uint32_t a = __shfl_sync(0xffffffffu, m1, src), c = __shfl_sync(0xffffffffu, m2, src);
            r1 += (a < m1) + (c < m1);
            r2 += (a < m2) + (c < m2);
        }
        const bool is1 = r1 == take - 1 && m1 != 0xFFFFFFFFu, is2 = r2 == take - 1 && m2 != 0xFFFFFFFFu;
        const uint32_t who = __ballot_sync(0xffffffffu, is1 || is2);
        if (who != 0u) {  // (always, for take <= n; kept as a guard)
            const uint32_t T0 = __shfl_sync(0xffffffffu, is1 ? m1 : m2, __ffs(who) - 1);
            hi = T0;
            int c0 = 0, c1 = 0;
#pragma unroll
            for (int i = 0; i < NK; i += 2) { c0 += pk[i] <= T0; c1 += pk[i + 1] <= T0; }
            const int cnt = __reduce_add_sync(0xffffffffu, c0 + c1);
            if (cnt <= 64) {
                // the candidates, in ascending block order, into the warp's shared list
                int base = 0;
#pragma unroll
                for (int i = 0; i < NK; ++i) {
                    const bool cand = pk[i] <= T0;
                    const uint32_t bal = __ballot_sync(0xffffffffu, cand);
                    if (cand) list[base + __popc(bal & lt_mask)] = (int)pk[i];
                    base += __popc(bal);
                }
                __syncwarp();
                const bool have_a = lane < cnt, have_b = lane + 32 < cnt;
                const uint32_t va = have_a ? (uint32_t)list[lane] : 0xFFFFFFFFu;
                const uint32_t vb = have_b ? (uint32_t)list[lane + 32] : 0xFFFFFFFFu;
                int ra = 0, rb = 0;
                for (int x = 0; x < cnt; ++x) {
                    const uint32_t v = (uint32_t)list[x];
                    ra += v < va;
                    rb += v < vb;
                }
                const bool ca = have_a && ra < take, cb = have_b && rb < take;
                const uint32_t bal_a = __ballot_sync(0xffffffffu, ca), bal_b = __ballot_sync(0xffffffffu, cb);
                if (ca) write_out(__popc(bal_a & lt_mask), (int)(va & idx_mask));
                if (cb) write_out(__popc(bal_a) + __popc(bal_b & lt_mask), (int)(vb & idx_mask));
                __syncwarp();  // the list is reused for the warp's next row
                done = true;
            }
        }
    }
    if (!done) {
        // General case: bisection on the count of words <= T, then an ordered compaction by ballots.
        while (lo < hi) {
            const uint32_t mid = lo + ((hi - lo) >> 1);
            int c0 = 0, c1 = 0, c2 = 0, c3 = 0;  // four chains: the adds of one are dependent
#pragma unroll
            for (int i = 0; i < NK; i += 4) {
                c0 += pk[i] <= mid; c1 += pk[i + 1] <= mid; c2 += pk[i + 2] <= mid; c3 += pk[i + 3] <= mid;
            }
            const int cnt = __reduce_add_sync(0xffffffffu, (c0 + c1) + (c2 + c3));
            if (cnt >= take) hi = mid; else lo = mid + 1u;
        }
        const uint32_t T = lo;
        // The chosen blocks are first listed in shared memory, then written out one per lane, so that the block-table
        // and score loads of different entries are in flight together instead of one load latency per register slot.
        const bool listed = take <= kSelListLen;
        int base = 0;
#pragma unroll
        for (int i = 0; i < NK; ++i) {
            if (base >= take) break;  // (uniform)
            const bool chosen = pk[i] <= T;
            const uint32_t bal = __ballot_sync(0xffffffffu, chosen);
            if (chosen) {
                const int pos = base + __popc(bal & lt_mask);
                const int j = i * 32 + lane;
                if (listed) list[pos] = j; else write_out(pos, j);
            }
            base += __popc(bal);
        }
        if (listed) {
            __syncwarp();
#pragma unroll
            for (int u = 0; u < kSelListLen / 32; ++u) {
                const int pos = u * 32 + lane;
                if (pos < take) write_out(pos, list[pos]);
            }
            __syncwarp();  // the list is reused for the warp's next row
        }
    }
    for (int i = take + lane; i < f.k; i += 32) {  // fewer than k entries: padding
        f.out_phys[obase + i] = 0;
        if (f.out_logical) f.out_logical[obase + i] = -1;
        if (f.out_scores) f.out_scores[obase + i] = -1;
    }
}

// MIN selects the per-token-minimum path; RW_T (sum mode only) and G_T are compile-time copies of the row
// width and group size for the common shapes, 0 = read them from the parameters; CH is the sum mode's
// chunk size.  ROW > 0 selects the token-row path for one kv head with ROW words per token (any group size).
template <bool MIN, int RW_T, int G_T, int CH, int ROW>
__global__ void __launch_bounds__(kRingThreads, 1)
scan_ring_kernel(const RingParams p)
{
    extern __shared__ __align__(128) uint8_t s_ring[];
    __shared__ __align__(8) uint64_t s_full[kRingWarps];
    __shared__ StageMeta s_meta[kRingWarps];
    __shared__ int s_cum[kRingMaxBatch + 1];  // s_cum[b] = work items before request b
    __shared__ int s_seq[kRingMaxBatch];      // seq_lens[b]
    __shared__ volatile int s_pool_empty;     // a warp of this CTA found the dynamic item pool exhausted
    __shared__ int s_warps_done;                // warps of this CTA out of work items (fused selection)
    __shared__ volatile int s_tail_state;       // 0 = scan still running somewhere, 1 = all scores complete, 2 = gave up waiting
    __shared__ volatile int s_epoch;            // the "all scored" word as this launch found it
    __shared__ volatile int s_leader;           // the warp that spoke for the CTA (valid once s_tail_state is set)
    __shared__ FusedSel s_sel;                  // the selection parameters, for the warps that select rows
    __shared__ int s_sel_list[kRingWarps][kSelListLen];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int Hout = p.reduce_kvhead ? 1 : p.Hkv;
    UCMR_STAMP(0);
    grid_launch_dependents();  // a scan launched right behind this one (the next layer's) may set itself up

    if (tid == 0) {
        for (int s = 0; s < kRingWarps; ++s) mbar_init(&s_full[s], 1);
        fence_mbar_init();
        s_pool_empty = 0;
        s_warps_done = 0;
        s_tail_state = 0;
        s_sel = p.sel;
    }
    // Launched early (programmatic dependent launch): the CTA is resident and its barriers are set up while the
    // kernel before it in the stream drains.  Nothing in global memory is read before the wait, because that kernel
    // may be the one that writes the sequence lengths or the block table - unless the caller has ruled that out
    // (early_setup): then the wait moves behind the resolution of the first work items.
    if (!p.early_setup) grid_dependency_wait();
    const bool fused = p.sel.enabled != 0;  // selection folded into the scan (see FusedSel)
    if (fused && !p.early_setup && tid == 0) s_epoch = ld_acquire_gpu(p.sel.all_scored);
    if (warp == 0) {  // prefix sum of items per request
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
    UCMR_STAMP(1);
    const int total_items = s_cum[p.B];

    // Work split.  Static part: CTA c takes flat items c, c + grid, ... and warp w every n_active-th of
    // those.  With a work counter (p.sched) only the first 7/8 of the items are split that way; the rest
    // is claimed item by item with an atomic, so that all SMs finish together whatever their luck with
    // the memory system (a fully dynamic split would serialise ~10^4 atomics on one address).
    auto mark_past_end = [&]() {  // scores of blocks past each request's length
        for (int64_t i = (int64_t)blockIdx.x * kRingThreads + tid; i < (int64_t)p.B * p.max_blocks;
             i += (int64_t)gridDim.x * kRingThreads) {
            const int b = (int)(i / p.max_blocks), j = (int)(i - (int64_t)b * p.max_blocks);
            const int nb = (s_seq[b] + p.BS - 1) / p.BS;
            if (j >= nb)
                for (int h = 0; h < Hout; ++h) p.out[((int64_t)b * Hout + h) * p.max_blocks + j] = -1;
        }
    };
    if (warp >= p.n_active) {
        if (p.early_setup) grid_dependency_wait();
        mark_past_end();
        return;
    }
    uint8_t* const stage = s_ring + (size_t)warp * p.stage_bytes;
    uint64_t* const full = &s_full[warp];
    const int lanes_total = gridDim.x * p.n_active;
    // (small launches stay static: every warp pays at least one atomic to learn that the pool is empty)
    const bool dynamic = p.sched != nullptr && total_items >= 4 * lanes_total;
    // (long scans - 16 items per warp or more - keep a quarter for the pool: SMs drift apart by some 10 % over
    // 150 us, and an SM that is still on its static share when the pool runs dry finishes that much later)
    const int pool_share = total_items >= 16 * lanes_total ? 4 : 8;
    const int static_items = dynamic ? (total_items - total_items / pool_share) / lanes_total * lanes_total : total_items;
    int static_k = 0;
    // claim_start returns a token (meaningful in lane 0); claim_finish turns it into a flat item index or
    // -1.  They are called one item apart so that the atomic's latency is hidden.
    auto claim_start = [&]() -> int {
        const int flat = blockIdx.x + (static_k * p.n_active + warp) * gridDim.x;
        if (flat < static_items || !dynamic) {
            ++static_k;
            return flat;
        }
        int t = total_items;
        if (lane == 0 && !s_pool_empty) {
            t = static_items + atomicAdd(p.sched, 1);
            if (t >= total_items) s_pool_empty = 1;  // spares the CTA's other warps their failing claim
        }
        return t;
    };
    auto claim_finish = [&](int token) -> int {
        const int flat = __shfl_sync(0xffffffffu, token, 0);
        return flat < total_items ? flat : -1;
    };
    // A claimed item resolved to (request, first block, length); lane i < bps holds the block-table entry
    // of block j0 + i (-1: past the end or out of range).  The global load of the entry is started here
    // and first needed one item later, so its latency is off the critical path.
    struct Item { int valid, b, j0, seq, phys; };
    auto resolve = [&](int flat) -> Item {
        Item r{0, 0, 0, 0, -1};
        if (flat < 0) return r;
        int lo = 0, hi = p.B - 1;  // last b with s_cum[b] <= flat
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (s_cum[mid] <= flat) lo = mid; else hi = mid - 1;
        }
        r.valid = 1; r.b = lo; r.j0 = (flat - s_cum[lo]) * p.bps; r.seq = s_seq[lo];
        const int nb = min(p.max_blocks, (r.seq + p.BS - 1) / p.BS);
        if (lane < p.bps && r.j0 + lane < nb) r.phys = p.bt[(int64_t)lo * p.bt_stride + r.j0 + lane];
        return r;
    };
    // Starts the copy of a resolved item into the warp's stage (which must be free).  All lanes call.
    auto issue = [&](const Item& r) {
        if (!r.valid) return;
        int ph = r.phys;
        if (lane < p.bps && ph != -1 && (ph < 0 || ph >= p.NB)) {
            flag_status(p.status, UCMR_DEV_BAD_BLOCK_ID);
            ph = -1;
        }
        const uint32_t mask = __ballot_sync(0xffffffffu, ph >= 0) & ((1u << p.bps) - 1u);
        if (lane == 0) {
            s_meta[warp] = StageMeta{r.b, r.j0, r.seq, mask};
            mbar_expect_tx(full, (uint32_t)(__popc(mask) * p.block_bytes));
        }
        __syncwarp();
        if (lane < p.bps && ph >= 0)
            bulk_g2s(stage + lane * p.block_stride, p.codes + (int64_t)ph * p.block_bytes, (uint32_t)p.block_bytes, full);
        __syncwarp();
    };

    Item cur = resolve(claim_finish(claim_start()));
    int token = claim_start();
    UCMR_STAMP(2);
    // (early_setup) up to here only the sequence lengths and the block table were read; the code cache, the query
    // codes and the score buffer may still be in use by the kernel before this one
    // (early_loads) the kernels still in flight only write the block that holds a request's newest token: the first
    // item's copy starts now unless it contains that block, and travels while those kernels finish.  Everything else
    // - query codes, score stores, the work counter - stays behind the wait.
    const bool first_early = p.early_loads && cur.valid && (int64_t)(cur.j0 + p.bps) * p.BS < (int64_t)cur.seq;
    if (first_early) issue(cur);
    if (first_early) UCMR_STAMP(3);
    if (p.early_setup) {
        grid_dependency_wait();
        if (fused && tid == 0) s_epoch = ld_acquire_gpu(p.sel.all_scored);  // (the kernel before this one may set it)
    }
    UCMR_STAMP(4);
    if (!first_early) issue(cur);
    if (!first_early) UCMR_STAMP(3);
    mark_past_end();  // while the first block is on its way
    Item nxt = resolve(claim_finish(token));
    token = claim_start();
    // refill the (free) stage with the next item and advance the two-deep claim/resolve pipeline
    auto advance = [&]() {
        issue(nxt);
        cur = nxt;
        nxt = resolve(claim_finish(token));
        token = claim_start();
    };
    int cur_b = -1;
    uint32_t phase = 0;
    if constexpr (ROW > 0) {
        // One kv head, ROW words per token (MLA: 512 + 64 bits = 18 words), up to 255 query codes per request.
        // A lane owns a token.  sum_g popc(k ^ q_g) only depends on c[i] = how many of the G query codes have
        // bit i set:  d = sum_i c[i] + G * popc(k) - 2 * sum_p 2^p * popc(k & Q_p),  Q_p = bit p of the counts
        // (bit-sliced), so a token costs (1 + log2 G) popcount sums instead of G, each taken over its ROW words
        // with carry-save adders.  The planes Q_p of the warp's current request live in shared memory.
        constexpr int W = ROW;
        constexpr int kQPlanes = 8;
        __shared__ uint32_t s_qp[kRingWarps][kQPlanes][ROW];
        uint32_t* const qp = &s_qp[warp][0][0];
        const int G = p.G;
        // Per request: the counts are stored minus their minimum cmin over the 32*ROW bit positions, so only
        // bits(max - min) planes are needed (query heads agree on most bits far less often than never or always:
        // the counts sit in a band), and  sum_i k_i c_i = cmin * popc(k) + sum_p 2^p popc(k & Q_p).
        int nq = 0, gk = G;  // planes in use; gk = G - 2 * cmin, the factor of popc(k)
        int ctot = 0;
        while (cur.valid) {
            if (!mbar_wait(full, phase)) { flag_status(p.status, UCMR_DEV_WAIT_TIMEOUT); break; }
            phase ^= 1u;
            const StageMeta m = s_meta[warp];
            if (m.b != cur_b) {
                uint32_t P[kQPlanes];
#pragma unroll
                for (int pl = 0; pl < kQPlanes; ++pl) P[pl] = 0u;
                int cpop = 0;
                if (lane < W) {
                    const uint32_t* qb = p.q + (int64_t)m.b * p.Hq * W + lane;
                    for (int g0 = 0; g0 < G; g0 += 8) {
                        uint32_t wv[8];
#pragma unroll
                        for (int u = 0; u < 8; ++u) wv[u] = (g0 + u < G) ? __ldg(qb + (int64_t)(g0 + u) * W) : 0u;
#pragma unroll
                        for (int u = 0; u < 8; ++u) {
                            uint32_t carry = wv[u];
                            cpop += __popc(carry);
#pragma unroll
                            for (int pl = 0; pl < kQPlanes; ++pl) {  // bit-sliced increment
                                const uint32_t t = P[pl] & carry;
                                P[pl] ^= carry;
                                carry = t;
                            }
                        }
                    }
                }
                // minimum and maximum count over all bit positions: bitwise search from the top plane
                int cmin = 0, cmax = 0;
                {
                    uint32_t mlo = lane < W ? 0xFFFFFFFFu : 0u, mhi = mlo;  // positions still tied for min / max
#pragma unroll
                    for (int pl = kQPlanes - 1; pl >= 0; --pl) {
                        const uint32_t z = mlo & ~P[pl];
                        if (__any_sync(0xffffffffu, z != 0u)) mlo = z; else cmin |= 1 << pl;
                        const uint32_t o = mhi & P[pl];
                        if (__any_sync(0xffffffffu, o != 0u)) { mhi = o; cmax |= 1 << pl; }
                    }
                }
                if (G == 1) cmin = 0;  // plane 0 is then used as the query code itself (see below)
                if (lane < W) {
                    uint32_t borrow = 0u;  // bit-sliced subtraction of the constant cmin
#pragma unroll
                    for (int pl = 0; pl < kQPlanes; ++pl) {
                        const uint32_t b = ((cmin >> pl) & 1) ? 0xFFFFFFFFu : 0u;
                        const uint32_t a = P[pl];
                        P[pl] = a ^ b ^ borrow;
                        borrow = (~a & (b | borrow)) | (b & borrow);
                    }
#pragma unroll
                    for (int pl = 0; pl < kQPlanes; ++pl) qp[pl * W + lane] = P[pl];
                }
                nq = 32 - __clz(cmax - cmin);  // 0 when every position has the same count
                gk = G - 2 * cmin;
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) cpop += __shfl_xor_sync(0xffffffffu, cpop, off);
                ctot = cpop;
                cur_b = m.b;
                __syncwarp();
            }
            // The blocks of a stage sit back to back, so the stage is one array of bps * BS token rows.  It is
            // walked 64 rows at a time, two rows per lane (two independent dependency chains, and every plane
            // word read from shared memory serves both).  BS is a power of two below 32 or a multiple of 32
            // (checked on the host), so each half of a step lies in one block or covers whole blocks.
            const uint32_t* sb = reinterpret_cast<const uint32_t*>(stage);
            const int n_rows = p.bps * p.BS;
            const int seg = min(p.BS, 32);  // lanes that share a block within a half step
            int agg = MIN ? INT_MAX : 0;    // running result of the block in progress (BS >= 32)
            bool reissued = false;
            for (int r0 = 0; r0 < n_rows; r0 += 64) {
                uint32_t k[2][W];
                int blk[2], within[2];
                bool ok[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int tt = r0 + 32 * h + lane;
                    blk[h] = tt / p.BS;
                    within[h] = tt - blk[h] * p.BS;
                    const bool have = tt < n_rows && ((m.valid_mask >> blk[h]) & 1u);
                    const int ntok = have ? min(p.BS, m.seq - (m.j0 + blk[h]) * p.BS) : 0;
                    ok[h] = within[h] < ntok;
                    if (ok[h]) {
                        if constexpr (W % 2 == 0) {
                            const uint2* rp = reinterpret_cast<const uint2*>(sb + (size_t)tt * W);
#pragma unroll
                            for (int i = 0; i < W / 2; ++i) { const uint2 v = rp[i]; k[h][2 * i] = v.x; k[h][2 * i + 1] = v.y; }
                        } else {
#pragma unroll
                            for (int i = 0; i < W; ++i) k[h][i] = sb[(size_t)tt * W + i];
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < W; ++i) k[h][i] = 0u;
                    }
                }
                if (r0 + 64 >= n_rows) {
                    __syncwarp();
                    advance();  // the stage's last words are in registers: refill it before the math
                    reissued = true;
                }
                int d[2], masked[2] = {0, 0};
                if (G == 1) {
                    // a single query code: plane 0 is the code itself, so the distance is popc(k ^ q) directly
                    uint32_t v0[W], v1[W];
#pragma unroll
                    for (int i = 0; i < W; ++i) {
                        const uint32_t qw = qp[i];
                        v0[i] = k[0][i] ^ qw;
                        v1[i] = k[1][i] ^ qw;
                    }
                    d[0] = hs_popc<W>(v0);
                    d[1] = hs_popc<W>(v1);
                } else {
                    d[0] = ctot + gk * hs_popc<W>(k[0]);
                    d[1] = ctot + gk * hs_popc<W>(k[1]);
                }
                for (int pl = 0; pl < (G == 1 ? 0 : nq); ++pl) {
                    uint32_t v0[W], v1[W];
#pragma unroll
                    for (int i = 0; i < W; ++i) {
                        const uint32_t qw = qp[pl * W + i];
                        v0[i] = k[0][i] & qw;
                        v1[i] = k[1][i] & qw;
                    }
                    masked[0] += hs_popc<W>(v0) << pl;
                    masked[1] += hs_popc<W>(v1) << pl;
                }
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    int v = ok[h] ? d[h] - 2 * masked[h] : (MIN ? INT_MAX : 0);
                    for (int off = 1; off < seg; off <<= 1) {
                        const int o = __shfl_xor_sync(0xffffffffu, v, off);
                        v = MIN ? min(v, o) : v + o;
                    }
                    const int tt0 = r0 + 32 * h;  // first row of this half step
                    if (tt0 >= n_rows) continue;
                    if (p.BS < 32) {
                        // whole blocks inside the half step: the first lane of each writes
                        const int j = m.j0 + blk[h];
                        if (within[h] == 0 && blk[h] < p.bps && j < p.max_blocks)
                            p.out[(int64_t)m.b * p.max_blocks + j] = ((m.valid_mask >> blk[h]) & 1u) ? v : -1;
                    } else {
                        agg = MIN ? min(agg, v) : agg + v;
                        if ((tt0 + 32) % p.BS == 0) {  // the block ends with this half step
                            const int bk = tt0 / p.BS, j = m.j0 + bk;
                            if (lane == 0 && j < p.max_blocks)
                                p.out[(int64_t)m.b * p.max_blocks + j] = ((m.valid_mask >> bk) & 1u) ? agg : -1;
                            agg = MIN ? INT_MAX : 0;
                        }
                    }
                }
            }
            if (!reissued) {
                __syncwarp();
                advance();
            }
        }
    } else if constexpr (!MIN) {
        bool small_done = false;
        if constexpr (RW_T == 32 && G_T > 0 && (CH == 16 || CH == 32)) {
            if (p.small_blocks) {
                // Small blocks (16 or 32 tokens of 128 bytes: vLLM's default block sizes with 8 kv heads x 128 bits).
                // Scanning such a block with the whole warp, one column per lane, spends more instructions on the
                // per-block bookkeeping (lengths, shuffles, stores) than on the 16 words a lane folds.  Here a lane
                // owns one 16-byte piece of the token row (4 consecutive words: a kv head of 128-bit codes, half a
                // head of 256-bit ones) in the blocks  lane / 8, lane / 8 + 4, ...  of the stage: it reads its piece
                // of every token with one 16-byte shared-memory load (the 8 lanes of a quarter warp cover the 128
                // bytes of a row, so no bank is hit twice), folds the four columns as four independent carry-save
                // chains and ends up with the whole head's score, so there is no cross-lane reduction for 128-bit
                // codes and the query words stay in registers across blocks.
                small_done = true;
                constexpr int kBlocksPerLane = (CH == 16) ? 2 : 1;  // the stage holds 8 (4) blocks, a lane group of 8 takes every 4th
                const int piece = lane & 7, grp = lane >> 3;
                const int head = (piece * 4) / p.W, w0 = (piece * 4) % p.W;
                uint32_t qv[4][G_T];  // [column of the piece][query head of the group]
                while (cur.valid) {
                    if (cur.b != cur_b) {  // (before the wait: the query words travel while the block does)
#pragma unroll
                        for (int g = 0; g < G_T; ++g) {
                            const uint4 v = __ldg(reinterpret_cast<const uint4*>(
                                p.q + ((int64_t)cur.b * p.Hq + head * G_T + g) * p.W + w0));
                            qv[0][g] = v.x; qv[1][g] = v.y; qv[2][g] = v.z; qv[3][g] = v.w;
                        }
#pragma unroll
                        for (int c = 0; c < 4; ++c) slice_query_counts<G_T>(qv[c]);
                        cur_b = cur.b;
                    }
                    if (!mbar_wait(full, phase)) { flag_status(p.status, UCMR_DEV_WAIT_TIMEOUT); break; }
                    phase ^= 1u;
                    const StageMeta m = s_meta[warp];
                    int score[kBlocksPerLane];
                    int ntoks[kBlocksPerLane];
#pragma unroll
                    for (int bi = 0; bi < kBlocksPerLane; ++bi) {
                        const int blk_e = grp + 4 * bi;
                        const int j = m.j0 + blk_e;
                        const bool have = blk_e < p.bps && ((m.valid_mask >> blk_e) & 1u);
                        const int ntok = have ? min(p.BS, m.seq - j * p.BS) : 0;
                        ntoks[bi] = have ? ntok : -1;
                        const uint4* sp = reinterpret_cast<const uint4*>(stage + blk_e * p.block_stride) + piece;
                        int acc = 0;
                        if constexpr (CH == 16) {
                            uint32_t x0[CH], x1[CH], x2[CH], x3[CH];
#pragma unroll
                            for (int t = 0; t < CH; ++t) {
                                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                                if (t < ntok) v = sp[t * 8];
                                x0[t] = v.x; x1[t] = v.y; x2[t] = v.z; x3[t] = v.w;
                            }
                            if (bi == kBlocksPerLane - 1) {  // the stage's last words are in registers: refill it first
                                __syncwarp();
                                advance();
                            }
                            acc = chunk_score<G_T, CH>(x0, ntok, G_T, qv[0]) + chunk_score<G_T, CH>(x1, ntok, G_T, qv[1]) +
                                  chunk_score<G_T, CH>(x2, ntok, G_T, qv[2]) + chunk_score<G_T, CH>(x3, ntok, G_T, qv[3]);
                        } else {
                            // 32 tokens: two columns at a time (64 registers of buffered words)
                            const uint2* sp2 = reinterpret_cast<const uint2*>(sp);
#pragma unroll
                            for (int half = 0; half < 2; ++half) {
                                uint32_t x0[CH], x1[CH];
#pragma unroll
                                for (int t = 0; t < CH; ++t) {
                                    uint2 v = make_uint2(0u, 0u);
                                    if (t < ntok) v = sp2[t * 16 + half];
                                    x0[t] = v.x; x1[t] = v.y;
                                }
                                if (half == 1) {
                                    __syncwarp();
                                    advance();
                                }
                                acc += chunk_score<G_T, CH>(x0, ntok, G_T, qv[2 * half]) +
                                       chunk_score<G_T, CH>(x1, ntok, G_T, qv[2 * half + 1]);
                            }
                        }
                        score[bi] = acc;
                    }
#pragma unroll
                    for (int bi = 0; bi < kBlocksPerLane; ++bi) {
                        const int blk_e = grp + 4 * bi;
                        const int j = m.j0 + blk_e;
                        int acc = score[bi];
                        // pieces of one head (256-bit codes: two), or of all heads, sit in neighbouring lanes
                        const int span = p.reduce_kvhead ? 8 : p.W / 4;
                        for (int off = 1; off < span; off <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
                        if (blk_e < p.bps && j < p.max_blocks) {
                            const int v = ntoks[bi] >= 0 ? acc : -1;  // -1: past the request's end or a bad block id
                            if (p.reduce_kvhead) {
                                if (piece == 0) p.out[(int64_t)m.b * p.max_blocks + j] = v;
                            } else if (w0 == 0) {
                                p.out[((int64_t)m.b * Hout + head) * p.max_blocks + j] = v;
                            }
                        }
                    }
                }
            }
        }
        if (!small_done) {
        // lane <-> (block in stage, column); a column is one 32-bit word of one kv head
        const int RW = RW_T > 0 ? RW_T : p.RW;
        const int G = G_T > 0 ? G_T : p.G;
        constexpr int GMAX = G_T > 0 ? G_T : kRingMaxG;
        const int cols = min(RW, 32);
        const int passes = RW / cols;
        const int blk = (RW < 32) ? lane / RW : 0;
        const int col0 = (RW < 32) ? lane % RW : lane;
        const int rot = (RW < 32) ? blk % max(p.BS, 1) : 0;  // see load_chunk
        // query words of the lane's column(s): kept across items of one request; rows of 64 words keep both
        // passes' sets, wider rows reload per pass
        constexpr int QP = (RW_T == 64) ? 2 : 1;
        uint32_t qw[QP][GMAX];
        const bool q_kept = passes <= QP;  // every pass has its own register set: loaded once per request
        [[maybe_unused]] bool first_item = true;  // (step timeline only)
        while (cur.valid) {
            if (q_kept && cur.b != cur_b) {  // (before the wait: the query words travel while the block does)
#pragma unroll
                for (int ps = 0; ps < QP; ++ps) {
                    const int col = col0 + ps * 32;
                    const int head = col / p.W, w = col - head * p.W;
#pragma unroll
                    for (int g = 0; g < GMAX; ++g)
                        if (ps < passes && g < G) qw[ps][g] = __ldg(p.q + ((int64_t)cur.b * p.Hq + head * G + g) * p.W + w);
                    slice_query_counts<G_T>(qw[ps]);
                }
                cur_b = cur.b;
            }
            if (!mbar_wait(full, phase)) { flag_status(p.status, UCMR_DEV_WAIT_TIMEOUT); break; }
            if (first_item) UCMR_STAMP(5);
            phase ^= 1u;
            const StageMeta m = s_meta[warp];
            bool reissued = false;
            // rows of 32 words or more: the blocks of a stage (several when they are small) are scanned one after
            // the other by the whole warp; narrower rows: one lane group per block, all at once
            const int seq_blocks = (RW < 32) ? 1 : p.bps;
            for (int sbi = 0; sbi < seq_blocks; ++sbi) {
            const int blk_e = (RW < 32) ? blk : sbi;
            const int j = m.j0 + blk_e;
            const bool have = blk_e < p.bps && ((m.valid_mask >> blk_e) & 1u);
            const int ntok = have ? min(p.BS, m.seq - j * p.BS) : 0;
            const uint8_t* sb = stage + blk_e * p.block_stride;
            int total = 0;  // per-head (or all-head) score, complete in the lanes that write
            // tokens are walked in chunks; with one lane group per block every group walks the whole block
            // capacity (rotated), else only the valid tokens
            const int walk = (RW < 32) ? p.BS : ntok;
            const int n_chunks = (__reduce_max_sync(0xffffffffu, walk) + CH - 1) / CH;
            const bool full_narrow = RW < 32 && p.BS == CH && __all_sync(0xffffffffu, ntok == CH);
            for (int ps = 0; ps < passes; ++ps) {
                const int col = col0 + ps * 32;
                const int head = col / p.W, w = col - head * p.W;
                const int qs = (QP == 2) ? ps : 0;
                if (!q_kept) {
#pragma unroll
                    for (int g = 0; g < GMAX; ++g)
                        if (g < G) qw[qs][g] = __ldg(p.q + ((int64_t)m.b * p.Hq + head * G + g) * p.W + w);
                    slice_query_counts<G_T>(qw[qs]);
                }
                const uint32_t* colp = reinterpret_cast<const uint32_t*>(sb) + col;
                int acc = 0;
                for (int c = 0; c < n_chunks; ++c) {
                    uint32_t x[CH];
                    load_chunk<RW_T, CH>(x, colp, c * CH, ntok, RW, rot, p.BS, full_narrow);
                    if (sbi == seq_blocks - 1 && ps == passes - 1 && c == n_chunks - 1) {
                        // the stage's last words are in registers: refill it before doing the math
                        __syncwarp();
                        advance();
                        reissued = true;
                    }
                    const int n_here = max(0, min(CH, ntok - ((RW < 32) ? 0 : c * CH)));
                    acc += chunk_score<G_T, CH>(x, (RW < 32) ? (c == 0 ? ntok : 0) : n_here, G, qw[qs]);
                }
                // fold the words of a head; with reduce_kvhead also the heads of this pass
                const int span = p.reduce_kvhead ? cols : p.W;
                for (int off = 1; off < span && off < 32; off <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
                if (p.reduce_kvhead) {
                    total += acc;
                } else if (have && w == 0) {
                    p.out[((int64_t)m.b * Hout + head) * p.max_blocks + j] = acc;
                }
            }
            if (p.reduce_kvhead && have && col0 == 0) p.out[(int64_t)m.b * p.max_blocks + j] = total;
            if (!have && blk_e < p.bps && col0 == 0 && j < p.max_blocks) {
                // block inside the stage but not loaded: past the request's end or a bad id
                for (int h = 0; h < Hout; ++h) p.out[((int64_t)m.b * Hout + h) * p.max_blocks + j] = -1;
            }
            }
            if (!reissued) {
                __syncwarp();
                advance();
            }
            if (first_item) UCMR_STAMP(6);
            first_item = false;
        }
        }  // (!small_done)
    } else {
        // lane <-> (block in stage, 16-byte piece of a token row, token slot)
        const int PW = p.W / 4, P = p.Hkv * PW;
        const int LG = 32 / p.bps;     // lanes per block
        const int TS = LG / P;         // token slots per block (>= 1 by construction)
        const int blk = lane / LG, lam = lane % LG;
        const int hp = lam % P, slot = lam / P;
        const int head = hp / PW, part = hp % PW;
        const int G = G_T > 0 ? G_T : p.G;
        constexpr int GMAX = G_T > 0 ? G_T : kRingMaxG;
        constexpr int kMinRounds = 16;  // 16-byte pieces a lane buffers in registers at a time
        uint4 qv[GMAX];
        // Groups of 2, 4 or 8 query heads: sum_g popc(k ^ q_g) only depends, bit position by bit position, on the key
        // bit and on c = how many of the G query codes have the bit set: the position contributes  k ? G - c : c.
        // With c and G - c kept bit-sliced per query (planes cnt[p], alt[p]), plane p of the contribution is the mux
        // k ? alt[p] : cnt[p] - one logic instruction per plane and word - and the distance is
        // sum_p 2^p popc(plane p): P = bits(G) + ... planes instead of G XOR-popcounts per word.  For even G plane 0
        // does not depend on k (G - c and c have the same parity) and is folded into a per-query constant.
        constexpr int kMuxPlanes = G_T >= 8 ? 4 : G_T >= 4 ? 3 : 2;
        constexpr int kMuxFirst = (G_T >= 2 && G_T % 2 == 0) ? 1 : 0;
        uint4 cnt[kMuxPlanes], alt[kMuxPlanes];
        int mux_const = 0;
        while (cur.valid) {
            if (cur.b != cur_b) {  // (before the wait: query words and planes are ready when the block lands)
                const uint4* q4 = reinterpret_cast<const uint4*>(p.q) + ((int64_t)cur.b * p.Hq + head * G) * PW + part;
#pragma unroll
                for (int g = 0; g < GMAX; ++g)
                    if (g < G) qv[g] = __ldg(q4 + g * PW);
                cur_b = cur.b;
                if constexpr (G_T >= 2) {
                    uint32_t* cw = reinterpret_cast<uint32_t*>(cnt);
                    uint32_t* aw = reinterpret_cast<uint32_t*>(alt);
                    mux_const = 0;
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
                        uint32_t pl[kMuxPlanes];
#pragma unroll
                        for (int q = 0; q < kMuxPlanes; ++q) pl[q] = 0u;
#pragma unroll
                        for (int g = 0; g < G_T; ++g) {  // bit-sliced increment by query code g
                            uint32_t carry = reinterpret_cast<const uint32_t*>(&qv[g])[w];
#pragma unroll
                            for (int q = 0; q < kMuxPlanes; ++q) {
                                const uint32_t t = pl[q] & carry;
                                pl[q] ^= carry;
                                carry = t;
                            }
                        }
                        uint32_t borrow = 0u;  // bit-sliced G - c
#pragma unroll
                        for (int q = 0; q < kMuxPlanes; ++q) {
                            const uint32_t gb = ((G_T >> q) & 1) ? 0xFFFFFFFFu : 0u;
                            const uint32_t c = pl[q];
                            cw[q * 4 + w] = c;
                            aw[q * 4 + w] = gb ^ c ^ borrow;
                            borrow = (~gb & (c | borrow)) | (c & borrow);
                        }
                        if (kMuxFirst == 1) mux_const += __popc(pl[0]);
                    }
                }
            }
            if (!mbar_wait(full, phase)) { flag_status(p.status, UCMR_DEV_WAIT_TIMEOUT); break; }
            phase ^= 1u;
            const StageMeta m = s_meta[warp];
            const int j = m.j0 + blk;
            const bool have = (m.valid_mask >> blk) & 1u;
            const int ntok = have ? min(p.BS, m.seq - j * p.BS) : 0;
            const uint4* sb = reinterpret_cast<const uint4*>(stage + blk * p.block_stride);
            int best = INT_MAX;
            const int rounds = (p.BS + TS - 1) / TS;  // same trip count in every lane (shuffles inside)
            for (int r0 = 0; r0 < rounds; r0 += kMinRounds) {
                uint4 kb[kMinRounds];
#pragma unroll
                for (int i = 0; i < kMinRounds; ++i) {
                    const int tok = (r0 + i) * TS + slot;
                    kb[i] = make_uint4(0u, 0u, 0u, 0u);
                    if (tok < ntok) kb[i] = sb[tok * P + hp];
                }
                if (r0 + kMinRounds >= rounds) {
                    __syncwarp();
                    advance();  // the stage's last words are in registers: refill it before the math
                }
#pragma unroll
                for (int i = 0; i < kMinRounds; ++i) {
                    const int tok = (r0 + i) * TS + slot;
                    int d = 0;
                    if constexpr (G_T >= 2) {
                        d = mux_const;
#pragma unroll
                        for (int q = kMuxFirst; q < kMuxPlanes; ++q) {
                            const uint4 k = kb[i], a = alt[q], c = cnt[q];
                            const int s = __popc((k.x & a.x) | (~k.x & c.x)) + __popc((k.y & a.y) | (~k.y & c.y)) +
                                          __popc((k.z & a.z) | (~k.z & c.z)) + __popc((k.w & a.w) | (~k.w & c.w));
                            d += s << q;
                        }
                    } else {
#pragma unroll
                        for (int g = 0; g < GMAX; ++g)
                            if (g < G)
                                d += __popc(kb[i].x ^ qv[g].x) + __popc(kb[i].y ^ qv[g].y) + __popc(kb[i].z ^ qv[g].z) +
                                     __popc(kb[i].w ^ qv[g].w);
                    }
                    for (int off = 1; off < PW; off <<= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
                    best = min(best, tok < ntok ? d : INT_MAX);
                }
            }
            // lanes of the same block that differ in the token slot (>= P), or with reduce_kvhead in
            // the head bits as well, fold by min
            for (int off = p.reduce_kvhead ? PW : P; off < LG; off <<= 1)
                best = min(best, __shfl_xor_sync(0xffffffffu, best, off));
            if (j < p.max_blocks) {
                if (p.reduce_kvhead) {
                    if (lam == 0) p.out[(int64_t)m.b * p.max_blocks + j] = have ? best : -1;
                } else if (slot == 0 && part == 0) {
                    p.out[((int64_t)m.b * Hout + head) * p.max_blocks + j] = have ? best : -1;
                }
            }
        }
    }
    UCMR_STAMP(7);
    if (fused) {
        // Out of work items: arrive (after this warp's score stores are visible device-wide).  The last warp of the
        // CTA to arrive speaks for the CTA: it makes the grid-level arrival and, unless that was the final one, polls
        // the grid's "all scored" word; its sibling warps watch a shared-memory copy, so that word's L2 line sees
        // one poller per SM.  The word counts launches: the final arrival sets it to the value read at the start of
        // this launch plus one (and clears the counters for the next launch), so nothing has to be reset afterwards.
        __threadfence();
        __syncwarp();
        const int grid = (int)gridDim.x;
        int state = 0;
        int cta_last = 0;
        if (lane == 0) cta_last = atomicAdd(&s_warps_done, 1) == p.n_active - 1;
        cta_last = __shfl_sync(0xffffffffu, cta_last, 0);
        if (lane == 0) {
            if (cta_last) {
                const int epoch = s_epoch;
                if (atom_add_release_gpu(p.sel.cta_done, 1) == grid - 1) {
                    *p.sel.cta_done = 0;
                    if (p.sched != nullptr) *p.sched = 0;  // (no warp of the grid claims work any more)
                    st_release_gpu(p.sel.all_scored, epoch + 1);
                    state = 1;
                } else {
                    // (the timer is only consulted every 1024 polls: reading it costs far more than a poll)
                    unsigned long long t0 = 0;
                    state = 2;
                    for (uint32_t polls = 1;; ++polls) {
                        if (ld_acquire_gpu(p.sel.all_scored) != epoch) { state = 1; break; }
                        if ((polls & 1023u) == 0u) {
                            const unsigned long long now = global_timer_ns();
                            if (t0 == 0) t0 = now;
                            else if (now - t0 > kWaitLimitNs) break;
                        }
                        __nanosleep(40);
                    }
                }
                s_leader = warp;
                __threadfence_block();
                s_tail_state = state;
            } else {
                unsigned long long t0 = 0;
                state = 2;
                for (uint32_t polls = 1;; ++polls) {
                    const int v = s_tail_state;
                    if (v != 0) { state = v; break; }
                    if ((polls & 1023u) == 0u) {
                        const unsigned long long now = global_timer_ns();
                        if (t0 == 0) t0 = now;
                        else if (now - t0 > kWaitLimitNs + kWaitLimitNs / 8) break;
                    }
                    __nanosleep(40);
                }
            }
        }
        state = __shfl_sync(0xffffffffu, state, 0);
        if (state != 1) {
            flag_status(p.status, UCMR_DEV_WAIT_TIMEOUT);  // part of the grid never finished scanning: rows not selected
        } else {
            __threadfence();  // the scores written by the other SMs are read after this point
            // Rows blockIdx.x, blockIdx.x + grid, ... belong to this CTA.  The warp that spoke for the CTA takes the
            // first of them (it learns of the completion first), its siblings the others in order of warp index.
            const int n_rows = p.B * p.sel.Hout;
            int slot;  // this warp's position among the CTA's row takers
            if (cta_last) slot = 0;
            else slot = 1 + warp - (warp > s_leader ? 1 : 0);
            for (int t = blockIdx.x + slot * grid; t < n_rows; t += lanes_total) {
                const int b = t / p.sel.Hout, h = t - b * p.sel.Hout;
                if (p.max_blocks <= 1024)
                    warp_select_row<32>(&s_sel, p.out, p.bt, p.bt_stride, p.max_blocks, p.BS, b, h, s_seq[b], s_sel_list[warp]);
                else
                    warp_select_row<kFuseMaxBlocks / 32>(&s_sel, p.out, p.bt, p.bt_stride, p.max_blocks, p.BS, b, h,
                                                         s_seq[b], s_sel_list[warp]);
            }
        }
    }
}

// UCMR_SMALL_BLOCKS=0 (read once per process) sends blocks of 16 / 32 tokens through the general column-per-lane code.
static bool small_blocks_enabled()
{
    static const bool v = [] {
        const char* env = getenv("UCMR_SMALL_BLOCKS");
        return !(env && env[0] == '0');
    }();
    return v;
}

// Returns UCMR_OK after launching, or UCMR_ERR_UNSUPPORTED when the shape is not covered (the caller
// then uses the register kernel).
int run_scan_ring(const uint32_t* codes, int64_t NB, int BS, int Hkv, int W, const uint32_t* q, int Hq,
                  const int32_t* bt, int max_blocks, int64_t bt_stride, const int32_t* seq_lens, int B,
                  int reduce_mode, int reduce_kvhead, int32_t* out, int32_t* status, int32_t* sched, cudaStream_t st,
                  const FusedSel* fuse)
{
    const bool inputs_stable = (reduce_mode & UCMR_FLAG_INPUTS_STABLE) != 0;
    const bool append_only = (reduce_mode & UCMR_FLAG_CACHE_APPEND_ONLY) != 0;
    reduce_mode &= 0xFF;
    const int G = Hq / Hkv;
    const int64_t RW = (int64_t)Hkv * W;
    // MLA codes: one latent "head" of 576 bits; blocks of 8, 16 or a multiple of 32 tokens
    const bool row_mode = Hkv == 1 && W == 18 && (BS % 32 == 0 || BS == 16 || BS == 8);
    if (!row_mode && (!is_pow2(W) || !is_pow2(Hkv) || W > 32 || RW < 4 || RW > 1024)) return UCMR_ERR_UNSUPPORTED;
    if ((row_mode ? G > 255 : G > kRingMaxG) || G < 1 || B > kRingMaxBatch) return UCMR_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(codes) % 16 != 0) return UCMR_ERR_UNSUPPORTED;
    const int64_t block_bytes = (int64_t)BS * RW * 4;
    if (block_bytes % 16 != 0 || block_bytes > 32 * 1024) return UCMR_ERR_UNSUPPORTED;
    const bool is_min = reduce_mode == UCMR_REDUCE_MIN;
    int bps = 1;
    if (row_mode) {
        // several blocks per stage, scanned one after the other
        while (bps < kRingMaxBps && block_bytes * (bps + 1) <= 16 * 1024) ++bps;
    } else if (is_min) {
        if (W % 4 != 0 || reinterpret_cast<uintptr_t>(q) % 16 != 0) return UCMR_ERR_UNSUPPORTED;
        const int P = Hkv * (W / 4);
        if (P > 32) return UCMR_ERR_UNSUPPORTED;
        // several small blocks share a stage (one lane group per block) as long as a group still covers a token
        while (bps < kRingMaxBps && 32 / (bps * 2) >= P && block_bytes * bps * 2 <= 16 * 1024) bps *= 2;
    } else {
        if (RW < 32) bps = (int)(32 / RW);
        else while (bps < kRingMaxBps && block_bytes * (bps + 1) <= 16 * 1024) ++bps;  // small blocks: several per stage
        if (bps > kRingMaxBps) return UCMR_ERR_UNSUPPORTED;
    }
    RingParams p{};
    p.codes = reinterpret_cast<const char*>(codes);
    p.NB = NB; p.BS = BS; p.Hkv = Hkv; p.W = W; p.G = G; p.Hq = Hq;
    p.q = q; p.bt = bt; p.max_blocks = max_blocks; p.bt_stride = bt_stride; p.seq_lens = seq_lens; p.B = B;
    p.reduce_kvhead = reduce_kvhead ? 1 : 0; p.out = out; p.status = status; p.sched = sched;
    p.RW = (int)RW; p.bps = bps; p.block_bytes = (int)block_bytes; p.early_setup = inputs_stable ? 1 : 0;
    p.early_loads = (inputs_stable && append_only) ? 1 : 0;
    // small blocks of full-width rows: the lane <-> row-piece mapping (W = 4 or 8, and a stage of exactly 8 or 4 blocks)
    p.small_blocks = (!row_mode && !is_min && RW == 32 && (W == 4 || W == 8) && (BS == 16 || BS == 32) &&
                      (G == 1 || G == 2 || G == 4 || G == 8) && bps == (BS == 16 ? 8 : 4) &&
                      reinterpret_cast<uintptr_t>(q) % 16 == 0 && small_blocks_enabled()) ? 1 : 0;
    if (fuse != nullptr) {
        if (max_blocks > kFuseMaxBlocks || B > kWsMaxBatch || fuse->key_bits + fuse->idx_bits > 31) return UCMR_ERR_BAD_ARG;
        p.sel = *fuse;
        p.sel.enabled = 1;
    }
    if (block_bytes % (row_mode ? 16 : 128) != 0) return UCMR_ERR_UNSUPPORTED;
    if (!is_min && RW < 32 && BS > 240) return UCMR_ERR_UNSUPPORTED;
    p.block_stride = (int)block_bytes;
    p.stage_bytes = bps * p.block_stride;
    p.n_active = kRingBytes / p.stage_bytes;
    if (p.n_active > kRingWarps) p.n_active = kRingWarps;
    // Sum mode keeps ten of the twelve stages in use: 148 x 10 x 16 KiB in flight still saturate the memory system,
    // and what is in flight beyond that only lengthens the queue - the first wave and the drain of a launch (measured
    // on 268 MB, block 128: 46.0 -> 45.0 us per launch, the decode step 57.5 -> 56.6 us; eight stages make the launch
    // faster still, 44.4 us, but not the step, whose scan starts on half of the SMs first and needs the headroom to
    // even that out; six lose bandwidth: 54 us).  The min and token-row modes need all twelve warps for their
    // arithmetic (block 128, G = 4: 54 us with twelve, 59-60 us with eight or ten).
    if (!is_min && !row_mode && p.n_active > 10) p.n_active = 10;
    if (p.n_active < 4) return UCMR_ERR_UNSUPPORTED;
    const size_t smem = (size_t)p.n_active * p.stage_bytes;

    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // upper bound of the work items; the kernel computes the exact count from seq_lens
    const int64_t max_items = (int64_t)B * ((max_blocks + bps - 1) / bps);
    const int grid = (int)(max_items < sms ? (max_items > 0 ? max_items : 1) : sms);

    void (*kernel)(const RingParams) = nullptr;
    if (row_mode) {
        kernel = is_min ? scan_ring_kernel<true, 0, 0, 128, 18> : scan_ring_kernel<false, 0, 0, 128, 18>;
    } else if (is_min) {
        switch (G) {
            case 1: kernel = scan_ring_kernel<true, 0, 1, 128, 0>; break;
            case 2: kernel = scan_ring_kernel<true, 0, 2, 128, 0>; break;
            case 4: kernel = scan_ring_kernel<true, 0, 4, 128, 0>; break;
            case 8: kernel = scan_ring_kernel<true, 0, 8, 128, 0>; break;
            default: kernel = scan_ring_kernel<true, 0, 0, 128, 0>;
        }
    } else {
        const bool short_blocks = BS <= 64;  // half-size register chunks (wide rows only)
#define UCMR_RING_CASE(RWV, GV, CHV) \
    if (p.RW == RWV && G == GV) kernel = scan_ring_kernel<false, RWV, GV, CHV, 0>;
#define UCMR_RING_ROW(RWV, CHV) \
    UCMR_RING_CASE(RWV, 1, CHV) UCMR_RING_CASE(RWV, 2, CHV) UCMR_RING_CASE(RWV, 4, CHV) UCMR_RING_CASE(RWV, 8, CHV)
        if (BS <= 16) {
            UCMR_RING_ROW(32, 16) UCMR_RING_ROW(64, 16)
        } else if (BS <= 32) {
            UCMR_RING_ROW(32, 32) UCMR_RING_ROW(64, 32)
        } else if (short_blocks) {
            UCMR_RING_ROW(32, 64) UCMR_RING_ROW(64, 64)
        }
        if (!kernel) {
            UCMR_RING_ROW(4, 128) UCMR_RING_ROW(8, 128) UCMR_RING_ROW(16, 128) UCMR_RING_ROW(32, 128) UCMR_RING_ROW(64, 128)
        }
#undef UCMR_RING_ROW
#undef UCMR_RING_CASE
        if (!kernel) kernel = scan_ring_kernel<false, 0, 0, 128, 0>;
    }
    // idempotent attribute, set on every call: cheap, and correct on every device of a process
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kRingBytes);
    if (e != cudaSuccess) { note_cuda_error(e); return UCMR_ERR_LAUNCH; }
    return launch_kernel_ex(kernel, dim3(grid), dim3(kRingThreads), smem, st, 1, true, p);
}

#ifdef UCMR_TRACE
UCMR_TRACE_READER(trace_read_scan)
#endif

}  // namespace ucmr

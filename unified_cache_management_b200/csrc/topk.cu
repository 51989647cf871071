// Exact per-row top-k over block scores (sm_100a): radix select in shared memory + ordered
// compaction.  One CTA per (request, kv head) row; a few very long rows are split over a thread-block cluster
// (distributed shared memory).  The same routine merges the candidate records of sequence shards, which arrive
// either through a collective or as peer-memory stores of the other GPUs' selection kernels (flag wait).
//
// Each candidate j has a key (forced block -> 0, valid block -> score + 1, past the request's length ->
// all ones).  Two or three 11-bit histogram passes find the k-th smallest key T and how many keys equal
// to T are still needed; a single ordered pass then emits every j with key < T and the first `need` j
// with key == T, which is exactly "first k under (key, id)", already in ascending id order.  No sort
// is involved.
//
// Stands in for torch.topk + torch.sort + torch.gather of the reference
// (ucm/sparse/gsa_on_device/hamming_topk.py:49-54) and for update_seq_lens (:7-12), with the
// (score, id) total order the reference leaves unspecified.
#include <limits.h>
#include <math.h>
#include <stdlib.h>

#include <cooperative_groups.h>

#include <type_traits>

#include "common.cuh"

namespace ucmr {

int run_scan(const uint32_t* codes, int64_t NB, int BS, int Hkv, int W, const uint32_t* q, int Hq,
             const int32_t* bt, int max_blocks, int64_t bt_stride, const int32_t* seq_lens, int B,
             int reduce_mode, int reduce_kvhead, int32_t* out, int32_t* status, int32_t* sched, cudaStream_t st,
             const FusedSel* fuse, bool* fused, void* row_scratch);
size_t rows_scratch_bytes(int B);

constexpr int kSelThreads = 512;
constexpr int kSelWarps = kSelThreads / 32;
constexpr int kSelMaxCachedKeys = 40 * 1024;  // 160 KiB of keys in shared memory at most
constexpr uint32_t kKeyInvalid = 0xFFFFFFFFu;
constexpr int kSelInlineKeys = 8 * kSelThreads;  // rows (slices) up to this many keys apply the forced-block rule while loading
// Rows longer than this are split over a thread-block cluster (2, 4 or 8 CTAs) when there are few enough rows.
// Measured: a cluster launch costs about 2 us more than a plain one and large grids of clusters schedule
// slowly, so shorter rows and launches of many rows stay with one CTA per row.
constexpr int kSelClusterSlice = 2048;

constexpr int kMaxPeers = 8;  // ranks of one NVLink domain that exchange candidate records directly

__device__ __forceinline__ void st_relaxed_sys(int32_t* p, int v)
{
    asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int32_t* p)
{
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

constexpr int kDigitBits = 11;
constexpr int kBins = 1 << kDigitBits;
constexpr int kBinsPerThread = kBins / kSelThreads;

struct SelScratch {
    int hist[3][kBins];  // one histogram per radix pass (keys have at most 32 bits: 3 passes of <= 11)
    int warp_a[kSelWarps], warp_b[kSelWarps];
    uint32_t w_lo[kSelWarps], w_hi[kSelWarps];  // per-warp partials of the key range ...
    int w_zero[kSelWarps], w_norm[kSelWarps];   // ... and of the forced / ordinary key counts (written once)
    uint32_t prefix;
    int remaining;
    uint32_t kmin, kmax;  // range of the ordinary keys
    int n_zero, n_normal;  // forced keys, ordinary keys
    int cta_lt, cta_eq;    // this CTA's slice: keys below / equal to the threshold
    // cluster-wide values, gathered by warp 0 from the other CTAs' scratch
    int g_zero, g_normal;
    uint32_t g_kmin, g_kmax;
    int base_lt, base_eq;
};

// Finds the first kb entries of keys[0..n) under (key, position) and calls emit(pos, j) for each,
// pos = rank of j among the chosen in ascending j.  Keys are below 2^key_bits.  key_of has two pure members:
// raw(j) does the global loads of entry j, key(j, raw) turns them into the key; key_fast may skip rules that
// fixup(s_keys, j_lo, n_cached) (called by all threads, between two barriers) applies to the cached keys
// afterwards.  All threads of the CTA must call this.
//
// Radix select from the most significant digit: ceil(key_bits / 11) histogram passes over 2048 bins
// each (a block score needs 17-20 bits, so two passes), every pass narrowing the candidates to the bin
// that holds the kb-th smallest key.  Then one ordered pass emits every j with key < T and the first
// `need` j with key == T: that is "first kb under (key, id)", already in ascending id order.
//
// CL = true: the CTAs of a thread-block cluster share one row.  CTA r works on the r-th slice of the row
// (its keys cached in its own shared memory).  Key range and emit offsets are combined by warp 0 reading the
// other CTAs' scratch through distributed shared memory after a cluster barrier (lane r reads CTA r: one
// remote latency); histograms are summed in CTA 0's shared memory with remote atomics on the non-empty bins,
// and every CTA derives the same threshold from that sum, so no result has to be broadcast.  A few very long
// rows (sequence shards) would otherwise leave most SMs idle during the selection.
// s_keys caches the first n_cached keys of the CTA's slice.
// Per-warp totals w[0..kSelWarps) -> (sum of the totals of the warps before `warp`, sum of all), by a shuffle scan
// over one lane per warp.  Called by whole warps.
__device__ __forceinline__ int2 warp_exclusive(const int* w, int warp, int lane)
{
    static_assert(kSelWarps <= 32 && (kSelWarps & (kSelWarps - 1)) == 0, "one lane per warp total");
    const int v = lane < kSelWarps ? w[lane] : 0;
    int incl = v;
#pragma unroll
    for (int off = 1; off < kSelWarps; off <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += o;
    }
    return make_int2(__shfl_sync(0xffffffffu, incl - v, warp), __shfl_sync(0xffffffffu, incl, kSelWarps - 1));
}

template <bool CL, typename KeyFn, typename EmitFn>
__device__ void select_row(int n, int kb, int key_bits, KeyFn key_of, EmitFn emit, uint32_t* s_keys, int n_cached,
                           SelScratch& sc)
{
    namespace cg = cooperative_groups;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (kb <= 0 || n <= 0) return;  // (the same for every CTA of a cluster)
    if (kb > n) kb = n;
    int crank = 0, csize = 1;
    if constexpr (CL) {
        crank = (int)cg::this_cluster().block_rank();
        csize = (int)cg::this_cluster().num_blocks();
    }
    auto cluster_sync = [&]() {
        if constexpr (CL) cg::this_cluster().sync();
    };
    auto remote = [&](int r) -> SelScratch* {
        if constexpr (CL) return cg::this_cluster().map_shared_rank(&sc, r);
        return &sc;
    };
    // slice of this CTA
    const int slice = CL ? ((n + csize - 1) / csize + 3) / 4 * 4 : n;
    const int j_lo = min(n, crank * slice), j_hi = min(n, j_lo + slice);
    const int len = j_hi - j_lo;
    n_cached = min(n_cached, len);

    // (the first pass's histogram; a later pass clears its own while the one before it runs)
    for (int i = tid; i < kBins; i += kSelThreads) sc.hist[0][i] = 0;
    const uint32_t key_top = key_bits >= 32 ? 0xFFFFFFFFu : (1u << key_bits) - 1u;  // "past the end" marker
    // Range of the ordinary keys (neither 0 = forced nor key_top).  Block scores cluster in a narrow band,
    // so radix digits are taken from (key - kmin): the histogram spreads over the band instead of piling
    // onto a few bins of the top digit, and one pass usually pins the k-th key.
    uint32_t r_lo = 0xFFFFFFFFu, r_hi = 0u;
    int zeros = 0, normals = 0;
    auto tally = [&](uint32_t key) {
        if (key == 0u) ++zeros;
        else if (key != key_top) { ++normals; r_lo = min(r_lo, key); r_hi = max(r_hi, key); }
    };
    // Keys into shared memory; the global loads of several entries are in flight together.  Rows of a few keys per
    // thread apply every rule while loading (key) and take the range from the registers on the way: one barrier
    // until the range is known.  Long rows use key_fast, which leaves out the forced-block rule; fixup() then applies
    // it to the few entries it concerns, and the range comes from a pass over the cached keys.
    const bool inline_rule = len <= kSelInlineKeys;
    // (U loads in flight per thread; short rows take the narrow form: predicated-off copies of the body still cost
    // issue slots, and a selection of a thousand keys is bound by those)
    // (inline_rule) what the thread needs to apply the rules to its keys tid, tid + kSelThreads, ... of the cached
    // slice without walking a list per key
    const auto ctx = key_of.thread_ctx(j_lo, inline_rule ? n_cached : 0, tid);
    auto load_keys = [&](auto u_tag) {
        constexpr int kU = decltype(u_tag)::value;
        for (int i0 = tid; i0 < n_cached; i0 += kSelThreads * kU) {
            decltype(key_of.raw(0)) raw[kU];
#pragma unroll
            for (int u = 0; u < kU; ++u) {
                const int i = i0 + u * kSelThreads;
                if (i < n_cached) raw[u] = key_of.raw(j_lo + i);
            }
#pragma unroll
            for (int u = 0; u < kU; ++u) {
                const int i = i0 + u * kSelThreads;
                if (i < n_cached) {
                    if (inline_rule) {
                        const uint32_t key = key_of.key_ctx(j_lo + i, raw[u], i / kSelThreads, ctx);
                        s_keys[i] = key;
                        tally(key);
                    } else {
                        s_keys[i] = key_of.key_fast(j_lo + i, raw[u]);
                    }
                }
            }
        }
    };
    if (n_cached <= 2 * kSelThreads) load_keys(std::integral_constant<int, 2>{});
    else if (n_cached <= 4 * kSelThreads) load_keys(std::integral_constant<int, 4>{});
    else load_keys(std::integral_constant<int, 8>{});
    auto get = [&](int j) -> uint32_t { return j - j_lo < n_cached ? s_keys[j - j_lo] : key_of.key(j, key_of.raw(j)); };
    if (inline_rule) {
        for (int j = j_lo + n_cached + tid; j < j_hi; j += kSelThreads) tally(get(j));  // (keys beyond the cache)
    } else {
        __syncthreads();
        key_of.fixup(s_keys, j_lo, n_cached);
        __syncthreads();
        for (int j = j_lo + tid; j < j_hi; j += kSelThreads) tally(get(j));
    }
    r_lo = __reduce_min_sync(0xffffffffu, r_lo);
    r_hi = __reduce_max_sync(0xffffffffu, r_hi);
    zeros = __reduce_add_sync(0xffffffffu, zeros);
    normals = __reduce_add_sync(0xffffffffu, normals);
    if (lane == 0) { sc.w_lo[warp] = r_lo; sc.w_hi[warp] = r_hi; sc.w_zero[warp] = zeros; sc.w_norm[warp] = normals; }
    __syncthreads();
    UCMR_STAMP(2);
    // every warp folds the per-warp partials itself (no atomics, no second barrier)
    static_assert(kSelWarps <= 32, "one lane per warp partial");
    r_lo = lane < kSelWarps ? sc.w_lo[lane] : 0xFFFFFFFFu;
    r_hi = lane < kSelWarps ? sc.w_hi[lane] : 0u;
    zeros = lane < kSelWarps ? sc.w_zero[lane] : 0;
    normals = lane < kSelWarps ? sc.w_norm[lane] : 0;
    r_lo = __reduce_min_sync(0xffffffffu, r_lo);
    r_hi = __reduce_max_sync(0xffffffffu, r_hi);
    zeros = __reduce_add_sync(0xffffffffu, zeros);
    normals = __reduce_add_sync(0xffffffffu, normals);
    int n_zero = zeros, n_normal = normals;
    uint32_t kmin = r_lo, kmax = r_hi;
    if constexpr (CL) {
        if (tid == 0) { sc.kmin = kmin; sc.kmax = kmax; sc.n_zero = n_zero; sc.n_normal = n_normal; }
        cluster_sync();
        if (warp == 0) {
            int z = 0, nn = 0;
            uint32_t glo = 0xFFFFFFFFu, ghi = 0u;
            if (lane < csize) {
                const SelScratch* o = remote(lane);
                z = o->n_zero; nn = o->n_normal; glo = o->kmin; ghi = o->kmax;
            }
#pragma unroll
            for (int off = 4; off > 0; off >>= 1) {  // clusters have at most 8 CTAs
                z += __shfl_xor_sync(0xffffffffu, z, off);
                nn += __shfl_xor_sync(0xffffffffu, nn, off);
                glo = min(glo, __shfl_xor_sync(0xffffffffu, glo, off));
                ghi = max(ghi, __shfl_xor_sync(0xffffffffu, ghi, off));
            }
            if (lane == 0) { sc.g_zero = z; sc.g_normal = nn; sc.g_kmin = glo; sc.g_kmax = ghi; }
        }
        __syncthreads();
        n_zero = sc.g_zero; n_normal = sc.g_normal; kmin = sc.g_kmin; kmax = sc.g_kmax;
    }
    uint32_t T;
    int need;
    if (kb <= n_zero) {
        T = 0u; need = kb;
    } else if (kb > n_zero + n_normal) {
        T = key_top; need = kb - n_zero - n_normal;
    } else {
        const uint32_t range = kmax - kmin;
        int hi = 32 - __clz(range | 1u);  // bits of (key - kmin) still undecided
        // every thread carries the decided prefix and the rank still to find; after a pass the one thread that
        // found the bin publishes both through shared memory
        uint32_t prefix = 0u;
        int rem = kb - n_zero;
        for (int pass = 0; hi > 0; ++pass) {
            const int width = min(kDigitBits, hi);
            const int shift = hi - width;
            const uint32_t dmask = (1u << width) - 1u;
            int* hist = sc.hist[pass];
            if (shift > 0)  // another pass will follow: its histogram is cleared now (used two barriers from here)
                for (int i = tid; i < kBins; i += kSelThreads) sc.hist[pass + 1][i] = 0;
            const int len_round = (len + kSelThreads - 1) / kSelThreads * kSelThreads;
            for (int i = tid; i < len_round; i += kSelThreads) {
                const uint32_t key = i < len ? get(j_lo + i) : 0u;
                const uint32_t rel = key - kmin;
                const bool hit = key != 0u && key != key_top && (hi >= 32 || (rel >> hi) == (prefix >> hi));
                const uint32_t digit = (rel >> shift) & dmask;
                int same;
                __match_all_sync(0xffffffffu, hit ? digit : 0xFFFFFFFFu, &same);
                if (same) {
                    if (hit && lane == 0) atomicAdd(&hist[digit], 32);
                } else if (hit) {
                    atomicAdd(&hist[digit], 1);
                }
            }
            __syncthreads();
            // exclusive scan over the (cluster-wide) bins, kBinsPerThread consecutive bins per thread
            int loc[kBinsPerThread];
            int sum = 0;
            if constexpr (CL) {
                int* const h0 = remote(0)->hist[pass];
                if (crank != 0) {
#pragma unroll
                    for (int i = 0; i < kBinsPerThread; ++i) {
                        const int v = hist[tid * kBinsPerThread + i];
                        if (v != 0) atomicAdd(&h0[tid * kBinsPerThread + i], v);
                    }
                }
                cluster_sync();
#pragma unroll
                for (int i = 0; i < kBinsPerThread; ++i) loc[i] = h0[tid * kBinsPerThread + i];
            } else {
#pragma unroll
                for (int i = 0; i < kBinsPerThread; ++i) loc[i] = hist[tid * kBinsPerThread + i];
            }
#pragma unroll
            for (int i = 0; i < kBinsPerThread; ++i) sum += loc[i];
            int incl = sum;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int o = __shfl_up_sync(0xffffffffu, incl, off);
                if (lane >= off) incl += o;
            }
            if (lane == 31) sc.warp_a[warp] = incl;
            __syncthreads();
            int excl = incl - sum + warp_exclusive(sc.warp_a, warp, lane).x;
            if (rem > excl && rem <= excl + sum) {  // exactly one thread
                int run = excl;
#pragma unroll
                for (int i = 0; i < kBinsPerThread; ++i) {
                    if (rem > run && rem <= run + loc[i]) {
                        sc.prefix = prefix | ((uint32_t)(tid * kBinsPerThread + i) << shift);
                        sc.remaining = rem - run;
                    }
                    run += loc[i];
                }
            }
            hi = shift;
            __syncthreads();
            prefix = sc.prefix;
            rem = sc.remaining;
        }
        T = kmin + prefix;
        need = rem;  // how many keys equal to T are taken, lowest positions first
    }

    UCMR_STAMP(3);
    const int ipt = (len + kSelThreads - 1) / kSelThreads;
    const int j_begin = min(j_hi, j_lo + tid * ipt), j_end = min(j_hi, j_begin + ipt);
    int lt = 0, eq = 0;
    for (int j = j_begin; j < j_end; ++j) {
        const uint32_t key = get(j);
        lt += key < T;
        eq += key == T;
    }
    int lt_incl = lt, eq_incl = eq;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int a = __shfl_up_sync(0xffffffffu, lt_incl, off);
        const int b = __shfl_up_sync(0xffffffffu, eq_incl, off);
        if (lane >= off) { lt_incl += a; eq_incl += b; }
    }
    if (lane == 31) { sc.warp_a[warp] = lt_incl; sc.warp_b[warp] = eq_incl; }
    __syncthreads();
    const int2 wl = warp_exclusive(sc.warp_a, warp, lane), we = warp_exclusive(sc.warp_b, warp, lane);
    int lt_before = lt_incl - lt + wl.x, eq_before = eq_incl - eq + we.x;
    const int cta_lt = wl.y, cta_eq = we.y;
    // entries of the row that precede this CTA's slice
    int base_lt = 0, base_eq = 0;
    if constexpr (CL) {
        if (tid == 0) { sc.cta_lt = cta_lt; sc.cta_eq = cta_eq; }
        __syncthreads();
        cluster_sync();  // also: every CTA is done reading CTA 0's histograms
        if (warp == 0) {
            int a = 0, b = 0;
            if (lane < crank) {
                const SelScratch* o = remote(lane);
                a = o->cta_lt; b = o->cta_eq;
            }
#pragma unroll
            for (int off = 4; off > 0; off >>= 1) {
                a += __shfl_xor_sync(0xffffffffu, a, off);
                b += __shfl_xor_sync(0xffffffffu, b, off);
            }
            if (lane == 0) { sc.base_lt = a; sc.base_eq = b; }
        }
        __syncthreads();
        base_lt = sc.base_lt; base_eq = sc.base_eq;
        cg::this_cluster().barrier_arrive();  // last remote access of this CTA is done; waited for at the end
    }
    lt_before += base_lt; eq_before += base_eq;
    // The chosen entries are first listed in shared memory (the histograms are free by now) and then emitted
    // one per thread, so that the global loads and stores of an emit are not chained inside one thread's walk.
    int* const sel = &sc.hist[0][0];
    const int pos_base = base_lt + min(base_eq, need);                           // first position this CTA emits
    const int n_mine = cta_lt + max(0, min(cta_eq, need - base_eq));             // how many it emits
    const bool listed = n_mine <= 3 * kBins;
    for (int j = j_begin; j < j_end; ++j) {
        const uint32_t key = get(j);
        int pos = -1;
        if (key < T) {
            pos = lt_before + min(eq_before, need);
            ++lt_before;
        } else if (key == T) {
            if (eq_before < need) pos = lt_before + eq_before;
            ++eq_before;
        }
        if (pos >= 0) {
            if (listed) sel[pos - pos_base] = j;
            else emit(pos, j);
        }
    }
    __syncthreads();
    UCMR_STAMP(4);
    if (listed)
        for (int i = tid; i < n_mine; i += kSelThreads) emit(pos_base + i, sel[i]);
    __syncthreads();
    if constexpr (CL) cg::this_cluster().barrier_wait();  // no CTA leaves while another may still read its scratch
}

struct SelectParams {
    const int32_t* scores;  // [B, Hout, max_blocks]
    int Hout, max_blocks, BS;
    const int32_t* bt;
    int64_t bt_stride;
    const int32_t* seq_local;
    const int32_t* seq_global;  // null = same as local
    int k;
    const int32_t* k_per_request;
    const uint8_t* mask;
    ForcedSpec forced;
    int id_offset;
    int n_cached;
    int key_bits;  // valid keys (score + 1) are below 2^key_bits - 1, which marks blocks past the end
    // block-id outputs
    int32_t *out_phys, *out_logical, *out_scores, *out_valid, *out_newseq;
    // candidate-record outputs
    float* cand_scores;
    int32_t* cand_ids;
    float scale;
    int32_t* sched;  // the scan's work counter, cleared here for the next launch
    int cluster;     // CTAs per row (thread-block cluster size), 1 = one CTA per row
    // Candidate records written straight into every rank's gather buffer over peer memory (n_peers > 0): entry r
    // points at this rank's slice of rank r's buffer; when the last CTA is done, the step number is stored to
    // this rank's flag word on every rank.
    // With step_word != null the step number is read on the device (*step_word + 1) instead of taken from `seq`,
    // and its parity picks one of two pointer sets: a launch captured in a CUDA graph then stays correct when
    // replayed, which a by-value step number does not.
    int n_peers;
    float* peer_scores[2][kMaxPeers];
    int32_t* peer_ids[2][kMaxPeers];
    int32_t* peer_flags[2][kMaxPeers];
    int seq;
    const int32_t* step_word;
    int32_t* arrive;  // CTA arrival counter (workspace header), zero between launches
};

// CL: p.cluster consecutive CTAs (one thread-block cluster) share a row.
template <bool CANDIDATES, bool CL>
__global__ void __launch_bounds__(kSelThreads) select_kernel(const SelectParams p)
{
    extern __shared__ uint32_t s_keys[];
    __shared__ SelScratch sc;
    // The forced-block rule walks its list with a run-time index.  On the kernel parameter that means loads through
    // a generic address into parameter space - measured at about a microsecond per selection - so the rule reads a
    // shared-memory copy (made with compile-time offsets, published by the barrier before the selection).
    __shared__ ForcedSpec s_forced;
    const int tid = threadIdx.x;
    if (tid == 0) s_forced = p.forced;
    UCMR_STAMP(0);
    const int row = CL ? blockIdx.x / p.cluster : blockIdx.x;
    const bool lead = !CL || blockIdx.x % p.cluster == 0;  // the CTA that writes the row's padding and scalars
    const int b = row / p.Hout;
    const int n = p.max_blocks;
    const int seq_l = p.seq_local[b];
    const int nb_l = min(n, (seq_l + p.BS - 1) / p.BS);
    const int seq_g = p.seq_global ? p.seq_global[b] : seq_l;
    const int nb_g = (seq_g + p.BS - 1) / p.BS;
    const int32_t* srow = p.scores + (int64_t)row * n;
    const int32_t* btrow = p.bt + (int64_t)b * p.bt_stride;
    int kb = p.k;
    if (p.k_per_request) kb = max(0, min(p.k_per_request[b], p.k));
    const bool masked = p.mask != nullptr && p.mask[b] == 0;
    const int64_t obase = (int64_t)row * p.k;
    // peer exchange: step number of this launch and the pointer set of its parity
    int step_no = p.seq, par = 0;
    if (CANDIDATES && p.n_peers > 0 && p.step_word != nullptr) {
        step_no = *p.step_word + 1;
        par = step_no & 1;
    }
    // the pointer set of this parity, in shared memory for the same reason as the forced-block list
    __shared__ float* s_peer_scores[kMaxPeers];
    __shared__ int32_t* s_peer_ids[kMaxPeers];
    __shared__ int32_t* s_peer_flags[kMaxPeers];
    if (CANDIDATES && p.n_peers > 0) {
        if (tid == 0) {
#pragma unroll
            for (int r = 0; r < kMaxPeers; ++r) {
                s_peer_scores[r] = par ? p.peer_scores[1][r] : p.peer_scores[0][r];
                s_peer_ids[r] = par ? p.peer_ids[1][r] : p.peer_ids[0][r];
                s_peer_flags[r] = par ? p.peer_flags[1][r] : p.peer_flags[0][r];
            }
        }
        __syncthreads();
    }
    float* const* const peer_scores = s_peer_scores;
    int32_t* const* const peer_ids = s_peer_ids;

    if (masked) grid_dependency_wait();  // pass-through rows copy scores below
    // Padding of the positions the selection will not write: it emits exactly min(kb, max_blocks) entries, each of
    // which stores its position (a record that turns out invalid stores the padding values itself), so only the
    // tail [min(kb, max_blocks), k) is padded here - usually nothing, and over peer memory every store saved before
    // the wait is a remote one.  Rows that are passed through unselected are written here in full.
    const int pad_from = masked ? 0 : max(0, min(kb, n));
    for (int i = pad_from + tid; lead && i < p.k; i += kSelThreads) {
        if (CANDIDATES) {
            if (p.n_peers > 0) {
                for (int r = 0; r < p.n_peers; ++r) {
                    peer_scores[r][obase + i] = INFINITY;
                    peer_ids[r][obase + i] = -1;
                }
            } else {
                p.cand_scores[obase + i] = INFINITY;
                p.cand_ids[obase + i] = -1;
            }
        } else {
            const bool pass = masked && i < kb;
            p.out_phys[obase + i] = pass ? btrow[i] : 0;
            if (p.out_logical) p.out_logical[obase + i] = pass ? i : -1;
            if (p.out_scores) p.out_scores[obase + i] = pass ? (i < nb_l ? srow[i] : -1) : -1;
        }
    }
    // per-request scalars: written at the end, so that nothing before the selection waits for the sequence length
    auto write_scalars = [&]() {
        if (!CANDIDATES && lead && tid == 0 && row % p.Hout == 0) {
            if (p.out_valid) p.out_valid[b] = min(kb, nb_l);
            if (p.out_newseq) {
                int ns = seq_l;
                if (!masked) {
                    const int over = max(seq_l - kb * p.BS, 0);
                    ns = seq_l - (over + p.BS - 1) / p.BS * p.BS;
                }
                p.out_newseq[b] = ns;
            }
        }
    };
    // Up to here only the sequence lengths and the block table were read and only outputs written: the scan
    // that produces the scores may still be running (programmatic dependent launch).
    grid_dependency_wait();
    UCMR_STAMP(1);
    UCMR_STAMP_LAST(13);
    if (blockIdx.x == 0 && tid == 0 && p.sched != nullptr) *p.sched = 0;
    if (masked) {
        write_scalars();
        return;
    }
    __syncthreads();  // padding stores precede the emits of the same CTA

    const uint32_t key_invalid = p.key_bits >= 32 ? kKeyInvalid : (1u << p.key_bits) - 1u;
    // (the functors below hold copies of what they need, never a reference to the kernel parameter: reached through
    // a reference that the compiler does not fold away, every field is a load through a generic address)
    struct KeyOf {
        const ForcedSpec& forced;
        const int32_t* srow;
        int nb_l, nb_g, seq_g, id_offset, BS;
        uint32_t key_invalid;
        // (unconditional: j is below max_blocks, and the load then does not wait for the sequence length)
        __device__ int raw(int j) const { return srow[j]; }
        __device__ uint32_t key_fast(int j, int s) const { return (j >= nb_l || s < 0) ? key_invalid : (uint32_t)s + 1u; }
        __device__ uint32_t key(int j, int s) const
        {
            if (j >= nb_l || s < 0) return key_invalid;
            if (block_is_forced(forced, j + id_offset, nb_g, seq_g, BS)) return 0u;
            return (uint32_t)s + 1u;
        }
        // Rows of a few keys per thread: bit t of the context says that the thread's t-th cached key (index tid +
        // t * kSelThreads of the slice) is a listed must-select block, so the list is walked once per thread
        // instead of once per key; sink and recent window are two comparisons.
        __device__ uint32_t thread_ctx(int j_lo, int n_cached, int tid) const
        {
            static_assert(kSelInlineKeys <= 32 * kSelThreads, "one context bit per key of the thread");
            uint32_t mask = 0u;
            if (n_cached == 0) return mask;
            for (int m = 0; m < forced.n_must; ++m) {
                const int jg = forced.must[m] >= 0 ? forced.must[m] : nb_g + forced.must[m];
                const int c = jg - id_offset - j_lo;
                if (jg >= 0 && jg < nb_g && c >= 0 && c < n_cached && c % kSelThreads == tid) mask |= 1u << (c / kSelThreads);
            }
            return mask;
        }
        __device__ uint32_t key_ctx(int j, int s, int t, uint32_t ctx) const
        {
            if (j >= nb_l || s < 0) return key_invalid;
            const int jg = j + id_offset;
            if (jg >= nb_g) return (uint32_t)s + 1u;
            const int lo = jg * BS, hi = min(lo + BS, seq_g);
            const bool f = ((ctx >> t) & 1u) || (forced.sink > 0 && lo < forced.sink) ||
                           (forced.recent > 0 && hi > seq_g - forced.recent);
            return f ? 0u : (uint32_t)s + 1u;
        }
        // Forced blocks are few: the listed ones, the first blocks (sink) and the last ones (recent window).
        __device__ void fixup(uint32_t* s_keys, int j_lo, int n_cached) const
        {
            const ForcedSpec& f = forced;
            const int n_sink = f.sink > 0 ? min(nb_g, (f.sink + BS - 1) / BS) : 0;
            const int first_recent = f.recent > 0 ? max(0, (seq_g - f.recent) / BS) : nb_g;
            const int n_recent = max(0, nb_g - first_recent);
            const int total = f.n_must + n_sink + n_recent;
            for (int i = threadIdx.x; i < total; i += blockDim.x) {
                int jg;  // global block index
                if (i < f.n_must) jg = f.must[i] >= 0 ? f.must[i] : nb_g + f.must[i];
                else if (i < f.n_must + n_sink) jg = i - f.n_must;
                else jg = first_recent + (i - f.n_must - n_sink);
                const int j = jg - id_offset;
                const int c = j - j_lo;  // index in this CTA's cached slice
                if (jg >= 0 && jg < nb_g && j >= 0 && j < nb_l && c >= 0 && c < n_cached && s_keys[c] != key_invalid &&
                    block_is_forced(f, jg, nb_g, seq_g, BS))
                    s_keys[c] = 0u;
            }
        }
    };
    const int id_offset = p.id_offset, BS = p.BS, n_peers = p.n_peers;
    const float scale = p.scale;
    float* const cand_scores = p.cand_scores;
    int32_t* const cand_ids = p.cand_ids;
    int32_t* const out_phys = p.out_phys;
    int32_t* const out_logical = p.out_logical;
    int32_t* const out_scores = p.out_scores;
    const ForcedSpec& forced = s_forced;
    const KeyOf key_of{forced, srow, nb_l, nb_g, seq_g, id_offset, BS, key_invalid};
    auto emit = [=, &forced](int pos, int j) {
        const bool valid = j < nb_l && srow[j] >= 0;
        if (CANDIDATES) {
            if (valid) {
                const bool is_forced = block_is_forced(forced, j + id_offset, nb_g, seq_g, BS);
                const float sc_v = is_forced ? -1.0f : (float)srow[j] * scale;
                if (n_peers > 0) {
                    for (int r = 0; r < n_peers; ++r) {
                        peer_scores[r][obase + pos] = sc_v;
                        peer_ids[r][obase + pos] = j + id_offset;
                    }
                } else {
                    cand_scores[obase + pos] = sc_v;
                    cand_ids[obase + pos] = j + id_offset;
                }
            } else if (n_peers > 0) {  // no block behind this position: the padding record
                for (int r = 0; r < n_peers; ++r) {
                    peer_scores[r][obase + pos] = INFINITY;
                    peer_ids[r][obase + pos] = -1;
                }
            } else {
                cand_scores[obase + pos] = INFINITY;
                cand_ids[obase + pos] = -1;
            }
        } else {
            out_phys[obase + pos] = btrow[j];
            if (out_logical) out_logical[obase + pos] = j;
            if (out_scores) out_scores[obase + pos] = valid ? srow[j] : -1;
        }
    };
    select_row<CL>(n, kb, p.key_bits, key_of, emit, s_keys, p.n_cached, sc);
    UCMR_STAMP(5);
    UCMR_STAMP_LAST(11);
    write_scalars();
    if (CANDIDATES && p.n_peers > 0) {
        // Records are in the peers' memory: they must be visible system-wide before the step number is.  The CTA
        // barrier orders every thread's stores before thread 0's fence (fences are cumulative), so one system fence
        // per CTA serves; the arrival is counted with acquire-release semantics, and the last CTA's release stores of
        // the step number follow one more fence that orders them behind all it has observed through that counter.
        __syncthreads();
        if (tid == 0) {
            __threadfence_system();
            UCMR_STAMP(6);
            UCMR_STAMP_LAST(12);
            const int done = atom_add_release_gpu(p.arrive, 1);
            if (done == (int)gridDim.x - 1) {
                *p.arrive = 0;
                // One fence, then relaxed stores: a release store per rank would put a system fence - a round trip
                // to the rank written just before - in front of each of them (measured: 15 us for 8 ranks).
                __threadfence_system();
                for (int r = 0; r < p.n_peers; ++r) st_relaxed_sys(s_peer_flags[r], step_no);
                UCMR_STAMP_ANY(7);
            }
        }
    }
}

__device__ __forceinline__ uint32_t f32_order_key(float x)
{
    const uint32_t u = __float_as_uint(x);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct MergeParams {
    const float* cand_scores;  // [R, B, H, kl]
    const int32_t* cand_ids;
    int64_t rank_stride;
    int R, B, H, kl, k, n_cached;
    float* out_scores;  // [B, H, k]
    int32_t* out_ids;
    int largest;        // 0: the k smallest scores win (distances); 1: the k largest (inner products)
    // records arrive from other GPUs: wait (bounded) until flag r holds wait_seq for every rank r < R
    const int32_t* wait_flags;
    int wait_seq;
    int32_t* status;
    // Replay-safe form: the step number is *step_word + 1, its parity selects the records (cand_* + parity *
    // parity_stride) and the flags (wait_flags + parity * flags_parity_stride); the launch's last CTA stores the
    // step number back to *step_word (arrive_word counts the CTAs and is zero between launches).
    int32_t* step_word;
    int32_t* arrive_word;
    int64_t parity_stride;
    int64_t flags_parity_stride;
};

__global__ void __launch_bounds__(kSelThreads) merge_kernel(const MergeParams p)
{
    extern __shared__ uint32_t s_keys[];
    __shared__ SelScratch sc;
    const int tid = threadIdx.x;
    UCMR_STAMP(8);
    const int row = blockIdx.x;  // b*H + h
    const int n = p.R * p.kl;
    const int64_t obase = (int64_t)row * p.k;
    for (int i = tid; i < p.k; i += kSelThreads) {
        p.out_scores[obase + i] = p.largest ? -INFINITY : INFINITY;
        p.out_ids[obase + i] = -1;
    }
    int wait_seq = p.wait_seq;
    const float* cand_scores = p.cand_scores;
    const int32_t* cand_ids = p.cand_ids;
    const int32_t* wait_flags = p.wait_flags;
    if (p.step_word != nullptr) {
        wait_seq = *p.step_word + 1;
        const int par = wait_seq & 1;
        cand_scores += par * p.parity_stride;
        cand_ids += par * p.parity_stride;
        wait_flags += par * p.flags_parity_stride;
    }
    // Every CTA has read the step word by the time it arrives here; the last one to arrive advances it.
    auto advance_step = [&]() {
        if (p.step_word == nullptr) return;
        __syncthreads();
        if (tid == 0) {
            __threadfence();
            if (atomicAdd(p.arrive_word, 1) == (int)gridDim.x - 1) {
                *p.arrive_word = 0;
                *p.step_word = wait_seq;
            }
        }
    };
    if (wait_flags != nullptr) {
        __shared__ int s_timed_out;
        if (tid == 0) s_timed_out = 0;
        __syncthreads();
        if (tid < p.R) {
            unsigned long long t0 = 0;
            uint32_t polls = 0;
            while (ld_acquire_sys(wait_flags + tid) != wait_seq) {
                if ((++polls & (kWaitPollsPerClockCheck - 1)) == 0) {
                    unsigned long long now;
                    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                    if (t0 == 0) t0 = now;
                    else if (now - t0 > kWaitLimitNs) { s_timed_out = 1; break; }
                }
            }
        }
        __syncthreads();
        UCMR_STAMP(9);
        if (s_timed_out) {  // a rank never delivered: leave the padding as the result and report
            if (tid == 0) flag_status(p.status, UCMR_DEV_WAIT_TIMEOUT);
            advance_step();
            return;
        }
    }
    __syncthreads();
    struct Rec { int32_t id; float score; };
    struct KeyOf {
        int kl, largest;
        int64_t rank_stride;
        int row;
        const float* cand_scores;
        const int32_t* cand_ids;
        __device__ int64_t at(int i) const
        {
            const int r = i / kl, c = i - r * kl;
            return (int64_t)r * rank_stride + (int64_t)row * kl + c;
        }
        __device__ Rec raw(int i) const
        {
            const int64_t a = at(i);
            return Rec{__ldcg(cand_ids + a), __ldcg(cand_scores + a)};
        }
        __device__ uint32_t key(int, Rec r) const
        {
            if (r.id < 0) return kKeyInvalid;
            const uint32_t k = f32_order_key(largest ? -r.score : r.score);
            return k == kKeyInvalid ? kKeyInvalid - 1u : k;
        }
        __device__ uint32_t key_fast(int i, Rec r) const { return key(i, r); }
        __device__ int thread_ctx(int, int, int) const { return 0; }
        __device__ uint32_t key_ctx(int i, Rec r, int, int) const { return key(i, r); }
        __device__ void fixup(uint32_t*, int, int) const {}
    };
    const KeyOf key_of{p.kl, p.largest, p.rank_stride, row, cand_scores, cand_ids};
    float* const out_scores = p.out_scores;
    int32_t* const out_ids = p.out_ids;
    auto emit = [=](int pos, int i) {
        const int64_t a = key_of.at(i);
        const int32_t id = __ldcg(cand_ids + a);
        if (id >= 0) {
            out_scores[obase + pos] = __ldcg(cand_scores + a);
            out_ids[obase + pos] = id;
        }
    };
    select_row<false>(n, min(p.k, n), 32, key_of, emit, s_keys, p.n_cached, sc);
    UCMR_STAMP(10);
    advance_step();
}

__global__ void update_seq_lens_kernel(const int32_t* seq, int B, int topk_tokens, int BS, int32_t* out)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= B) return;
    const int s = seq[i];
    const int over = max(s - topk_tokens, 0);
    out[i] = s - (over + BS - 1) / BS * BS;
}

static int fill_forced(ForcedSpec& f, const int32_t* must, int n_must, int sink, int recent)
{
    if (n_must < 0 || n_must > UCMR_MAX_MUST_SELECT || (n_must > 0 && !must)) return UCMR_ERR_BAD_ARG;
    if (sink < 0 || recent < 0) return UCMR_ERR_BAD_ARG;
    for (int i = 0; i < n_must; ++i) f.must[i] = must[i];
    f.n_must = n_must; f.sink = sink; f.recent = recent;
    return UCMR_OK;
}

template <typename K>
static int set_dyn_smem(K kernel, size_t bytes)
{
    // static + dynamic shared memory above 48 KiB needs the opt-in; the kernels hold ~25 KiB statically
    if (bytes > 16 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) { note_cuda_error(e); return UCMR_ERR_LAUNCH; }
    }
    return UCMR_OK;
}

static size_t scores_bytes(int B, int Hout, int max_blocks)
{
    size_t b = (size_t)B * Hout * max_blocks * sizeof(int32_t);
    return (b + 255) / 256 * 256;
}

}  // namespace ucmr

using namespace ucmr;

extern "C" size_t ucmr_hamming_topk_workspace_bytes(int B, int Hkv, int max_blocks, int reduce_kvhead)
{
    if (B < 0 || Hkv <= 0 || max_blocks <= 0) return 0;
    // header, block scores, and for one kv head (where the codes may be token rows) the query planes of the row scan
    return UCMR_WORKSPACE_HEADER_BYTES + scores_bytes(B, reduce_kvhead ? 1 : Hkv, max_blocks) +
           (Hkv == 1 ? rows_scratch_bytes(B) : 0);
}

extern "C" int ucmr_workspace_init(void* workspace, size_t bytes, void* stream)
{
    if (!workspace || bytes < UCMR_WORKSPACE_HEADER_BYTES) return UCMR_ERR_WORKSPACE;
    cudaError_t e = cudaMemsetAsync(workspace, 0, UCMR_WORKSPACE_HEADER_BYTES, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) { note_cuda_error(e); return UCMR_ERR_LAUNCH; }
    return UCMR_OK;
}

extern "C" int ucmr_workspace_status(const void* workspace, int* host_status, void* stream)
{
    if (!workspace || !host_status) return UCMR_ERR_BAD_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(host_status, workspace, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) { note_cuda_error(e); return UCMR_ERR_LAUNCH; }
    return *host_status == 0 ? UCMR_OK : UCMR_ERR_DEVICE;
}

// Value of the UCMR_SEL_CLUSTER environment switch, looked up on the first call only (-1 = not set).
static int sel_cluster_override()
{
    static const int v = [] {
        const char* env = getenv("UCMR_SEL_CLUSTER");
        return env ? atoi(env) : -1;
    }();
    return v;
}

// UCMR_FUSED_SELECT=1 (read once per process) lets the staged scan run the selection itself for rows of at most
// kFuseMaxBlocks blocks (one launch instead of two).  Off by default: measured on B200 the in-kernel hand-over (grid-wide
// arrival, then one warp per row) takes as long as the second launch it saves - 55.6 vs 54.7 us for 16 x 1024-block rows
// x 8 heads, 25.5 vs 23.3 us for 8 x 2048-block rows - so it only pays where launches are expensive (no CUDA graph).
static bool fused_select_enabled()
{
    static const bool v = [] {
        const char* env = getenv("UCMR_FUSED_SELECT");
        return env != nullptr && env[0] == '1';
    }();
    return v;
}

struct PeerDest {
    int n_peers, seq;
    float* scores[2][kMaxPeers];   // [parity][rank]; the by-value form fills parity 0 only
    int32_t* ids[2][kMaxPeers];
    int32_t* flags[2][kMaxPeers];
    const int32_t* step_word;      // null = step number given by value (seq)
};

static int run_select(bool candidates, const uint32_t* codes, int64_t NB, int BS, int Hkv, int W,
                      const uint32_t* q_codes, int Hq, const int32_t* bt, int max_blocks, int64_t bt_stride,
                      const int32_t* seq_local, const int32_t* seq_global, int B, int k,
                      const int32_t* k_per_request, const uint8_t* mask, int reduce_mode, int reduce_kvhead,
                      const int32_t* must, int n_must, int sink, int recent, int id_offset, float scale,
                      int32_t* out_phys, int32_t* out_logical, int32_t* out_scores, int32_t* out_valid,
                      int32_t* out_newseq, float* cand_scores, int32_t* cand_ids, void* workspace,
                      size_t workspace_bytes, cudaStream_t st, const PeerDest* peers = nullptr)
{
    if (k < 0 || k > max_blocks) return UCMR_ERR_BAD_ARG;
    if (candidates ? (!peers && (!cand_scores || !cand_ids)) : !out_phys) return UCMR_ERR_BAD_ARG;
    if (k == 0 && peers) return UCMR_ERR_BAD_ARG;
    if (!workspace) return UCMR_ERR_WORKSPACE;
    if (workspace_bytes < ucmr_hamming_topk_workspace_bytes(B, Hkv, max_blocks, reduce_kvhead)) return UCMR_ERR_WORKSPACE;
    SelectParams p{};
    int rc = fill_forced(p.forced, must, n_must, sink, recent);
    if (rc != UCMR_OK) return rc;
    int32_t* status = static_cast<int32_t*>(workspace);
    int32_t* scores = reinterpret_cast<int32_t*>(static_cast<char*>(workspace) + UCMR_WORKSPACE_HEADER_BYTES);
    int32_t* sched = status + 2;  // work counter of the scan; zero between launches
    const int scan_mode = reduce_mode;  // with its UCMR_FLAG_* bits
    reduce_mode &= 0xFF;
    {
        const int G = Hkv > 0 ? Hq / Hkv : 1;
        int64_t max_score = (int64_t)G * W * 32;
        if (reduce_mode == UCMR_REDUCE_SUM) max_score *= (int64_t)BS * (reduce_kvhead ? Hkv : 1);
        p.key_bits = 1;
        while (p.key_bits < 32 && ((int64_t)1 << p.key_bits) - 1 <= max_score + 1) ++p.key_bits;
    }
    // Rows short enough for one warp each are selected inside the scan (no second launch): see FusedSel.
    FusedSel fs{};
    bool try_fuse = false;
    if (!candidates && k > 0 && max_blocks <= kFuseMaxBlocks && B <= kWsMaxBatch && fused_select_enabled()) {
        int idx_bits = 1;
        while ((1 << idx_bits) < max_blocks) ++idx_bits;
        if (p.key_bits + idx_bits <= 31) {
            try_fuse = true;
            fs.Hout = reduce_kvhead ? 1 : Hkv; fs.k = k; fs.key_bits = p.key_bits; fs.idx_bits = idx_bits;
            fs.k_per_request = k_per_request; fs.mask = mask; fs.forced = p.forced;
            fs.out_phys = out_phys; fs.out_logical = out_logical; fs.out_scores = out_scores;
            fs.out_valid = out_valid; fs.out_newseq = out_newseq;
            fs.cta_done = status + 4;
            fs.all_scored = status + 36;
        }
    }
    bool fused = false;
    void* row_scratch = Hkv == 1 ? static_cast<char*>(workspace) + UCMR_WORKSPACE_HEADER_BYTES +
                                       scores_bytes(B, 1, max_blocks)
                                 : nullptr;
    rc = run_scan(codes, NB, BS, Hkv, W, q_codes, Hq, bt, max_blocks, bt_stride, seq_local, B, scan_mode,
                  reduce_kvhead, scores, status, sched, st, try_fuse ? &fs : nullptr, &fused, row_scratch);
    if (rc != UCMR_OK || B == 0 || fused) return rc;
    // From here on the scan is enqueued and will leave its work counter non-zero; the selection kernel clears it.
    // If that kernel cannot be launched, clear it here, or the next call on this workspace would skip work items.
    auto fail_after_scan = [&](int code) {
        (void)cudaMemsetAsync(sched, 0, sizeof(int32_t), st);
        return code;
    };
    if (k == 0) {  // no selection kernel will run: clear the counter here
        cudaError_t e = cudaMemsetAsync(sched, 0, sizeof(int32_t), st);
        if (e != cudaSuccess) { note_cuda_error(e); return UCMR_ERR_LAUNCH; }
        return UCMR_OK;
    }

    p.scores = scores;
    p.Hout = reduce_kvhead ? 1 : Hkv; p.max_blocks = max_blocks; p.BS = BS;
    p.bt = bt; p.bt_stride = bt_stride;
    p.seq_local = seq_local; p.seq_global = seq_global;
    p.k = k; p.k_per_request = k_per_request; p.mask = mask;
    p.id_offset = id_offset;
    p.n_cached = max_blocks < kSelMaxCachedKeys ? max_blocks : kSelMaxCachedKeys;
    p.out_phys = out_phys; p.out_logical = out_logical; p.out_scores = out_scores;
    p.out_valid = out_valid; p.out_newseq = out_newseq;
    p.cand_scores = cand_scores; p.cand_ids = cand_ids; p.scale = scale; p.sched = sched;
    if (peers) {
        p.n_peers = peers->n_peers; p.seq = peers->seq; p.step_word = peers->step_word; p.arrive = status + 3;
        for (int par = 0; par < 2; ++par)
            for (int r = 0; r < peers->n_peers; ++r) {
                p.peer_scores[par][r] = peers->scores[par][r]; p.peer_ids[par][r] = peers->ids[par][r];
                p.peer_flags[par][r] = peers->flags[par][r];
            }
    }
    const int rows = B * p.Hout;
    // Few long rows: split each over a thread-block cluster so that the selection uses more than `rows` SMs.
    p.cluster = 1;
    while (p.cluster < 8 && rows * p.cluster * 2 <= 160 && max_blocks > p.cluster * kSelClusterSlice) p.cluster *= 2;
    // (8 CTAs per row only while each still gets more than 4096 keys: 16 rows x 8 CTAs do not always fit the GPCs in
    // one wave; rows of 32768 blocks measured 5 us faster with 4, rows of 65536 blocks 11 us faster with 8)
    if (p.cluster == 8 && max_blocks <= 8 * 2 * kSelClusterSlice) p.cluster = 4;
    bool use_cluster = p.cluster > 1;
    {   // tuning aid UCMR_SEL_CLUSTER (read once per process): 0 = never split, 1/2/4/8 = force that size
        const int v = sel_cluster_override();
        if (v == 0) { p.cluster = 1; use_cluster = false; }
        else if (v == 1 || v == 2 || v == 4 || v == 8) { p.cluster = v; use_cluster = true; }
    }
    if (use_cluster) {
        const int slice = ((max_blocks + p.cluster - 1) / p.cluster + 3) / 4 * 4;
        p.n_cached = slice < kSelMaxCachedKeys ? slice : kSelMaxCachedKeys;
    }
    const size_t smem = (size_t)p.n_cached * sizeof(uint32_t);
    void (*kernel)(const SelectParams) =
        candidates ? (use_cluster ? select_kernel<true, true> : select_kernel<true, false>)
                   : (use_cluster ? select_kernel<false, true> : select_kernel<false, false>);
    rc = set_dyn_smem(kernel, smem);
    if (rc != UCMR_OK) return fail_after_scan(rc);
    // (not launched early: selection CTAs that sit on SMs waiting for the scan to end cost more than the launch
    // latency they would hide - measured 1 to 8 us slower)
    rc = launch_kernel_ex(kernel, dim3(rows * (use_cluster ? p.cluster : 1)), dim3(kSelThreads), smem, st,
                          use_cluster ? p.cluster : 1, false, p);
    return rc == UCMR_OK ? rc : fail_after_scan(rc);
}

extern "C" int ucmr_hamming_topk(const uint32_t* codes, int64_t NB, int BS, int Hkv, int W,
                                 const uint32_t* q_codes, int Hq, const int32_t* block_table, int max_blocks,
                                 int64_t block_table_stride, const int32_t* seq_lens, int B, int k,
                                 const int32_t* k_per_request, const uint8_t* request_mask, int reduce_mode,
                                 int reduce_kvhead, const int32_t* must_select, int n_must, int sink_tokens,
                                 int recent_tokens, int32_t* out_physical, int32_t* out_logical,
                                 int32_t* out_scores, int32_t* out_valid_count, int32_t* out_new_seq_lens,
                                 void* workspace, size_t workspace_bytes, void* stream)
{
    return run_select(false, codes, NB, BS, Hkv, W, q_codes, Hq, block_table, max_blocks, block_table_stride,
                      seq_lens, nullptr, B, k, k_per_request, request_mask, reduce_mode, reduce_kvhead,
                      must_select, n_must, sink_tokens, recent_tokens, 0, 1.0f, out_physical, out_logical,
                      out_scores, out_valid_count, out_new_seq_lens, nullptr, nullptr, workspace,
                      workspace_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" int ucmr_topk_candidates(const uint32_t* codes, int64_t NB, int BS, int Hkv, int W,
                                    const uint32_t* q_codes, int Hq, const int32_t* block_table, int max_blocks,
                                    int64_t block_table_stride, const int32_t* seq_lens_local,
                                    const int32_t* seq_lens_global, int B, int k, int block_id_offset,
                                    float score_scale, int reduce_mode, int reduce_kvhead,
                                    const int32_t* must_select, int n_must, int sink_tokens, int recent_tokens,
                                    float* cand_scores, int32_t* cand_ids, void* workspace,
                                    size_t workspace_bytes, void* stream)
{
    if (block_id_offset < 0) return UCMR_ERR_BAD_ARG;
    return run_select(true, codes, NB, BS, Hkv, W, q_codes, Hq, block_table, max_blocks, block_table_stride,
                      seq_lens_local, seq_lens_global, B, k, nullptr, nullptr, reduce_mode, reduce_kvhead,
                      must_select, n_must, sink_tokens, recent_tokens, block_id_offset, score_scale, nullptr,
                      nullptr, nullptr, nullptr, nullptr, cand_scores, cand_ids, workspace, workspace_bytes,
                      static_cast<cudaStream_t>(stream));
}

namespace ucmr {
int run_merge(const float* cand_scores, const int32_t* cand_ids, int64_t rank_stride, int R, int B, int Hout, int kl, int k,
              int largest, float* out_scores, int32_t* out_ids, cudaStream_t st);
struct MergeStep {  // replay-safe step counting, see MergeParams
    int32_t* step_word;
    int32_t* arrive_word;
    int64_t parity_stride, flags_parity_stride;
};
static int run_merge_wait(const float* cand_scores, const int32_t* cand_ids, int64_t rank_stride, int R, int B, int Hout,
                          int kl, int k, int largest, float* out_scores, int32_t* out_ids, const int32_t* wait_flags,
                          int wait_seq, int32_t* status, cudaStream_t st, const MergeStep* step = nullptr);
}

extern "C" int ucmr_merge_topk(const float* cand_scores, const int32_t* cand_ids, int64_t rank_stride, int R,
                               int B, int Hout, int kl, int k, float* out_scores, int32_t* out_ids, void* stream)
{
    return run_merge(cand_scores, cand_ids, rank_stride, R, B, Hout, kl, k, 0, out_scores, out_ids,
                     static_cast<cudaStream_t>(stream));
}

int ucmr::run_merge(const float* cand_scores, const int32_t* cand_ids, int64_t rank_stride, int R, int B, int Hout, int kl,
                    int k, int largest, float* out_scores, int32_t* out_ids, cudaStream_t stream)
{
    return run_merge_wait(cand_scores, cand_ids, rank_stride, R, B, Hout, kl, k, largest, out_scores, out_ids, nullptr, 0,
                          nullptr, stream);
}

static int ucmr::run_merge_wait(const float* cand_scores, const int32_t* cand_ids, int64_t rank_stride, int R, int B,
                                int Hout, int kl, int k, int largest, float* out_scores, int32_t* out_ids,
                                const int32_t* wait_flags, int wait_seq, int32_t* status, cudaStream_t stream,
                                const MergeStep* step)
{
    if (rank_stride == 0) rank_stride = (int64_t)B * Hout * kl;
    if (rank_stride < (int64_t)B * Hout * kl) return UCMR_ERR_BAD_ARG;
    if (!cand_scores || !cand_ids || !out_scores || !out_ids) return UCMR_ERR_BAD_ARG;
    if (R <= 0 || B < 0 || Hout <= 0 || kl <= 0 || k < 0) return UCMR_ERR_BAD_ARG;
    if ((int64_t)R * kl > INT_MAX) return UCMR_ERR_UNSUPPORTED;
    if (B == 0 || k == 0) return UCMR_OK;
    if (wait_flags && R > kSelThreads) return UCMR_ERR_UNSUPPORTED;
    MergeParams p{cand_scores, cand_ids, rank_stride, R, B, Hout, kl, k, 0, out_scores, out_ids, largest ? 1 : 0,
                  wait_flags, wait_seq, status, nullptr, nullptr, 0, 0};
    if (step) {
        p.step_word = step->step_word; p.arrive_word = step->arrive_word;
        p.parity_stride = step->parity_stride; p.flags_parity_stride = step->flags_parity_stride;
    }
    const int n = R * kl;
    p.n_cached = n < kSelMaxCachedKeys ? n : kSelMaxCachedKeys;
    const size_t smem = (size_t)p.n_cached * sizeof(uint32_t);
    int rc = set_dyn_smem(merge_kernel, smem);
    if (rc != UCMR_OK) return rc;
    return launch_kernel(merge_kernel, dim3(B * Hout), dim3(kSelThreads), smem, stream, p);
}

extern "C" int ucmr_update_seq_lens(const int32_t* seq_lens, int B, int topk_tokens, int BS, int32_t* out,
                                    void* stream)
{
    if (!seq_lens || !out || B < 0 || BS <= 0 || topk_tokens < 0) return UCMR_ERR_BAD_ARG;
    if (B == 0) return UCMR_OK;
    update_seq_lens_kernel<<<(B + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(seq_lens, B, topk_tokens, BS, out);
    return check_launch();
}

/* Peer-memory form of the sequence-sharded exchange (see include/ucmr.h). */
extern "C" int ucmr_topk_candidates_p2p(const uint32_t* codes, int64_t NB, int BS, int Hkv, int W,
                                        const uint32_t* q_codes, int Hq, const int32_t* block_table, int max_blocks,
                                        int64_t block_table_stride, const int32_t* seq_lens_local,
                                        const int32_t* seq_lens_global, int B, int k, int block_id_offset,
                                        float score_scale, int reduce_mode, int reduce_kvhead,
                                        const int32_t* must_select, int n_must, int sink_tokens, int recent_tokens,
                                        float* const* peer_scores, int32_t* const* peer_ids,
                                        int32_t* const* peer_flags, int n_peers, int seq, void* workspace,
                                        size_t workspace_bytes, void* stream)
{
    if (block_id_offset < 0 || !peer_scores || !peer_ids || !peer_flags || n_peers <= 0 || n_peers > kMaxPeers)
        return UCMR_ERR_BAD_ARG;
    PeerDest pd{};
    pd.n_peers = n_peers; pd.seq = seq;
    for (int r = 0; r < n_peers; ++r) {
        if (!peer_scores[r] || !peer_ids[r] || !peer_flags[r]) return UCMR_ERR_BAD_ARG;
        pd.scores[0][r] = peer_scores[r]; pd.ids[0][r] = peer_ids[r]; pd.flags[0][r] = peer_flags[r];
    }
    return run_select(true, codes, NB, BS, Hkv, W, q_codes, Hq, block_table, max_blocks, block_table_stride,
                      seq_lens_local, seq_lens_global, B, k, nullptr, nullptr, reduce_mode, reduce_kvhead,
                      must_select, n_must, sink_tokens, recent_tokens, block_id_offset, score_scale, nullptr,
                      nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, workspace, workspace_bytes,
                      static_cast<cudaStream_t>(stream), &pd);
}

extern "C" int ucmr_merge_topk_wait(const float* cand_scores, const int32_t* cand_ids, int64_t rank_stride, int R, int B,
                                    int Hout, int kl, int k, float* out_scores, int32_t* out_ids,
                                    const int32_t* flags, int seq, int32_t* status_word, void* stream)
{
    if (!flags) return UCMR_ERR_BAD_ARG;
    return run_merge_wait(cand_scores, cand_ids, rank_stride, R, B, Hout, kl, k, 0, out_scores, out_ids, flags, seq,
                          status_word, static_cast<cudaStream_t>(stream));
}

/* Replay-safe forms of the peer-memory exchange: the step number lives in a device word (see include/ucmr.h). */
extern "C" int ucmr_topk_candidates_p2p_step(const uint32_t* codes, int64_t NB, int BS, int Hkv, int W,
                                             const uint32_t* q_codes, int Hq, const int32_t* block_table,
                                             int max_blocks, int64_t block_table_stride,
                                             const int32_t* seq_lens_local, const int32_t* seq_lens_global, int B,
                                             int k, int block_id_offset, float score_scale, int reduce_mode,
                                             int reduce_kvhead, const int32_t* must_select, int n_must,
                                             int sink_tokens, int recent_tokens, float* const* peer_scores,
                                             int32_t* const* peer_ids, int32_t* const* peer_flags, int n_peers,
                                             const int32_t* step_word, void* workspace, size_t workspace_bytes,
                                             void* stream)
{
    if (block_id_offset < 0 || !peer_scores || !peer_ids || !peer_flags || !step_word || n_peers <= 0 ||
        n_peers > kMaxPeers)
        return UCMR_ERR_BAD_ARG;
    PeerDest pd{};
    pd.n_peers = n_peers; pd.seq = 0; pd.step_word = step_word;
    for (int par = 0; par < 2; ++par)
        for (int r = 0; r < n_peers; ++r) {
            const int i = par * n_peers + r;
            if (!peer_scores[i] || !peer_ids[i] || !peer_flags[i]) return UCMR_ERR_BAD_ARG;
            pd.scores[par][r] = peer_scores[i]; pd.ids[par][r] = peer_ids[i]; pd.flags[par][r] = peer_flags[i];
        }
    return run_select(true, codes, NB, BS, Hkv, W, q_codes, Hq, block_table, max_blocks, block_table_stride,
                      seq_lens_local, seq_lens_global, B, k, nullptr, nullptr, reduce_mode, reduce_kvhead,
                      must_select, n_must, sink_tokens, recent_tokens, block_id_offset, score_scale, nullptr,
                      nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, workspace, workspace_bytes,
                      static_cast<cudaStream_t>(stream), &pd);
}

extern "C" int ucmr_merge_topk_wait_step(const float* cand_scores, const int32_t* cand_ids, int64_t parity_stride,
                                         int64_t rank_stride, int R, int B, int Hout, int kl, int k,
                                         float* out_scores, int32_t* out_ids, const int32_t* flags,
                                         int64_t flags_parity_stride, int32_t* step_word, int32_t* arrive_word,
                                         int32_t* status_word, void* stream)
{
    if (!flags || !step_word || !arrive_word || parity_stride < 0 || flags_parity_stride < 0) return UCMR_ERR_BAD_ARG;
    const MergeStep ms{step_word, arrive_word, parity_stride, flags_parity_stride};
    return run_merge_wait(cand_scores, cand_ids, rank_stride, R, B, Hout, kl, k, 0, out_scores, out_ids, flags, 0,
                          status_word, static_cast<cudaStream_t>(stream), &ms);
}

#ifdef UCMR_TRACE
namespace ucmr { UCMR_TRACE_READER(trace_read_select) }
#endif

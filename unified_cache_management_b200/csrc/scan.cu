// Hamming scan over the paged hash-code cache (sm_100a).
//
// One CTA of 128 threads owns NBLK consecutive logical blocks of one request.  The physical block
// is one contiguous run of BS*Hkv*W words, so the CTA streams it with 16-byte loads, eight of them
// in flight per thread, XORs each against the query codes held in registers, popcounts, and
// reduces to one score per (block, kv head) with warp shuffles and a handful of shared-memory
// atomics.  No per-token score is ever written: the only output is int32 [B, Hout, max_blocks].
//
// Stands in for HammingScoreContiKernel + the torch.min that follows it in the reference
// (ucm/sparse/gsa_on_device/csrc/cuda/ham_dist/paged_ham_dist_mla.cu:111-248,
//  ucm/sparse/gsa_on_device/hamming_topk.py:45-47).
#include <limits.h>
#include <stdlib.h>

#include <cuda_fp16.h>

#include "common.cuh"

namespace ucmr {

constexpr int kScanThreads = 128;
constexpr int kScanLoads = 8;     // 16-byte loads in flight per thread
constexpr int kScanMaxHeads = 64;  // kv heads per device the fast kernel supports
constexpr int kGenericMaxQWords = 8192;

struct ScanParams {
    const uint4* codes;
    int64_t NB;
    int BS, Hkv, W;
    const uint32_t* q;
    int Hq, G;
    const int32_t* bt;
    int max_blocks;
    int64_t bt_stride;
    const int32_t* seq_lens;
    int reduce_kvhead;
    int32_t* out;     // [B, Hout, max_blocks]
    int32_t* status;  // may be null
    int P, PW, logP, logPW;
    int u4_per_block;
};

__device__ __forceinline__ int popc4(const uint4& a, const uint4& b)
{
    return __popc(a.x ^ b.x) + __popc(a.y ^ b.y) + __popc(a.z ^ b.z) + __popc(a.w ^ b.w);
}

// G = query heads per kv head as a compile-time constant (register-resident query codes), or 0 for
// "any G", which keeps the query codes in shared memory.
template <int NBLK, int G, bool MIN>
__global__ void __launch_bounds__(kScanThreads) scan_kernel(const ScanParams p)
{
    constexpr int UNROLL = kScanLoads / NBLK;
    constexpr int GQ = (G > 0) ? G : 1;
    __shared__ int s_acc[NBLK][kScanMaxHeads];
    __shared__ int s_valid[NBLK];
    extern __shared__ uint4 s_q[];  // only used when G == 0

    const int tid = threadIdx.x, lane = tid & 31;
    const int b = blockIdx.y;
    const int j0 = blockIdx.x * NBLK;
    const int Hout = p.reduce_kvhead ? 1 : p.Hkv;
    int32_t* out_row = p.out + (int64_t)b * Hout * p.max_blocks;

    const int seq = p.seq_lens[b];
    const int nb = (seq + p.BS - 1) / p.BS;

    if (j0 >= nb) {  // nothing valid here: mark the scores and leave
        for (int idx = tid; idx < NBLK * Hout; idx += kScanThreads) {
            const int n = idx / Hout, h = idx - n * Hout;
            if (j0 + n < p.max_blocks) out_row[(int64_t)h * p.max_blocks + j0 + n] = -1;
        }
        return;
    }

    int phys[NBLK];
#pragma unroll
    for (int n = 0; n < NBLK; ++n) {
        const int j = j0 + n;
        int v = -1;
        if (j < nb && j < p.max_blocks) {
            v = p.bt[(int64_t)b * p.bt_stride + j];
            if (v < 0 || v >= p.NB) {
                if (tid == 0) flag_status(p.status, UCMR_DEV_BAD_BLOCK_ID);
                v = -1;
            }
        }
        phys[n] = v;
    }

    const int hp = tid & (p.P - 1);
    const int head = hp >> p.logPW;
    const int part = hp & (p.PW - 1);

    uint4 qv[GQ];
    if constexpr (G > 0) {
        const uint4* q4 = reinterpret_cast<const uint4*>(p.q) + ((int64_t)b * p.Hq + head * G) * p.PW + part;
#pragma unroll
        for (int g = 0; g < G; ++g) qv[g] = __ldg(q4 + g * p.PW);
    } else {
        const uint4* q4 = reinterpret_cast<const uint4*>(p.q) + (int64_t)b * p.Hq * p.PW;
        for (int i = tid; i < p.Hq * p.PW; i += kScanThreads) s_q[i] = __ldg(q4 + i);
    }
    for (int i = tid; i < NBLK * kScanMaxHeads; i += kScanThreads) (&s_acc[0][0])[i] = MIN ? INT_MAX : 0;
    if (tid == 0) {  // every thread holds the same phys[]
#pragma unroll
        for (int n = 0; n < NBLK; ++n) s_valid[n] = phys[n] >= 0;
    }
    __syncthreads();

    int acc[NBLK];
#pragma unroll
    for (int n = 0; n < NBLK; ++n) acc[n] = MIN ? INT_MAX : 0;

    for (int base = 0; base < p.u4_per_block; base += kScanThreads * UNROLL) {
        uint4 kv[NBLK][UNROLL];
        bool ok[NBLK][UNROLL];
#pragma unroll
        for (int n = 0; n < NBLK; ++n) {
#pragma unroll
            for (int i = 0; i < UNROLL; ++i) {
                const int u = base + i * kScanThreads + tid;
                const int tok = u >> p.logP;
                const bool good = phys[n] >= 0 && u < p.u4_per_block && (j0 + n) * p.BS + tok < seq;
                ok[n][i] = good;
                kv[n][i] = make_uint4(0u, 0u, 0u, 0u);
                if (good) kv[n][i] = ld_stream_u4(p.codes + (int64_t)phys[n] * p.u4_per_block + u);
            }
        }
#pragma unroll
        for (int n = 0; n < NBLK; ++n) {
#pragma unroll
            for (int i = 0; i < UNROLL; ++i) {
                int d = 0;
                if constexpr (G > 0) {
#pragma unroll
                    for (int g = 0; g < G; ++g) d += popc4(kv[n][i], qv[g]);
                } else {
                    const uint4* sq = s_q + (head * p.G) * p.PW + part;
                    for (int g = 0; g < p.G; ++g) d += popc4(kv[n][i], sq[g * p.PW]);
                }
                if constexpr (MIN) {
                    // a token's distance spans PW adjacent lanes: complete it before taking the min
                    for (int off = 1; off < p.PW && off < 32; off <<= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
                    acc[n] = min(acc[n], ok[n][i] ? d : INT_MAX);
                } else {
                    acc[n] += ok[n][i] ? d : 0;
                }
            }
        }
    }

    // Lanes that differ only in their token bits (>= P) hold the same kv head; in sum mode the part
    // bits (< PW) fold in as well.
#pragma unroll
    for (int n = 0; n < NBLK; ++n) {
        int v = acc[n];
        for (int off = 1; off < 32; off <<= 1) {
            const bool fold = (off >= p.P) || (!MIN && off < p.PW);
            if (fold) {
                const int o = __shfl_xor_sync(0xffffffffu, v, off);
                v = MIN ? min(v, o) : v + o;
            }
        }
        const bool publish = ((lane & (p.PW - 1)) == 0) && ((lane >> p.logP) == 0);
        if (publish) {
            if (MIN) atomicMin(&s_acc[n][head], v);
            else atomicAdd(&s_acc[n][head], v);
        }
    }
    __syncthreads();

    for (int idx = tid; idx < NBLK * Hout; idx += kScanThreads) {
        const int n = idx / Hout, h = idx - n * Hout;
        const int j = j0 + n;
        if (j >= p.max_blocks) continue;
        int v = -1;
        if (j < nb && s_valid[n]) {
            if (p.reduce_kvhead) {
                v = s_acc[n][0];
                for (int hh = 1; hh < p.Hkv; ++hh) v = MIN ? min(v, s_acc[n][hh]) : v + s_acc[n][hh];
            } else {
                v = s_acc[n][h];
            }
        }
        out_row[(int64_t)h * p.max_blocks + j] = v;
    }
}

// Any W / Hkv / G: one thread per (token, kv head), word loads, query codes in shared memory.
// Used for shapes the 16-byte kernel does not cover (e.g. 576-bit MLA codes, W = 18).
__global__ void __launch_bounds__(kScanThreads) scan_generic_kernel(const ScanParams p, int mode_min)
{
    extern __shared__ uint32_t s_qw[];  // [Hq*W] then [Hkv] accumulators
    int* s_acc = reinterpret_cast<int*>(s_qw + p.Hq * p.W);
    const int tid = threadIdx.x;
    const int b = blockIdx.y, j = blockIdx.x;
    const int Hout = p.reduce_kvhead ? 1 : p.Hkv;
    int32_t* out_row = p.out + (int64_t)b * Hout * p.max_blocks;
    const int seq = p.seq_lens[b];
    const int nb = (seq + p.BS - 1) / p.BS;
    int phys = -1;
    if (j < nb) {
        phys = p.bt[(int64_t)b * p.bt_stride + j];
        if (phys < 0 || phys >= p.NB) {
            if (tid == 0) flag_status(p.status, UCMR_DEV_BAD_BLOCK_ID);
            phys = -1;
        }
    }
    if (phys < 0) {
        for (int h = tid; h < Hout; h += kScanThreads) out_row[(int64_t)h * p.max_blocks + j] = -1;
        return;
    }
    for (int i = tid; i < p.Hq * p.W; i += kScanThreads) s_qw[i] = p.q[(int64_t)b * p.Hq * p.W + i];
    for (int i = tid; i < p.Hkv; i += kScanThreads) s_acc[i] = mode_min ? INT_MAX : 0;
    __syncthreads();
    const int ntok = min(p.BS, seq - j * p.BS);
    const uint32_t* blk = reinterpret_cast<const uint32_t*>(p.codes) + (int64_t)phys * p.BS * p.Hkv * p.W;
    for (int e = tid; e < ntok * p.Hkv; e += kScanThreads) {
        const int h = e % p.Hkv;
        const uint32_t* kc = blk + (int64_t)e * p.W;
        int d = 0;
        for (int g = 0; g < p.G; ++g) {
            const uint32_t* qc = s_qw + (h * p.G + g) * p.W;
            for (int w = 0; w < p.W; ++w) d += __popc(kc[w] ^ qc[w]);
        }
        if (mode_min) atomicMin(&s_acc[h], d);
        else atomicAdd(&s_acc[h], d);
    }
    __syncthreads();
    for (int h = tid; h < Hout; h += kScanThreads) {
        int v;
        if (p.reduce_kvhead) {
            v = s_acc[0];
            for (int hh = 1; hh < p.Hkv; ++hh) v = mode_min ? min(v, s_acc[hh]) : v + s_acc[hh];
        } else {
            v = s_acc[h];
        }
        out_row[(int64_t)h * p.max_blocks + j] = v;
    }
}

template <int NBLK, bool MIN>
static int launch_scan_g(const ScanParams& p, int B, cudaStream_t st)
{
    dim3 grid((p.max_blocks + NBLK - 1) / NBLK, B);
    switch (p.G) {
        case 1: scan_kernel<NBLK, 1, MIN><<<grid, kScanThreads, 0, st>>>(p); break;
        case 2: scan_kernel<NBLK, 2, MIN><<<grid, kScanThreads, 0, st>>>(p); break;
        case 4: scan_kernel<NBLK, 4, MIN><<<grid, kScanThreads, 0, st>>>(p); break;
        case 8: scan_kernel<NBLK, 8, MIN><<<grid, kScanThreads, 0, st>>>(p); break;
        default: {
            const size_t smem = (size_t)p.Hq * p.PW * sizeof(uint4);
            scan_kernel<NBLK, 0, MIN><<<grid, kScanThreads, smem, st>>>(p);
        }
    }
    return check_launch();
}

template <bool MIN>
static int launch_scan_m(const ScanParams& p, int B, cudaStream_t st)
{
    if (p.u4_per_block >= kScanThreads * 8) return launch_scan_g<1, MIN>(p, B, st);
    if (p.u4_per_block >= kScanThreads * 4) return launch_scan_g<2, MIN>(p, B, st);
    if (p.u4_per_block >= kScanThreads * 2) return launch_scan_g<4, MIN>(p, B, st);
    return launch_scan_g<8, MIN>(p, B, st);
}

static int ilog2(int v)
{
    int l = 0;
    while ((1 << l) < v) ++l;
    return l;
}

int validate_scan_args(const void* codes, int64_t NB, int BS, int Hkv, int W, const void* q, int Hq,
                       const void* bt, int max_blocks, int64_t bt_stride, const void* seq_lens, int B)
{
    if (!codes || !q || !bt || !seq_lens) return UCMR_ERR_BAD_ARG;
    if (NB <= 0 || BS <= 0 || Hkv <= 0 || W <= 0 || Hq <= 0 || max_blocks <= 0 || B < 0) return UCMR_ERR_BAD_ARG;
    if (Hq % Hkv != 0) return UCMR_ERR_BAD_ARG;
    if (bt_stride < max_blocks) return UCMR_ERR_BAD_ARG;
    if (B > 65535) return UCMR_ERR_UNSUPPORTED;
    if ((int64_t)max_blocks * BS > INT_MAX) return UCMR_ERR_UNSUPPORTED;
    return UCMR_OK;
}

int run_scan_ring(const uint32_t* codes, int64_t NB, int BS, int Hkv, int W, const uint32_t* q, int Hq,
                  const int32_t* bt, int max_blocks, int64_t bt_stride, const int32_t* seq_lens, int B,
                  int reduce_mode, int reduce_kvhead, int32_t* out, int32_t* status, int32_t* sched, cudaStream_t st,
                  const FusedSel* fuse);

int run_scan_rows(const uint32_t* codes, int64_t NB, int BS, int Hkv, int W, const uint32_t* q, int Hq,
                  const int32_t* bt, int max_blocks, int64_t bt_stride, const int32_t* seq_lens, int B,
                  int reduce_mode, int reduce_kvhead, int32_t* out, int32_t* status, void* scratch, cudaStream_t st);

// UCMR_SCAN=register routes every scan through the register kernel of this file (debug aid; the
// staged kernel in scan_ring.cu is the default wherever it covers the shape).
static bool force_register_scan()
{
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("UCMR_SCAN");
        v = (e && e[0] == 'r') ? 1 : 0;
    }
    return v == 1;
}

// Launches the scan into `out` ([B,Hout,max_blocks] int32).  Shared by the C entry points.  `sched` is an
// optional zero-initialised int32 the staged kernel uses as its work counter; whoever passes it resets it
// to zero after the launch (stream-ordered).  `row_scratch` (optional, rows_scratch_bytes(B) bytes) enables the
// producer / consumer kernel for token-row codes.  With `fuse` the staged kernel also runs the selection (and clears the
// counter itself); *fused says whether it did - false when the shape went to a kernel that cannot.
int run_scan(const uint32_t* codes, int64_t NB, int BS, int Hkv, int W, const uint32_t* q, int Hq,
             const int32_t* bt, int max_blocks, int64_t bt_stride, const int32_t* seq_lens, int B,
             int reduce_mode, int reduce_kvhead, int32_t* out, int32_t* status, int32_t* sched, cudaStream_t st,
             const FusedSel* fuse, bool* fused, void* row_scratch)
{
    if (fused) *fused = false;
    int rc = validate_scan_args(codes, NB, BS, Hkv, W, q, Hq, bt, max_blocks, bt_stride, seq_lens, B);
    if (rc != UCMR_OK) return rc;
    if (!out) return UCMR_ERR_BAD_ARG;
    const int mode_flags = reduce_mode & ~0xFF;  // UCMR_FLAG_* bits travel with the mode
    reduce_mode &= 0xFF;
    if (mode_flags & ~(UCMR_FLAG_INPUTS_STABLE | UCMR_FLAG_CACHE_APPEND_ONLY)) return UCMR_ERR_BAD_ARG;
    if (reduce_mode != UCMR_REDUCE_MIN && reduce_mode != UCMR_REDUCE_SUM) return UCMR_ERR_BAD_ARG;
    if (B == 0) return UCMR_OK;

    if (!force_register_scan() && fuse == nullptr && row_scratch != nullptr) {
        // token-row codes (one kv head, 18 words): the producer / consumer kernel, which needs scratch for the planes
        rc = run_scan_rows(codes, NB, BS, Hkv, W, q, Hq, bt, max_blocks, bt_stride, seq_lens, B, reduce_mode, reduce_kvhead,
                           out, status, row_scratch, st);
        if (rc != UCMR_ERR_UNSUPPORTED) return rc;
    }
    if (!force_register_scan()) {
        rc = run_scan_ring(codes, NB, BS, Hkv, W, q, Hq, bt, max_blocks, bt_stride, seq_lens, B, reduce_mode | mode_flags,
                           reduce_kvhead, out, status, sched, st, fuse);
        if (rc != UCMR_ERR_UNSUPPORTED) {
            if (fused) *fused = rc == UCMR_OK && fuse != nullptr;
            return rc;
        }
    }

    ScanParams p{};
    p.codes = reinterpret_cast<const uint4*>(codes);
    p.NB = NB; p.BS = BS; p.Hkv = Hkv; p.W = W;
    p.q = q; p.Hq = Hq; p.G = Hq / Hkv;
    p.bt = bt; p.max_blocks = max_blocks; p.bt_stride = bt_stride;
    p.seq_lens = seq_lens;
    p.reduce_kvhead = reduce_kvhead ? 1 : 0;
    p.out = out; p.status = status;

    const bool aligned = (reinterpret_cast<uintptr_t>(codes) % 16 == 0) && (reinterpret_cast<uintptr_t>(q) % 16 == 0);
    const bool fast = aligned && (W % 4 == 0) && is_pow2(W / 4) && is_pow2(Hkv) && Hkv <= kScanMaxHeads &&
                      (Hkv * (W / 4) <= kScanThreads) && ((int64_t)BS * Hkv * (W / 4) <= (1 << 24)) &&
                      ((int64_t)Hq * (W / 4) * 16 <= 40 * 1024);
    if (fast) {
        p.PW = W / 4; p.P = Hkv * p.PW;
        p.logPW = ilog2(p.PW); p.logP = ilog2(p.P);
        p.u4_per_block = BS * p.P;
        return reduce_mode == UCMR_REDUCE_MIN ? launch_scan_m<true>(p, B, st) : launch_scan_m<false>(p, B, st);
    }
    if ((int64_t)Hq * W > kGenericMaxQWords) return UCMR_ERR_UNSUPPORTED;
    const size_t smem = ((size_t)Hq * W + Hkv) * sizeof(uint32_t);
    dim3 grid(max_blocks, B);
    scan_generic_kernel<<<grid, kScanThreads, smem, st>>>(p, reduce_mode == UCMR_REDUCE_MIN);
    return check_launch();
}

// ---- per-token fp16 scores of the old op -------------------------------------------------------
__global__ void hamming_score_kernel(const uint32_t* __restrict__ codes, int64_t NB, int BS, int Hkv, int W,
                                     const uint32_t* __restrict__ q, int Hq, const int32_t* __restrict__ bt,
                                     int max_blocks, int64_t bt_stride, const int32_t* __restrict__ seq_lens,
                                     int sink, int recent, int reduce_kvhead, __half* __restrict__ out)
{
    const int b = blockIdx.y;
    const int64_t max_seq = (int64_t)max_blocks * BS;
    const int Hout = reduce_kvhead ? 1 : Hkv;
    const int G = Hq / Hkv;
    const int seq = seq_lens[b];
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < max_seq * Hout;
         e += (int64_t)gridDim.x * blockDim.x) {
        const int ho = (int)(e / max_seq);
        const int pos = (int)(e - (int64_t)ho * max_seq);
        __half* o = out + ((int64_t)b * Hout + ho) * max_seq + pos;
        if (pos >= seq) { *o = __ushort_as_half(0x7C00); continue; }
        if (pos < sink || pos >= seq - recent) { *o = __float2half(0.f); continue; }
        int phys = bt[(int64_t)b * bt_stride + pos / BS];
        if (phys < 0 || phys >= NB) phys = 0;  // the reference reads block 0 for bad slots
        const uint32_t* tokc = codes + ((int64_t)phys * BS + pos % BS) * Hkv * W;
        int best = INT_MAX;
        const int h0 = reduce_kvhead ? 0 : ho, h1 = reduce_kvhead ? Hkv : ho + 1;
        for (int h = h0; h < h1; ++h) {
            int d = 0;
            for (int g = 0; g < G; ++g) {
                const uint32_t* qc = q + ((int64_t)b * Hq + h * G + g) * W;
                for (int w = 0; w < W; ++w) d += __popc(tokc[h * W + w] ^ __ldg(qc + w));
            }
            best = min(best, d);
        }
        *o = __float2half((float)best);
    }
}

}  // namespace ucmr

using namespace ucmr;

extern "C" int ucmr_block_scores(const uint32_t* codes, int64_t NB, int BS, int Hkv, int W,
                                 const uint32_t* q_codes, int Hq, const int32_t* block_table, int max_blocks,
                                 int64_t block_table_stride, const int32_t* seq_lens, int B, int reduce_mode,
                                 int reduce_kvhead, int32_t* out_scores, int32_t* status_word, void* stream)
{
    return run_scan(codes, NB, BS, Hkv, W, q_codes, Hq, block_table, max_blocks, block_table_stride, seq_lens,
                    B, reduce_mode, reduce_kvhead, out_scores, status_word, nullptr, static_cast<cudaStream_t>(stream),
                    nullptr, nullptr, nullptr);
}

extern "C" int ucmr_hamming_score(const uint32_t* codes, int64_t NB, int BS, int Hkv, int W,
                                  const uint32_t* q_codes, int Hq, const int32_t* block_table, int max_blocks,
                                  int64_t block_table_stride, const int32_t* seq_lens, int B, int sink_tokens,
                                  int recent_tokens, int reduce_kvhead, void* out_fp16, void* stream)
{
    int rc = validate_scan_args(codes, NB, BS, Hkv, W, q_codes, Hq, block_table, max_blocks,
                                block_table_stride, seq_lens, B);
    if (rc != UCMR_OK) return rc;
    if (!out_fp16 || sink_tokens < 0 || recent_tokens < 0) return UCMR_ERR_BAD_ARG;
    if (B == 0) return UCMR_OK;
    const int64_t per_req = (int64_t)max_blocks * BS * (reduce_kvhead ? 1 : Hkv);
    int gx = (int)((per_req + 255) / 256);
    if (gx > 148 * 16) gx = 148 * 16;
    hamming_score_kernel<<<dim3(gx, B), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        codes, NB, BS, Hkv, W, q_codes, Hq, block_table, max_blocks, block_table_stride, seq_lens, sink_tokens,
        recent_tokens, reduce_kvhead ? 1 : 0, static_cast<__half*>(out_fp16));
    return check_launch();
}

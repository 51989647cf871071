// Float block retrieval on the device (sm_100a): block representations and inner-product block scores, the
// path the reference's ESA / KVStar plugins run on CPU worker threads.
//
//   block_repr_kernel   representation of a KV block = mean of its keys over groups of `merge` tokens
//                       (ESA: merge = BS, one vector per block, ucm/sparse/esa/esa.py:254-263; KVStar: merge =
//                       blk_repre_inner_token_merge, ucm/sparse/kvstar/multistep.py:322-327).  float32 accumulation,
//                       one rounding to the cache's dtype, like torch's mean.  Reads every key once: HBM-bound.
//   dot_scores_kernel   score(request b, candidate i) = <q_b, repr[indexes[b][i]]> over all heads' dims in float32
//                       (ucm/sparse/esa/retrieval/cpy/retrieval_backend.cpp:206-219), one warp per candidate,
//                       written next to the candidate's index; the selection kernel of the sharded merge then
//                       returns the k largest.  HBM-bound on the representations.
//
// Numerics: float32 sums in a fixed order that differs from the reference's scalar loop, so scores agree to
// float32 rounding of the sum, not bit for bit.
#include <cuda_bf16.h>
#include <math.h>

#include "common.cuh"

namespace ucmr {

int run_merge(const float* cand_scores, const int32_t* cand_ids, int64_t rank_stride, int R, int B, int Hout, int kl, int k,
              int largest, float* out_scores, int32_t* out_ids, cudaStream_t st);

struct ReprParams {
    const __nv_bfloat16* k_cache;  // [NB, BS, row] with strides (elements)
    int64_t NB;
    int BS, row;                   // row = heads * head_dim elements per token (contiguous)
    int64_t stride_block, stride_t;
    const int32_t* block_ids;      // [n]
    int64_t n;
    int merge;                     // tokens per representation; divides BS
    __nv_bfloat16* out;            // [n, BS / merge, row]
    int32_t* status;
};

__device__ __forceinline__ void add_bf16x8(float (&acc)[8], uint4 v)
{
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        acc[2 * i] += f.x;
        acc[2 * i + 1] += f.y;
    }
}

// grid.x = n * (BS / merge); a thread owns eight consecutive elements of the row.
__global__ void __launch_bounds__(128) block_repr_kernel(const ReprParams p)
{
    const int groups = p.BS / p.merge;
    const int64_t item = blockIdx.x;
    const int64_t bi = item / groups;
    const int m = (int)(item - bi * groups);
    const int id = p.block_ids[bi];
    if (id < 0 || id >= p.NB) {
        if (threadIdx.x == 0) flag_status(p.status, UCMR_DEV_BAD_BLOCK_ID);
        return;
    }
    const __nv_bfloat16* src = p.k_cache + (int64_t)id * p.stride_block + (int64_t)m * p.merge * p.stride_t;
    __nv_bfloat16* dst = p.out + (bi * groups + m) * (int64_t)p.row;
    const float inv = 1.0f / (float)p.merge;
    for (int e = threadIdx.x * 8; e < p.row; e += blockDim.x * 8) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        constexpr int UN = 8;  // token rows in flight
        for (int t0 = 0; t0 < p.merge; t0 += UN) {
            uint4 v[UN];
#pragma unroll
            for (int u = 0; u < UN; ++u)
                if (t0 + u < p.merge) v[u] = ld_stream_u4(reinterpret_cast<const uint4*>(src + (int64_t)(t0 + u) * p.stride_t + e));
#pragma unroll
            for (int u = 0; u < UN; ++u)
                if (t0 + u < p.merge) add_bf16x8(acc, v[u]);
        }
        __nv_bfloat162 o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) o[i] = __floats2bfloat162_rn(acc[2 * i] * inv, acc[2 * i + 1] * inv);
        *reinterpret_cast<uint4*>(dst + e) = *reinterpret_cast<const uint4*>(o);
    }
}

struct DotParams {
    const __nv_bfloat16* repr;  // [N, dim]
    int64_t N;
    int dim;                    // multiple of 8
    const __nv_bfloat16* q;     // [B, dim]
    const int32_t* indexes;     // [B, n]; entries < 0 or >= N are not candidates
    int B, n;
    float* scores;              // [B, n]
    int32_t* ids;               // [B, n] (-1 = not a candidate)
};

constexpr int kDotWarps = 8;

// grid = (ceil(n / kDotWarps), B): the CTA's query sits in shared memory as float32, one warp per candidate.
__global__ void __launch_bounds__(kDotWarps * 32) dot_scores_kernel(const DotParams p)
{
    extern __shared__ float s_q[];  // [dim]
    const int b = blockIdx.y;
    for (int e = threadIdx.x; e < p.dim; e += blockDim.x) s_q[e] = __bfloat162float(p.q[(int64_t)b * p.dim + e]);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int i = blockIdx.x * kDotWarps + warp;
    if (i >= p.n) return;
    const int idx = p.indexes[(int64_t)b * p.n + i];
    const int64_t o = (int64_t)b * p.n + i;
    if (idx < 0 || idx >= p.N) {
        if (lane == 0) { p.scores[o] = -INFINITY; p.ids[o] = -1; }
        return;
    }
    const uint4* row = reinterpret_cast<const uint4*>(p.repr + (int64_t)idx * p.dim);
    float acc = 0.f;
    for (int c = lane; c < p.dim / 8; c += 32) {
        const uint4 v = ld_stream_u4(row + c);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
        const float* qv = s_q + c * 8;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h[j]);
            acc = fmaf(f.x, qv[2 * j], acc);
            acc = fmaf(f.y, qv[2 * j + 1], acc);
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0) { p.scores[o] = acc; p.ids[o] = idx; }
}

// ---- softmax-sum block scores (KVStar) -------------------------------------------------------------------
// ucm/sparse/kvstar/retrieve/core/domain/retrieve_task/simd_compute_kernel.cpp:884-960: for every query row (token x,
// query head H of kv head h) the inner products with all S = n_blocks * M representations of that kv head, a softmax
// over the S values, and the block score = sum over rows and over the block's M representations of the softmax.
struct SoftmaxParams {
    const __nv_bfloat16* repr;  // [S, Hkv, D]
    const __nv_bfloat16* q;     // [X, Hq, D]
    int S, Hkv, Hq, D, X, n_blocks, M;
    float* logits;              // [X * Hq, S]
    float* stats;               // [X * Hq, 2]: row max, 1 / sum of exp (or 1 when the sum is tiny)
    float* out;                 // [n_blocks]
    int32_t* ids;               // [n_blocks] = 0, 1, 2, ...
};

// grid = (ceil(S / reps per CTA), X * Hkv): a group of lanes per representation (16 lanes for D = 128, so two
// representations per warp); the representation is read once and multiplied with the G query heads of its kv head,
// whose vectors sit in shared memory as float32.
constexpr int kLogitMaxG = 16;

__global__ void __launch_bounds__(kDotWarps * 32) kv_logits_kernel(const SoftmaxParams p)
{
    extern __shared__ float s_q[];  // [G][D]
    const int G = p.Hq / p.Hkv;
    const int x = blockIdx.y / p.Hkv, h = blockIdx.y % p.Hkv;
    const int row0 = x * p.Hq + h * G;  // first query row of this kv head
    for (int e = threadIdx.x; e < G * p.D; e += blockDim.x) s_q[e] = __bfloat162float(p.q[(int64_t)row0 * p.D + e]);
    __syncthreads();
    const int chunks = p.D / 8;
    int lanes_per = 1;
    while (lanes_per < chunks && lanes_per < 32) lanes_per <<= 1;
    const int reps_per_warp = 32 / lanes_per;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane / lanes_per, sl = lane % lanes_per;
    const int sidx = (blockIdx.x * kDotWarps + warp) * reps_per_warp + sub;
    const bool live = sidx < p.S;
    float acc[kLogitMaxG];
#pragma unroll
    for (int g = 0; g < kLogitMaxG; ++g) acc[g] = 0.f;
    if (live) {
        const uint4* kr = reinterpret_cast<const uint4*>(p.repr + ((int64_t)sidx * p.Hkv + h) * p.D);
        for (int c = sl; c < chunks; c += lanes_per) {
            const uint4 v = __ldg(kr + c);
            const __nv_bfloat162* hv = reinterpret_cast<const __nv_bfloat162*>(&v);
            float kf[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(hv[j]); kf[2 * j] = f.x; kf[2 * j + 1] = f.y; }
#pragma unroll
            for (int g = 0; g < kLogitMaxG; ++g) {
                if (g < G) {
                    const float* qv = s_q + g * p.D + c * 8;
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[g] = fmaf(kf[j], qv[j], acc[g]);
                }
            }
        }
    }
#pragma unroll
    for (int g = 0; g < kLogitMaxG; ++g) {
        if (g < G) {  // (G is the same for the whole warp)
            float a = acc[g];
            for (int off = lanes_per >> 1; off > 0; off >>= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
            if (live && sl == 0) p.logits[(int64_t)(row0 + g) * p.S + sidx] = a;
        }
    }
}

// One CTA per row: max, then sum of exp(l - max).
__global__ void __launch_bounds__(256) softmax_stats_kernel(const SoftmaxParams p)
{
    __shared__ float s_red[8];
    const float* l = p.logits + (int64_t)blockIdx.x * p.S;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < p.S; i += blockDim.x) mx = fmaxf(mx, l[i]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    if (lane == 0) s_red[warp] = mx;
    __syncthreads();
    mx = s_red[0];
    for (int w = 1; w < 8; ++w) mx = fmaxf(mx, s_red[w]);
    __syncthreads();
    float sum = 0.f;
    for (int i = threadIdx.x; i < p.S; i += blockDim.x) sum += expf(l[i] - mx);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    if (lane == 0) s_red[warp] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int w = 0; w < 8; ++w) t += s_red[w];
        p.stats[2 * blockIdx.x] = mx;
        p.stats[2 * blockIdx.x + 1] = t > 1e-9f ? 1.0f / t : 1.0f;  // the reference skips the division for a tiny sum
    }
}

// A warp per block: sum over rows and over the block's M representations of the normalised exponentials.
__global__ void __launch_bounds__(kDotWarps * 32) softmax_block_sum_kernel(const SoftmaxParams p)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * kDotWarps + warp;
    if (n >= p.n_blocks) return;
    const int rows = p.X * p.Hq;
    float acc = 0.f;
    for (int e = lane; e < rows * p.M; e += 32) {
        const int row = e / p.M, m = e - row * p.M;
        acc += expf(p.logits[(int64_t)row * p.S + (int64_t)n * p.M + m] - p.stats[2 * row]) * p.stats[2 * row + 1];
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0) { p.out[n] = acc; p.ids[n] = n; }
}

}  // namespace ucmr

using namespace ucmr;

extern "C" int ucmr_block_repr_mean(const void* k_cache, int64_t NB, int BS, int row_elems, int64_t stride_block,
                                    int64_t stride_t, const int32_t* block_ids, int64_t n_blocks, int merge, void* out,
                                    int32_t* status_word, void* stream)
{
    if (!k_cache || !out || NB <= 0 || BS <= 0 || row_elems <= 0 || n_blocks < 0 || merge <= 0) return UCMR_ERR_BAD_ARG;
    if (n_blocks > 0 && !block_ids) return UCMR_ERR_BAD_ARG;
    if (BS % merge != 0 || stride_t < row_elems || stride_block < stride_t) return UCMR_ERR_BAD_ARG;
    if (row_elems % 8 != 0 || stride_t % 8 != 0 || stride_block % 8 != 0 || reinterpret_cast<uintptr_t>(k_cache) % 16 != 0 ||
        reinterpret_cast<uintptr_t>(out) % 16 != 0)
        return UCMR_ERR_UNSUPPORTED;
    const int64_t items = n_blocks * (BS / merge);
    if (items == 0) return UCMR_OK;
    if (items > 0x7FFFFFFF) return UCMR_ERR_UNSUPPORTED;
    ReprParams p{};
    p.k_cache = static_cast<const __nv_bfloat16*>(k_cache); p.NB = NB; p.BS = BS; p.row = row_elems;
    p.stride_block = stride_block; p.stride_t = stride_t; p.block_ids = block_ids; p.n = n_blocks; p.merge = merge;
    p.out = static_cast<__nv_bfloat16*>(out); p.status = status_word;
    return launch_kernel(block_repr_kernel, dim3((unsigned)items), dim3(128), 0, static_cast<cudaStream_t>(stream), p);
}

extern "C" size_t ucmr_dot_topk_workspace_bytes(int B, int n)
{
    if (B < 0 || n < 0) return 0;
    return (size_t)B * n * (sizeof(float) + sizeof(int32_t));
}

extern "C" int ucmr_dot_topk(const void* repr, int64_t N, int dim, const void* q, const int32_t* indexes, int B, int n,
                             int k, float* out_scores, int32_t* out_ids, void* workspace, size_t workspace_bytes,
                             void* stream)
{
    if (!repr || !q || !indexes || !out_scores || !out_ids || N <= 0 || dim <= 0 || B < 0 || n <= 0 || k < 0) return UCMR_ERR_BAD_ARG;
    if (dim % 8 != 0 || dim > 8192 || reinterpret_cast<uintptr_t>(repr) % 16 != 0) return UCMR_ERR_UNSUPPORTED;
    if (!workspace || workspace_bytes < ucmr_dot_topk_workspace_bytes(B, n)) return UCMR_ERR_WORKSPACE;
    if (B == 0 || k == 0) return UCMR_OK;
    if (B > 65535) return UCMR_ERR_UNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    DotParams p{};
    p.repr = static_cast<const __nv_bfloat16*>(repr); p.N = N; p.dim = dim; p.q = static_cast<const __nv_bfloat16*>(q);
    p.indexes = indexes; p.B = B; p.n = n;
    p.scores = static_cast<float*>(workspace);
    p.ids = reinterpret_cast<int32_t*>(p.scores + (size_t)B * n);
    int rc = launch_kernel(dot_scores_kernel, dim3((unsigned)((n + kDotWarps - 1) / kDotWarps), (unsigned)B),
                           dim3(kDotWarps * 32), (size_t)dim * sizeof(float), st, p);
    if (rc != UCMR_OK) return rc;
    // the k largest scores, ties to the earlier candidate; rows come out in candidate order
    return run_merge(p.scores, p.ids, 0, 1, B, 1, n, k, 1, out_scores, out_ids, st);
}

extern "C" size_t ucmr_softmax_topk_workspace_bytes(int X, int Hq, int n_blocks, int M)
{
    if (X < 0 || Hq < 0 || n_blocks < 0 || M < 0) return 0;
    const size_t rows = (size_t)X * Hq;
    return rows * (size_t)n_blocks * M * sizeof(float) + rows * 2 * sizeof(float) + (size_t)n_blocks * 8 + 64;
}

extern "C" int ucmr_softmax_topk(const void* repr, int n_blocks, int M, int Hkv, int D, const void* q, int X, int Hq, int k,
                                 float* out_block_scores, float* out_scores, int32_t* out_ids, void* workspace,
                                 size_t workspace_bytes, void* stream)
{
    if (!repr || !q || n_blocks <= 0 || M <= 0 || Hkv <= 0 || D <= 0 || X <= 0 || Hq <= 0 || k < 0) return UCMR_ERR_BAD_ARG;
    if (Hq % Hkv != 0 || (k > 0 && (!out_scores || !out_ids))) return UCMR_ERR_BAD_ARG;
    if (D % 8 != 0 || D > 8192 || reinterpret_cast<uintptr_t>(repr) % 16 != 0) return UCMR_ERR_UNSUPPORTED;
    if ((int64_t)n_blocks * M > 0x7FFFFFFF || (int64_t)X * Hq > 65535) return UCMR_ERR_UNSUPPORTED;
    if (!workspace || workspace_bytes < ucmr_softmax_topk_workspace_bytes(X, Hq, n_blocks, M)) return UCMR_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    SoftmaxParams p{};
    p.repr = static_cast<const __nv_bfloat16*>(repr); p.q = static_cast<const __nv_bfloat16*>(q);
    p.S = n_blocks * M; p.Hkv = Hkv; p.Hq = Hq; p.D = D; p.X = X; p.n_blocks = n_blocks; p.M = M;
    const int rows = X * Hq;
    p.logits = static_cast<float*>(workspace);
    p.stats = p.logits + (size_t)rows * p.S;
    float* scores = p.stats + (size_t)rows * 2;
    p.out = out_block_scores ? out_block_scores : scores;
    p.ids = reinterpret_cast<int32_t*>(scores + n_blocks);
    if (Hq / Hkv > kLogitMaxG || (size_t)(Hq / Hkv) * D * sizeof(float) > 48 * 1024) return UCMR_ERR_UNSUPPORTED;
    int lanes_per = 1;
    while (lanes_per < D / 8 && lanes_per < 32) lanes_per <<= 1;
    const int reps_per_cta = kDotWarps * (32 / lanes_per);
    int rc = launch_kernel(kv_logits_kernel, dim3((unsigned)((p.S + reps_per_cta - 1) / reps_per_cta), (unsigned)(X * Hkv)),
                           dim3(kDotWarps * 32), (size_t)(Hq / Hkv) * D * sizeof(float), st, p);
    if (rc != UCMR_OK) return rc;
    rc = launch_kernel(softmax_stats_kernel, dim3((unsigned)rows), dim3(256), 0, st, p);
    if (rc != UCMR_OK) return rc;
    rc = launch_kernel(softmax_block_sum_kernel, dim3((unsigned)((n_blocks + kDotWarps - 1) / kDotWarps)),
                       dim3(kDotWarps * 32), 0, st, p);
    if (rc != UCMR_OK || k == 0) return rc;
    return run_merge(p.out, p.ids, 0, 1, 1, 1, n_blocks, k, 1, out_scores, out_ids, st);
}

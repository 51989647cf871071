// Paged-KV gather (sm_100a): copies the selected physical blocks of the K and V pools into one
// contiguous buffer per request.
//
// Whole-block mode moves data with the bulk-copy (TMA) engine only: a persistent CTA per SM drives
// a ring of shared-memory stages; one thread issues cp.async.bulk global->shared for chunk i+LAG
// while chunk i goes shared->global.  No thread ever touches the payload.
// Per-head mode (each kv head selects its own blocks) copies D*elem-size rows with 16-byte
// loads/stores.
//
// Device-to-device form of the reference's kv_cache[block_ids]
// (ucm/sparse/gsa_on_device/gsa_on_device.py:579-580) and of CudaCopyKernel's
// scattered-blocks-to-one-buffer overload (ucm/shared/trans/cuda/cuda_sm_kernel.cu:66-78).
// ucmr_copy_blocks is the pointer-list form of all three CudaCopyKernel overloads (:52-92: list -> list,
// list -> contiguous, contiguous -> list) on the same copy-engine loop.
#include "common.cuh"

namespace ucmr {

constexpr int kGatherStages = 8;
constexpr int kGatherChunk = 16 * 1024;  // bytes per stage
constexpr int kGatherLag = 2;             // stores trail loads by STAGES - LAG chunks

struct GatherParams {
    const char* pool[2];
    char* out[2];
    int n_pools;
    int64_t NB, block_bytes;
    const int32_t* sel;  // [n_sel]
    int64_t n_sel;
    int chunks_per_block;
    int32_t* status;
};

// Where chunk c of a copy job comes from and goes to; false = skip it (bad id / misaligned pointer, flagged).
struct GatherLocator {
    GatherParams p;
    __device__ int64_t total() const { return p.n_sel * p.n_pools * p.chunks_per_block; }
    __device__ bool operator()(int64_t c, const char*& src, char*& dst, uint32_t& bytes) const
    {
        // The one thread that drives a CTA's copies resolves two chunks per 16 KiB moved; 64-bit divisions here
        // (a few hundred cycles each) would cost more than the copy engine needs per chunk, so chunk numbers that
        // fit 32 bits - all practical sizes - are split with 32-bit arithmetic.
        int chunk, which;
        int64_t s;
        if (c <= 0xFFFFFFFFll) {
            const uint32_t c32 = (uint32_t)c, cpb = (uint32_t)p.chunks_per_block;
            const uint32_t t = c32 / cpb;
            chunk = (int)(c32 - t * cpb);
            const uint32_t s32 = p.n_pools == 2 ? (t >> 1) : t;
            which = p.n_pools == 2 ? (int)(t & 1u) : 0;
            s = s32;
        } else {
            chunk = (int)(c % p.chunks_per_block);
            const int64_t t = c / p.chunks_per_block;
            which = (int)(t % p.n_pools);
            s = t / p.n_pools;
        }
        const int phys = p.sel[s];
        const int64_t off = (int64_t)chunk * kGatherChunk;
        const int64_t left = p.block_bytes - off;
        bytes = (uint32_t)(left < kGatherChunk ? left : kGatherChunk);
        if (phys < 0 || phys >= p.NB) return false;
        // (picked with compile-time offsets: a run-time index into the kernel parameter means generic-address loads)
        src = (which ? p.pool[1] : p.pool[0]) + (int64_t)phys * p.block_bytes + off;
        dst = (which ? p.out[1] : p.out[0]) + s * p.block_bytes + off;
        return true;
    }
    __device__ int32_t* status() const { return p.status; }
};

// Pointer-list form: block i goes from src_ptrs[i] (or src_base + i*size) to dst_ptrs[i] (or dst_base + i*size).
struct CopyListParams {
    const void* const* src_ptrs;
    const char* src_base;
    void* const* dst_ptrs;
    char* dst_base;
    int64_t size, num;
    int chunks_per_block;
    int32_t* status;
};

struct ListLocator {
    CopyListParams p;
    __device__ int64_t total() const { return p.num * p.chunks_per_block; }
    __device__ bool operator()(int64_t c, const char*& src, char*& dst, uint32_t& bytes) const
    {
        int chunk;
        int64_t i;
        if (c <= 0xFFFFFFFFll) {  // 32-bit split, see GatherLocator
            const uint32_t c32 = (uint32_t)c, cpb = (uint32_t)p.chunks_per_block;
            const uint32_t q = c32 / cpb;
            chunk = (int)(c32 - q * cpb);
            i = q;
        } else {
            chunk = (int)(c % p.chunks_per_block);
            i = c / p.chunks_per_block;
        }
        const int64_t off = (int64_t)chunk * kGatherChunk;
        const int64_t left = p.size - off;
        bytes = (uint32_t)(left < kGatherChunk ? left : kGatherChunk);
        const char* sb = p.src_ptrs ? static_cast<const char*>(p.src_ptrs[i]) : p.src_base + i * p.size;
        char* db = p.dst_ptrs ? static_cast<char*>(p.dst_ptrs[i]) : p.dst_base + i * p.size;
        // the copy engine needs 16-byte aligned addresses; a null or misaligned entry is skipped and flagged
        if (!sb || !db || (reinterpret_cast<uintptr_t>(sb) & 15u) || (reinterpret_cast<uintptr_t>(db) & 15u)) return false;
        src = sb + off;
        dst = db + off;
        return true;
    }
    __device__ int32_t* status() const { return p.status; }
};

template <typename Locator>
__global__ void __launch_bounds__(32) bulk_copy_kernel(const Locator loc)
{
    extern __shared__ __align__(128) char s_buf[];
    __shared__ __align__(8) uint64_t s_full[kGatherStages];
    __shared__ char* s_dst[kGatherStages];       // where the chunk in each stage goes (null: nothing to store)
    __shared__ uint32_t s_bytes[kGatherStages];
    if (threadIdx.x != 0) return;  // a single thread drives the copy engine

    for (int s = 0; s < kGatherStages; ++s) mbar_init(&s_full[s], 1);
    fence_mbar_init();

    const int64_t total = loc.total();
    const int64_t first = blockIdx.x, step = gridDim.x;
    const int64_t my_count = first < total ? (total - first + step - 1) / step : 0;
    constexpr int AHEAD = kGatherStages - kGatherLag;  // loads in flight before the first store
    bool dead = false;

    for (int64_t it = 0; it < my_count + AHEAD; ++it) {
        if (it < my_count && !dead) {
            const int stage = (int)(it % kGatherStages);
            // the store that last read this stage was committed LAG groups ago
            if (it >= kGatherStages) bulk_wait_read<kGatherLag - 1>();
            // the chunk is resolved once, here; its destination waits in shared memory for the store side (a second
            // resolution there would put another dependent load of the selection on this thread's critical path)
            const char* src; char* dst; uint32_t bytes;
            if (loc(first + it * step, src, dst, bytes)) {
                s_dst[stage] = dst;
                s_bytes[stage] = bytes;
                mbar_expect_tx(&s_full[stage], bytes);
                bulk_g2s(s_buf + (size_t)stage * kGatherChunk, src, bytes, &s_full[stage]);
            } else {
                s_dst[stage] = nullptr;
                flag_status(loc.status(), UCMR_DEV_BAD_BLOCK_ID);
                mbar_arrive(&s_full[stage]);  // keep the phase sequence; nothing is stored for it
            }
        }
        const int64_t c = it - AHEAD;
        if (c >= 0 && c < my_count && !dead) {
            const int stage = (int)(c % kGatherStages);
            const uint32_t parity = (uint32_t)((c / kGatherStages) & 1);
            if (!mbar_wait(&s_full[stage], parity)) {
                flag_status(loc.status(), UCMR_DEV_WAIT_TIMEOUT);
                dead = true;
            } else {
                char* const dst = s_dst[stage];
                if (dst != nullptr) bulk_s2g(dst, s_buf + (size_t)stage * kGatherChunk, s_bytes[stage]);
                bulk_commit();  // one group per chunk, empty or not, so the wait counts stay aligned
            }
        }
    }
    bulk_wait_all<0>();
}

template <typename Locator>
static int launch_bulk_copy(const Locator& loc, int64_t total_chunks, cudaStream_t st)
{
    const size_t smem = (size_t)kGatherStages * kGatherChunk;
    cudaError_t e = cudaFuncSetAttribute(bulk_copy_kernel<Locator>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { note_cuda_error(e); return UCMR_ERR_LAUNCH; }
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int grid = (int)(total_chunks < sms ? total_chunks : sms);
    bulk_copy_kernel<Locator><<<grid, 32, smem, st>>>(loc);
    return check_launch();
}

struct GatherRowsParams {
    const uint4* pool[2];
    uint4* out[2];
    int n_pools;
    int64_t NB;
    const int32_t* sel;  // [B, Hkv, k]
    int B, k, BS, Hkv;
    int u4_per_row;
    int32_t* status;
};

__global__ void __launch_bounds__(256) gather_rows_kernel(const GatherRowsParams p)
{
    // one item = one 16-byte piece of one (request, slot i, token t, head h) row
    const int64_t rows = (int64_t)p.B * p.k * p.BS * p.Hkv;
    const int64_t total = rows * p.u4_per_row;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    constexpr int UN = 4;
    for (int64_t base = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; base < total; base += stride * UN) {
        uint4 v[2][UN];
        int64_t dsti[UN];
        bool ok[UN];
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            const int64_t e = base + u * stride;
            ok[u] = e < total;
            dsti[u] = e;
            if (!ok[u]) continue;
            const int piece = (int)(e % p.u4_per_row);
            int64_t r = e / p.u4_per_row;
            const int h = (int)(r % p.Hkv); r /= p.Hkv;
            const int t = (int)(r % p.BS); r /= p.BS;
            const int i = (int)(r % p.k);
            const int b = (int)(r / p.k);
            const int phys = p.sel[((int64_t)b * p.Hkv + h) * p.k + i];
            if (phys < 0 || phys >= p.NB) {
                flag_status(p.status, UCMR_DEV_BAD_BLOCK_ID);
                ok[u] = false;
                continue;
            }
            const int64_t srci = (((int64_t)phys * p.BS + t) * p.Hkv + h) * p.u4_per_row + piece;
#pragma unroll
            for (int w = 0; w < 2; ++w)  // (compile-time pool index, see GatherLocator)
                if (w < p.n_pools) v[w][u] = ld_stream_u4(p.pool[w] + srci);
        }
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            if (!ok[u]) continue;
#pragma unroll
            for (int w = 0; w < 2; ++w)
                if (w < p.n_pools) st_stream_u4(p.out[w] + dsti[u], v[w][u]);
        }
    }
}

}  // namespace ucmr

using namespace ucmr;

extern "C" int ucmr_gather_kv(const void* k_pool, const void* v_pool, int64_t NB, int64_t block_bytes,
                              const int32_t* sel, int B, int k, int per_head, int BS, int Hkv,
                              int64_t row_bytes, void* out_k, void* out_v, int32_t* status_word, void* stream)
{
    if (!sel || B < 0 || k < 0 || NB <= 0 || block_bytes <= 0) return UCMR_ERR_BAD_ARG;
    if ((k_pool == nullptr) != (out_k == nullptr) || (v_pool == nullptr) != (out_v == nullptr)) return UCMR_ERR_BAD_ARG;
    if (!k_pool && !v_pool) return UCMR_ERR_BAD_ARG;
    if (block_bytes % 16 != 0) return UCMR_ERR_UNSUPPORTED;
    const void* pools[2]; void* outs[2]; int n = 0;
    if (k_pool) { pools[n] = k_pool; outs[n] = out_k; ++n; }
    if (v_pool) { pools[n] = v_pool; outs[n] = out_v; ++n; }
    for (int i = 0; i < n; ++i)
        if (reinterpret_cast<uintptr_t>(pools[i]) % 16 || reinterpret_cast<uintptr_t>(outs[i]) % 16) return UCMR_ERR_UNSUPPORTED;
    if (B == 0 || k == 0) return UCMR_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    if (!per_head) {
        GatherParams p{};
        for (int i = 0; i < n; ++i) { p.pool[i] = static_cast<const char*>(pools[i]); p.out[i] = static_cast<char*>(outs[i]); }
        p.n_pools = n; p.NB = NB; p.block_bytes = block_bytes; p.sel = sel; p.n_sel = (int64_t)B * k;
        p.chunks_per_block = (int)((block_bytes + kGatherChunk - 1) / kGatherChunk);
        p.status = status_word;
        return launch_bulk_copy(GatherLocator{p}, p.n_sel * n * p.chunks_per_block, st);
    }

    if (BS <= 0 || Hkv <= 0 || row_bytes <= 0 || row_bytes % 16 != 0) return UCMR_ERR_UNSUPPORTED;
    if ((int64_t)BS * Hkv * row_bytes != block_bytes) return UCMR_ERR_BAD_ARG;
    GatherRowsParams p{};
    for (int i = 0; i < n; ++i) { p.pool[i] = static_cast<const uint4*>(pools[i]); p.out[i] = static_cast<uint4*>(outs[i]); }
    p.n_pools = n; p.NB = NB; p.sel = sel; p.B = B; p.k = k; p.BS = BS; p.Hkv = Hkv;
    p.u4_per_row = (int)(row_bytes / 16); p.status = status_word;
    const int64_t total = (int64_t)B * k * BS * Hkv * p.u4_per_row;
    int64_t want = (total + 256 * 4 - 1) / (256 * 4);
    int grid = (int)(want < 148 * 8 ? want : 148 * 8);
    if (grid < 1) grid = 1;
    gather_rows_kernel<<<grid, 256, 0, st>>>(p);
    return check_launch();
}

extern "C" int ucmr_copy_blocks(const void* const* src_ptrs, const void* src_base, void* const* dst_ptrs, void* dst_base,
                                int64_t size, int64_t num, int32_t* status_word, void* stream)
{
    if ((src_ptrs == nullptr) == (src_base == nullptr) || (dst_ptrs == nullptr) == (dst_base == nullptr)) return UCMR_ERR_BAD_ARG;
    if (size <= 0 || num < 0) return UCMR_ERR_BAD_ARG;
    if (size % 16 != 0) return UCMR_ERR_UNSUPPORTED;
    if ((src_base && reinterpret_cast<uintptr_t>(src_base) % 16) || (dst_base && reinterpret_cast<uintptr_t>(dst_base) % 16))
        return UCMR_ERR_UNSUPPORTED;
    if (num == 0) return UCMR_OK;
    CopyListParams p{};
    p.src_ptrs = src_ptrs; p.src_base = static_cast<const char*>(src_base);
    p.dst_ptrs = dst_ptrs; p.dst_base = static_cast<char*>(dst_base);
    p.size = size; p.num = num; p.chunks_per_block = (int)((size + kGatherChunk - 1) / kGatherChunk);
    p.status = status_word;
    return launch_bulk_copy(ListLocator{p}, num * p.chunks_per_block, static_cast<cudaStream_t>(stream));
}

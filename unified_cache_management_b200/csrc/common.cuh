// Shared helpers of the sm_100a retrieval kernels: status plumbing, cache-hinted loads,
// mbarrier / bulk-copy wrappers with bounded waits.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "ucmr.h"

namespace ucmr {

// Records the last CUDA runtime error text for ucmr_last_cuda_error().
void note_cuda_error(cudaError_t e);

inline int check_launch()
{
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        note_cuda_error(e);
        return UCMR_ERR_LAUNCH;
    }
    return UCMR_OK;
}

inline bool is_pow2(int64_t v) { return v > 0 && (v & (v - 1)) == 0; }

// Blocks that are selected whatever their score: listed block indices (>= 0 from the start, < 0 from the request's
// block count) and every block that overlaps the first `sink` or the last `recent` tokens.
struct ForcedSpec {
    int must[UCMR_MAX_MUST_SELECT];
    int n_must, sink, recent;
};

// Workspace header (int32 words, UCMR_WORKSPACE_HEADER_BYTES in all): [0] device status, [2] the scan's work
// counter, [3] CTA arrival counter of the peer exchange, and for a scan that also runs the selection [4] scan CTAs
// that have scored all their blocks and [36] the "all blocks scored" word, which counts such launches.  The block
// scores follow the header.  Every counter is zero between launches.
constexpr int kWsMaxBatch = 1024;

// Selection folded into the staged scan (scan_ring.cu) for rows of at most kFuseMaxBlocks blocks: what the scan needs
// to know to select the rows itself once every block has been scored.
constexpr int kFuseMaxBlocks = 2048;
struct FusedSel {
    int enabled;
    int Hout, k, key_bits, idx_bits;
    const int32_t* k_per_request;
    const uint8_t* mask;
    ForcedSpec forced;
    int32_t *out_phys, *out_logical, *out_scores, *out_valid, *out_newseq;
    int32_t* cta_done;    // scan CTAs whose warps have all run out of work items (zero between launches)
    int32_t* all_scored;  // bumped by one when the last CTA has arrived: every block score is in memory
};


// Launches `kernel` on `st` and turns a refused launch into UCMR_ERR_LAUNCH.
template <typename... KArgs, typename... Args>
inline int launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cfg.attrs = nullptr;
    cfg.numAttrs = 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
    if (e != cudaSuccess) {
        note_cuda_error(e);
        (void)cudaGetLastError();
        return UCMR_ERR_LAUNCH;
    }
    return UCMR_OK;
}

// Programmatic dependent launch (UCMR_PDL=0 turns it off): a kernel launched with `early = true` may start while
// the kernel before it in the stream is still running, once that kernel has executed grid_launch_dependents() in
// all its CTAs (or has finished); it must call grid_dependency_wait() before touching anything the earlier kernel
// writes - or reads anything that kernel might write: the kernel before it can be any kernel of the caller.  That
// hides the launch latency of the scan and lets its CTAs take over SMs one by one as the earlier kernel drains.
inline bool pdl_enabled()
{
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("UCMR_PDL");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

// Same as launch_kernel, optionally as a thread-block cluster launch (cluster_x > 1: that many consecutive CTAs
// form a cluster, grid.x % cluster_x == 0) and / or as a programmatic dependent launch (early).
template <typename... KArgs, typename... Args>
inline int launch_kernel_ex(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                            int cluster_x, bool early, Args... args)
{
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (cluster_x > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = (unsigned)cluster_x;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    if (early && pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cfg.attrs = n ? attr : nullptr;
    cfg.numAttrs = n;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
    if (e != cudaSuccess) {
        note_cuda_error(e);
        (void)cudaGetLastError();
        return UCMR_ERR_LAUNCH;
    }
    return UCMR_OK;
}

// Same, with `cluster_x` consecutive CTAs of the grid forming a thread-block cluster (grid.x % cluster_x == 0).
template <typename... KArgs, typename... Args>
inline int launch_kernel_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                 int cluster_x, Args... args)
{
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cluster_x;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
    if (e != cudaSuccess) {
        note_cuda_error(e);
        (void)cudaGetLastError();
        return UCMR_ERR_LAUNCH;
    }
    return UCMR_OK;
}

// Time bound of every spin-wait in this library.  A wait that runs out sets UCMR_DEV_WAIT_TIMEOUT in
// the status word and the kernel winds down without touching the data.
constexpr unsigned long long kWaitLimitNs = 1000ull * 1000ull * 1000ull;  // 1 s
constexpr uint32_t kWaitPollsPerClockCheck = 2048;

#ifdef __CUDACC__

// See launch_kernel_ex.
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ void flag_status(int32_t* status, int bits)
{
    if (status != nullptr) atomicOr(status, bits);
}

__device__ __forceinline__ bool block_is_forced(const ForcedSpec& f, int j, int nb, int seq, int BS)
{
    if (j >= nb) return false;
    for (int m = 0; m < f.n_must; ++m) {
        const int t = f.must[m] >= 0 ? f.must[m] : nb + f.must[m];
        if (t == j) return true;
    }
    const int lo = j * BS;
    const int hi = min(lo + BS, seq);
    if (f.sink > 0 && lo < f.sink) return true;
    if (f.recent > 0 && hi > seq - f.recent) return true;
    return false;
}

// Atomic add / exchange with release semantics at device scope: everything this thread has observed or written
// before is visible to whoever reads the new value with an acquire load (one instruction instead of fence + atomic).
__device__ __forceinline__ int atom_add_release_gpu(int32_t* p, int v)
{
    int old;
    asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
    return old;
}
__device__ __forceinline__ void st_release_gpu(int32_t* p, int v)
{
    asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ int ld_acquire_gpu(const int32_t* p)
{
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Streaming 16-byte load: read-only path, no L1 allocation (each code word is read once per scan).
__device__ __forceinline__ uint4 ld_stream_u4(const uint4* p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ void st_stream_u4(uint4* p, const uint4& v)
{
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
                 "r"(v.w)
                 : "memory");
}

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier -------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_inval(uint64_t* bar)
{
    asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)));
}
__device__ __forceinline__ void fence_mbar_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Non-blocking phase test (try_wait may suspend the thread for a while when the phase is not complete).
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_timer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Step timeline (builds with -DUCMR_TRACE only): thread 0 of CTA 0 stores %globaltimer at numbered points of the
// decode-step kernels (encode, scan, selection: one table per translation unit) and ucmr_trace_read copies a table
// to the host.  Without the define the macro expands to nothing and ucmr_trace_read reports "unsupported".
#ifdef UCMR_TRACE
static __device__ unsigned long long g_trace[UCMR_TRACE_SLOTS];
#define UCMR_STAMP(i)                                                                    \
    do {                                                                                 \
        if (blockIdx.x == 0 && threadIdx.x == 0) g_trace[(i)] = global_timer_ns();       \
    } while (0)
#define UCMR_STAMP_ANY(i) (g_trace[(i)] = global_timer_ns()) /* whichever thread gets there */
#define UCMR_STAMP_LAST(i) /* thread 0 of every CTA: the latest one stays */ \
    do {                                                                      \
        if (threadIdx.x == 0) atomicMax(&g_trace[(i)], global_timer_ns());     \
    } while (0)
#define UCMR_TRACE_READER(name)                                                                             \
    int name(unsigned long long* host)                                                                      \
    {                                                                                                       \
        return cudaMemcpyFromSymbol(host, g_trace, sizeof(g_trace)) == cudaSuccess ? UCMR_OK : UCMR_ERR_LAUNCH; \
    }
#else
#define UCMR_STAMP(i) ((void)0)
#define UCMR_STAMP_ANY(i) ((void)0)
#define UCMR_STAMP_LAST(i) ((void)0)
#endif

// Bounded wait.  Returns false when the time limit ran out (the caller must stop using the
// barrier's data, flag the status word and leave).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity)
{
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_timer_ns();
    for (;;) {
        for (uint32_t i = 0; i < kWaitPollsPerClockCheck; ++i) {
            if (mbar_try_wait(bar, parity)) return true;
        }
        if (global_timer_ns() - t0 > kWaitLimitNs) return false;
    }
}

// ---- untiled bulk copies (TMA engine, 16-byte aligned addresses and sizes) -----------------------
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes,
                                         uint64_t* bar)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
            "r"(smem_u32(smem_dst)),
        "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* gdst, const void* smem_src, uint32_t bytes)
{
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst),
                 "r"(smem_u32(smem_src)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit()
{
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_read()
{
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_all()
{
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

#endif  // __CUDACC__

}  // namespace ucmr

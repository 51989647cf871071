// Retrieval without a caller-provided workspace.
//
// Some callers of this library cannot hand over scratch memory: a serving engine that gave every free
// byte of the GPU to its KV-cache pool at start-up has nothing left to cudaMalloc from later, and a
// plugin hook that runs inside the engine's forward pass has no allocator of its own to ask.  For them
// the block scores that travel from the scan kernel to the selection kernel live in a fixed array inside
// the library image instead.
//
// The array belongs to the loaded module: every GPU that loads the library holds kStaticScratchBytes
// until the process exits, whether or not this entry point is ever called.
#include <mutex>

#include "common.cuh"

namespace ucmr {

constexpr size_t kStaticScratchBytes = 4u << 20;  // 4 MiB: header + up to ~1M block scores
constexpr int kMaxDevices = 64;

// File-scope device array.  In host code this name is only a handle for cudaGetSymbolAddress; it is not
// a device address and must never be passed to a kernel directly.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

static std::mutex g_setup_mutex;
static void* g_scratch_ptr[kMaxDevices] = {};

// Device address of the array on the current device, resolved once per device.
static int static_scratch(void** out)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { note_cuda_error(e); return UCMR_ERR_LAUNCH; }
    if (dev < 0 || dev >= kMaxDevices) return UCMR_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_ptr[dev] == nullptr) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_static_scratch);  // with device `dev` current
        if (e != cudaSuccess || ptr == nullptr) {
            if (e != cudaSuccess) note_cuda_error(e);
            return UCMR_ERR_LAUNCH;
        }
        g_scratch_ptr[dev] = ptr;
    }
    *out = g_scratch_ptr[dev];
    return UCMR_OK;
}

}  // namespace ucmr

using namespace ucmr;

extern "C" size_t ucmr_static_workspace_capacity(void) { return kStaticScratchBytes; }

extern "C" int ucmr_hamming_topk_static(const uint32_t* codes, int64_t NB, int BS, int Hkv, int W,
                                        const uint32_t* q_codes, int Hq, const int32_t* block_table, int max_blocks,
                                        int64_t block_table_stride, const int32_t* seq_lens, int B, int k,
                                        const int32_t* k_per_request, const uint8_t* request_mask, int reduce_mode,
                                        int reduce_kvhead, const int32_t* must_select, int n_must, int sink_tokens,
                                        int recent_tokens, int32_t* out_physical, int32_t* out_logical,
                                        int32_t* out_scores, int32_t* out_valid_count, int32_t* out_new_seq_lens,
                                        void* stream)
{
    const size_t need = ucmr_hamming_topk_workspace_bytes(B, Hkv, max_blocks, reduce_kvhead);
    if (need == 0) return UCMR_ERR_BAD_ARG;
    if (need > kStaticScratchBytes) return UCMR_ERR_WORKSPACE;  // shapes beyond the built-in scratch
    void* ws = nullptr;
    int rc = static_scratch(&ws);
    if (rc != UCMR_OK) return rc;
    // The array keeps what the previous call left in it.  The header (status word, the scan's work counter)
    // must start at zero; the scores are fully rewritten by the scan before the selection reads them.
    cudaError_t e = cudaMemsetAsync(ws, 0, UCMR_WORKSPACE_HEADER_BYTES, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) { note_cuda_error(e); return UCMR_ERR_LAUNCH; }
    return ucmr_hamming_topk(codes, NB, BS, Hkv, W, q_codes, Hq, block_table, max_blocks, block_table_stride, seq_lens,
                             B, k, k_per_request, request_mask, reduce_mode, reduce_kvhead, must_select, n_must,
                             sink_tokens, recent_tokens, out_physical, out_logical, out_scores, out_valid_count,
                             out_new_seq_lens, ws, kStaticScratchBytes, stream);
}

// Version, status strings and the per-thread record of the last CUDA runtime error.
#include <string.h>

#include "common.cuh"

namespace ucmr {

static thread_local char g_last_error[256] = "";

void note_cuda_error(cudaError_t e)
{
    const char* s = cudaGetErrorString(e);
    strncpy(g_last_error, s ? s : "unknown CUDA error", sizeof(g_last_error) - 1);
    g_last_error[sizeof(g_last_error) - 1] = '\0';
}

}  // namespace ucmr

#ifdef UCMR_TRACE
namespace ucmr {
int trace_read_encode(unsigned long long* host);
int trace_read_scan(unsigned long long* host);
int trace_read_select(unsigned long long* host);
}  // namespace ucmr
#endif

extern "C" int ucmr_trace_read(int unit, unsigned long long* stamps)
{
    if (stamps == nullptr) return UCMR_ERR_BAD_ARG;
#ifdef UCMR_TRACE
    switch (unit) {
        case UCMR_TRACE_ENCODE: return ucmr::trace_read_encode(stamps);
        case UCMR_TRACE_SCAN: return ucmr::trace_read_scan(stamps);
        case UCMR_TRACE_SELECT: return ucmr::trace_read_select(stamps);
        default: return UCMR_ERR_BAD_ARG;
    }
#else
    (void)unit;
    return UCMR_ERR_UNSUPPORTED;
#endif
}

extern "C" int ucmr_version(void) { return UCMR_VERSION; }

extern "C" const char* ucmr_last_cuda_error(void) { return ucmr::g_last_error; }

extern "C" const char* ucmr_status_string(int status)
{
    switch (status) {
        case UCMR_OK: return "ok";
        case UCMR_ERR_BAD_ARG: return "bad argument";
        case UCMR_ERR_UNSUPPORTED: return "unsupported shape or alignment";
        case UCMR_ERR_LAUNCH: return "CUDA launch or runtime call failed";
        case UCMR_ERR_DEVICE: return "a kernel recorded a problem in the status word";
        case UCMR_ERR_WORKSPACE: return "workspace missing or too small";
        default: return "unknown status";
    }
}

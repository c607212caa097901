// nb_gemm_w4a4_noalloc: nb_gemm_w4a4 with its scratch block in a fixed device array of this module, for callers that
// cannot hand the library a scratch allocation.  The kernels are the ones nb_gemm_w4a4 launches; only the origin of
// the scratch pointer differs.  Nothing here allocates or frees device or host memory.
#include <mutex>

#include "nb_common.cuh"

namespace nb {
int record_cuda_error(cudaError_t e);

// One array per device context (the module is loaded once per device).  Every byte a GEMM kernel reads from it is
// written by the same call's pre-pass first, so the contents never have to start at zero and are never cleared.
static __device__ __align__(256) unsigned char g_noalloc_scratch[NB_NOALLOC_SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
static std::mutex g_noalloc_mutex;
static void* g_noalloc_ptr[MAX_DEVICES] = {};

// Address of the array on the current device, looked up once per device.
static int noalloc_scratch(void** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return record_cuda_error(e);
    if (dev < 0 || dev >= MAX_DEVICES) return NB_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (!g_noalloc_ptr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess) return record_cuda_error(e);
        if (!p || (reinterpret_cast<uintptr_t>(p) & 255)) return NB_ERR_INVALID;
        g_noalloc_ptr[dev] = p;
    }
    *out = g_noalloc_ptr[dev];
    return NB_OK;
}
}  // namespace nb

extern "C" int nb_gemm_w4a4_noalloc(const nb_gemm_args* args, const void* epi, int epi_kind, void* stream) {
    if (!args) return NB_ERR_INVALID;
    const int64_t need = nb_gemm_w4a4_scratch_bytes(args, epi, epi_kind);
    if (need < 0) return NB_ERR_INVALID;
    if (need > (int64_t)NB_NOALLOC_SCRATCH_BYTES) return NB_ERR_TOO_LARGE;
    nb_gemm_args a = *args;
    a.scratch = nullptr;
    a.scratch_bytes = 0;
    if (need > 0) {
        void* p = nullptr;
        const int rc = nb::noalloc_scratch(&p);
        if (rc != NB_OK) return rc;
        a.scratch = p;
        a.scratch_bytes = NB_NOALLOC_SCRATCH_BYTES;
    }
    return nb_gemm_w4a4(&a, epi, epi_kind, stream);
}

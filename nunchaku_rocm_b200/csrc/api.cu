// Status strings and launch-error bookkeeping of the C ABI.
#include "nb_common.cuh"

namespace nb {
static thread_local cudaError_t g_last_error = cudaSuccess;
static thread_local const char* g_detail = "";
// one static string saying which check of a launcher refused the call (read by nb_last_error_detail)
int fail_with(int status, const char* detail) {
    g_detail = detail;
    return status;
}
int record_cuda_error(cudaError_t e) {
    g_last_error = e;
    (void)cudaGetLastError();  // clear the sticky-less error so the next launch starts clean
    return NB_ERR_LAUNCH;
}
}  // namespace nb

extern "C" const char* nb_strerror(int status) {
    switch (status) {
        case NB_OK: return "ok";
        case NB_ERR_INVALID: return "invalid argument (shape, alignment or null pointer)";
        case NB_ERR_UNSUPPORTED: return "unsupported call for the selected kernel";
        case NB_ERR_LAUNCH: return "CUDA launch error";
        case NB_ERR_DEVICE: return "a kernel gave up on a bounded wait";
        case NB_ERR_TOO_LARGE: return "size beyond the fixed capacity of this entry point";
        default: return "unknown status";
    }
}
extern "C" int nb_last_cuda_error(void) {
    int e = (int)nb::g_last_error;
    nb::g_last_error = cudaSuccess;
    return e;
}
extern "C" const char* nb_last_cuda_error_string(void) { return cudaGetErrorString(nb::g_last_error); }
extern "C" const char* nb_last_error_detail(void) {
    const char* d = nb::g_detail;
    nb::g_detail = "";
    return d;
}
extern "C" int nb_version(void) { return 101; }
extern "C" int nb_num_sms(void) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return -1;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
    return n;
}

// ------------------------------------------------------------------------------------------------
// nb_debug_expire_wait: the bounded-wait path of the kernels, exercised on purpose.  One warp waits on an mbarrier that
// nothing will ever arrive on, with the limit the caller gives; the wait gives up after that time, the kernel stores the
// code in *status exactly as the GEMM and attention kernels do, and returns.  Nothing spins beyond the limit and the
// context stays usable.
// ------------------------------------------------------------------------------------------------
namespace nb {
__global__ void expire_wait_kernel(int* status, unsigned long long limit_ns, int code) {
    __shared__ uint64_t barrier;
    __shared__ int abort_word;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&barrier), 1);
        abort_word = 0;
        fence_barrier_init();
    }
    __syncthreads();
    bool ok = true;
    if (threadIdx.x == 0) ok = mbar_wait(smem_u32(&barrier), 0, &abort_word, code, 200, limit_ns);
    __syncthreads();
    if (threadIdx.x == 0 && !ok && status) atomicCAS(status, 0, abort_word);
}
}  // namespace nb

extern "C" int nb_debug_expire_wait(void* status, int64_t limit_us, void* stream) {
    if (!status || limit_us < 1 || limit_us > 1000000) return NB_ERR_INVALID;  // at most one second
    nb::expire_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<int*>(status),
                                                                             (unsigned long long)limit_us * 1000ull, 0x7E1);
    NB_CUDA_CHECK(cudaGetLastError());
    return NB_OK;
}

// Status strings and launch-error bookkeeping of the C ABI.
#include "nb_common.cuh"

namespace nb {
static thread_local cudaError_t g_last_error = cudaSuccess;
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
extern "C" int nb_version(void) { return 100; }
extern "C" int nb_num_sms(void) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return -1;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
    return n;
}

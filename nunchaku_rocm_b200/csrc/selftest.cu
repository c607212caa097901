// nb_selftest: the tensor-core and the generic W4A4 kernels against each other on small seeded problems (int4 with and
// without load-time prepared weights, NVFP4 on the wide tile).
#include <cmath>
#include <cstring>
#include <vector>

#include "nb_common.cuh"

namespace nb {
int record_cuda_error(cudaError_t e);
namespace {
struct DevBuf {
    void* p = nullptr;
    ~DevBuf() { if (p) cudaFree(p); }
    cudaError_t alloc(size_t n) { return cudaMalloc(&p, n); }
};
uint32_t lcg(uint32_t& s) { s = s * 1664525u + 1013904223u; return s >> 8; }
uint16_t bf16_of(float f) {  // round to nearest even
    uint32_t u;
    memcpy(&u, &f, 4);
    return (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}
float f32_of(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
bool close_bf16(const std::vector<uint16_t>& a, const std::vector<uint16_t>& b) {
    for (size_t i = 0; i < a.size(); ++i) {
        const float x = f32_of(a[i]), y = f32_of(b[i]);
        if (!(fabsf(x - y) <= 2.0f * 0.0078125f * fmaxf(fabsf(x), fabsf(y)) + 1e-3f)) return false;
    }
    return true;
}

// NVFP4: 136 x 512 x 512, rank 16, per-channel scales and alpha: the block-scaled kernel (128 x 256 tile) against the generic one
int selftest_fp4() {
    constexpr int M = 136, N = 512, K = 512, R = 16, G = K / 16;
    uint32_t seed = 777u;
    std::vector<uint8_t> act((size_t)M * K / 2), wgt((size_t)N * K / 2), asc((size_t)G * M), wsc((size_t)G * N);
    for (auto& b : act) b = (uint8_t)lcg(seed);
    for (auto& b : wgt) b = (uint8_t)lcg(seed);
    for (auto& b : asc) b = (uint8_t)(0x28 + lcg(seed) % 0x18);  // e4m3 0.0625 .. 1.75
    for (auto& b : wsc) b = (uint8_t)(0x20 + lcg(seed) % 0x18);
    std::vector<uint16_t> bias(N), wcs(N), lu((size_t)N * R);
    for (auto& v : bias) v = bf16_of(((int)(lcg(seed) % 2001) - 1000) * 1e-2f);
    for (auto& v : wcs) v = bf16_of(0.5f + (lcg(seed) % 1000) * 5e-4f);
    for (auto& v : lu) v = bf16_of(((int)(lcg(seed) % 2001) - 1000) * 2e-4f);
    std::vector<float> la((size_t)M * R);
    for (auto& v : la) v = ((int)(lcg(seed) % 2001) - 1000) * 1e-2f;
    DevBuf d_act, d_wgt, d_asc, d_wsc, d_bias, d_wcs, d_lu, d_la, d_out[2], d_status;
    struct Up { DevBuf* b; const void* h; size_t n; } ups[] = {
        {&d_act, act.data(), act.size()}, {&d_wgt, wgt.data(), wgt.size()}, {&d_asc, asc.data(), asc.size()},
        {&d_wsc, wsc.data(), wsc.size()}, {&d_bias, bias.data(), bias.size() * 2}, {&d_wcs, wcs.data(), wcs.size() * 2},
        {&d_lu, lu.data(), lu.size() * 2}, {&d_la, la.data(), la.size() * 4}};
    cudaError_t e;
    for (auto& u : ups) {
        e = u.b->alloc(u.n);
        if (e == cudaSuccess) e = cudaMemcpy(u.b->p, u.h, u.n, cudaMemcpyHostToDevice);
        if (e != cudaSuccess) return record_cuda_error(e);
    }
    e = d_status.alloc(4);
    if (e == cudaSuccess) e = cudaMemset(d_status.p, 0, 4);
    if (e != cudaSuccess) return record_cuda_error(e);
    nb_gemm_args a = {};
    a.act = d_act.p; a.wgt = d_wgt.p; a.ascales = d_asc.p; a.wscales = d_wsc.p; a.bias = d_bias.p; a.wcscales = d_wcs.p;
    a.lora_act = d_la.p; a.lora_up = d_lu.p;
    a.M = M; a.N = N; a.K = K; a.actual_m = M; a.R = R; a.dtype = NB_DTYPE_BF16; a.fp4 = 1; a.alpha = 0.75f;
    a.stride_am = K / 2; a.stride_wn = K / 2; a.stride_asg = M; a.stride_wsg = N; a.stride_om = N;
    a.stride_lam = R; a.stride_lun = R; a.status = d_status.p;
    const int impls[2] = {NB_IMPL_TCGEN05, NB_IMPL_GENERIC};
    std::vector<uint16_t> o[2] = {std::vector<uint16_t>((size_t)M * N), std::vector<uint16_t>((size_t)M * N)};
    for (int i = 0; i < 2; ++i) {
        e = d_out[i].alloc((size_t)M * N * 2);
        if (e != cudaSuccess) return record_cuda_error(e);
        a.impl = impls[i];
        a.out = d_out[i].p;
        const int64_t need = nb_gemm_w4a4_scratch_bytes(&a, nullptr, NB_EPI_STORE);
        DevBuf scratch;
        if (need > 0 && (e = scratch.alloc((size_t)need)) != cudaSuccess) return record_cuda_error(e);
        a.scratch = scratch.p; a.scratch_bytes = need;
        const int st = nb_gemm_w4a4(&a, nullptr, NB_EPI_STORE, nullptr);
        e = cudaDeviceSynchronize();
        if (st != NB_OK) return st;
        if (e == cudaSuccess) e = cudaMemcpy(o[i].data(), d_out[i].p, o[i].size() * 2, cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) return record_cuda_error(e);
    }
    int status = 0;
    e = cudaMemcpy(&status, d_status.p, 4, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return record_cuda_error(e);
    return (status == 0 && close_bf16(o[0], o[1])) ? NB_OK : NB_ERR_DEVICE;
}
}  // namespace
}  // namespace nb

extern "C" int nb_selftest(void) {
    using namespace nb;
    constexpr int M = 136, N = 264, K = 256, R = 16, G = K / 64;
    uint32_t seed = 12345u;
    std::vector<uint8_t> act((size_t)M * K / 2), wgt((size_t)N * K / 2);
    for (auto& b : act) b = (uint8_t)lcg(seed);
    for (auto& b : wgt) b = (uint8_t)lcg(seed);
    std::vector<uint16_t> asc((size_t)G * M), wsc((size_t)G * N), bias(N), lu((size_t)N * R);
    for (auto& v : asc) v = bf16_of(0.05f + (lcg(seed) % 1000) * 1e-4f);
    for (auto& v : wsc) v = bf16_of(0.005f + (lcg(seed) % 1000) * 1e-5f);
    for (auto& v : bias) v = bf16_of(((int)(lcg(seed) % 2001) - 1000) * 1e-3f);
    for (auto& v : lu) v = bf16_of(((int)(lcg(seed) % 2001) - 1000) * 2e-5f);
    std::vector<float> la((size_t)M * R);
    for (auto& v : la) v = ((int)(lcg(seed) % 2001) - 1000) * 1e-3f;

    DevBuf d_act, d_wgt, d_asc, d_wsc, d_bias, d_lu, d_la, d_out[2], d_p[2], d_scratch, d_status;
    struct Up { DevBuf* b; const void* h; size_t n; } ups[] = {
        {&d_act, act.data(), act.size()}, {&d_wgt, wgt.data(), wgt.size()}, {&d_asc, asc.data(), asc.size() * 2},
        {&d_wsc, wsc.data(), wsc.size() * 2}, {&d_bias, bias.data(), bias.size() * 2}, {&d_lu, lu.data(), lu.size() * 2},
        {&d_la, la.data(), la.size() * 4}};
    for (auto& u : ups) {
        cudaError_t e = u.b->alloc(u.n);
        if (e == cudaSuccess) e = cudaMemcpy(u.b->p, u.h, u.n, cudaMemcpyHostToDevice);
        if (e != cudaSuccess) return record_cuda_error(e);
    }
    for (int i = 0; i < 2; ++i) {
        cudaError_t e = d_out[i].alloc((size_t)M * N * 2);
        if (e == cudaSuccess) e = d_p[i].alloc((size_t)G * M * N * 4);
        if (e != cudaSuccess) return record_cuda_error(e);
    }
    cudaError_t e = d_status.alloc(4);
    if (e == cudaSuccess) e = cudaMemset(d_status.p, 0, 4);
    if (e != cudaSuccess) return record_cuda_error(e);

    nb_gemm_args a = {};
    a.act = d_act.p; a.wgt = d_wgt.p; a.ascales = d_asc.p; a.wscales = d_wsc.p; a.bias = d_bias.p;
    a.lora_act = d_la.p; a.lora_up = d_lu.p;
    a.M = M; a.N = N; a.K = K; a.actual_m = M; a.R = R; a.dtype = NB_DTYPE_BF16; a.alpha = 1.0f;
    a.stride_am = K / 2; a.stride_wn = K / 2; a.stride_asg = M; a.stride_wsg = N; a.stride_om = N;
    a.stride_lam = R; a.stride_lun = R; a.status = d_status.p;
    const int impls[2] = {NB_IMPL_TCGEN05, NB_IMPL_GENERIC};
    for (int i = 0; i < 2; ++i) {
        a.impl = impls[i];
        a.out = d_out[i].p;
        const int64_t need = nb_gemm_w4a4_scratch_bytes(&a, nullptr, NB_EPI_STORE);
        DevBuf scratch;
        if (need > 0) {
            e = scratch.alloc((size_t)need);
            if (e != cudaSuccess) return record_cuda_error(e);
        }
        a.scratch = scratch.p; a.scratch_bytes = need;
        int st = nb_gemm_w4a4(&a, nullptr, NB_EPI_STORE, nullptr);
        if (st == NB_OK) st = nb_gemm_w4a4_group_sums(&a, static_cast<int32_t*>(d_p[i].p), nullptr);
        e = cudaDeviceSynchronize();
        if (st != NB_OK) return st;
        if (e != cudaSuccess) return record_cuda_error(e);
    }
    int status = 0;
    std::vector<uint16_t> o0((size_t)M * N), o1((size_t)M * N);
    std::vector<int32_t> p0((size_t)G * M * N), p1((size_t)G * M * N);
    e = cudaMemcpy(&status, d_status.p, 4, cudaMemcpyDeviceToHost);
    if (e == cudaSuccess) e = cudaMemcpy(o0.data(), d_out[0].p, o0.size() * 2, cudaMemcpyDeviceToHost);
    if (e == cudaSuccess) e = cudaMemcpy(o1.data(), d_out[1].p, o1.size() * 2, cudaMemcpyDeviceToHost);
    if (e == cudaSuccess) e = cudaMemcpy(p0.data(), d_p[0].p, p0.size() * 4, cudaMemcpyDeviceToHost);
    if (e == cudaSuccess) e = cudaMemcpy(p1.data(), d_p[1].p, p1.size() * 4, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return record_cuda_error(e);
    if (status != 0) return NB_ERR_DEVICE;
    if (p0 != p1) return NB_ERR_DEVICE;
    if (!close_bf16(o0, o1)) return NB_ERR_DEVICE;

    // the same call with the weights prepared once: bit-identical to the call that widened them itself
    {
        a.impl = NB_IMPL_TCGEN05;
        const int64_t pbytes = nb_gemm_w4a4_prepared_bytes(&a);
        if (pbytes <= 0) return NB_ERR_DEVICE;
        DevBuf prep, scratch, out2;
        e = prep.alloc((size_t)pbytes);
        if (e == cudaSuccess) e = out2.alloc((size_t)M * N * 2);
        if (e != cudaSuccess) return record_cuda_error(e);
        int st = nb_gemm_w4a4_prepare_weights(&a, prep.p, pbytes, nullptr);
        if (st != NB_OK) return st;
        a.wgt_prepared = prep.p; a.wgt_prepared_bytes = pbytes;
        a.out = out2.p;
        const int64_t need = nb_gemm_w4a4_scratch_bytes(&a, nullptr, NB_EPI_STORE);
        if (need > 0 && (e = scratch.alloc((size_t)need)) != cudaSuccess) return record_cuda_error(e);
        a.scratch = scratch.p; a.scratch_bytes = need;
        st = nb_gemm_w4a4(&a, nullptr, NB_EPI_STORE, nullptr);
        e = cudaDeviceSynchronize();
        if (st != NB_OK) return st;
        std::vector<uint16_t> o2((size_t)M * N);
        if (e == cudaSuccess) e = cudaMemcpy(o2.data(), out2.p, o2.size() * 2, cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) return record_cuda_error(e);
        if (o2 != o0) return NB_ERR_DEVICE;
    }
    return selftest_fp4();
}

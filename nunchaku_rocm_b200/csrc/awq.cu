// AWQ W4A16: streaming dequant-GEMV for small batches (HBM-bound) and the dense dequantiser.
//
// Weight layout (TinyChat, reference: nunchaku/ops/triton/awq.py:8-18 and 28-46): the packed tensor is
// int16 B[n/4, k]; stored column e = c*64 + b*16 + d of packed row a holds, in nibble m (bits 4m..4m+3),
// the logical element (n, k) = (4a + b, 64c + (d/8)*32 + 8m + d%8).  One aligned group of 8 stored
// int16 (16 bytes) therefore is 32 consecutive logical k of ONE output channel, inside ONE scale group:
// k = 64c + 32h + 8m + j, j = 0..7 the int16 index, h = (d/8).
//
// Arithmetic (awq.py:121-183): out[row, n] = sum_c ( s[c,n] * sum_{k in c} x[k] q[n,k] + z[c,n] * sum_{k in c} x[k] ),
// fp32 accumulation, one rounding to T.  A nibble becomes the fp32 value 128 + q by OR-ing it into the
// mantissa of 128.0f (exact), so the inner loop is one shift, one logic op and one FMA per element and the
// 128 is folded into the zero-point term: s*(sum (128+q) x) + (z - 128 s) * sum x.
#include "nb_common.cuh"

namespace nb {
namespace {

template <typename T, int MR>
__global__ void __launch_bounds__(256) awq_gemv_kernel(const T* __restrict__ x, const uint16_t* __restrict__ kernel,
                                                       const T* __restrict__ scales, const T* __restrict__ zeros,
                                                       T* __restrict__ out, int m, int n, int k, long long stride_xm,
                                                       long long stride_kn, long long stride_sg, long long stride_om) {
    extern __shared__ float xs[];  // [MR][k] activations in fp32
    for (int i = threadIdx.x; i < MR * k; i += 256) {
        const int r = i / k, c = i - r * k;
        xs[i] = r < m ? to_f32<T>(x[(long long)r * stride_xm + c]) : 0.f;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int a = blockIdx.x * 8 + warp;
    if (a >= n / 4) return;
    const uint4* row = reinterpret_cast<const uint4*>(kernel + (long long)a * stride_kn);
    const int b = (lane >> 1) & 3, h = lane & 1;
    const int ncol = 4 * a + b;

    float acc[MR];
#pragma unroll
    for (int r = 0; r < MR; ++r) acc[r] = 0.f;

    for (int e0 = lane * 8; e0 < k; e0 += 256) {
        const uint4 w4 = __ldg(row + (e0 >> 3));
        const int c = e0 >> 6;
        const int kbase = 64 * c + 32 * h;
        const uint32_t w[4] = {w4.x, w4.y, w4.z, w4.w};
        const float s = to_f32<T>(scales[(long long)c * stride_sg + ncol]);
        const float z = to_f32<T>(zeros[(long long)c * stride_sg + ncol]);
        float dot[MR], xsum[MR];
#pragma unroll
        for (int r = 0; r < MR; ++r) dot[r] = xsum[r] = 0.f;
#pragma unroll
        for (int m4 = 0; m4 < 4; ++m4) {
            float q[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                // nibble m4 of int16 j -> bits 16..19 of the fp32 pattern of 128.0f
                const int sh = 16 * (j & 1) + 4 * m4;
                const uint32_t bits = sh <= 16 ? (w[j >> 1] << (16 - sh)) : (w[j >> 1] >> (sh - 16));
                q[j] = __uint_as_float((bits & 0x000F0000u) | 0x43000000u);
            }
#pragma unroll
            for (int r = 0; r < MR; ++r) {
                const float4 x0 = *reinterpret_cast<const float4*>(xs + r * k + kbase + 8 * m4);
                const float4 x1 = *reinterpret_cast<const float4*>(xs + r * k + kbase + 8 * m4 + 4);
                dot[r] = fmaf(q[0], x0.x, dot[r]); dot[r] = fmaf(q[1], x0.y, dot[r]);
                dot[r] = fmaf(q[2], x0.z, dot[r]); dot[r] = fmaf(q[3], x0.w, dot[r]);
                dot[r] = fmaf(q[4], x1.x, dot[r]); dot[r] = fmaf(q[5], x1.y, dot[r]);
                dot[r] = fmaf(q[6], x1.z, dot[r]); dot[r] = fmaf(q[7], x1.w, dot[r]);
                xsum[r] += ((x0.x + x0.y) + (x0.z + x0.w)) + ((x1.x + x1.y) + (x1.z + x1.w));
            }
        }
        const float zc = z - 128.0f * s;
#pragma unroll
        for (int r = 0; r < MR; ++r) acc[r] += s * dot[r] + zc * xsum[r];
    }
    // lanes sharing an output channel differ in bit 0 (h) and bits 3, 4 (scale group within the 256-wide step)
#pragma unroll
    for (int r = 0; r < MR; ++r) {
        float v = acc[r];
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 8);
        v += __shfl_xor_sync(0xffffffffu, v, 16);
        if ((lane & 0x19) == 0 && r < m) out[(long long)r * stride_om + ncol] = from_f32<T>(v);
    }
}

template <typename T>
__global__ void __launch_bounds__(256) awq_dequant_kernel(const uint16_t* __restrict__ kernel,
                                                          const T* __restrict__ scales, const T* __restrict__ zeros,
                                                          T* __restrict__ out, int n, int k, int group,
                                                          long long stride_kn, long long stride_sg,
                                                          long long stride_on) {
    const long long unit = (long long)blockIdx.x * 256 + threadIdx.x;  // 16-byte units of the packed tensor
    const int upr = k / 8;
    if (unit >= (long long)(n / 4) * upr) return;
    const int a = (int)(unit / upr), e0 = (int)(unit % upr) * 8;
    const uint4 w4 = __ldg(reinterpret_cast<const uint4*>(kernel + (long long)a * stride_kn + e0));
    const uint32_t w[4] = {w4.x, w4.y, w4.z, w4.w};
    const int c = e0 >> 6, b = (e0 >> 4) & 3, h = (e0 >> 3) & 1;
    const int ncol = 4 * a + b;
    T* orow = out + (long long)ncol * stride_on;
#pragma unroll
    for (int m4 = 0; m4 < 4; ++m4) {
        const int k0 = 64 * c + 32 * h + 8 * m4;
        const int g = k0 / group;
        const float s = to_f32<T>(scales[(long long)g * stride_sg + ncol]);
        const float z = to_f32<T>(zeros[(long long)g * stride_sg + ncol]);
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = (float)((w[j >> 1] >> (16 * (j & 1) + 4 * m4)) & 0xF) * s + z;
        uint4 o;
        o.x = pack2<T>(v[0], v[1]); o.y = pack2<T>(v[2], v[3]); o.z = pack2<T>(v[4], v[5]); o.w = pack2<T>(v[6], v[7]);
        *reinterpret_cast<uint4*>(orow + k0) = o;
    }
}

template <typename T, int MR>
int launch_gemv_t(const void* x, const void* kernel, const void* scales, const void* zeros, void* out, int m, int n,
                  int k, long long sxm, long long skn, long long ssg, long long som, cudaStream_t s) {
    const size_t smem = (size_t)MR * k * sizeof(float);
    auto kern = awq_gemv_kernel<T, MR>;
    NB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    kern<<<(n / 4 + 7) / 8, 256, smem, s>>>(static_cast<const T*>(x), static_cast<const uint16_t*>(kernel),
                                            static_cast<const T*>(scales), static_cast<const T*>(zeros),
                                            static_cast<T*>(out), m, n, k, sxm, skn, ssg, som);
    NB_CUDA_CHECK(cudaGetLastError());
    return NB_OK;
}

template <typename T>
int launch_gemv(const void* x, const void* kernel, const void* scales, const void* zeros, void* out, int m, int n,
                int k, long long sxm, long long skn, long long ssg, long long som, cudaStream_t s) {
    // rows are processed in slabs of at most 8 so that the activations stay in shared memory
    for (int r0 = 0; r0 < m; r0 += 8) {
        const int mr = min(8, m - r0);
        const T* xr = static_cast<const T*>(x) + (long long)r0 * sxm;
        T* outr = static_cast<T*>(out) + (long long)r0 * som;
        int st;
        if (mr == 1) st = launch_gemv_t<T, 1>(xr, kernel, scales, zeros, outr, mr, n, k, sxm, skn, ssg, som, s);
        else if (mr == 2) st = launch_gemv_t<T, 2>(xr, kernel, scales, zeros, outr, mr, n, k, sxm, skn, ssg, som, s);
        else if (mr <= 4) st = launch_gemv_t<T, 4>(xr, kernel, scales, zeros, outr, mr, n, k, sxm, skn, ssg, som, s);
        else st = launch_gemv_t<T, 8>(xr, kernel, scales, zeros, outr, mr, n, k, sxm, skn, ssg, som, s);
        if (st != NB_OK) return st;
    }
    return NB_OK;
}

}  // namespace
}  // namespace nb

extern "C" int nb_awq_gemv(const void* x, const void* kernel, const void* scales, const void* zeros, void* out,
                           int32_t m, int32_t n, int32_t k, int64_t stride_xm, int64_t stride_kn, int64_t stride_sg,
                           int64_t stride_om, int32_t dtype, void* stream) {
    using namespace nb;
    NB_REQUIRE(x && kernel && scales && zeros && out);
    NB_REQUIRE(m >= 0 && n > 0 && k > 0 && n % 4 == 0 && k % 64 == 0);
    NB_REQUIRE(dtype == NB_DTYPE_BF16 || dtype == NB_DTYPE_FP16);
    NB_REQUIRE(aligned16(kernel) && stride_kn % 8 == 0);
    if ((size_t)8 * k * 4 > 200 * 1024) return NB_ERR_UNSUPPORTED;
    if (m == 0) return NB_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return dtype == NB_DTYPE_BF16
               ? launch_gemv<__nv_bfloat16>(x, kernel, scales, zeros, out, m, n, k, stride_xm, stride_kn, stride_sg, stride_om, s)
               : launch_gemv<__half>(x, kernel, scales, zeros, out, m, n, k, stride_xm, stride_kn, stride_sg, stride_om, s);
}

extern "C" int nb_awq_dequant(const void* kernel, const void* scales, const void* zeros, void* out, int32_t n,
                              int32_t k, int32_t group, int64_t stride_kn, int64_t stride_sg, int64_t stride_on,
                              int32_t dtype, void* stream) {
    using namespace nb;
    NB_REQUIRE(kernel && scales && zeros && out);
    NB_REQUIRE(n > 0 && k > 0 && n % 4 == 0 && k % 64 == 0 && group >= 8 && group % 8 == 0 && k % group == 0);
    NB_REQUIRE(dtype == NB_DTYPE_BF16 || dtype == NB_DTYPE_FP16);
    NB_REQUIRE(aligned16(kernel) && stride_kn % 8 == 0 && aligned16(out) && stride_on % 8 == 0);
    const long long units = (long long)(n / 4) * (k / 8);
    const int blocks = (int)((units + 255) / 256);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == NB_DTYPE_BF16)
        awq_dequant_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(
            static_cast<const uint16_t*>(kernel), static_cast<const __nv_bfloat16*>(scales),
            static_cast<const __nv_bfloat16*>(zeros), static_cast<__nv_bfloat16*>(out), n, k, group, stride_kn,
            stride_sg, stride_on);
    else
        awq_dequant_kernel<__half><<<blocks, 256, 0, s>>>(
            static_cast<const uint16_t*>(kernel), static_cast<const __half*>(scales),
            static_cast<const __half*>(zeros), static_cast<__half*>(out), n, k, group, stride_kn, stride_sg,
            stride_on);
    NB_CUDA_CHECK(cudaGetLastError());
    return NB_OK;
}

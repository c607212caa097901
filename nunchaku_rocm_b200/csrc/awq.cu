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
#include <type_traits>

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

// ------------------------------------------------------------------------------------------------
// Batches of up to 8 rows on mma.sync.m16n8k16: the HBM stream of the weights is the only large cost.
//
// A warp owns 16 output channels (4 packed rows x 4) and a contiguous range of 64-wide scale groups.  The weights are
// the A operand (16 channels x 16 k), the activations the B operand (16 k x 8 batch rows).  A dot product does not see
// a permutation of k applied to both operands, so the k-slots of an MMA are chosen to fit the packing: the four lanes
// of a quad read the 32 contiguous bytes that hold one channel's 64 k of a group (8 bytes each), and MMA i of the group
// (i = 0..3) takes nibble i of every int16: slot 2 t + {0, 1} and 2 t + 8 + {0, 1} of lane t are
// k = 64 c + 32 (t >> 1) + 8 i + 4 (t & 1) + {0, 1, 2, 3}.  A nibble pair becomes two 16-bit floats OFF + q by one
// shift and one logic operation (OFF = 128 for bf16, 1024 for fp16; exact), and OFF is folded into the zero-point term:
// out = sum_c s (sum (OFF + q) x) + (z - OFF s) sum x.  The per-group sums of x come from a fifth MMA per step whose A
// operand is all ones; the activations (as T) are staged in shared memory once per CTA.
// A CTA is 8 warps = (8 / KS) channel blocks x KS group ranges; the KS partial results are added in a fixed order.
// The first weight loads are issued before the staging so that the two latencies overlap.
// ------------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void mma16816_f32(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816_f32<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816_f32<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

constexpr int GV_UNROLL = 4;  // scale groups per batch; two batches of loads are in flight
constexpr int GV_WARPS = 8;

template <typename T, int KS>
__global__ void __launch_bounds__(GV_WARPS * 32) awq_gemv_mma_kernel(const T* __restrict__ x, const uint16_t* __restrict__ kernel,
                                                                     const T* __restrict__ scales, const T* __restrict__ zeros,
                                                                     T* __restrict__ out, int m, int n, int k, long long stride_xm,
                                                                     long long stride_kn, long long stride_sg, long long stride_om) {
    constexpr int CB = GV_WARPS / KS;  // channel blocks (of 16) per CTA
    constexpr int CH = 16 * CB;        // channels per CTA
    constexpr int NT = GV_WARPS * 32;
    constexpr bool BF = std::is_same<T, __nv_bfloat16>::value;
    constexpr uint32_t MAGIC2 = BF ? 0x43004300u : 0x64006400u;  // OFF twice, as T
    constexpr uint32_t ONE2 = BF ? 0x3F803F80u : 0x3C003C00u;    // 1.0 twice, as T
    constexpr float OFF = BF ? 128.0f : 1024.0f;
    const int G = k / 64, KP = k + 8;  // padded row of the staged activations (elements)
    extern __shared__ __align__(16) uint8_t gv_smem[];
    T* xs = reinterpret_cast<T*>(gv_smem);  // [8][KP]
    const int ch0 = blockIdx.x * CH;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gid = lane >> 2, tig = lane & 3;
    const int cb = warp % CB, ks = warp / CB;
    const int gpw = (G + KS - 1) / KS;  // groups per warp
    const int c_begin = ks * gpw, c_end = min(G, c_begin + gpw);
    // MMA rows gid and gid + 8 of this lane are the ADJACENT channels ch0 + 16 cb + 2 gid + {0, 1} (any assignment of
    // rows to channels is allowed), so that one 32-bit load fetches both channels' scales; packed row ch / 4, block ch % 4
    const int chA = ch0 + 16 * cb + 2 * gid, chB = chA + 1;
    const bool okA = chA < n, okB = chB < n;
    const uint16_t* rowA = kernel + (long long)(chA >> 2) * stride_kn + (chA & 3) * 16 + 4 * tig;
    const uint16_t* rowB = kernel + (long long)(chB >> 2) * stride_kn + (chB & 3) * 16 + 4 * tig;
    const T* xlane = xs + gid * KP + 32 * (tig >> 1) + 4 * (tig & 1);  // + 64 c + 8 i
    const bool pair_ok = okB && ((reinterpret_cast<uintptr_t>(scales) | reinterpret_cast<uintptr_t>(zeros)) & 3) == 0 &&
                         (stride_sg & 1) == 0;  // chA is even: the pair is 4-byte aligned when the rows are

    // weights and scale / zero pairs of a batch of groups
    struct Batch { uint2 wa[GV_UNROLL], wb[GV_UNROLL]; uint32_t s2[GV_UNROLL], z2[GV_UNROLL]; };
    auto load_batch = [&](Batch& bt, int c0) {
#pragma unroll
        for (int u = 0; u < GV_UNROLL; ++u) {
            const int c = c0 + u;
            const bool in = c < c_end;
            bt.wa[u] = in && okA ? __ldg(reinterpret_cast<const uint2*>(rowA + c * 64)) : make_uint2(0, 0);
            bt.wb[u] = in && okB ? __ldg(reinterpret_cast<const uint2*>(rowB + c * 64)) : make_uint2(0, 0);
            const unsigned short* sp = reinterpret_cast<const unsigned short*>(scales) + (long long)c * stride_sg + chA;
            const unsigned short* zp = reinterpret_cast<const unsigned short*>(zeros) + (long long)c * stride_sg + chA;
            if (in && pair_ok) {
                bt.s2[u] = __ldg(reinterpret_cast<const uint32_t*>(sp));
                bt.z2[u] = __ldg(reinterpret_cast<const uint32_t*>(zp));
            } else {
                bt.s2[u] = (in && okA ? (uint32_t)__ldg(sp) : 0u) | (in && okB ? (uint32_t)__ldg(sp + 1) << 16 : 0u);
                bt.z2[u] = (in && okA ? (uint32_t)__ldg(zp) : 0u) | (in && okB ? (uint32_t)__ldg(zp + 1) << 16 : 0u);
            }
        }
    };
    Batch b0, b1;
    load_batch(b0, c_begin);
    load_batch(b1, c_begin + GV_UNROLL);

    // ---- stage the activations as T (rows >= m are zero)
    for (int i = threadIdx.x; i < 8 * (k / 8); i += NT) {
        const int r = i / (k / 8), c8 = (i % (k / 8)) * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < m) v = __ldg(reinterpret_cast<const uint4*>(x + (long long)r * stride_xm + c8));
        *reinterpret_cast<uint4*>(xs + r * KP + c8) = v;
    }
    __syncthreads();

    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    auto compute = [&](const Batch& bt, int c0) {
#pragma unroll
        for (int u = 0; u < GV_UNROLL; ++u) {
            const int c = c0 + u;
            if (c < c_end) {
                float d[4] = {0.f, 0.f, 0.f, 0.f}, ones[4] = {0.f, 0.f, 0.f, 0.f};
                const uint32_t a1[4] = {ONE2, ONE2, ONE2, ONE2};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint32_t a[4];
                    a[0] = ((bt.wa[u].x >> (4 * i)) & 0x000F000Fu) | MAGIC2;
                    a[1] = ((bt.wb[u].x >> (4 * i)) & 0x000F000Fu) | MAGIC2;
                    a[2] = ((bt.wa[u].y >> (4 * i)) & 0x000F000Fu) | MAGIC2;
                    a[3] = ((bt.wb[u].y >> (4 * i)) & 0x000F000Fu) | MAGIC2;
                    const uint2 b = *reinterpret_cast<const uint2*>(xlane + 64 * c + 8 * i);
                    mma16816_f32<T>(d, a, b.x, b.y);
                    mma16816_f32<T>(ones, a1, b.x, b.y);  // every row: the sum of the group's activations per batch row
                }
                // d[0..1]: channel A x batch rows 2 tig, 2 tig + 1; d[2..3]: channel B; ones[0..1]: the activation sums
                const float2 sf = unpack2<T>(bt.s2[u]), zf = unpack2<T>(bt.z2[u]);
                const float zA = zf.x - OFF * sf.x, zB = zf.y - OFF * sf.y;
                acc[0] += sf.x * d[0] + zA * ones[0];
                acc[1] += sf.x * d[1] + zA * ones[1];
                acc[2] += sf.y * d[2] + zB * ones[0];
                acc[3] += sf.y * d[3] + zB * ones[1];
            }
        }
    };
    // two batches in flight: while one is multiplied the next one's loads are outstanding
    for (int c0 = c_begin; c0 < c_end; c0 += 2 * GV_UNROLL) {
        compute(b0, c0);
        load_batch(b0, c0 + 2 * GV_UNROLL);
        compute(b1, c0 + GV_UNROLL);
        load_batch(b1, c0 + 3 * GV_UNROLL);
    }

    // ---- fixed-order sum over the KS group ranges, then the store
    __syncthreads();  // the staged activations are dead; reuse their memory: [warp][16][8]
    float* red = reinterpret_cast<float*>(gv_smem);
    {
        float* mine = red + warp * 128;
        // stored by channel inside the block: 2 gid and 2 gid + 1
        mine[(2 * gid) * 8 + 2 * tig] = acc[0];
        mine[(2 * gid) * 8 + 2 * tig + 1] = acc[1];
        mine[(2 * gid + 1) * 8 + 2 * tig] = acc[2];
        mine[(2 * gid + 1) * 8 + 2 * tig + 1] = acc[3];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < CH * 8; i += NT) {
        const int r = i / CH, chl = i % CH;  // consecutive threads -> consecutive channels of one batch row
        const int cbl = chl >> 4, row = chl & 15;
        float v = 0.f;
#pragma unroll
        for (int q = 0; q < KS; ++q) v += red[(q * CB + cbl) * 128 + row * 8 + r];
        if (r < m && ch0 + chl < n) out[(long long)r * stride_om + ch0 + chl] = from_f32<T>(v);
    }
}

template <typename T, int KS>
int launch_gemv_mma_t(const void* x, const void* kernel, const void* scales, const void* zeros, void* out, int m, int n,
                      int k, long long sxm, long long skn, long long ssg, long long som, cudaStream_t s) {
    constexpr int CH = 16 * (GV_WARPS / KS);
    const int G = k / 64;
    // the staged activations; the reduction buffer of 16 x 128 floats reuses the memory
    size_t smem = (size_t)8 * (k + 8) * 2;
    if (smem < (size_t)GV_WARPS * 128 * sizeof(float)) smem = (size_t)GV_WARPS * 128 * sizeof(float);
    (void)G;
    auto kern = awq_gemv_mma_kernel<T, KS>;
    NB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<(n + CH - 1) / CH, GV_WARPS * 32, smem, s>>>(static_cast<const T*>(x), static_cast<const uint16_t*>(kernel),
                                              static_cast<const T*>(scales), static_cast<const T*>(zeros),
                                              static_cast<T*>(out), m, n, k, sxm, skn, ssg, som);
    NB_CUDA_CHECK(cudaGetLastError());
    return NB_OK;
}

// Shared memory of the tensor-core GEMV for the widest channel block, or 0 when the call does not fit its rules.
inline size_t gemv_mma_smem(int k, int ks) {
    (void)ks;
    const size_t b = (size_t)8 * (k + 8) * 2;
    return b < (size_t)GV_WARPS * 512 ? (size_t)GV_WARPS * 512 : b;
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
    int dev = 0, sms = 0;
    NB_CUDA_CHECK(cudaGetDevice(&dev));
    NB_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    // tensor-core kernel: 16-byte aligned activation rows; a CTA of 8 warps covers (8 / ks) blocks of 16 channels, with
    // ks chosen so that there are about two CTAs per SM
    int ks = 1;
    while (ks < GV_WARPS && 2 * (((n + 15) / 16 + (GV_WARPS / ks) - 1) / (GV_WARPS / ks)) < 3 * sms && ks * 2 <= k / 64) ks *= 2;
    const bool mma_ok = n % 4 == 0 && aligned16(x) && sxm % 8 == 0 && gemv_mma_smem(k, ks) <= 200 * 1024;
    for (int r0 = 0; r0 < m; r0 += 8) {
        const int mr = min(8, m - r0);
        const T* xr = static_cast<const T*>(x) + (long long)r0 * sxm;
        T* outr = static_cast<T*>(out) + (long long)r0 * som;
        int st;
        if (mma_ok) {
            switch (ks) {
                case 1: st = launch_gemv_mma_t<T, 1>(xr, kernel, scales, zeros, outr, mr, n, k, sxm, skn, ssg, som, s); break;
                case 2: st = launch_gemv_mma_t<T, 2>(xr, kernel, scales, zeros, outr, mr, n, k, sxm, skn, ssg, som, s); break;
                case 4: st = launch_gemv_mma_t<T, 4>(xr, kernel, scales, zeros, outr, mr, n, k, sxm, skn, ssg, som, s); break;
                default: st = launch_gemv_mma_t<T, 8>(xr, kernel, scales, zeros, outr, mr, n, k, sxm, skn, ssg, som, s); break;
            }
            if (st != NB_OK) return st;
            continue;
        }
        if (mr == 1) st = launch_gemv_t<T, 1>(xr, kernel, scales, zeros, outr, mr, n, k, sxm, skn, ssg, som, s);
        else if (mr == 2) st = launch_gemv_t<T, 2>(xr, kernel, scales, zeros, outr, mr, n, k, sxm, skn, ssg, som, s);
        else if (mr <= 4) st = launch_gemv_t<T, 4>(xr, kernel, scales, zeros, outr, mr, n, k, sxm, skn, ssg, som, s);
        else st = launch_gemv_t<T, 8>(xr, kernel, scales, zeros, outr, mr, n, k, sxm, skn, ssg, som, s);
        if (st != NB_OK) return st;
    }
    return NB_OK;
}

}  // namespace

// ------------------------------------------------------------------------------------------------
// W4A16 GEMM for larger batches (reference: awq_gemm_w4a16, nunchaku/ops/triton/awq.py:232-251 = dequantise, then a
// dense matmul): one kernel, the weight never exists in dense form outside shared memory.
//
// A CTA owns 128 rows x 128 output channels and walks K in steps of 64.  Per step its 256 threads copy the activations
// (128 x 64 T) to shared memory and each thread widens ONE 16-byte packed unit (32 nibbles of one channel: k = 64 c + 32 h
// + 8 m4 + j) to q * s + z rounded to T, exactly as awq_dequant_kernel does, into the channel-major weight tile.  Eight
// warps (4 along the rows x 2 along the channels, 32 x 64 each) multiply with mma.sync.m16n8k16 (fp32 accumulators) from
// ldmatrix fragments; rows of both tiles are padded by 16 bytes so that the eight rows of an 8 x 8 matrix fall into
// different bank groups.  The next step's global loads are issued before the current step's MMAs.
// ------------------------------------------------------------------------------------------------
constexpr int GM_BM = 128, GM_BN = 128, GM_BK = 64, GM_PITCH = GM_BK + 8;  // pitch in T elements (144 bytes)

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
template <typename T>
__device__ __forceinline__ void mma16816_acc(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if (std::is_same<T, __nv_bfloat16>::value)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename T>
__global__ void __launch_bounds__(256) awq_gemm_kernel(const T* __restrict__ x, const uint16_t* __restrict__ kernel,
                                                       const T* __restrict__ scales, const T* __restrict__ zeros,
                                                       T* __restrict__ out, int m, int n, int k, int group,
                                                       long long stride_xm, long long stride_kn, long long stride_sg,
                                                       long long stride_om) {
    __shared__ __align__(16) T xs[GM_BM * GM_PITCH];
    __shared__ __align__(16) T ws[GM_BN * GM_PITCH];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int m0 = blockIdx.y * GM_BM, n0 = blockIdx.x * GM_BN;
    const int wm = (warp & 3) * 32, wn = (warp >> 2) * 64;  // this warp's 32 x 64 corner of the tile

    // this thread's packed unit of a step: packed row a (4 channels), channel b of it, 32-wide half h
    const int ua = tid >> 3, ub = (tid >> 1) & 3, uh = tid & 1;
    const int ch = 4 * ua + ub;                      // channel inside the tile
    const bool ch_ok = n0 + ch < n;
    const uint16_t* wsrc = kernel + (long long)(n0 / 4 + ua) * stride_kn + 16 * ub + 8 * uh;
    // this thread's activation units of a step: row tid / 2, 32-element half tid % 2 (four 16-byte units)
    const int xr = tid >> 1, xh = tid & 1;
    const bool x_ok = m0 + xr < m;
    const T* xsrc = x + (long long)(m0 + xr) * stride_xm + 32 * xh;

    float acc[2][8][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;

    uint4 wreg = make_uint4(0, 0, 0, 0), xreg[4];
    float sc = 0.f, zp = 0.f;
    auto fetch = [&](int c) {
        wreg = ch_ok ? __ldg(reinterpret_cast<const uint4*>(wsrc + 64 * c)) : make_uint4(0, 0, 0, 0);
        const int g = (64 * c + 32 * uh) / group;
        sc = ch_ok ? to_f32<T>(__ldg(scales + (long long)g * stride_sg + n0 + ch)) : 0.f;
        zp = ch_ok ? to_f32<T>(__ldg(zeros + (long long)g * stride_sg + n0 + ch)) : 0.f;
#pragma unroll
        for (int u = 0; u < 4; ++u)
            xreg[u] = x_ok ? __ldg(reinterpret_cast<const uint4*>(xsrc + 64 * c) + u) : make_uint4(0, 0, 0, 0);
    };
    const int steps = k / GM_BK;
    fetch(0);
    for (int c = 0; c < steps; ++c) {
        __syncthreads();  // the previous step's fragments have been read
        {
            const uint32_t w[4] = {wreg.x, wreg.y, wreg.z, wreg.w};
#pragma unroll
            for (int m4 = 0; m4 < 4; ++m4) {
                float v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = (float)((w[j >> 1] >> (16 * (j & 1) + 4 * m4)) & 0xF) * sc + zp;
                uint4 o;
                o.x = pack2<T>(v[0], v[1]); o.y = pack2<T>(v[2], v[3]); o.z = pack2<T>(v[4], v[5]); o.w = pack2<T>(v[6], v[7]);
                *reinterpret_cast<uint4*>(ws + ch * GM_PITCH + 32 * uh + 8 * m4) = o;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) *reinterpret_cast<uint4*>(xs + xr * GM_PITCH + 32 * xh + 8 * u) = xreg[u];
        }
        __syncthreads();
        if (c + 1 < steps) fetch(c + 1);  // in flight during the MMAs
#pragma unroll
        for (int kk = 0; kk < GM_BK; kk += 16) {
            uint32_t a[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i)
                ldmatrix_x4(a[i], smem_u32(xs + (wm + 16 * i + (lane & 15)) * GM_PITCH + kk + 8 * (lane >> 4)));
#pragma unroll
            for (int jp = 0; jp < 4; ++jp) {
                // two 8-channel blocks per load: matrices (channels 0-7, k 0-7), (0-7, k 8-15), (8-15, k 0-7), (8-15, k 8-15)
                uint32_t b[4];
                ldmatrix_x4(b, smem_u32(ws + (wn + 16 * jp + (lane & 7) + 8 * (lane >> 4)) * GM_PITCH + kk + 8 * ((lane >> 3) & 1)));
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    mma16816_acc<T>(acc[i][2 * jp], a[i], b[0], b[1]);
                    mma16816_acc<T>(acc[i][2 * jp + 1], a[i], b[2], b[3]);
                }
            }
        }
    }
    // C fragment: rows gid, gid + 8 of a 16-row block, columns 2 tig + {0, 1} of an 8-column block
    const int gid = lane >> 2, tig = lane & 3;
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int col = n0 + wn + 8 * j + 2 * tig;
            if (col >= n) continue;  // (n is a multiple of 4 and col is even: col + 1 < n as well)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int row = m0 + wm + 16 * i + gid + 8 * h;
                if (row < m)
                    *reinterpret_cast<uint32_t*>(out + (long long)row * stride_om + col) = pack2<T>(acc[i][j][2 * h], acc[i][j][2 * h + 1]);
            }
        }
}

template <typename T>
static int launch_gemm(const void* x, const void* kernel, const void* scales, const void* zeros, void* out, int m, int n, int k,
                       int group, long long sxm, long long skn, long long ssg, long long som, cudaStream_t s) {
    dim3 grid((n + GM_BN - 1) / GM_BN, (m + GM_BM - 1) / GM_BM);
    awq_gemm_kernel<T><<<grid, 256, 0, s>>>(static_cast<const T*>(x), static_cast<const uint16_t*>(kernel),
                                            static_cast<const T*>(scales), static_cast<const T*>(zeros), static_cast<T*>(out), m, n,
                                            k, group, sxm, skn, ssg, som);
    NB_CUDA_CHECK(cudaGetLastError());
    return NB_OK;
}

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

extern "C" int nb_awq_gemm(const void* x, const void* kernel, const void* scales, const void* zeros, void* out, int32_t m,
                           int32_t n, int32_t k, int32_t group, int64_t stride_xm, int64_t stride_kn, int64_t stride_sg,
                           int64_t stride_om, int32_t dtype, void* stream) {
    using namespace nb;
    NB_REQUIRE(x && kernel && scales && zeros && out);
    NB_REQUIRE(m >= 0 && n > 0 && k > 0 && n % 4 == 0 && k % 64 == 0 && group >= 32 && group % 32 == 0 && k % group == 0);
    NB_REQUIRE(dtype == NB_DTYPE_BF16 || dtype == NB_DTYPE_FP16);
    NB_REQUIRE(aligned16(kernel) && stride_kn % 8 == 0 && aligned16(x) && stride_xm % 8 == 0);
    NB_REQUIRE((reinterpret_cast<uintptr_t>(out) & 3) == 0 && stride_om % 2 == 0);
    if (m == 0) return NB_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return dtype == NB_DTYPE_BF16
               ? launch_gemm<__nv_bfloat16>(x, kernel, scales, zeros, out, m, n, k, group, stride_xm, stride_kn, stride_sg, stride_om, s)
               : launch_gemm<__half>(x, kernel, scales, zeros, out, m, n, k, group, stride_xm, stride_kn, stride_sg, stride_om, s);
}

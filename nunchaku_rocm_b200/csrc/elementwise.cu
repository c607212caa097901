// The two element-wise steps that surround every quantised linear layer of a DiT block, each as ONE pass over HBM:
//
//   layernorm_modulate:  out = LayerNorm(x) * (scale[b] + scale_add) + shift[b]      (no affine, eps inside the root)
//   gated_residual:      out = x + gate[b] * (y [+ y2])
//
// The reference runs them as separate torch kernels (AdaLayerNormZero: nunchaku/models/normalization.py:60-159; the
// gated residuals of the blocks: nunchaku/models/transformers/transformer_flux_v2.py:174-343): LayerNorm, a broadcast
// multiply and a broadcast add, each rounding to the 16-bit dtype and each a full trip through HBM.  Here every
// intermediate is rounded to the 16-bit dtype at the same points (so the quantizers that follow see the values the
// reference's sequence gives them), but nothing leaves the registers.  scale / shift / gate are (batch, dim) views with
// an element stride (they are columns of the modulation linear's interleaved [dim, n] output), read through the
// read-only cache.
#include "nb_common.cuh"

namespace nb {
namespace {

struct EwParams {
    const void* x; const void* y; const void* y2; void* out;
    const void* a; const void* b;  // layernorm: scale, shift; gated: gate, unused
    int rows, rows_per_batch, dim;
    long long stride_xr, stride_yr, stride_y2r, stride_or;  // elements between rows
    long long stride_ab, stride_ad;                          // scale / shift / gate: elements between batches, between channels
    float scale_add, eps;
    int vec_ab;  // scale / shift / gate are contiguous along the channels and 16-byte aligned: read them 8 at a time
};

template <typename T>
__device__ __forceinline__ void widen(const uint4& r, float (&v)[8]) {
    float2 f;
    f = unpack2<T>(r.x); v[0] = f.x; v[1] = f.y;
    f = unpack2<T>(r.y); v[2] = f.x; v[3] = f.y;
    f = unpack2<T>(r.z); v[4] = f.x; v[5] = f.y;
    f = unpack2<T>(r.w); v[6] = f.x; v[7] = f.y;
}
template <typename T>
__device__ __forceinline__ float rnd(float v) { return to_f32<T>(from_f32<T>(v)); }  // one rounding to the 16-bit dtype
template <typename T>
__device__ __forceinline__ uint4 narrow(const float (&v)[8]) {
    return make_uint4(pack2<T>(v[0], v[1]), pack2<T>(v[2], v[3]), pack2<T>(v[4], v[5]), pack2<T>(v[6], v[7]));
}

// One CTA of 128 threads per row; a thread keeps U 16-byte units of the row in registers (dim = 128 * 8 * U).
template <typename T, int U>
__global__ void __launch_bounds__(128) layernorm_modulate_kernel(const EwParams p) {
    __shared__ float red[2][4];
    const int row = blockIdx.x, t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int bidx = row / p.rows_per_batch;
    const T* x = static_cast<const T*>(p.x) + (long long)row * p.stride_xr;
    float v[U][8];
    float sum = 0.f;
#pragma unroll
    for (int u = 0; u < U; ++u) {
        widen<T>(__ldg(reinterpret_cast<const uint4*>(x) + u * 128 + t), v[u]);
#pragma unroll
        for (int j = 0; j < 8; ++j) sum += v[u][j];
    }
    auto block_sum = [&](float s, int which) {
#pragma unroll
        for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) red[which][warp] = s;
        __syncthreads();
        return (red[which][0] + red[which][1]) + (red[which][2] + red[which][3]);
    };
    const float mean = block_sum(sum, 0) / (float)p.dim;
    float sq = 0.f;
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float d = v[u][j] - mean;
            sq = fmaf(d, d, sq);
        }
    const float rstd = rsqrtf(block_sum(sq, 1) / (float)p.dim + p.eps);
    const T* sc = static_cast<const T*>(p.a) + (long long)bidx * p.stride_ab;
    const T* sh = static_cast<const T*>(p.b) + (long long)bidx * p.stride_ab;
    T* out = static_cast<T*>(p.out) + (long long)row * p.stride_or;
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int c0 = (u * 128 + t) * 8;
        float o[8], sv[8], hv[8];
        if (p.vec_ab) {
            widen<T>(__ldg(reinterpret_cast<const uint4*>(sc + c0)), sv);
            widen<T>(__ldg(reinterpret_cast<const uint4*>(sh + c0)), hv);
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                sv[j] = to_f32<T>(__ldg(sc + (long long)(c0 + j) * p.stride_ad));
                hv[j] = to_f32<T>(__ldg(sh + (long long)(c0 + j) * p.stride_ad));
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            // layer_norm -> T, scale + scale_add -> T, product -> T, sum -> T
            const float s = rnd<T>(sv[j] + p.scale_add);
            o[j] = rnd<T>(rnd<T>((v[u][j] - mean) * rstd) * s) + hv[j];
        }
        reinterpret_cast<uint4*>(out)[u * 128 + t] = narrow<T>(o);
    }
}

// 16-byte units of the (rows, dim) tensor, grid-stride.
template <typename T>
__global__ void __launch_bounds__(256) gated_residual_kernel(const EwParams p) {
    const int upr = p.dim / 8;
    const long long total = (long long)p.rows * upr;
    for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
        const int row = (int)(i / upr), u = (int)(i % upr);
        const int bidx = row / p.rows_per_batch;
        float xv[8], yv[8], o[8];
        widen<T>(__ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(p.x) + (long long)row * p.stride_xr) + u), xv);
        widen<T>(__ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(p.y) + (long long)row * p.stride_yr) + u), yv);
        if (p.y2) {
            float zv[8];
            widen<T>(__ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(p.y2) + (long long)row * p.stride_y2r) + u), zv);
#pragma unroll
            for (int j = 0; j < 8; ++j) yv[j] = rnd<T>(yv[j] + zv[j]);
        }
        const T* g = static_cast<const T*>(p.a) + (long long)bidx * p.stride_ab + (long long)u * 8 * p.stride_ad;
        float gv[8];
        if (p.vec_ab) {
            widen<T>(__ldg(reinterpret_cast<const uint4*>(g)), gv);
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) gv[j] = to_f32<T>(__ldg(g + (long long)j * p.stride_ad));
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rnd<T>(gv[j] * yv[j]) + xv[j];
        reinterpret_cast<uint4*>(static_cast<T*>(p.out) + (long long)row * p.stride_or)[u] = narrow<T>(o);
    }
}

template <typename T>
int launch_ln(const EwParams& p, cudaStream_t s) {
    switch (p.dim / 1024) {
        case 1: layernorm_modulate_kernel<T, 1><<<p.rows, 128, 0, s>>>(p); break;
        case 2: layernorm_modulate_kernel<T, 2><<<p.rows, 128, 0, s>>>(p); break;
        case 3: layernorm_modulate_kernel<T, 3><<<p.rows, 128, 0, s>>>(p); break;
        case 4: layernorm_modulate_kernel<T, 4><<<p.rows, 128, 0, s>>>(p); break;
        default: return NB_ERR_UNSUPPORTED;
    }
    NB_CUDA_CHECK(cudaGetLastError());
    return NB_OK;
}

}  // namespace
}  // namespace nb

extern "C" int nb_layernorm_modulate(const void* x, const void* scale, const void* shift, void* out, int32_t rows,
                                     int32_t rows_per_batch, int32_t dim, int64_t stride_xr, int64_t stride_or,
                                     int64_t stride_sb, int64_t stride_sd, float scale_add, float eps, int32_t dtype,
                                     void* stream) {
    using namespace nb;
    NB_REQUIRE(x && scale && shift && out);
    NB_REQUIRE(rows >= 0 && rows_per_batch > 0 && dim > 0);
    NB_REQUIRE(dtype == NB_DTYPE_BF16 || dtype == NB_DTYPE_FP16);
    if (dim % 1024 || dim > 4096) return NB_ERR_UNSUPPORTED;
    NB_REQUIRE(aligned16(x) && aligned16(out) && stride_xr % 8 == 0 && stride_or % 8 == 0);
    if (rows == 0) return NB_OK;
    EwParams p = {};
    p.x = x; p.out = out; p.a = scale; p.b = shift;
    p.rows = rows; p.rows_per_batch = rows_per_batch; p.dim = dim;
    p.stride_xr = stride_xr; p.stride_or = stride_or; p.stride_ab = stride_sb; p.stride_ad = stride_sd;
    p.scale_add = scale_add; p.eps = eps;
    p.vec_ab = stride_sd == 1 && stride_sb % 8 == 0 && aligned16(scale) && aligned16(shift);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return dtype == NB_DTYPE_BF16 ? launch_ln<__nv_bfloat16>(p, s) : launch_ln<__half>(p, s);
}

extern "C" int nb_gated_residual(const void* x, const void* gate, const void* y, const void* y2, void* out, int32_t rows,
                                 int32_t rows_per_batch, int32_t dim, int64_t stride_xr, int64_t stride_yr,
                                 int64_t stride_y2r, int64_t stride_or, int64_t stride_gb, int64_t stride_gd,
                                 int32_t dtype, void* stream) {
    using namespace nb;
    NB_REQUIRE(x && gate && y && out);
    NB_REQUIRE(rows >= 0 && rows_per_batch > 0 && dim > 0 && dim % 8 == 0);
    NB_REQUIRE(dtype == NB_DTYPE_BF16 || dtype == NB_DTYPE_FP16);
    NB_REQUIRE(aligned16(x) && aligned16(y) && aligned16(out) && stride_xr % 8 == 0 && stride_yr % 8 == 0 && stride_or % 8 == 0);
    NB_REQUIRE(!y2 || (aligned16(y2) && stride_y2r % 8 == 0));
    if (rows == 0) return NB_OK;
    EwParams p = {};
    p.x = x; p.y = y; p.y2 = y2; p.out = out; p.a = gate;
    p.rows = rows; p.rows_per_batch = rows_per_batch; p.dim = dim;
    p.stride_xr = stride_xr; p.stride_yr = stride_yr; p.stride_y2r = stride_y2r; p.stride_or = stride_or;
    p.stride_ab = stride_gb; p.stride_ad = stride_gd;
    p.vec_ab = stride_gd == 1 && stride_gb % 8 == 0 && aligned16(gate);
    const long long units = (long long)rows * (dim / 8);
    int sms = 148;
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long want = (units + 255) / 256;
    const int blocks = (int)(want < (long long)sms * 8 ? want : (long long)sms * 8);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == NB_DTYPE_BF16) gated_residual_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(p);
    else gated_residual_kernel<__half><<<blocks, 256, 0, s>>>(p);
    NB_CUDA_CHECK(cudaGetLastError());
    return NB_OK;
}

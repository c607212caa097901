// Generic W4A4 GEMM on CUDA cores plus the row-wise epilogue kernels.
//
// This is the kernel for calls the tcgen05 kernels do not take (NVFP4 calls outside the block-scaled
// kernel's shapes, unaligned strides, ranks or widths off the tile grid); it plays the role of the
// reference's generic `_gemm_w4a4_kernel` (nunchaku/ops/triton/gemm_w4a4.py:230-373) next to its int4
// fast path.  Arithmetic: one exact int32 dot (dp4a) per 64-group, `acc += float(p) * as * ws`
// (gemm_w4a4.py:477-483); NVFP4: exact fp32 dot per 16-group of decoded e2m1 values, scales decoded
// from e4m3.  Then `_w4a4_epilogue` order (gemm_w4a4.py:155-209): wcscale, alpha, LoRA-up with
// lora_act rounded to T, bias, SiLU.  The fused epilogues run afterwards as row kernels on the fp32
// tile kept in scratch, so their input is the unrounded value, as in the fused kernels.
#include "nb_common.cuh"

namespace nb {

struct GenericParams {
    const uint8_t* act;
    const uint8_t* wgt;
    void* out;
    float* acc_out;  // optional (M, N) fp32 copy of the post-epilogue tile
    int32_t* p_out;  // optional (K/64, M, N) int32 group sums (debug)
    const void* ascales;
    const void* wscales;
    const void* bias;
    const float* lora_act;
    const void* lora_up;
    const void* wcscales;
    int M, N, K, actual_m, R;
    int act_unsigned, fp4, fuse_silu;
    float alpha;
    long long stride_am, stride_wn, stride_asg, stride_wsg, stride_om, stride_lam, stride_lun;
};

namespace {

constexpr int GT = 64;  // tile edge
constexpr int GPITCH = 80;  // bytes per decoded int8 row (64 + 16 pad)

// byte of 2 nibbles -> two sign- or zero-extended int8 packed in the low 16 bits
__device__ __forceinline__ uint32_t widen_byte(uint32_t b, bool is_signed) {
    int lo = b & 0xF, hi = (b >> 4) & 0xF;
    if (is_signed) {
        lo = (lo ^ 8) - 8;
        hi = (hi ^ 8) - 8;
    }
    return (uint32_t)(lo & 0xFF) | ((uint32_t)(hi & 0xFF) << 8);
}

template <typename T>
__global__ void __launch_bounds__(256) gemm_generic_kernel(const GenericParams p) {
    __shared__ __align__(16) uint8_t a_s[GT * GPITCH];
    __shared__ __align__(16) uint8_t w_s[GT * GPITCH];
    __shared__ float af_s[GT][65];  // fp4: decoded values
    __shared__ float wf_s[GT][65];
    __shared__ float as_s[4][GT], ws_s[4][GT];

    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * GT, n0 = blockIdx.x * GT;
    float acc[4][4] = {};

    for (int k0 = 0; k0 < p.K; k0 += 64) {
        const int kw = min(64, p.K - k0);  // fp4 allows K % 64 == 16, 32, 48
        // ---- stage: 64 rows x 32 bytes per operand, one byte pair per thread iteration
        for (int e = tid; e < GT * 32; e += 256) {
            const int r = e >> 5, b = e & 31;
            uint32_t ab = 0, wb = 0;
            if (2 * b < kw) {
                if (m0 + r < p.M) ab = p.act[(long long)(m0 + r) * p.stride_am + (k0 >> 1) + b];
                if (n0 + r < p.N) wb = p.wgt[(long long)(n0 + r) * p.stride_wn + (k0 >> 1) + b];
            }
            if (p.fp4) {
                af_s[r][2 * b] = e2m1_decode(ab & 0xF);
                af_s[r][2 * b + 1] = e2m1_decode(ab >> 4);
                wf_s[r][2 * b] = e2m1_decode(wb & 0xF);
                wf_s[r][2 * b + 1] = e2m1_decode(wb >> 4);
            } else {
                *reinterpret_cast<uint16_t*>(a_s + r * GPITCH + 2 * b) = (uint16_t)widen_byte(ab, !p.act_unsigned);
                *reinterpret_cast<uint16_t*>(w_s + r * GPITCH + 2 * b) = (uint16_t)widen_byte(wb, true);
            }
        }
        // ---- scales of this 64-block: 1 group (int4) or up to 4 groups (fp4)
        const int ng = p.fp4 ? (kw >> 4) : 1;
        for (int e = tid; e < 2 * 4 * GT; e += 256) {
            const int which = e / (4 * GT), gi = (e / GT) & 3, r = e % GT;
            float s = 0.f;
            if (gi < ng) {
                const long long g = p.fp4 ? (k0 >> 4) + gi : (k0 >> 6);
                if (which == 0 && m0 + r < p.M) {
                    s = p.fp4 ? e4m3_to_f32(static_cast<const uint8_t*>(p.ascales)[g * p.stride_asg + m0 + r])
                              : to_f32<T>(static_cast<const T*>(p.ascales)[g * p.stride_asg + m0 + r]);
                } else if (which == 1 && n0 + r < p.N) {
                    s = p.fp4 ? e4m3_to_f32(static_cast<const uint8_t*>(p.wscales)[g * p.stride_wsg + n0 + r])
                              : to_f32<T>(static_cast<const T*>(p.wscales)[g * p.stride_wsg + n0 + r]);
                }
            }
            (which == 0 ? as_s : ws_s)[gi][r] = s;
        }
        __syncthreads();

        if (!p.fp4) {
            int dot[4][4] = {};
#pragma unroll 4
            for (int kk = 0; kk < 16; ++kk) {
                int av[4], wv[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    av[i] = *reinterpret_cast<const int*>(a_s + (ty * 4 + i) * GPITCH + kk * 4);
                    wv[i] = *reinterpret_cast<const int*>(w_s + (tx * 4 + i) * GPITCH + kk * 4);
                }
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) dot[i][j] = __dp4a(av[i], wv[j], dot[i][j]);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] += (float)dot[i][j] * as_s[0][ty * 4 + i] * ws_s[0][tx * 4 + j];
                    if (p.p_out) {
                        const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
                        if (m < p.M && n < p.N) p.p_out[((long long)(k0 >> 6) * p.M + m) * p.N + n] = dot[i][j];
                    }
                }
        } else {
            for (int gi = 0; gi < ng; ++gi) {
                float dot[4][4] = {};
#pragma unroll 4
                for (int kk = 0; kk < 16; ++kk) {
                    float av[4], wv[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        av[i] = af_s[ty * 4 + i][gi * 16 + kk];
                        wv[i] = wf_s[tx * 4 + i][gi * 16 + kk];
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i)
#pragma unroll
                        for (int j = 0; j < 4; ++j) dot[i][j] = fmaf(av[i], wv[j], dot[i][j]);
                }
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[i][j] += dot[i][j] * as_s[gi][ty * 4 + i] * ws_s[gi][tx * 4 + j];
            }
        }
        __syncthreads();
    }

    // ---- epilogue stage 1
    const T* bias = static_cast<const T*>(p.bias);
    const T* lora_up = static_cast<const T*>(p.lora_up);
    const T* wcs = static_cast<const T*>(p.wcscales);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= p.M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= p.N) continue;
            float v = acc[i][j];
            if (wcs) v *= to_f32<T>(wcs[n]);
            v *= p.alpha;
            if (p.R > 0) {
                float l = 0.f;
                for (int r = 0; r < p.R; ++r)
                    l = fmaf(to_f32<T>(from_f32<T>(p.lora_act[(long long)m * p.stride_lam + r])),
                             to_f32<T>(lora_up[(long long)n * p.stride_lun + r]), l);
                v += l;
            }
            if (bias) v += to_f32<T>(bias[n]);
            if (p.fuse_silu) v = silu(v);
            if (p.acc_out) p.acc_out[(long long)m * p.N + n] = v;
            if (p.out && m < p.actual_m) static_cast<T*>(p.out)[(long long)m * p.stride_om + n] = from_f32<T>(v);
        }
    }
}

// ---- per-head RMSNorm + RoPE on the Q and K thirds (gemm_w4a4.py:498-521, 781-831) -----------------
// One warp per (row, head); SRC is float (fused path, unrounded tile) or T (in place on a stored tile).  In place, the V
// third is not touched at all (`heads` then counts the Q and K heads only).  VEC: rows and pointers are 16-byte aligned,
// so a lane's four values, weights and rotary entries move as one access each.
template <typename T, typename SRC, bool VEC>
__global__ void qk_rows_kernel(const SRC* src, long long stride_sm, T* out, long long stride_om, int M, int N, int heads,
                               const T* norm_q, const T* norm_k, const float* rot, long long stride_rm, int rot_rows,
                               float eps) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= M * heads) return;
    const int m = warp / heads, h = warp % heads;
    const int part = (h * 128) / (N / 3);
    const SRC* s = src + (long long)m * stride_sm + h * 128 + lane * 4;
    float x[4];
    if (VEC && sizeof(SRC) == 2) {
        const uint2 raw = *reinterpret_cast<const uint2*>(s);
        const float2 a = unpack2<T>(raw.x), b = unpack2<T>(raw.y);
        x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
    } else if (VEC) {
        const float4 raw = *reinterpret_cast<const float4*>(s);
        x[0] = raw.x; x[1] = raw.y; x[2] = raw.z; x[3] = raw.w;
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) x[i] = (float)s[i];
    }
    if (part < 2) {
        float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
#pragma unroll
        for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float rstd = rsqrtf(ss / 128.0f + eps);
        const T* w = (part == 0 ? norm_q : norm_k) + lane * 4;
        const float* rr = rot + (long long)(m % rot_rows) * stride_rm + lane * 4;
        float wf[4], rf[4];
        if (VEC) {
            const uint2 wr = __ldg(reinterpret_cast<const uint2*>(w));
            const float2 a = unpack2<T>(wr.x), b = unpack2<T>(wr.y);
            wf[0] = a.x; wf[1] = a.y; wf[2] = b.x; wf[3] = b.y;
            const float4 r4 = __ldg(reinterpret_cast<const float4*>(rr));
            rf[0] = r4.x; rf[1] = r4.y; rf[2] = r4.z; rf[3] = r4.w;
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) { wf[i] = to_f32<T>(w[i]); rf[i] = rr[i]; }
        }
#pragma unroll
        for (int pr = 0; pr < 2; ++pr) {
            const float xe = x[2 * pr] * rstd * wf[2 * pr];
            const float xo = x[2 * pr + 1] * rstd * wf[2 * pr + 1];
            const float sn = rf[2 * pr], cs = rf[2 * pr + 1];
            x[2 * pr] = xe * cs - xo * sn;
            x[2 * pr + 1] = xe * sn + xo * cs;
        }
    }
    T* o = out + (long long)m * stride_om + h * 128 + lane * 4;
    if (VEC) {
        *reinterpret_cast<uint2*>(o) = make_uint2(pack2<T>(x[0], x[1]), pack2<T>(x[2], x[3]));
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) o[i] = from_f32<T>(x[i]);
    }
}

// ---- GELU / SwiGLU + LoRA-down + int4 re-quantisation of an fp32 tile (gemm_w4a4.py:723-778) --------
// One CTA (128 threads) per row.  mode 0: x = gelu(lin[n]), unsigned codes; mode 1: x = silu(gate) * up with
// gate / up in 16-row interleaved blocks (native/w4a4.py:349-359), signed codes.
template <typename T>
__global__ void __launch_bounds__(128) requant_rows_kernel(const float* lin, int M, int N, int mode, uint8_t* qout,
                                                           long long stride_qm, T* oscales, long long stride_osg,
                                                           const T* smooth, const T* lora_down, long long stride_ld,
                                                           float* lora_act_out, long long stride_lom, int R2,
                                                           float shift) {
    extern __shared__ float xrow[];  // Nq activated values of this row
    const int m = blockIdx.x, tid = threadIdx.x;
    const int Nq = mode == 0 ? N : N / 2;
    const float* l = lin + (long long)m * N;
    for (int n = tid; n < Nq; n += 128) {
        float x;
        if (mode == 0) {
            x = gelu_tanh(l[n]);
        } else {
            const int blk = n >> 4, w = n & 15;
            x = silu(l[blk * 32 + w]) * l[blk * 32 + 16 + w];
        }
        xrow[n] = x;
    }
    __syncthreads();
    // LoRA-down from the activated value rounded to T, before shift and smoothing; one rank per thread,
    // summed in index order
    for (int r = tid; r < R2; r += 128) {
        float s = 0.f;
        for (int n = 0; n < Nq; ++n)
            s = fmaf(to_f32<T>(from_f32<T>(xrow[n])), to_f32<T>(lora_down[(long long)n * stride_ld + r]), s);
        lora_act_out[(long long)m * stride_lom + r] = s;
    }
    // quantise: one warp per 64-group
    const int warp = tid >> 5, lane = tid & 31;
    for (int g = warp; g < Nq / 64; g += 4) {
        float v0 = xrow[g * 64 + 2 * lane] + shift, v1 = xrow[g * 64 + 2 * lane + 1] + shift;
        if (smooth) {
            v0 *= 1.0f / to_f32<T>(smooth[g * 64 + 2 * lane]);
            v1 *= 1.0f / to_f32<T>(smooth[g * 64 + 2 * lane + 1]);
        }
        float mx = mode == 0 ? fmaxf(v0, v1) : fmaxf(fabsf(v0), fabsf(v1));
#pragma unroll
        for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        mx = fmaxf(mx, 0.f);
        const float scale = mx / (mode == 0 ? 15.0f : 7.0f);
        const float inv = 1.0f / (scale == 0.f ? 1.0f : scale);
        const float lo = mode == 0 ? 0.f : -8.f, hi = mode == 0 ? 15.f : 7.f;
        const int q0 = (int)fminf(fmaxf(rint_small(__fmul_rn(v0, inv)), lo), hi);
        const int q1 = (int)fminf(fmaxf(rint_small(__fmul_rn(v1, inv)), lo), hi);
        qout[(long long)m * stride_qm + g * 32 + lane] = (uint8_t)((q0 & 0xF) | ((q1 & 0xF) << 4));
        if (lane == 0) oscales[(long long)g * stride_osg + m] = from_f32<T>(scale);
    }
}

}  // namespace

template <typename T>
static int launch_generic_t(const GenericParams& p, cudaStream_t s) {
    dim3 grid((p.N + GT - 1) / GT, (p.M + GT - 1) / GT);
    gemm_generic_kernel<T><<<grid, 256, 0, s>>>(p);
    NB_CUDA_CHECK(cudaGetLastError());
    return NB_OK;
}

int launch_generic(const GenericParams& p, int dtype, cudaStream_t s) {
    return dtype == NB_DTYPE_BF16 ? launch_generic_t<__nv_bfloat16>(p, s) : launch_generic_t<__half>(p, s);
}

template <typename T>
static int launch_qk_rows_t(const float* src_f, void* out, long long stride_om, int M, int N, const nb_qk_args* qk,
                            cudaStream_t s) {
    const int heads = src_f ? N / 128 : 2 * (N / 3) / 128;  // in place: Q and K only
    const long long warps = (long long)M * heads;
    const int blocks = (int)((warps + 7) / 8);
    const bool vec = aligned16(out) && stride_om % 8 == 0 && aligned16(qk->norm_q) && aligned16(qk->norm_k) &&
                     aligned16(qk->rot) && qk->stride_rm % 4 == 0 && (!src_f || (aligned16(src_f) && N % 4 == 0));
    auto go = [&](auto kern, auto* src, long long stride_sm) {
        kern<<<blocks, 256, 0, s>>>(src, stride_sm, static_cast<T*>(out), stride_om, M, N, heads,
                                    static_cast<const T*>(qk->norm_q), static_cast<const T*>(qk->norm_k), qk->rot,
                                    qk->stride_rm, qk->rot_rows, qk->eps);
    };
    if (src_f) {
        if (vec) go(qk_rows_kernel<T, float, true>, src_f, (long long)N);
        else go(qk_rows_kernel<T, float, false>, src_f, (long long)N);
    } else {
        if (vec) go(qk_rows_kernel<T, T, true>, static_cast<const T*>(out), stride_om);
        else go(qk_rows_kernel<T, T, false>, static_cast<const T*>(out), stride_om);
    }
    NB_CUDA_CHECK(cudaGetLastError());
    return NB_OK;
}

// src_f == nullptr: in place on `out`
int launch_qk_rows(const float* src_f, void* out, long long stride_om, int M, int N, int dtype, const nb_qk_args* qk,
                   cudaStream_t s) {
    if (M == 0) return NB_OK;
    return dtype == NB_DTYPE_BF16 ? launch_qk_rows_t<__nv_bfloat16>(src_f, out, stride_om, M, N, qk, s)
                                  : launch_qk_rows_t<__half>(src_f, out, stride_om, M, N, qk, s);
}

template <typename T>
static int launch_requant_rows_t(const float* lin, int M, int N, int mode, const nb_requant_args* q, cudaStream_t s) {
    const int Nq = mode == 0 ? N : N / 2;
    const size_t smem = (size_t)Nq * sizeof(float);
    NB_CUDA_CHECK(cudaFuncSetAttribute(requant_rows_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    const bool lora = q->lora_down && q->lora_act_out && q->R2 > 0;
    requant_rows_kernel<T><<<M, 128, smem, s>>>(lin, M, N, mode, static_cast<uint8_t*>(q->qout), q->stride_qm,
                                                 static_cast<T*>(q->oscales), q->stride_osg,
                                                 static_cast<const T*>(q->smooth), static_cast<const T*>(q->lora_down),
                                                 q->stride_ld, q->lora_act_out, q->stride_lom, lora ? q->R2 : 0,
                                                 q->shift);
    NB_CUDA_CHECK(cudaGetLastError());
    return NB_OK;
}

int launch_requant_rows(const float* lin, int M, int N, int mode, int dtype, const nb_requant_args* q,
                        cudaStream_t s) {
    if (M == 0) return NB_OK;
    const int Nq = mode == 0 ? N : N / 2;
    if ((size_t)Nq * 4 > 200 * 1024) return NB_ERR_UNSUPPORTED;
    return dtype == NB_DTYPE_BF16 ? launch_requant_rows_t<__nv_bfloat16>(lin, M, N, mode, q, s)
                                  : launch_requant_rows_t<__half>(lin, M, N, mode, q, s);
}

}  // namespace nb

extern "C" int nb_qk_norm_rope(void* out, int32_t M, int32_t N, int64_t stride_om, int32_t dtype,
                               const nb_qk_args* qk, void* stream) {
    using namespace nb;
    NB_REQUIRE(out && qk && qk->norm_q && qk->norm_k && qk->rot);
    NB_REQUIRE(N % 3 == 0 && (N / 3) % 128 == 0 && qk->rot_rows > 0);
    NB_REQUIRE(dtype == NB_DTYPE_BF16 || dtype == NB_DTYPE_FP16);
    return launch_qk_rows(nullptr, out, stride_om, M, N, dtype, qk, static_cast<cudaStream_t>(stream));
}

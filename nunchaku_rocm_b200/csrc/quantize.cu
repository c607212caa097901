// Activation quantizer with fused LoRA-down (HBM-bound).
//
// Semantics follow `_quantize_tile_kernel` of the reference (nunchaku/ops/triton/gemm_w4a4.py:1338-1462):
// optional GLU / GELU, LoRA-down from the un-shifted, un-smoothed row rounded to the 16-bit dtype,
// then shift, reciprocal-multiply by smooth, per-group max, scale = max / qmax (stored rounded,
// transposed (K/G, M)), codes from the unrounded scale with round-half-even, low nibble first.
//
// Work split: a CTA owns 16 rows and splits K over its warps (4, 8 or 16 of them, chosen so that the grid fills the
// machine): warp w takes the 64-wide K groups g = w, w + warps, ...  A lane holds rows {gid, gid + 8} x columns
// {8 tig .. 8 tig + 7} and {32 + 8 tig ..}, read with 128-bit loads kept three iterations in flight; the per-group
// maximum is a 2-step warp shuffle over the 4 lanes that share a row.  The same registers are the A fragments of the
// LoRA-down mma.sync.m16n8k16 (a dot product does not care about a permutation of k applied to both operands, so the
// B fragments are fetched with ldmatrix.trans from the matching rows of the lora_down chunk, staged in shared memory
// by cp.async).  The warps' partial sums are added in a fixed order through shared memory, so the result is
// run-to-run identical.
#include <cuda_fp8.h>

#include "nb_common.cuh"

namespace nb {
namespace {

constexpr int QT_ROWS = 16;
constexpr int QT_MAX_WARPS = 16;

// Byte offset of the 16-byte unit c of k-row `krow` inside a staged lora_down chunk (64 k-rows x U units, U = ranks / 8
// in {2, 4, 8}).  Rows are packed into 128-byte lines; the unit index inside a line is XOR-ed with bits of the k-row so
// that the eight rows one ldmatrix 8x8 tile reads (k = 8 t + e + const, t < 4, e < 2) fall into eight different
// 16-byte bank groups.
__device__ __forceinline__ int ld_unit_offset(int krow, int c, int U) {
    const int t = (krow >> 3) & 3, e = krow & 1;
    int line, u, sw;
    if (U == 8) { line = krow; u = c; sw = e | (t << 1); }
    else if (U == 4) { line = krow >> 1; u = ((krow & 1) << 2) | c; sw = t; }
    else { line = krow >> 2; u = ((krow & 3) << 1) | c; sw = (t & 1) | ((t >> 1) << 2); }
    return line * 128 + ((u ^ sw) << 4);
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <typename T>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                                        uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

struct QParams {
    const void* input;
    uint8_t* output;
    void* oscales;
    const void* lora_down;
    float* lora_act_out;
    const void* smooth;
    int M, K, R;
    int fuse_glu, fuse_gelu, fp4, is_unsigned, do_lora;
    float shift;
    long long stride_im, stride_om, stride_sg, stride_ld, stride_lam;
};

// One 16-byte load of 8 T values, zero when the row is out of range, and its conversion to fp32.
__device__ __forceinline__ uint4 load_raw(const void* p, bool ok) {
    return ok ? __ldg(reinterpret_cast<const uint4*>(p)) : make_uint4(0, 0, 0, 0);
}
template <typename T>
__device__ __forceinline__ void widen8(const uint4& raw, float (&v)[8]) {
    float2 f;
    f = unpack2<T>(raw.x); v[0] = f.x; v[1] = f.y;
    f = unpack2<T>(raw.y); v[2] = f.x; v[3] = f.y;
    f = unpack2<T>(raw.z); v[4] = f.x; v[5] = f.y;
    f = unpack2<T>(raw.w); v[6] = f.x; v[7] = f.y;
}
template <typename T>
__device__ __forceinline__ void load8(const T* p, bool ok, float (&v)[8]) {
    widen8<T>(load_raw(p, ok), v);
}

template <typename T, int RC>  // RC: LoRA ranks per grid.y slice (16, 32 or 64)
__global__ void __launch_bounds__(QT_MAX_WARPS * 32) quantize_kernel(const QParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KS = blockDim.x >> 5;  // K slices = warps
    const int gid = lane >> 2, tig = lane & 3;
    const int kq = warp;
    const int m0 = blockIdx.x * QT_ROWS;
    const int r0 = blockIdx.y * RC;                    // first LoRA rank of this slice
    const int rn = p.do_lora ? min(RC, p.R - r0) : 0;  // ranks in this slice: 16, 32, 48 (RC = 64 only) or 64
    const bool quantize = blockIdx.y == 0;
    const int G = p.K / 64;  // 64-wide column blocks; an NVFP4 block holds four 16-groups

    // per-warp double buffer for the lora_down chunk: 64 k-rows x RC ranks
    constexpr int U = RC / 8;             // 16-byte units per k-row
    constexpr int CHUNK = 64 * RC * 2;    // bytes
    uint8_t* ld_buf = smem + warp * (2 * CHUNK);
    const T* x = static_cast<const T*>(p.input);
    const T* ldw = static_cast<const T*>(p.lora_down);
    const T* smooth = static_cast<const T*>(p.smooth);

    const int row_a = m0 + gid, row_b = m0 + gid + 8;
    const bool ok_a = row_a < p.M, ok_b = row_b < p.M;

    float acc[RC / 8][4];
#pragma unroll
    for (int i = 0; i < RC / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

    auto stage_ld = [&](int g, int buf) {
        // 64 k-rows x RC ranks in 16-byte units, 32 / U rows per pass of the warp (units beyond rn stay unwritten and
        // are never multiplied); the loop unrolls, so the swizzled offsets fold to a few operations each
        const uint32_t dst0 = smem_u32(ld_buf + buf * CHUNK);
        const int c = lane % U, kr0 = lane / U;
        const T* src = ldw + (long long)(g * 64 + kr0) * p.stride_ld + r0 + c * 8;
        if (c * 8 < rn) {
#pragma unroll
            for (int j = 0; j < 2 * U; ++j)
                cp_async16(dst0 + ld_unit_offset(kr0 + j * (32 / U), c, U), src + (long long)j * (32 / U) * p.stride_ld);
        }
    };
    // The x block of a warp iteration is four 16-byte loads per lane.  Three iterations' loads are kept in flight (the
    // kernel is HBM-bound and a warp's own iteration is far shorter than the memory latency).
    auto issue_x = [&](int g, uint4(&r)[4]) {
        const bool in = g < G;
        const int c0 = (in ? g : 0) * 64 + 8 * tig;
        r[0] = load_raw(x + (long long)row_a * p.stride_im + c0, ok_a && in);
        r[1] = load_raw(x + (long long)row_a * p.stride_im + c0 + 32, ok_a && in);
        r[2] = load_raw(x + (long long)row_b * p.stride_im + c0, ok_b && in);
        r[3] = load_raw(x + (long long)row_b * p.stride_im + c0 + 32, ok_b && in);
    };
    uint4 xr0[4], xr1[4], xr2[4];
    issue_x(kq, xr0);
    issue_x(kq + KS, xr1);

    int it = 0;
    if (rn > 0 && kq < G) stage_ld(kq, 0);
    cp_async_commit();

    for (int g = kq; g < G; g += KS, ++it) {
        if (rn > 0 && g + KS < G) stage_ld(g + KS, (it + 1) & 1);
        cp_async_commit();
        issue_x(g + 2 * KS, xr2);

        // ---- the 16 x 64 block: rows {gid, gid+8}, columns {8 tig.., 32 + 8 tig..}
        float v[2][16];
        const int c0 = g * 64 + 8 * tig;
        widen8<T>(xr0[0], *reinterpret_cast<float(*)[8]>(&v[0][0]));
        widen8<T>(xr0[1], *reinterpret_cast<float(*)[8]>(&v[0][8]));
        widen8<T>(xr0[2], *reinterpret_cast<float(*)[8]>(&v[1][0]));
        widen8<T>(xr0[3], *reinterpret_cast<float(*)[8]>(&v[1][8]));
        // the 16-bit words themselves: the LoRA-down operands when no activation function changes the values
        const uint32_t raw_w[2][8] = {{xr0[0].x, xr0[0].y, xr0[0].z, xr0[0].w, xr0[1].x, xr0[1].y, xr0[1].z, xr0[1].w},
                                      {xr0[2].x, xr0[2].y, xr0[2].z, xr0[2].w, xr0[3].x, xr0[3].y, xr0[3].z, xr0[3].w}};
        const bool raw_ok = !p.fuse_glu && !p.fuse_gelu;
#pragma unroll
        for (int i = 0; i < 4; ++i) { xr0[i] = xr1[i]; xr1[i] = xr2[i]; }
        if (p.fuse_glu) {
            float gate[2][16];
            load8<T>(x + (long long)row_a * p.stride_im + p.K + c0, ok_a, *reinterpret_cast<float(*)[8]>(&gate[0][0]));
            load8<T>(x + (long long)row_a * p.stride_im + p.K + c0 + 32, ok_a,
                     *reinterpret_cast<float(*)[8]>(&gate[0][8]));
            load8<T>(x + (long long)row_b * p.stride_im + p.K + c0, ok_b, *reinterpret_cast<float(*)[8]>(&gate[1][0]));
            load8<T>(x + (long long)row_b * p.stride_im + p.K + c0 + 32, ok_b,
                     *reinterpret_cast<float(*)[8]>(&gate[1][8]));
#pragma unroll
            for (int r = 0; r < 2; ++r)
#pragma unroll
                for (int i = 0; i < 16; ++i) v[r][i] = v[r][i] * silu(gate[r][i]);
        }
        if (p.fuse_gelu) {
#pragma unroll
            for (int r = 0; r < 2; ++r)
#pragma unroll
                for (int i = 0; i < 16; ++i) v[r][i] = gelu_tanh(v[r][i]);
        }

        // ---- LoRA-down on the un-shifted, un-smoothed values rounded to T
        if (rn > 0) {
            cp_async_wait<1>();
            __syncwarp();
            const uint32_t base = smem_u32(ld_buf + (it & 1) * CHUNK);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                // A fragment i: k-slots (2 tig, 2 tig + 1) = elements 4i, 4i+1; slots (2 tig + 8, +9) = 4i+2, 4i+3
                uint32_t a[4];
                if (raw_ok) {
                    a[0] = raw_w[0][2 * i]; a[1] = raw_w[1][2 * i]; a[2] = raw_w[0][2 * i + 1]; a[3] = raw_w[1][2 * i + 1];
                } else {
                    a[0] = pack2<T>(v[0][4 * i], v[0][4 * i + 1]);
                    a[1] = pack2<T>(v[1][4 * i], v[1][4 * i + 1]);
                    a[2] = pack2<T>(v[0][4 * i + 2], v[0][4 * i + 3]);
                    a[3] = pack2<T>(v[1][4 * i + 2], v[1][4 * i + 3]);
                }
                // k-slot s of fragment i is column (i < 2 ? 0 : 32) + 8 (s % 8 / 2) + 4 (i % 2) + 2 (s / 8) + s % 2
                // ldmatrix.x4: lanes 0-7 give the rows of matrix 0 (slots 0-7, ranks +0), 8-15 matrix 1
                // (slots 8-15, ranks +0), 16-23 matrix 2 (slots 0-7, ranks +8), 24-31 matrix 3 (slots 8-15, +8)
                const int s = (lane & 7) + ((lane >> 3) & 1) * 8;
                const int krow = (i < 2 ? 0 : 32) + 8 * ((s & 7) >> 1) + 4 * (i & 1) + 2 * (s >> 3) + (s & 1);
#pragma unroll
                for (int nt = 0; nt < RC / 8; nt += 2) {
                    if (nt * 8 < rn) {
                        uint32_t b[4];
                        ldmatrix_x4_trans(b, base + ld_unit_offset(krow, nt + (lane >> 4), U));
                        mma16816<T>(acc[nt], a, b[0], b[1]);
                        mma16816<T>(acc[nt + 1], a, b[2], b[3]);
                    }
                }
            }
            __syncwarp();
        }

        if (!quantize) continue;

        // ---- shift, smooth, per-group max, codes
        if (p.shift != 0.f) {
#pragma unroll
            for (int r = 0; r < 2; ++r)
#pragma unroll
                for (int i = 0; i < 16; ++i) v[r][i] += p.shift;
        }
        if (smooth) {
            // The 8 lanes with the same tig hold the same 16 columns.  Each of them takes the correctly rounded reciprocal
            // (as 1.0f / s) of two of those columns and the others fetch it by shuffle: 2 reciprocals per lane, not 16.
            const int i0 = 2 * gid;  // element index of this lane's pair among the 16
            const float2 s2 = unpack2<T>(__ldg(reinterpret_cast<const uint32_t*>(smooth + c0 + (i0 < 8 ? i0 : 24 + i0))));
            const float r0v = __frcp_rn(s2.x), r1v = __frcp_rn(s2.y);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float inv = __shfl_sync(0xffffffffu, (i & 1) ? r1v : r0v, (i >> 1) * 4 + tig);
                v[0][i] *= inv;
                v[1][i] *= inv;
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int row = r ? row_b : row_a;
            const bool ok = r ? ok_b : ok_a;
            uint8_t* orow = p.output + (long long)row * p.stride_om;
            if (!p.fp4) {
                float mx = p.is_unsigned ? v[r][0] : fabsf(v[r][0]);
#pragma unroll
                for (int i = 1; i < 16; ++i) mx = fmaxf(mx, p.is_unsigned ? v[r][i] : fabsf(v[r][i]));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                mx = fmaxf(mx, 0.f);
                const float scale = mx / (p.is_unsigned ? 15.0f : 7.0f);
                const float inv = __frcp_rn(scale == 0.f ? 1.0f : scale);
                // |v| <= mx and inv = 1 / (mx / qmax) bound v * inv by qmax * (1 + 2^-22), which rounds to qmax: only the
                // lower bound of the unsigned format (negative inputs) needs a clamp, and clamping to an integer bound
                // commutes with the rounding
                // round half-even by the magic add: the low mantissa bits of 1.5 * 2^23 + q are the two's-complement code
                uint32_t w[2] = {0, 0};
                if (p.is_unsigned) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const uint32_t u = __float_as_uint(__fadd_rn(fmaxf(__fmul_rn(v[r][i], inv), 0.f), 12582912.0f));
                        asm("bfi.b32 %0, %1, %0, %2, 4;" : "+r"(w[i >> 3]) : "r"(u), "r"(4 * (i & 7)));
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const uint32_t u = __float_as_uint(__fadd_rn(__fmul_rn(v[r][i], inv), 12582912.0f));
                        asm("bfi.b32 %0, %1, %0, %2, 4;" : "+r"(w[i >> 3]) : "r"(u), "r"(4 * (i & 7)));
                    }
                }
                if (ok) {
                    *reinterpret_cast<uint32_t*>(orow + (c0 >> 1)) = w[0];
                    *reinterpret_cast<uint32_t*>(orow + ((c0 + 32) >> 1)) = w[1];
                    if (tig == 0) static_cast<T*>(p.oscales)[(long long)g * p.stride_sg + row] = from_f32<T>(scale);
                }
            } else {
                // four 16-groups per 64 block: lanes (tig 0,1) share group 0 / 2, lanes (2,3) group 1 / 3
                uint32_t w[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    float mx = 0.f;
#pragma unroll
                    for (int i = 0; i < 8; ++i) mx = fmaxf(mx, fabsf(v[r][8 * h + i]));
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                    const float scale = mx / 6.0f;
                    const float inv = 1.0f / (scale == 0.f ? 1.0f : scale);
                    uint32_t ww = 0;
#pragma unroll
                    for (int i = 0; i < 8; ++i) ww |= e2m1_encode(__fmul_rn(v[r][8 * h + i], inv)) << (4 * i);
                    w[h] = ww;
                    if (ok && (tig & 1) == 0) {
                        const int g16 = g * 4 + 2 * h + (tig >> 1);
                        static_cast<uint8_t*>(p.oscales)[(long long)g16 * p.stride_sg + row] =
                            (uint8_t)__nv_cvt_float_to_fp8(scale, __NV_SATFINITE, __NV_E4M3);
                    }
                }
                if (ok) {
                    *reinterpret_cast<uint32_t*>(orow + (c0 >> 1)) = w[0];
                    *reinterpret_cast<uint32_t*>(orow + ((c0 + 32) >> 1)) = w[1];
                }
            }
        }
    }
    cp_async_wait<0>();

    // ---- fixed-order sum of the warps' partials
    if (rn > 0) {
        __syncthreads();  // lora_down buffers are dead; reuse shared memory: [warp][16 rows][RC]
        float* red = reinterpret_cast<float*>(smem);
        float* mine = red + (warp * 16) * RC;
#pragma unroll
        for (int nt = 0; nt < RC / 8; ++nt) {
            const int c = nt * 8 + 2 * tig;
            mine[gid * RC + c] = acc[nt][0];
            mine[gid * RC + c + 1] = acc[nt][1];
            mine[(gid + 8) * RC + c] = acc[nt][2];
            mine[(gid + 8) * RC + c + 1] = acc[nt][3];
        }
        __syncthreads();
        for (int e = threadIdx.x; e < QT_ROWS * rn; e += blockDim.x) {
            const int row = e / rn, c = e % rn;
            float s = 0.f;
            for (int q = 0; q < KS; ++q) s += red[(q * 16 + row) * RC + c];
            const int m = m0 + row;
            if (m < p.M) p.lora_act_out[(long long)m * p.stride_lam + r0 + c] = s;
        }
    }
}

}  // namespace
}  // namespace nb

extern "C" int nb_quantize_w4a4(const nb_quant_args* a, void* stream) {
    using namespace nb;
    NB_REQUIRE(a && a->input && a->output && a->oscales);
    NB_REQUIRE(a->M >= 0 && a->K > 0 && a->K % 64 == 0);
    NB_REQUIRE(a->dtype == NB_DTYPE_BF16 || a->dtype == NB_DTYPE_FP16);
    const bool lora = a->lora_down != nullptr && a->lora_act_out != nullptr && a->R > 0;
    if (lora) NB_REQUIRE(a->R % 16 == 0 && a->stride_ld % 8 == 0 && aligned16(a->lora_down));
    NB_REQUIRE(aligned16(a->input) && a->stride_im % 8 == 0);
    NB_REQUIRE((reinterpret_cast<uintptr_t>(a->output) & 3) == 0 && a->stride_om % 4 == 0);
    if (a->smooth) NB_REQUIRE(aligned16(a->smooth));
    if (a->M == 0) return NB_OK;

    QParams p;
    p.input = a->input;
    p.output = static_cast<uint8_t*>(a->output);
    p.oscales = a->oscales;
    p.lora_down = a->lora_down;
    p.lora_act_out = a->lora_act_out;
    p.smooth = a->smooth;
    p.M = a->M; p.K = a->K; p.R = lora ? a->R : 0;
    p.fuse_glu = a->fuse_glu; p.fuse_gelu = a->fuse_gelu; p.fp4 = a->fp4; p.is_unsigned = a->is_unsigned;
    p.do_lora = lora;
    p.shift = a->shift;
    p.stride_im = a->stride_im; p.stride_om = a->stride_om; p.stride_sg = a->stride_sg;
    p.stride_ld = a->stride_ld; p.stride_lam = a->stride_lam;

    // rank chunk per grid.y slice and K slices per CTA: enough warps to cover the memory latency of every SM
    const int RC = !lora || a->R <= 16 ? 16 : (a->R <= 32 ? 32 : 64);
    const int row_blocks = (a->M + QT_ROWS - 1) / QT_ROWS;
    int dev = 0, sms = 0;
    NB_CUDA_CHECK(cudaGetDevice(&dev));
    NB_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    int ks = 4;
    while (ks < QT_MAX_WARPS && (long long)row_blocks * ks < 14LL * sms && ks * 2 <= a->K / 64) ks *= 2;
    dim3 grid(row_blocks, lora ? (a->R + RC - 1) / RC : 1);
    const size_t smem = (size_t)ks * 2 * 64 * RC * 2;  // also covers the reduction buffer (ks x 16 x RC floats)
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    auto launch = [&](auto kern) -> int {
        NB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kern<<<grid, ks * 32, smem, s>>>(p);
        return NB_OK;
    };
    int rc;
    if (a->dtype == NB_DTYPE_BF16)
        rc = RC == 16 ? launch(quantize_kernel<__nv_bfloat16, 16>) : RC == 32 ? launch(quantize_kernel<__nv_bfloat16, 32>) : launch(quantize_kernel<__nv_bfloat16, 64>);
    else
        rc = RC == 16 ? launch(quantize_kernel<__half, 16>) : RC == 32 ? launch(quantize_kernel<__half, 32>) : launch(quantize_kernel<__half, 64>);
    if (rc != NB_OK) return rc;
    NB_CUDA_CHECK(cudaGetLastError());
    return NB_OK;
}

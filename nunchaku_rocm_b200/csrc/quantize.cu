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

#include <type_traits>

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

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// x / C, correctly rounded, for the three divisors the formats use: q = x * (1 / C), one residual step.  Compared with
// the division itself over every non-negative finite float: identical for 7 and 15 everywhere and for 6 from 2^-125
// up (below that the division runs).
template <int C>
__device__ __forceinline__ float div_const(float x) {
    constexpr float c = (float)C, rc = 1.0f / c;
    if (C == 6 && x < 1e-30f) return x / c;
    const float q = __fmul_rn(x, rc);
    return __fmaf_rn(__fmaf_rn(-c, q, x), rc, q);
}

// Eight e2m1 codes (low nibble first) of eight floats with the conversion instruction, which rounds ties to even.
__device__ __forceinline__ uint32_t cvt_e2m1x8(const float (&x)[8]) {
    uint32_t w;
    asm("{\n.reg .b8 b0, b1, b2, b3;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n"
        "mov.b32 %0, {b0, b1, b2, b3};\n}"
        : "=r"(w)
        : "f"(x[0]), "f"(x[1]), "f"(x[2]), "f"(x[3]), "f"(x[4]), "f"(x[5]), "f"(x[6]), "f"(x[7]));
    return w;
}

// The same eight codes by comparison with the reference's thresholds (the rare words that hold a tie).
__device__ __noinline__ uint32_t e2m1_encode_x8(const float (&x)[8]) {
    uint32_t w = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) w |= e2m1_encode(x[i]) << (4 * i);
    return w;
}

constexpr int QM_S4 = 0, QM_U4 = 1, QM_FP4 = 2;

template <typename T, int RC, int MODE, bool ACT>  // RC: LoRA ranks per grid.y slice (16, 32 or 64); ACT: GLU / GELU in front
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

    // per-warp double buffer for the lora_down chunk (64 k-rows x RC ranks), then two strips of 64 reciprocals per warp
    constexpr int U = RC / 8;             // 16-byte units per k-row
    constexpr int CHUNK = 64 * RC * 2;    // bytes
    const uint32_t ld_buf = smem_u32(smem) + warp * (2 * CHUNK);
    float* rcp_strip = reinterpret_cast<float*>(smem + KS * (2 * CHUNK)) + warp * 128;
    const T* x = static_cast<const T*>(p.input);
    const T* ldw = static_cast<const T*>(p.lora_down);
    const T* smooth = static_cast<const T*>(p.smooth);

    const int row_a = m0 + gid, row_b = m0 + gid + 8;
    const bool ok_a = row_a < p.M, ok_b = row_b < p.M;
    // everything an iteration adds a multiple of g to is set up here: the loop itself is bound by instruction issue
    // (rows past M read the last row instead: rows never mix, and nothing of theirs is stored)
    const T* xa = x + (long long)min(row_a, p.M - 1) * p.stride_im + 8 * tig;
    const T* xb = x + (long long)min(row_b, p.M - 1) * p.stride_im + 8 * tig;
    uint8_t* oa = p.output + (long long)row_a * p.stride_om + 4 * tig;
    uint8_t* ob = p.output + (long long)row_b * p.stride_om + 4 * tig;

    // Staging of a lora_down chunk: a lane copies, for one 16-byte unit, the k-rows that share one swizzle pattern (their
    // destinations then differ by constants): rows 32 a + 8 t + 2 b + e (U = 4, 8: eight rows) or 32 a + 8 t + 4 b1 +
    // 2 b0 + e (U = 2: four rows).
    constexpr int ST_TASKS = U == 8 ? 2 : 1, ST_ROWS = U == 2 ? 4 : 8;
    uint32_t st_dst[ST_TASKS];
    const T* st_src[ST_TASKS];
    bool st_on[ST_TASKS];
#pragma unroll
    for (int k = 0; k < ST_TASKS; ++k) {
        const int idx = lane + 32 * k;
        int c, krow;
        if (U == 8) { c = idx & 7; krow = ((idx >> 3) & 1) + 8 * (idx >> 4); }
        else if (U == 4) { c = idx & 3; krow = ((idx >> 2) & 1) + 8 * (idx >> 3); }
        else { c = idx & 1; krow = ((idx >> 1) & 1) + 2 * ((idx >> 2) & 1) + 8 * (idx >> 3); }
        st_dst[k] = ld_unit_offset(krow, c, U);
        st_src[k] = ldw + (long long)krow * p.stride_ld + r0 + c * 8;
        st_on[k] = c * 8 < rn;  // (units beyond rn stay unwritten and are never multiplied)
    }
    // (the source walks its rows by two pointer increments: to the next row of a half, and across to the other half)
    constexpr int ST_STEP = U == 2 ? 4 : 2, ST_HALF = ST_ROWS / 2;
    const long long ld_step = (long long)ST_STEP * p.stride_ld, ld_jump = (32 - ST_STEP * (ST_HALF - 1)) * p.stride_ld;
    const long long ld_group = 64 * p.stride_ld;
    auto stage_ld = [&](int g, int buf) {
        const uint32_t dst0 = ld_buf + buf * CHUNK;
#pragma unroll
        for (int k = 0; k < ST_TASKS; ++k) {
            if (!st_on[k]) continue;
            const T* src = st_src[k] + g * ld_group;
#pragma unroll
            for (int j = 0; j < ST_ROWS; ++j) {
                // row j of the task: half a = j / ST_HALF, then b = j % ST_HALF rows of step ST_STEP
                const int drow = 32 * (j / ST_HALF) + ST_STEP * (j % ST_HALF);  // k-rows after the task's first
                cp_async16(dst0 + st_dst[k] + drow * (16 * U), src);
                src += j == ST_HALF - 1 ? ld_jump : ld_step;
            }
        }
    };
    // ldmatrix addresses of the B fragments: k-slot s of A fragment i is column (i < 2 ? 0 : 32) + 8 (s % 8 / 2) +
    // 4 (i % 2) + 2 (s / 8) + s % 2; lanes 0-7 give the rows of matrix 0 (slots 0-7, ranks +0), 8-15 matrix 1 (slots
    // 8-15, ranks +0), 16-23 matrix 2 (slots 0-7, ranks +8), 24-31 matrix 3 (slots 8-15, +8).  The fragment index only
    // adds a constant to the k-row (0, 4, 32, 36), which leaves the swizzle pattern alone.
    uint32_t lm_off[RC / 16];
    {
        const int s = (lane & 7) + ((lane >> 3) & 1) * 8;
        const int krow = 8 * ((s & 7) >> 1) + 2 * (s >> 3) + (s & 1);
#pragma unroll
        for (int k = 0; k < RC / 16; ++k) lm_off[k] = ld_unit_offset(krow, 2 * k + (lane >> 4), U);
    }

    float acc[RC / 8][4];
#pragma unroll
    for (int i = 0; i < RC / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

    // The x block of a warp iteration is four 16-byte loads per lane.  Two iterations' loads are kept in flight (an
    // iteration lasts several times the memory latency); the loop body is instantiated once per buffer, so no register
    // is copied to rotate them.
    auto issue_x = [&](int g, uint4(&r)[4]) {
        if (g < G) {
            const long long c0 = (long long)g * 64;
            r[0] = __ldg(reinterpret_cast<const uint4*>(xa + c0));
            r[1] = __ldg(reinterpret_cast<const uint4*>(xa + c0 + 32));
            r[2] = __ldg(reinterpret_cast<const uint4*>(xb + c0));
            r[3] = __ldg(reinterpret_cast<const uint4*>(xb + c0 + 32));
        }
    };
    auto load_smooth = [&](int g) -> uint32_t {
        // the two smoothing factors whose reciprocals this lane takes for the warp: columns 2 lane, 2 lane + 1
        return smooth != nullptr && g < G ? __ldg(reinterpret_cast<const uint32_t*>(smooth + g * 64 + 2 * lane)) : 0u;
    };
    uint4 xr0[4], xr1[4];
    issue_x(kq, xr0);
    issue_x(kq + KS, xr1);
    uint32_t sm_next = quantize ? load_smooth(kq) : 0u;

    if (rn > 0 && kq < G) stage_ld(kq, 0);
    cp_async_commit();

    auto body = [&](const int g, const int it, uint4(&xr)[4]) {
        if (rn > 0 && g + KS < G) stage_ld(g + KS, (it + 1) & 1);
        cp_async_commit();
        const uint32_t sm_raw = sm_next;
        if (quantize) sm_next = load_smooth(g + KS);

        // ---- the 16 x 64 block: rows {gid, gid+8}, columns {8 tig.., 32 + 8 tig..}
        float v[2][16];
        widen8<T>(xr[0], *reinterpret_cast<float(*)[8]>(&v[0][0]));
        widen8<T>(xr[1], *reinterpret_cast<float(*)[8]>(&v[0][8]));
        widen8<T>(xr[2], *reinterpret_cast<float(*)[8]>(&v[1][0]));
        widen8<T>(xr[3], *reinterpret_cast<float(*)[8]>(&v[1][8]));
        const bool raw_ok = !ACT;
        if (ACT && p.fuse_glu) {
            const long long c0 = (long long)g * 64 + p.K;
            float gate[2][16];
            load8<T>(xa + c0, true, *reinterpret_cast<float(*)[8]>(&gate[0][0]));
            load8<T>(xa + c0 + 32, true, *reinterpret_cast<float(*)[8]>(&gate[0][8]));
            load8<T>(xb + c0, true, *reinterpret_cast<float(*)[8]>(&gate[1][0]));
            load8<T>(xb + c0 + 32, true, *reinterpret_cast<float(*)[8]>(&gate[1][8]));
#pragma unroll
            for (int r = 0; r < 2; ++r)
#pragma unroll
                for (int i = 0; i < 16; ++i) v[r][i] = v[r][i] * silu(gate[r][i]);
        }
        if (ACT && p.fuse_gelu) {
#pragma unroll
            for (int r = 0; r < 2; ++r)
#pragma unroll
                for (int i = 0; i < 16; ++i) v[r][i] = gelu_tanh(v[r][i]);
        }

        // ---- LoRA-down on the un-shifted, un-smoothed values rounded to T
        if (rn > 0) {
            cp_async_wait<1>();
            __syncwarp();
            const uint32_t base = ld_buf + (it & 1) * CHUNK;
            // the 16-bit words themselves are the operands when no activation function changed the values
            const uint32_t raw_w[2][8] = {{xr[0].x, xr[0].y, xr[0].z, xr[0].w, xr[1].x, xr[1].y, xr[1].z, xr[1].w},
                                          {xr[2].x, xr[2].y, xr[2].z, xr[2].w, xr[3].x, xr[3].y, xr[3].z, xr[3].w}};
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
                constexpr int KI[4] = {0, 4, 32, 36};
#pragma unroll
                for (int k = 0; k < RC / 16; ++k) {
                    if (k * 16 < rn) {
                        uint32_t b[4];
                        ldmatrix_x4_trans(b, base + lm_off[k] + KI[i] * (16 * U));
                        mma16816<T>(acc[2 * k], a, b[0], b[1]);
                        mma16816<T>(acc[2 * k + 1], a, b[2], b[3]);
                    }
                }
            }
            __syncwarp();
        }
        issue_x(g + 2 * KS, xr);  // this buffer's next block (its registers are free from here on)

        if (!quantize) return;

        // ---- shift, smooth, per-group max, codes
        if (p.shift != 0.f) {
#pragma unroll
            for (int r = 0; r < 2; ++r)
#pragma unroll
                for (int i = 0; i < 16; ++i) v[r][i] += p.shift;
        }
        if (smooth) {
            // 1 / smooth (correctly rounded) of the block's 64 columns: two per lane, handed round through shared memory
            float* strip = rcp_strip + (it & 1) * 64;
            const float2 s2 = unpack2<T>(sm_raw);
            *reinterpret_cast<float2*>(strip + 2 * lane) = make_float2(__frcp_rn(s2.x), __frcp_rn(s2.y));
            __syncwarp();
#pragma unroll
            for (int h = 0; h < 4; ++h) {
                const ulonglong2 iv = *reinterpret_cast<const ulonglong2*>(strip + (h >> 1) * 32 + 8 * tig + (h & 1) * 4);
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const float2 lo = unpack_f32x2(mul_f32x2(pack_f32x2(v[r][4 * h], v[r][4 * h + 1]), iv.x));
                    const float2 hi = unpack_f32x2(mul_f32x2(pack_f32x2(v[r][4 * h + 2], v[r][4 * h + 3]), iv.y));
                    v[r][4 * h] = lo.x; v[r][4 * h + 1] = lo.y; v[r][4 * h + 2] = hi.x; v[r][4 * h + 3] = hi.y;
                }
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int row = r ? row_b : row_a;
            const bool ok = r ? ok_b : ok_a;
            uint8_t* orow = (r ? ob : oa) + g * 32;
            if (MODE != QM_FP4) {
                float mx;
                if (MODE == QM_U4) {
                    // negative values take code 0 whatever the scale: clamp them before the product (the scale is positive)
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[r][i] = fmaxf(v[r][i], 0.f);
                    float m4[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) m4[i] = max3(v[r][i], v[r][i + 4], v[r][i + 8]);
#pragma unroll
                    for (int i = 0; i < 4; ++i) m4[i] = fmaxf(m4[i], v[r][i + 12]);
                    mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
                } else {
                    // (two-input maxima here: the absolute value folds into them, not into the three-input form)
                    float m4[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) m4[i] = fmaxf(fabsf(v[r][i]), fabsf(v[r][i + 4]));
#pragma unroll
                    for (int i = 8; i < 16; ++i) m4[i & 3] = fmaxf(m4[i & 3], fabsf(v[r][i]));
                    mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
                }
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                mx = fmaxf(mx, 0.f);
                const float scale = MODE == QM_U4 ? div_const<15>(mx) : div_const<7>(mx);
                const float inv = __frcp_rn(scale == 0.f ? 1.0f : scale);
                // |v| <= mx and inv = 1 / (mx / qmax) bound v * inv by qmax * (1 + 2^-22), which rounds to qmax.  Round
                // half-even by the magic add: the low mantissa bits of 1.5 * 2^23 + q are the two's-complement code.
                // (The product is rounded to fp32 before the magic number is added, as the reference does.  ptxas contracts a
                // packed multiply feeding a packed ADD into one fused operation even with explicit rounding modifiers; it
                // leaves a multiply feeding a fused multiply-add alone, so the addition is written as p * 1 + magic.)
                const uint64_t inv2 = pack_f32x2(inv, inv), magic2 = pack_f32x2(12582912.0f, 12582912.0f);
                const uint64_t one2 = pack_f32x2(1.0f, 1.0f);
                // a pair's two nibbles make a byte (one bit-field insert), four bytes a word (three byte permutes)
                uint32_t t[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint64_t u = fma_f32x2(mul_f32x2(pack_f32x2(v[r][2 * i], v[r][2 * i + 1]), inv2), one2, magic2);
                    asm("bfi.b32 %0, %1, %2, 4, 4;" : "=r"(t[i]) : "r"((uint32_t)(u >> 32)), "r"((uint32_t)u));
                }
                uint32_t w[2];
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    w[h] = __byte_perm(__byte_perm(t[4 * h], t[4 * h + 1], 0x0040),
                                       __byte_perm(t[4 * h + 2], t[4 * h + 3], 0x0040), 0x5410);
                if (ok) {
                    *reinterpret_cast<uint32_t*>(orow) = w[0];
                    *reinterpret_cast<uint32_t*>(orow + 16) = w[1];
                    if (tig == 0) static_cast<T*>(p.oscales)[(long long)g * p.stride_sg + row] = from_f32<T>(scale);
                }
            } else {
                // four 16-groups per 64 block: lanes (tig 0,1) share group 0 / 2, lanes (2,3) group 1 / 3
                uint32_t w[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    float m2[2];
#pragma unroll
                    for (int i = 0; i < 2; ++i) m2[i] = fmaxf(fabsf(v[r][8 * h + i]), fabsf(v[r][8 * h + i + 2]));
#pragma unroll
                    for (int i = 4; i < 8; ++i) m2[i & 1] = fmaxf(m2[i & 1], fabsf(v[r][8 * h + i]));
                    float mx = fmaxf(m2[0], m2[1]);
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                    const float scale = div_const<6>(mx);
                    const float inv = __frcp_rn(scale == 0.f ? 1.0f : scale);
                    // The reference's thresholds send a tie to the larger magnitude and a negative zero to code 0; the
                    // conversion instruction rounds ties to even.  So: products with +0 added (one rounding, -0 becomes
                    // +0), converted twice, as they are and one unit in the last place further from zero.  Where the
                    // reference differs from round-to-even the two conversions differ too (the value is a tie), and
                    // those rare words are encoded by comparison.
                    const uint64_t inv2 = pack_f32x2(inv, inv);
                    float xq[8], xn[8];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 q2 = unpack_f32x2(
                            fma_f32x2(pack_f32x2(v[r][8 * h + 2 * i], v[r][8 * h + 2 * i + 1]), inv2, 0ull));
                        xq[2 * i] = q2.x; xq[2 * i + 1] = q2.y;
                    }
#pragma unroll
                    for (int i = 0; i < 8; ++i) xn[i] = __uint_as_float(__float_as_uint(xq[i]) + 1u);
                    uint32_t ww = cvt_e2m1x8(xq);
                    if (ww != cvt_e2m1x8(xn)) ww = e2m1_encode_x8(xq);
                    w[h] = ww;
                    if (ok && (tig & 1) == 0) {
                        const int g16 = g * 4 + 2 * h + (tig >> 1);
                        static_cast<uint8_t*>(p.oscales)[(long long)g16 * p.stride_sg + row] =
                            (uint8_t)__nv_cvt_float_to_fp8(scale, __NV_SATFINITE, __NV_E4M3);
                    }
                }
                if (ok) {
                    *reinterpret_cast<uint32_t*>(orow) = w[0];
                    *reinterpret_cast<uint32_t*>(orow + 16) = w[1];
                }
            }
        }
    };

    for (int g = kq, it = 0; g < G;) {
        body(g, it, xr0); g += KS; ++it;
        if (g >= G) break;
        body(g, it, xr1); g += KS; ++it;
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
    // K slices (warps) per CTA: 128 registers per thread leave an SM 16 warps, i.e. 16 / ks CTAs.  Take the split with the
    // fewest (waves of CTAs) x (K groups per warp); among equals the one with fewer waves.
    const int G = a->K / 64;
    int ks = 4;
    long long best = -1;
    for (int c = 4; c <= QT_MAX_WARPS; c *= 2) {
        if (c > 4 && c > G) break;
        const long long waves = (row_blocks + (long long)sms * (16 / c) - 1) / ((long long)sms * (16 / c));
        const long long cost = waves * ((G + c - 1) / c) * 64 + waves;
        if (best < 0 || cost < best) { best = cost; ks = c; }
    }
    dim3 grid(row_blocks, lora ? (a->R + RC - 1) / RC : 1);
    // lora_down double buffers (they also cover the reduction buffer, ks x 16 x RC floats) + the reciprocal strips
    const size_t smem = (size_t)ks * 2 * 64 * RC * 2 + (size_t)ks * 512;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    auto launch = [&](auto kern) -> int {
        NB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kern<<<grid, ks * 32, smem, s>>>(p);
        return NB_OK;
    };
    auto by_mode = [&](auto t, auto rc_tag) -> int {
        using T = decltype(t);
        constexpr int RCV = decltype(rc_tag)::value;
        if (a->fuse_glu || a->fuse_gelu) {
            if (a->fp4) return launch(quantize_kernel<T, RCV, QM_FP4, true>);
            return a->is_unsigned ? launch(quantize_kernel<T, RCV, QM_U4, true>) : launch(quantize_kernel<T, RCV, QM_S4, true>);
        }
        if (a->fp4) return launch(quantize_kernel<T, RCV, QM_FP4, false>);
        return a->is_unsigned ? launch(quantize_kernel<T, RCV, QM_U4, false>) : launch(quantize_kernel<T, RCV, QM_S4, false>);
    };
    auto by_rc = [&](auto t) -> int {
        if (RC == 16) return by_mode(t, std::integral_constant<int, 16>{});
        if (RC == 32) return by_mode(t, std::integral_constant<int, 32>{});
        return by_mode(t, std::integral_constant<int, 64>{});
    };
    const int rc = a->dtype == NB_DTYPE_BF16 ? by_rc(__nv_bfloat16{}) : by_rc(__half{});
    if (rc != NB_OK) return rc;
    NB_CUDA_CHECK(cudaGetLastError());
    return NB_OK;
}

// W4A4 int4 GEMM on the 5th-generation tensor cores (tcgen05.mma kind::i8, int32 accumulators in
// tensor memory), with the low-rank branch and the fused epilogues.
//
// Arithmetic contract (reference: nunchaku/ops/triton/gemm_w4a4.py:446-488 and :155-209): for every
// 64-wide K group g one EXACT int32 dot p_g[m,n]; acc += float(p_g) * as[g,m] * ws[g,n] in fp32;
// then + T(lora_act) . lora_up^T (16-bit operands, fp32 accumulate), + bias, one rounding to T.
//
// Pipeline of one persistent CTA (512 threads, one CTA per SM, static contiguous tile range):
//   warp 0      TMA producer: packed int4 rows of A (128 x 32 B) and W (BN x 32 B) of one K group, plus
//               that group's scale rows, into a 4-deep ring (no multicast, no cluster).
//   warps 2-7   widen: nibble n -> int8 16*n (n<<4 keeps the sign in the top bit; the factor 256 on
//               the product is folded into the activation scale) written in the K-major no-swizzle
//               UMMA layout (8-row x 16-byte core matrices, one 16-byte K chunk after another);
//               scales converted to fp32.  The same permutation of k inside the group is applied to
//               A and W, which a dot product does not see.  For the low-rank branch they stage
//               T(lora_act) and lora_up as bf16/fp16 operands through the same buffers.
//   warp 1      MMA issuer: two 128 x BN x 32 kind::i8 MMAs per group into one of two TMEM slots;
//               tcgen05.commit releases the operand buffer and publishes the slot.  The low-rank
//               product is kind::f16 into an fp32 slot of the same ring.
//   warps 8-15  drain: tcgen05.ld of the slot, int->float by the magic-number add, two FMAs per
//               element, into fp32 registers (one output row per thread, BN/2 columns); after the
//               last group the epilogue (bias, optional per-head RMSNorm + RoPE, rounding) and a
//               coalesced store through a padded per-warp staging tile.
// Every wait on an mbarrier is bounded (~2 s); on expiry the CTA records a code in the status word,
// unwinds without touching more data and frees its tensor memory.
#include <cuda.h>

#include <type_traits>

#include "nb_common.cuh"

namespace nb {
namespace tc {

constexpr int BM = 128;
constexpr int PK_STAGES = 4;
constexpr int WD_STAGES = 3;
constexpr int SC_STAGES = 4;
constexpr int NTHREADS = 512;
constexpr int WIDEN_THREADS = 192;  // warps 2..7
constexpr int WIDEN_WARPS = 6;
constexpr int DRAIN_WARPS = 8;      // warps 8..15
constexpr uint32_t MAGIC_BITS = 0x4B400000u;  // 1.5 * 2^23
constexpr float MAGIC_F = 12582912.0f;

template <int BN>
struct Cfg {
    static constexpr int PK_A = BM * 32, PK_W = BN * 32, PK_AS = BM * 2, PK_WS = BN * 2;
    static constexpr int PK_BYTES = PK_A + PK_W + PK_AS + PK_WS;
    static constexpr int WD_A = BM * 64, WD_W = BN * 64;
    static constexpr int WD_BYTES = WD_A + WD_W;
    static constexpr int SC_BYTES = BN * 4 + BM * 4 * 2;
    static constexpr int COLS = BN / 2;  // columns one drain warp owns
    static constexpr int STG_PITCH = COLS * 2 + 16;
    static constexpr int STG_BYTES = DRAIN_WARPS * 32 * STG_PITCH;
    static constexpr int OFF_PK = 0;
    static constexpr int OFF_WD = OFF_PK + PK_STAGES * PK_BYTES;
    static constexpr int OFF_SC = OFF_WD + WD_STAGES * WD_BYTES;
    static constexpr int OFF_STG = OFF_SC + SC_STAGES * SC_BYTES;
    static constexpr int OFF_BAR = OFF_STG + STG_BYTES;
    static constexpr int SMEM_BYTES = OFF_BAR + 512 + 1024;  // + slack to align the base to 1 KB
    static constexpr int TMEM_COLS = 2 * BN;                 // two accumulator slots (256 or 512: powers of two)
};

enum {  // barrier indices
    B_PK_FULL = 0,
    B_PK_EMPTY = B_PK_FULL + PK_STAGES,
    B_WD_FULL = B_PK_EMPTY + PK_STAGES,
    B_WD_EMPTY = B_WD_FULL + WD_STAGES,
    B_SC_FULL = B_WD_EMPTY + WD_STAGES,
    B_SC_EMPTY = B_SC_FULL + SC_STAGES,
    B_ACC_FULL = B_SC_EMPTY + SC_STAGES,
    B_ACC_EMPTY = B_ACC_FULL + 2,
    B_COUNT = B_ACC_EMPTY + 2
};

struct TcParams {
    void* out;
    const void* bias;
    const float* lora_act;
    const void* lora_up;
    int32_t* p_out;  // debug: (K/64, M, N) group sums
    int M, N, K, actual_m, R;
    int act_unsigned;
    long long stride_om, stride_lam, stride_lun;
    int* status;
    // QK epilogue
    const void* norm_q;
    const void* norm_k;
    const float* rot;
    long long stride_rm;
    int rot_rows;
    float eps;
};

// error codes written to *status: role * 16 + barrier kind
enum { E_PROD = 0x10, E_WIDEN = 0x20, E_MMA = 0x30, E_DRAIN = 0x40 };

template <int BN, int EPI, typename T, bool DEBUG_P>
__global__ void __launch_bounds__(NTHREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w,
               const __grid_constant__ CUtensorMap tm_as, const __grid_constant__ CUtensorMap tm_ws,
               const TcParams p) {
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t s_base = smem_u32(smem);
    const uint32_t s_bar = s_base + C::OFF_BAR;
    uint32_t* tmem_ptr_s = reinterpret_cast<uint32_t*>(smem + C::OFF_BAR + 8 * B_COUNT);
    volatile int* abort_s = reinterpret_cast<volatile int*>(smem + C::OFF_BAR + 8 * B_COUNT + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    auto bar = [&](int i) { return s_bar + 8u * i; };

    if (threadIdx.x == 0) {
        for (int i = 0; i < PK_STAGES; ++i) { mbar_init(bar(B_PK_FULL + i), 1); mbar_init(bar(B_PK_EMPTY + i), WIDEN_WARPS); }
        for (int i = 0; i < WD_STAGES; ++i) { mbar_init(bar(B_WD_FULL + i), WIDEN_WARPS); mbar_init(bar(B_WD_EMPTY + i), 1); }
        for (int i = 0; i < SC_STAGES; ++i) { mbar_init(bar(B_SC_FULL + i), WIDEN_WARPS); mbar_init(bar(B_SC_EMPTY + i), DRAIN_WARPS); }
        for (int i = 0; i < 2; ++i) { mbar_init(bar(B_ACC_FULL + i), 1); mbar_init(bar(B_ACC_EMPTY + i), DRAIN_WARPS); }
        *abort_s = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_ptr_s), C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr_s;

    // static contiguous tile range of this CTA; tile t = m_blk * NT + n_blk
    const int MT = (p.M + BM - 1) / BM, NT = (p.N + BN - 1) / BN;
    const int total = MT * NT;
    const int per = (total + gridDim.x - 1) / gridDim.x;
    const int t_begin = min(total, (int)blockIdx.x * per), t_end = min(total, t_begin + per);
    const int G = p.K / 64;
    const int LCH = (p.R + 31) / 32;  // low-rank chunks of 32 ranks

    if (warp < 8) {
        setmaxnreg_dec_56();
        if (warp == 0) {
            // ================================ TMA producer ================================
            if (lane == 0) {
                tma_prefetch_desc(&tm_a); tma_prefetch_desc(&tm_w); tma_prefetch_desc(&tm_as); tma_prefetch_desc(&tm_ws);
                uint32_t it = 0;
                bool ok = true;
                for (int t = t_begin; t < t_end && ok; ++t) {
                    const int m0 = (t / NT) * BM, n0 = (t % NT) * BN;
                    for (int g = 0; g < G; ++g, ++it) {
                        const int s = it % PK_STAGES;
                        if (!mbar_wait(bar(B_PK_EMPTY + s), ((it / PK_STAGES) & 1) ^ 1, abort_s, E_PROD | 1)) { ok = false; break; }
                        const uint32_t dst = s_base + C::OFF_PK + s * C::PK_BYTES;
                        mbar_expect_tx(bar(B_PK_FULL + s), C::PK_BYTES);
                        tma_load_2d(dst, &tm_a, bar(B_PK_FULL + s), g * 32, m0);
                        tma_load_2d(dst + C::PK_A, &tm_w, bar(B_PK_FULL + s), g * 32, n0);
                        tma_load_2d(dst + C::PK_A + C::PK_W, &tm_as, bar(B_PK_FULL + s), m0, g);
                        tma_load_2d(dst + C::PK_A + C::PK_W + C::PK_AS, &tm_ws, bar(B_PK_FULL + s), n0, g);
                    }
                }
                if (!ok) {
                    // let copies already in flight land before the CTA goes away (bounded)
                    for (int s = 0; s < PK_STAGES; ++s) {
                        const uint32_t issued = it > (uint32_t)s ? (it - 1 - s) / PK_STAGES + 1 : 0;  // fills of stage s
                        if (issued) {
                            uint64_t t0 = globaltimer_ns();
                            while (!mbar_try_wait(bar(B_PK_FULL + s), (issued - 1) & 1) && globaltimer_ns() - t0 < 200000000ull) {}
                        }
                    }
                }
            }
        } else if (warp == 1) {
            // ================================ MMA issuer ================================
            if (lane == 0) {
                const uint32_t idesc_i8 = umma_idesc(2u, p.act_unsigned ? 0u : 1u, 1u, BN);
                const uint32_t f16fmt = sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
                const uint32_t idesc_lr = umma_idesc(1u, f16fmt, f16fmt, BN);
                uint32_t wit = 0, ait = 0;
                bool ok = true;
                for (int t = t_begin; t < t_end && ok; ++t) {
                    for (int g = 0; g < G && ok; ++g, ++wit, ++ait) {
                        const int w = wit % WD_STAGES, slot = ait & 1;
                        if (!mbar_wait(bar(B_WD_FULL + w), (wit / WD_STAGES) & 1, abort_s, E_MMA | 1)) { ok = false; break; }
                        if (!mbar_wait(bar(B_ACC_EMPTY + slot), ((ait >> 1) & 1) ^ 1, abort_s, E_MMA | 2)) { ok = false; break; }
                        tc_fence_after();
                        const uint32_t a_addr = s_base + C::OFF_WD + w * C::WD_BYTES;
                        const uint32_t w_addr = a_addr + C::WD_A;
                        const uint32_t d = tmem_base + slot * BN;
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const uint64_t ad = umma_desc_kmajor(a_addr + h * 2 * (BM * 16), BM * 16, 128);
                            const uint64_t bd = umma_desc_kmajor(w_addr + h * 2 * (BN * 16), BN * 16, 128);
                            mma_i8(d, ad, bd, idesc_i8, h);
                        }
                        tc_commit(bar(B_WD_EMPTY + w));
                        tc_commit(bar(B_ACC_FULL + slot));
                    }
                    if (ok && LCH > 0) {
                        const int slot = ait & 1;
                        if (!mbar_wait(bar(B_ACC_EMPTY + slot), ((ait >> 1) & 1) ^ 1, abort_s, E_MMA | 3)) { ok = false; break; }
                        for (int c = 0; c < LCH && ok; ++c, ++wit) {
                            const int w = wit % WD_STAGES;
                            if (!mbar_wait(bar(B_WD_FULL + w), (wit / WD_STAGES) & 1, abort_s, E_MMA | 4)) { ok = false; break; }
                            tc_fence_after();
                            const uint32_t a_addr = s_base + C::OFF_WD + w * C::WD_BYTES;
                            const uint32_t w_addr = a_addr + C::WD_A;
                            const uint32_t d = tmem_base + slot * BN;
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                const uint64_t ad = umma_desc_kmajor(a_addr + h * 2 * (BM * 16), BM * 16, 128);
                                const uint64_t bd = umma_desc_kmajor(w_addr + h * 2 * (BN * 16), BN * 16, 128);
                                mma_f16(d, ad, bd, idesc_lr, (c | h) ? 1u : 0u);
                            }
                            tc_commit(bar(B_WD_EMPTY + w));
                        }
                        if (ok) { tc_commit(bar(B_ACC_FULL + slot)); ++ait; }
                    }
                }
            }
        } else {
            // ================================ widen warps ================================
            const int wt = threadIdx.x - 64;
            uint32_t it = 0, wit = 0, sit = 0;
            bool ok = true;
            for (int t = t_begin; t < t_end && ok; ++t) {
                const int m0 = (t / NT) * BM, n0 = (t % NT) * BN;
                for (int g = 0; g < G; ++g, ++it, ++wit, ++sit) {
                    const int s = it % PK_STAGES, w = wit % WD_STAGES, c = sit % SC_STAGES;
                    if (!mbar_wait(bar(B_PK_FULL + s), (it / PK_STAGES) & 1, abort_s, E_WIDEN | 1)) { ok = false; break; }
                    if (!mbar_wait(bar(B_WD_EMPTY + w), ((wit / WD_STAGES) & 1) ^ 1, abort_s, E_WIDEN | 2)) { ok = false; break; }
                    if (!mbar_wait(bar(B_SC_EMPTY + c), ((sit / SC_STAGES) & 1) ^ 1, abort_s, E_WIDEN | 3)) { ok = false; break; }
                    const uint8_t* pk = smem + C::OFF_PK + s * C::PK_BYTES;
                    uint8_t* wd = smem + C::OFF_WD + w * C::WD_BYTES;
                    // 16-byte units: unit u = 32 blk + l -> row 16 blk + (l & 15), half l >> 4
#pragma unroll
                    for (int u = wt; u < (BM + BN) * 2; u += WIDEN_THREADS) {
                        const int blk = u >> 5, l = u & 31;
                        const int row_all = blk * 16 + (l & 15), half = l >> 4;
                        const bool is_w = row_all >= BM;
                        const int row = is_w ? row_all - BM : row_all;
                        const uint4 v = *reinterpret_cast<const uint4*>(pk + (is_w ? C::PK_A : 0) + row * 32 + half * 16);
                        uint4 lo, hi;
                        lo.x = (v.x << 4) & 0xF0F0F0F0u; hi.x = v.x & 0xF0F0F0F0u;
                        lo.y = (v.y << 4) & 0xF0F0F0F0u; hi.y = v.y & 0xF0F0F0F0u;
                        lo.z = (v.z << 4) & 0xF0F0F0F0u; hi.z = v.z & 0xF0F0F0F0u;
                        lo.w = (v.w << 4) & 0xF0F0F0F0u; hi.w = v.w & 0xF0F0F0F0u;
                        const int rows = is_w ? BN : BM;
                        uint8_t* dst = wd + (is_w ? C::WD_A : 0) + (2 * half) * rows * 16 + row * 16;
                        *reinterpret_cast<uint4*>(dst) = lo;
                        *reinterpret_cast<uint4*>(dst + rows * 16) = hi;
                    }
                    // scales -> fp32: ws[n]; as' = as / 256; cm = -MAGIC * as'
                    {
                        const T* as_t = reinterpret_cast<const T*>(pk + C::PK_A + C::PK_W);
                        const T* ws_t = reinterpret_cast<const T*>(pk + C::PK_A + C::PK_W + C::PK_AS);
                        float* ws_f = reinterpret_cast<float*>(smem + C::OFF_SC + c * C::SC_BYTES);
                        float* as_f = ws_f + BN;
                        float* cm_f = as_f + BM;
                        for (int i = wt; i < BN; i += WIDEN_THREADS) ws_f[i] = to_f32<T>(ws_t[i]);
                        for (int i = wt; i < BM; i += WIDEN_THREADS) {
                            const float a = to_f32<T>(as_t[i]) * (1.0f / 256.0f);
                            as_f[i] = a;
                            cm_f[i] = -MAGIC_F * a;
                        }
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(bar(B_WD_FULL + w));
                        mbar_arrive(bar(B_SC_FULL + c));
                        mbar_arrive(bar(B_PK_EMPTY + s));
                    }
                }
                if (!ok) break;
                // ---- low-rank operands: T(lora_act[m0.., 32 ranks]) and lora_up[n0.., 32 ranks]
                for (int lc = 0; lc < LCH; ++lc, ++wit) {
                    const int w = wit % WD_STAGES;
                    if (!mbar_wait(bar(B_WD_EMPTY + w), ((wit / WD_STAGES) & 1) ^ 1, abort_s, E_WIDEN | 4)) { ok = false; break; }
                    uint8_t* wd = smem + C::OFF_WD + w * C::WD_BYTES;
                    const int r0 = lc * 32, rw = min(32, p.R - r0);
                    for (int u = wt; u < BM * 4; u += WIDEN_THREADS) {
                        const int ch = u / BM, row = u % BM;
                        const int m = m0 + row;
                        uint4 o = make_uint4(0, 0, 0, 0);
                        if (m < p.M && ch * 8 < rw) {
                            const float4* src = reinterpret_cast<const float4*>(p.lora_act + (long long)m * p.stride_lam + r0 + ch * 8);
                            const float4 x = __ldg(src), y = __ldg(src + 1);
                            o.x = pack2<T>(x.x, x.y); o.y = pack2<T>(x.z, x.w);
                            o.z = pack2<T>(y.x, y.y); o.w = pack2<T>(y.z, y.w);
                        }
                        *reinterpret_cast<uint4*>(wd + ch * (BM * 16) + row * 16) = o;
                    }
                    for (int u = wt; u < BN * 4; u += WIDEN_THREADS) {
                        const int ch = u / BN, row = u % BN;
                        const int n = n0 + row;
                        uint4 o = make_uint4(0, 0, 0, 0);
                        if (n < p.N && ch * 8 < rw)
                            o = __ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(p.lora_up) + (long long)n * p.stride_lun + r0 + ch * 8));
                        *reinterpret_cast<uint4*>(wd + C::WD_A + ch * (BN * 16) + row * 16) = o;
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar(B_WD_FULL + w));
                }
            }
        }
    } else {
        // ================================ drain + epilogue ================================
        setmaxnreg_inc_200();
        const int dw = warp - 8;
        const int q = dw & 3;       // TMEM lane quarter this warp may read
        const int half = dw >> 2;   // column half
        const int row = q * 32 + lane;
        constexpr int COLS = C::COLS;
        const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
        uint8_t* stg = smem + C::OFF_STG + dw * 32 * C::STG_PITCH;
        uint32_t ait = 0, sit = 0;
        bool ok = true;
        float acc[COLS];

        for (int t = t_begin; t < t_end && ok; ++t) {
            const int m0 = (t / NT) * BM, n0 = (t % NT) * BN;
            const int nc0 = n0 + half * COLS;  // first global column of this thread
#pragma unroll
            for (int i = 0; i < COLS; ++i) acc[i] = 0.f;

            for (int g = 0; g < G; ++g, ++ait, ++sit) {
                const int slot = ait & 1, c = sit % SC_STAGES;
                if (!mbar_wait(bar(B_ACC_FULL + slot), (ait >> 1) & 1, abort_s, E_DRAIN | 1)) { ok = false; break; }
                if (!mbar_wait(bar(B_SC_FULL + c), (sit / SC_STAGES) & 1, abort_s, E_DRAIN | 2)) { ok = false; break; }
                tc_fence_after();
                const float* ws_f = reinterpret_cast<const float*>(smem + C::OFF_SC + c * C::SC_BYTES) + half * COLS;
                const float as_v = reinterpret_cast<const float*>(smem + C::OFF_SC + c * C::SC_BYTES)[BN + row];
                const float cm_v = reinterpret_cast<const float*>(smem + C::OFF_SC + c * C::SC_BYTES)[BN + BM + row];
                const uint32_t taddr = tmem_base + lane_addr + slot * BN + half * COLS;
                uint32_t v[2][16];
                tmem_ld16(taddr, v[0]);
#pragma unroll
                for (int j = 0; j < COLS / 16; ++j) {
                    tmem_wait_ld();
                    if (j + 1 < COLS / 16) tmem_ld16(taddr + (j + 1) * 16, v[(j + 1) & 1]);
#pragma unroll
                    for (int i = 0; i < 16; i += 4) {
                        const float4 w4 = *reinterpret_cast<const float4*>(ws_f + j * 16 + i);
                        const uint32_t* vv = v[j & 1];
                        acc[j * 16 + i + 0] = fmaf(fmaf(__uint_as_float(vv[i + 0] + MAGIC_BITS), as_v, cm_v), w4.x, acc[j * 16 + i + 0]);
                        acc[j * 16 + i + 1] = fmaf(fmaf(__uint_as_float(vv[i + 1] + MAGIC_BITS), as_v, cm_v), w4.y, acc[j * 16 + i + 1]);
                        acc[j * 16 + i + 2] = fmaf(fmaf(__uint_as_float(vv[i + 2] + MAGIC_BITS), as_v, cm_v), w4.z, acc[j * 16 + i + 2]);
                        acc[j * 16 + i + 3] = fmaf(fmaf(__uint_as_float(vv[i + 3] + MAGIC_BITS), as_v, cm_v), w4.w, acc[j * 16 + i + 3]);
                    }
                    if (DEBUG_P) {
                        const int m = m0 + row;
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const int n = nc0 + j * 16 + i;
                            if (m < p.M && n < p.N) p.p_out[((long long)g * p.M + m) * p.N + n] = ((int)v[j & 1][i]) >> 8;
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(bar(B_ACC_EMPTY + slot));
                    mbar_arrive(bar(B_SC_EMPTY + c));
                }
            }
            if (!ok) break;
            if (LCH > 0) {
                const int slot = ait & 1;
                if (!mbar_wait(bar(B_ACC_FULL + slot), (ait >> 1) & 1, abort_s, E_DRAIN | 3)) { ok = false; break; }
                tc_fence_after();
                const uint32_t taddr = tmem_base + lane_addr + slot * BN + half * COLS;
                uint32_t v[2][16];
                tmem_ld16(taddr, v[0]);
#pragma unroll
                for (int j = 0; j < COLS / 16; ++j) {
                    tmem_wait_ld();
                    if (j + 1 < COLS / 16) tmem_ld16(taddr + (j + 1) * 16, v[(j + 1) & 1]);
#pragma unroll
                    for (int i = 0; i < 16; ++i) acc[j * 16 + i] += __uint_as_float(v[j & 1][i]);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(B_ACC_EMPTY + slot));
                ++ait;
            }

            // ---------------- epilogue: bias, optional RMSNorm + RoPE, rounding, staged store ----------------
            const int m = m0 + row;
            if (p.bias) {
                const T* b = static_cast<const T*>(p.bias) + nc0;
#pragma unroll
                for (int i = 0; i < COLS; i += 8) {
                    if (nc0 + i < p.N) {
                        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(b + i));
                        float2 f;
                        f = unpack2<T>(raw.x); acc[i + 0] += f.x; acc[i + 1] += f.y;
                        f = unpack2<T>(raw.y); acc[i + 2] += f.x; acc[i + 3] += f.y;
                        f = unpack2<T>(raw.z); acc[i + 4] += f.x; acc[i + 5] += f.y;
                        f = unpack2<T>(raw.w); acc[i + 6] += f.x; acc[i + 7] += f.y;
                    }
                }
            }
            if (EPI == NB_EPI_QK_NORM_ROPE) {
                // BN = 256: each thread owns exactly one 128-wide head of its row
                const int part = nc0 / (p.N / 3);
                if (part < 2 && nc0 < p.N) {
                    float ss = 0.f;
#pragma unroll
                    for (int i = 0; i < COLS; ++i) ss = fmaf(acc[i], acc[i], ss);
                    const float rstd = rsqrtf(ss / 128.0f + p.eps);
                    const T* wn = static_cast<const T*>(part == 0 ? p.norm_q : p.norm_k);
                    const int mr = m < p.actual_m ? m % p.rot_rows : 0;
                    const float4* rr = reinterpret_cast<const float4*>(p.rot + (long long)mr * p.stride_rm);
#pragma unroll
                    for (int i = 0; i < COLS; i += 8) {
                        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(wn + i));
                        float wv[8];
                        float2 f;
                        f = unpack2<T>(raw.x); wv[0] = f.x; wv[1] = f.y;
                        f = unpack2<T>(raw.y); wv[2] = f.x; wv[3] = f.y;
                        f = unpack2<T>(raw.z); wv[4] = f.x; wv[5] = f.y;
                        f = unpack2<T>(raw.w); wv[6] = f.x; wv[7] = f.y;
#pragma unroll
                        for (int pr = 0; pr < 4; pr += 2) {
                            const float4 sc = __ldg(rr + (i + 2 * pr) / 4);  // (sin, cos, sin, cos) of two pairs
                            {
                                const float xe = acc[i + 2 * pr] * rstd * wv[2 * pr];
                                const float xo = acc[i + 2 * pr + 1] * rstd * wv[2 * pr + 1];
                                acc[i + 2 * pr] = xe * sc.y - xo * sc.x;
                                acc[i + 2 * pr + 1] = xe * sc.x + xo * sc.y;
                            }
                            {
                                const float xe = acc[i + 2 * pr + 2] * rstd * wv[2 * pr + 2];
                                const float xo = acc[i + 2 * pr + 3] * rstd * wv[2 * pr + 3];
                                acc[i + 2 * pr + 2] = xe * sc.w - xo * sc.z;
                                acc[i + 2 * pr + 3] = xe * sc.z + xo * sc.w;
                            }
                        }
                    }
                }
            }
            // round and transpose through the per-warp staging tile: thread -> its row, then 2 rows per pass
            __syncwarp();
#pragma unroll
            for (int i = 0; i < COLS; i += 8) {
                uint4 o;
                o.x = pack2<T>(acc[i + 0], acc[i + 1]); o.y = pack2<T>(acc[i + 2], acc[i + 3]);
                o.z = pack2<T>(acc[i + 4], acc[i + 5]); o.w = pack2<T>(acc[i + 6], acc[i + 7]);
                *reinterpret_cast<uint4*>(stg + lane * C::STG_PITCH + i * 2) = o;
            }
            __syncwarp();
            {
                constexpr int UPR = COLS / 8;        // 16-byte units per row
                constexpr int RPP = 32 / UPR;        // rows per pass
                const int ur = lane / UPR, uc = lane % UPR;
#pragma unroll
                for (int r = 0; r < 32; r += RPP) {
                    const int rr = r + ur;
                    const int mm = m0 + q * 32 + rr, nn = nc0 + uc * 8;
                    const uint4 o = *reinterpret_cast<const uint4*>(stg + rr * C::STG_PITCH + uc * 16);
                    if (mm < p.actual_m && nn < p.N)
                        *reinterpret_cast<uint4*>(static_cast<T*>(p.out) + (long long)mm * p.stride_om + nn) = o;
                }
            }
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_s && p.status) atomicCAS(p.status, 0, *abort_s);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

// 2-D row-major tensor map: `inner` elements per row, `rows` rows, row pitch in bytes, box (bi x br)
static bool make_map(CUtensorMap* m, CUtensorMapDataType dt, int esize, const void* base, uint64_t inner, uint64_t rows,
                     uint64_t pitch_bytes, uint32_t bi, uint32_t br) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {inner, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {bi, br};
    cuuint32_t estr[2] = {1, 1};
    (void)esize;
    return fn(m, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) ==
           CUDA_SUCCESS;
}

template <int BN, int EPI, typename T, bool DEBUG_P>
static int launch_t(const nb_gemm_args* a, const TcParams& p, cudaStream_t s) {
    using C = Cfg<BN>;
    CUtensorMap tm_a, tm_w, tm_as, tm_ws;
    const CUtensorMapDataType sdt = CU_TENSOR_MAP_DATA_TYPE_UINT16;  // scales move as opaque 16-bit words
    if (!make_map(&tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a->act, a->K / 2, a->M, a->stride_am, 32, BM) ||
        !make_map(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a->wgt, a->K / 2, a->N, a->stride_wn, 32, BN) ||
        !make_map(&tm_as, sdt, 2, a->ascales, a->M, a->K / 64, a->stride_asg * 2, BM, 1) ||
        !make_map(&tm_ws, sdt, 2, a->wscales, a->N, a->K / 64, a->stride_wsg * 2, BN, 1))
        return NB_ERR_UNSUPPORTED;
    int dev = 0, sms = 0;
    NB_CUDA_CHECK(cudaGetDevice(&dev));
    NB_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int total = ((a->M + BM - 1) / BM) * ((a->N + BN - 1) / BN);
    const int grid = total < sms ? total : sms;
    auto kern = gemm_tc_kernel<BN, EPI, T, DEBUG_P>;
    NB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    kern<<<grid, NTHREADS, C::SMEM_BYTES, s>>>(tm_a, tm_w, tm_as, tm_ws, p);
    NB_CUDA_CHECK(cudaGetLastError());
    return NB_OK;
}

}  // namespace tc

// Why the tcgen05 kernel cannot take this call, or nullptr (the role of `unsupported_reason`,
// nunchaku/ops/triton/native/w4a4.py:164-231).
const char* tc_unsupported_reason(const nb_gemm_args* a, const void* epi, int epi_kind) {
    if (a->fp4) return "NVFP4";
    if (a->wcscales || a->alpha != 1.0f || a->fuse_silu) return "wcscales / alpha / SiLU";
    if (epi_kind != NB_EPI_STORE && epi_kind != NB_EPI_QK_NORM_ROPE) return "epilogue";
    if (a->K % 64 || a->N % 8 || a->M < 1) return "K % 64, N % 8";
    if (!aligned16(a->act) || !aligned16(a->wgt) || a->stride_am % 16 || a->stride_wn % 16) return "act / wgt alignment";
    if (!aligned16(a->ascales) || !aligned16(a->wscales) || a->stride_asg % 8 || a->stride_wsg % 8) return "scale alignment";
    if (a->out && (!aligned16(a->out) || a->stride_om % 8)) return "out alignment";
    if (!a->out) return "no 16-bit output";
    if (a->bias && !aligned16(a->bias)) return "bias alignment";
    if (a->R > 0) {
        if (a->R % 16 || !a->lora_act || !a->lora_up) return "rank";
        if (!aligned16(a->lora_act) || a->stride_lam % 4 || !aligned16(a->lora_up) || a->stride_lun % 8) return "LoRA alignment";
    }
    if (epi_kind == NB_EPI_QK_NORM_ROPE) {
        const nb_qk_args* q = static_cast<const nb_qk_args*>(epi);
        if (a->N % 3 || (a->N / 3) % 128) return "N is not three sets of 128-wide heads";
        if (!aligned16(q->norm_q) || !aligned16(q->norm_k) || !aligned16(q->rot) || q->stride_rm % 4) return "QK alignment";
    }
    return nullptr;
}

int launch_tc(const nb_gemm_args* a, const void* epi, int epi_kind, int32_t* p_out, cudaStream_t s) {
    tc::TcParams p = {};
    p.out = a->out; p.bias = a->bias; p.lora_act = static_cast<const float*>(a->lora_act); p.lora_up = a->lora_up;
    p.p_out = p_out;
    p.M = a->M; p.N = a->N; p.K = a->K; p.actual_m = a->actual_m; p.R = a->R;
    p.act_unsigned = a->act_unsigned;
    p.stride_om = a->stride_om; p.stride_lam = a->stride_lam; p.stride_lun = a->stride_lun;
    p.status = static_cast<int*>(a->status);
    if (epi_kind == NB_EPI_QK_NORM_ROPE) {
        const nb_qk_args* q = static_cast<const nb_qk_args*>(epi);
        p.norm_q = q->norm_q; p.norm_k = q->norm_k; p.rot = q->rot; p.stride_rm = q->stride_rm;
        p.rot_rows = q->rot_rows; p.eps = q->eps;
    }
    const bool bf = a->dtype == NB_DTYPE_BF16;
    if (p_out) {
        return bf ? tc::launch_t<256, NB_EPI_STORE, __nv_bfloat16, true>(a, p, s)
                  : tc::launch_t<256, NB_EPI_STORE, __half, true>(a, p, s);
    }
    if (epi_kind == NB_EPI_QK_NORM_ROPE)
        return bf ? tc::launch_t<256, NB_EPI_QK_NORM_ROPE, __nv_bfloat16, false>(a, p, s)
                  : tc::launch_t<256, NB_EPI_QK_NORM_ROPE, __half, false>(a, p, s);
    // few tiles: halve the tile width so more SMs get work
    const long long tiles256 = (long long)((a->M + 127) / 128) * ((a->N + 255) / 256);
    if (tiles256 < 100)
        return bf ? tc::launch_t<128, NB_EPI_STORE, __nv_bfloat16, false>(a, p, s)
                  : tc::launch_t<128, NB_EPI_STORE, __half, false>(a, p, s);
    return bf ? tc::launch_t<256, NB_EPI_STORE, __nv_bfloat16, false>(a, p, s)
              : tc::launch_t<256, NB_EPI_STORE, __half, false>(a, p, s);
}

}  // namespace nb

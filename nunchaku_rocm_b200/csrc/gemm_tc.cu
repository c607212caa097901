// W4A4 int4 GEMM on the 5th-generation tensor cores (tcgen05.mma kind::i8, int32 accumulators in
// tensor memory), with the low-rank branch and the fused epilogues.
//
// Arithmetic contract (reference: nunchaku/ops/triton/gemm_w4a4.py:446-488 and :155-209): for every
// 64-wide K group g one EXACT int32 dot p_g[m,n]; acc += float(p_g) * as[g,m] * ws[g,n] in fp32;
// then + T(lora_act) . lora_up^T (16-bit operands, fp32 accumulate), + bias, one rounding to T.
//
// Pipeline of one persistent CTA (512 threads, one CTA per SM, static contiguous range of 128 x 128 tiles):
//   warp 0      TMA producer: packed int4 rows of A and W (128 x 32 B each, 32-byte swizzle) of one K group,
//               plus that group's scale rows, into a ring (no multicast, no cluster).
//   warps 2-7   widen: nibble n -> int8 16*n (n << 4 keeps the sign in the top bit; the factor 256 on the
//               product is folded into the activation scale) written in the K-major no-swizzle UMMA layout
//               (8-row x 16-byte core matrices, one 16-byte K chunk after another); scales converted to
//               fp32.  The same permutation of k inside the group is applied to A and W, which a dot
//               product does not see.  For the low-rank branch they stage T(lora_act) and lora_up as
//               bf16/fp16 operands through the same buffers.
//   warp 1      MMA issuer: two 128 x 128 x 32 kind::i8 MMAs per group into one of FOUR tensor-memory
//               slots, so the tensor pipe runs up to three groups ahead of the drain; tcgen05.commit
//               releases the operand buffer and publishes the slot.  The low-rank product is kind::f16
//               into an fp32 slot of the same ring.
//   warps 8-15  drain: a warp owns 32 rows x 64 columns.  tcgen05.ld.16x256b gives a thread the
//               accumulator-fragment layout (4 rows x 16 columns), so it needs 4 row scales and 16 column
//               scales per group; int -> float by the magic-number add, then two packed fp32x2 FMAs per
//               column pair.  Loads of the next 16-lane chunk (of this or the next group) are in flight
//               while a chunk is scaled.  After the last group: bias, optional per-head RMSNorm + RoPE,
//               rounding, and a coalesced store through a padded per-warp staging tile.
// Every wait on an mbarrier is bounded (~2 s); on expiry the CTA records a code in the status word,
// unwinds without touching more data and frees its tensor memory.
#include <cuda.h>

#include <cstdlib>
#include <type_traits>

#include "nb_common.cuh"

namespace nb {
namespace tc {

constexpr int BM = 128;
constexpr int BN = 128;
constexpr int PK_STAGES = 6;
constexpr int WD_STAGES = 4;
constexpr int SC_STAGES = 6;
constexpr int NSLOT = 4;            // tensor-memory accumulator slots of BN columns
constexpr int NTHREADS = 512;
constexpr int WIDEN_THREADS = 192;  // warps 2..7
constexpr int WIDEN_WARPS = 6;
constexpr int DRAIN_WARPS = 8;      // warps 8..15
constexpr int COLS = BN / 2;        // columns one drain warp owns
constexpr uint32_t MAGIC_BITS = 0x4B400000u;  // 1.5 * 2^23
constexpr float MAGIC_F = 12582912.0f;

struct Cfg {
    static constexpr int PK_A = BM * 32, PK_W = BN * 32, PK_AS = BM * 2, PK_WS = BN * 2;
    static constexpr int PK_BYTES = PK_A + PK_W + PK_AS + PK_WS;
    static constexpr int WD_A = BM * 64, WD_W = BN * 64;
    static constexpr int WD_BYTES = WD_A + WD_W;
    static constexpr int SC_BYTES = BN * 4 + BM * 4 * 2;
    static constexpr int STG_PITCH = COLS * 2 + 16;
    static constexpr int STG_BYTES = DRAIN_WARPS * 32 * STG_PITCH;
    static constexpr int XCH_BYTES = DRAIN_WARPS * 32 * 4;  // per-row partial sums exchanged between column halves
    static constexpr int OFF_PK = 0;
    static constexpr int OFF_WD = OFF_PK + PK_STAGES * PK_BYTES;
    static constexpr int OFF_SC = OFF_WD + WD_STAGES * WD_BYTES;
    static constexpr int OFF_STG = OFF_SC + SC_STAGES * SC_BYTES;
    static constexpr int OFF_XCH = OFF_STG + STG_BYTES;
    static constexpr int OFF_BAR = OFF_XCH + XCH_BYTES;
    static constexpr int SMEM_BYTES = OFF_BAR + 512 + 1024;  // + slack to align the base to 1 KB
    static constexpr int TMEM_COLS = NSLOT * BN;             // 512
};
static_assert(Cfg::OFF_WD % 1024 == 0 && Cfg::PK_BYTES % 256 == 0, "TMA destinations must stay 256-byte aligned");

enum {  // barrier indices
    B_PK_FULL = 0,
    B_PK_EMPTY = B_PK_FULL + PK_STAGES,
    B_WD_FULL = B_PK_EMPTY + PK_STAGES,
    B_WD_EMPTY = B_WD_FULL + WD_STAGES,
    B_SC_FULL = B_WD_EMPTY + WD_STAGES,
    B_SC_EMPTY = B_SC_FULL + SC_STAGES,
    B_ACC_FULL = B_SC_EMPTY + SC_STAGES,
    B_ACC_EMPTY = B_ACC_FULL + NSLOT,
    B_XCH = B_ACC_EMPTY + NSLOT,  // one per TMEM lane quarter: the two warps that share rows
    B_COUNT = B_XCH + 4
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

#ifdef NB_TRACE
// Timeline instrumentation (debug builds only): CTA 0 records clock64() per pipeline event and step.
__device__ unsigned long long* g_trace = nullptr;
#define NB_TR(step, ev)                                                                      \
    do {                                                                                     \
        if (g_trace && blockIdx.x == 0 && (step) < 256) g_trace[(step)*16 + (ev)] = clock64(); \
    } while (0)
#else
#define NB_TR(step, ev) \
    do {                \
    } while (0)
#endif

// error codes written to *status: role * 16 + barrier kind
enum { E_PROD = 0x10, E_WIDEN = 0x20, E_MMA = 0x30, E_DRAIN = 0x40 };

template <int EPI, typename T, bool DEBUG_P>
__global__ void __launch_bounds__(NTHREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w,
               const __grid_constant__ CUtensorMap tm_as, const __grid_constant__ CUtensorMap tm_ws,
               const TcParams p) {
    using C = Cfg;
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
        for (int i = 0; i < NSLOT; ++i) { mbar_init(bar(B_ACC_FULL + i), 1); mbar_init(bar(B_ACC_EMPTY + i), DRAIN_WARPS); }
        for (int i = 0; i < 4; ++i) mbar_init(bar(B_XCH + i), 2);
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
        setmaxnreg_dec_80();
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
                        if (!mbar_wait(bar(B_PK_EMPTY + s), ((it / PK_STAGES) & 1) ^ 1, abort_s, E_PROD | 1, 128)) { ok = false; break; }
                        NB_TR(it, 0);
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
                const uint32_t f16fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
                const uint32_t idesc_lr = umma_idesc(1u, f16fmt, f16fmt, BN);
                uint32_t wit = 0, ait = 0;
                bool ok = true;
                for (int t = t_begin; t < t_end && ok; ++t) {
                    for (int g = 0; g < G && ok; ++g, ++wit, ++ait) {
                        const int w = wit % WD_STAGES, slot = ait % NSLOT;
                        if (!mbar_wait(bar(B_WD_FULL + w), (wit / WD_STAGES) & 1, abort_s, E_MMA | 1)) { ok = false; break; }
                        NB_TR(ait, 4);
                        if (!mbar_wait(bar(B_ACC_EMPTY + slot), ((ait / NSLOT) & 1) ^ 1, abort_s, E_MMA | 2)) { ok = false; break; }
                        NB_TR(ait, 5);
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
                        const int slot = ait % NSLOT;
                        if (!mbar_wait(bar(B_ACC_EMPTY + slot), ((ait / NSLOT) & 1) ^ 1, abort_s, E_MMA | 3)) { ok = false; break; }
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
                    if (!mbar_wait(bar(B_PK_FULL + s), (it / PK_STAGES) & 1, abort_s, E_WIDEN | 1, 128)) { ok = false; break; }
                    if (wt == 0) NB_TR(sit, 1);
                    if (!mbar_wait(bar(B_WD_EMPTY + w), ((wit / WD_STAGES) & 1) ^ 1, abort_s, E_WIDEN | 2, 128)) { ok = false; break; }
                    if (!mbar_wait(bar(B_SC_EMPTY + c), ((sit / SC_STAGES) & 1) ^ 1, abort_s, E_WIDEN | 3, 128)) { ok = false; break; }
                    if (wt == 0) NB_TR(sit, 2);
                    const uint8_t* pk = smem + C::OFF_PK + s * C::PK_BYTES;
                    uint8_t* wd = smem + C::OFF_WD + w * C::WD_BYTES;
                    // 16-byte units: unit u = 32 blk + l -> row 16 blk + (l & 15), half l >> 4.  The TMA wrote the
                    // rows with the 32-byte swizzle: the two 16-byte halves of a row swap when bit 2 of the row is
                    // set, which makes the 16 rows a half-warp reads hit 16 different bank groups.
#ifdef NB_EXP_NOWIDEN
                    for (int u = wt; u < 0; u += WIDEN_THREADS) {
#else
                    for (int u = wt; u < (BM + BN) * 2; u += WIDEN_THREADS) {
#endif
                        const int blk = u >> 5, l = u & 31;
                        const int row_all = blk * 16 + (l & 15), half = l >> 4;
                        const bool is_w = row_all >= BM;
                        const int row = is_w ? row_all - BM : row_all;
                        const int phys_half = half ^ ((row >> 2) & 1);
                        const uint4 v = *reinterpret_cast<const uint4*>(pk + (is_w ? C::PK_A : 0) + row * 32 + phys_half * 16);
                        uint4 lo, hi;
                        lo.x = (v.x << 4) & 0xF0F0F0F0u; hi.x = v.x & 0xF0F0F0F0u;
                        lo.y = (v.y << 4) & 0xF0F0F0F0u; hi.y = v.y & 0xF0F0F0F0u;
                        lo.z = (v.z << 4) & 0xF0F0F0F0u; hi.z = v.z & 0xF0F0F0F0u;
                        lo.w = (v.w << 4) & 0xF0F0F0F0u; hi.w = v.w & 0xF0F0F0F0u;
                        const int rows = is_w ? BN : BM;
                        uint8_t* dst = wd + (is_w ? C::WD_A : 0) + (2 * half) * rows * 16 + row * 16;
#ifndef NB_EXP_NOSTS
                        *reinterpret_cast<uint4*>(dst) = lo;
                        *reinterpret_cast<uint4*>(dst + rows * 16) = hi;
#else
                        if (lo.x == 0x12345 && hi.y == 0x777) *reinterpret_cast<uint4*>(dst) = lo;
#endif
                    }
                    // scales -> fp32: ws[n] (permuted for the drain's fragment layout); as' = as / 256; cm = -MAGIC * as'
                    {
                        const T* as_t = reinterpret_cast<const T*>(pk + C::PK_A + C::PK_W);
                        const T* ws_t = reinterpret_cast<const T*>(pk + C::PK_A + C::PK_W + C::PK_AS);
                        float* ws_f = reinterpret_cast<float*>(smem + C::OFF_SC + c * C::SC_BYTES);
                        float* as_f = ws_f + BN;
                        float* cm_f = as_f + BM;
                        if (wt < BN) {
                            // column i of the tile -> [warp half][pair of 8-col blocks][tig][4]: one 128-bit load of a
                            // drain thread is (cols c, c+1 of block j, cols c, c+1 of block j+1)
                            const int i = wt;
                            const int hf = i / COLS, cc = i % COLS;
                            const int blk = cc >> 3, tg = (cc >> 1) & 3, e = cc & 1;
                            ws_f[hf * COLS + (blk >> 1) * 16 + tg * 4 + (blk & 1) * 2 + e] = to_f32<T>(ws_t[i]);
                        }
                        if (wt < BM) {
                            const float a = to_f32<T>(as_t[wt]) * (1.0f / 256.0f);
                            as_f[wt] = a;
                            cm_f[wt] = -MAGIC_F * a;
                        }
                    }
#ifndef NB_EXP_NOFENCE
                    fence_proxy_async_smem();
#endif
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(bar(B_WD_FULL + w));
                        mbar_arrive(bar(B_SC_FULL + c));
                        mbar_arrive(bar(B_PK_EMPTY + s));
                    }
                    if (wt == 0) NB_TR(sit, 3);
                }
                if (!ok) break;
                // ---- low-rank operands: T(lora_act[m0.., 32 ranks]) and lora_up[n0.., 32 ranks]
                for (int lc = 0; lc < LCH; ++lc, ++wit) {
                    const int w = wit % WD_STAGES;
                    if (!mbar_wait(bar(B_WD_EMPTY + w), ((wit / WD_STAGES) & 1) ^ 1, abort_s, E_WIDEN | 4, 128)) { ok = false; break; }
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
        // A warp owns 32 rows (its TMEM lane quarter) x 64 columns.  tcgen05.ld.16x256b.x8 hands a thread, for one
        // 16-lane block, rows {gid, gid + 8} and the column pairs 8 j + 2 tig + {0, 1}, j = 0..7: register
        // 4 j + 2 rs + e.  The two 16-lane blocks of a group are two "chunks"; while one is scaled the load of the
        // next chunk (of this group or, when the tensor pipe is ahead, of the next group) is in flight.
        setmaxnreg_inc_176();
        const int dw = warp - 8;
        const int q = dw & 3;       // TMEM lane quarter this warp may read
        const int half = dw >> 2;   // column half of the tile
        const int gid = lane >> 2, tig = lane & 3;
        uint8_t* stg = smem + C::OFF_STG + dw * 32 * C::STG_PITCH;
        float* xch = reinterpret_cast<float*>(smem + C::OFF_XCH);
        const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16) + half * COLS;
        uint32_t ait = 0, sit = 0, xph = 0;
        bool ok = true;
        uint64_t acc[32];  // [chunk lb][j][row select] pairs of fp32
        uint32_t v[2][32];

        for (int t = t_begin; t < t_end && ok; ++t) {
            const int m0 = (t / NT) * BM, n0 = (t % NT) * BN;
            const int nc0 = n0 + half * COLS;  // first global column of this warp
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[i] = 0ull;
            const int nsteps = G + (LCH > 0 ? 1 : 0);

            // chunk 0 of the tile's first group
            if (!mbar_wait(bar(B_ACC_FULL + ait % NSLOT), (ait / NSLOT) & 1, abort_s, E_DRAIN | 1)) { ok = false; break; }
            tc_fence_after();
            tmem_ld_16x256b_x8(lane_base + (ait % NSLOT) * BN, v[0]);

            for (int g = 0; g < nsteps; ++g, ++ait) {
                const bool lowrank = g >= G;
                const int slot = ait % NSLOT;
                const int c = sit % SC_STAGES;
                if (dw == 0 && lane == 0) NB_TR(ait, 6);
                if (!lowrank && !mbar_wait(bar(B_SC_FULL + c), (sit / SC_STAGES) & 1, abort_s, E_DRAIN | 2)) { ok = false; break; }
                if (dw == 0 && lane == 0) NB_TR(ait, 7);
                const float* sc_f = reinterpret_cast<const float*>(smem + C::OFF_SC + c * C::SC_BYTES);
                const float4* ws4 = reinterpret_cast<const float4*>(sc_f + half * COLS) + tig;
                bool prefetched = false;
#pragma unroll
                for (int lb = 0; lb < 2; ++lb) {
                    tmem_wait_ld();  // chunk lb of this group is in v[lb]
                    if (dw == 0 && lane == 0) NB_TR(ait, 9 + 3 * lb);
                    if (lb == 0) {
                        tmem_ld_16x256b_x8(lane_base + (16u << 16) + slot * BN, v[1]);
                    } else {
                        // both chunks of the slot are in registers: hand it back, then start on the next group if
                        // its accumulator is already complete
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar(B_ACC_EMPTY + slot));
                        if (g + 1 < nsteps) {
                            const uint32_t nx = ait + 1;
                            prefetched = mbar_try_wait(bar(B_ACC_FULL + nx % NSLOT), (nx / NSLOT) & 1);
                            if (prefetched) {
                                tc_fence_after();
                                tmem_ld_16x256b_x8(lane_base + (nx % NSLOT) * BN, v[0]);
                            }
                        }
                    }
                    if (dw == 0 && lane == 0) NB_TR(ait, 10 + 3 * lb);
                    uint32_t(&vv)[32] = v[lb];
#ifdef NB_EXP_NOMATH
                    if (false) {
#else
                    if (!lowrank) {
#endif
                        uint64_t as2[2], cm2[2];
#pragma unroll
                        for (int rs = 0; rs < 2; ++rs) {
                            const int row = q * 32 + lb * 16 + rs * 8 + gid;
                            as2[rs] = pack_f32x2(sc_f[BN + row], sc_f[BN + row]);
                            cm2[rs] = pack_f32x2(sc_f[BN + BM + row], sc_f[BN + BM + row]);
                        }
#pragma unroll
                        for (int j = 0; j < 8; j += 2) {
                            const float4 w = ws4[(j >> 1) * 4];
                            const uint64_t w0 = pack_f32x2(w.x, w.y), w1 = pack_f32x2(w.z, w.w);
#pragma unroll
                            for (int jj = 0; jj < 2; ++jj) {
#pragma unroll
                                for (int rs = 0; rs < 2; ++rs) {
                                    const int vi = 4 * (j + jj) + 2 * rs;
                                    const uint64_t x = pack_u32x2(vv[vi] + MAGIC_BITS, vv[vi + 1] + MAGIC_BITS);
                                    const uint64_t tt = fma_f32x2(x, as2[rs], cm2[rs]);
                                    uint64_t& a = acc[(lb * 8 + j + jj) * 2 + rs];
                                    a = fma_f32x2(tt, jj ? w1 : w0, a);
                                }
                            }
                        }
                        if (DEBUG_P) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                const int m = m0 + q * 32 + lb * 16 + ((i >> 1) & 1) * 8 + gid;
                                const int n = nc0 + (i >> 2) * 8 + 2 * tig + (i & 1);
                                if (m < p.M && n < p.N) p.p_out[((long long)g * p.M + m) * p.N + n] = ((int)vv[i]) >> 8;
                            }
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
#pragma unroll
                            for (int rs = 0; rs < 2; ++rs) {
                                uint64_t& a = acc[(lb * 8 + j) * 2 + rs];
                                a = add_f32x2(a, pack_u32x2(vv[4 * j + 2 * rs], vv[4 * j + 2 * rs + 1]));
                            }
                    }
                }
                if (!lowrank) {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar(B_SC_EMPTY + c));
                    ++sit;
                }
                if (g + 1 < nsteps && !prefetched) {
                    const uint32_t nx = ait + 1;
                    if (!mbar_wait(bar(B_ACC_FULL + nx % NSLOT), (nx / NSLOT) & 1, abort_s, E_DRAIN | 3)) { ok = false; break; }
                    tc_fence_after();
                    tmem_ld_16x256b_x8(lane_base + (nx % NSLOT) * BN, v[0]);
                }
                if (dw == 0 && lane == 0) NB_TR(ait, 8);
            }
            if (!ok) break;

            // ---------------- epilogue: bias, optional RMSNorm + RoPE, rounding, staged store ----------------
            // element (lb, j, rs, e): row q*32 + lb*16 + rs*8 + gid, column nc0 + 8j + 2 tig + e
            float sumsq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int lb = 0; lb < 2; ++lb)
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int col = nc0 + 8 * j + 2 * tig;
                    float2 b = make_float2(0.f, 0.f);
                    if (p.bias && col < p.N) b = unpack2<T>(__ldg(reinterpret_cast<const uint32_t*>(static_cast<const T*>(p.bias) + col)));
#pragma unroll
                    for (int rs = 0; rs < 2; ++rs) {
                        float2 a = unpack_f32x2(acc[(lb * 8 + j) * 2 + rs]);
                        a.x += b.x;
                        a.y += b.y;
                        acc[(lb * 8 + j) * 2 + rs] = pack_f32x2(a.x, a.y);
                        if (EPI == NB_EPI_QK_NORM_ROPE) sumsq[lb * 2 + rs] = fmaf(a.x, a.x, fmaf(a.y, a.y, sumsq[lb * 2 + rs]));
                    }
                }
            if (EPI == NB_EPI_QK_NORM_ROPE) {
                // the 128-column tile is one head: the 4 lanes of a quad share a row inside the warp, and the
                // warp that owns the other 64 columns of the same rows is dw ^ 4
                const int part = n0 / (p.N / 3);
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    float s = sumsq[r];
                    s += __shfl_xor_sync(0xffffffffu, s, 1);
                    s += __shfl_xor_sync(0xffffffffu, s, 2);
                    sumsq[r] = s;
                    if (tig == 0) xch[dw * 32 + (r >> 1) * 16 + (r & 1) * 8 + gid] = s;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(B_XCH + q));
                if (!mbar_wait(bar(B_XCH + q), xph & 1, abort_s, E_DRAIN | 4)) { ok = false; break; }
                ++xph;
                if (part < 2) {
                    float rstd[4];
#pragma unroll
                    for (int r = 0; r < 4; ++r)
                        rstd[r] = rsqrtf((sumsq[r] + xch[(dw ^ 4) * 32 + (r >> 1) * 16 + (r & 1) * 8 + gid]) / 128.0f + p.eps);
                    const T* wn = static_cast<const T*>(part == 0 ? p.norm_q : p.norm_k);
#pragma unroll
                    for (int lb = 0; lb < 2; ++lb)
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const int hc = half * COLS + 8 * j + 2 * tig;  // column inside the head (even)
                            const float2 w = unpack2<T>(__ldg(reinterpret_cast<const uint32_t*>(wn + hc)));
#pragma unroll
                            for (int rs = 0; rs < 2; ++rs) {
                                const int m = m0 + q * 32 + lb * 16 + rs * 8 + gid;
                                const int mr = m < p.actual_m ? m % p.rot_rows : 0;
                                const float2 sc = __ldg(reinterpret_cast<const float2*>(p.rot + (long long)mr * p.stride_rm + hc));
                                const float2 a = unpack_f32x2(acc[(lb * 8 + j) * 2 + rs]);
                                const float xe = a.x * rstd[lb * 2 + rs] * w.x, xo = a.y * rstd[lb * 2 + rs] * w.y;
                                acc[(lb * 8 + j) * 2 + rs] = pack_f32x2(xe * sc.y - xo * sc.x, xe * sc.x + xo * sc.y);
                            }
                        }
                }
                // the partner must have read this warp's sums before the next tile overwrites them
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(B_XCH + q));
                if (!mbar_wait(bar(B_XCH + q), xph & 1, abort_s, E_DRAIN | 5)) { ok = false; break; }
                ++xph;
            }
            // round, transpose through the per-warp staging tile, store whole 128-byte row segments
            __syncwarp();
#pragma unroll
            for (int lb = 0; lb < 2; ++lb)
#pragma unroll
                for (int j = 0; j < 8; ++j)
#pragma unroll
                    for (int rs = 0; rs < 2; ++rs) {
                        const float2 a = unpack_f32x2(acc[(lb * 8 + j) * 2 + rs]);
                        *reinterpret_cast<uint32_t*>(stg + (lb * 16 + rs * 8 + gid) * C::STG_PITCH + (8 * j + 2 * tig) * 2) = pack2<T>(a.x, a.y);
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
static bool make_map(CUtensorMap* m, CUtensorMapDataType dt, const void* base, uint64_t inner, uint64_t rows,
                     uint64_t pitch_bytes, uint32_t bi, uint32_t br, CUtensorMapSwizzle sw) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {inner, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {bi, br};
    cuuint32_t estr[2] = {1, 1};
    return fn(m, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int EPI, typename T, bool DEBUG_P>
static int launch_t(const nb_gemm_args* a, const TcParams& p, cudaStream_t s) {
    using C = Cfg;
    CUtensorMap tm_a, tm_w, tm_as, tm_ws;
    const CUtensorMapDataType sdt = CU_TENSOR_MAP_DATA_TYPE_UINT16;  // scales move as opaque 16-bit words
    if (!make_map(&tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, a->act, a->K / 2, a->M, a->stride_am, 32, BM, CU_TENSOR_MAP_SWIZZLE_32B) ||
        !make_map(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, a->wgt, a->K / 2, a->N, a->stride_wn, 32, BN, CU_TENSOR_MAP_SWIZZLE_32B) ||
        !make_map(&tm_as, sdt, a->ascales, a->M, a->K / 64, a->stride_asg * 2, BM, 1, CU_TENSOR_MAP_SWIZZLE_NONE) ||
        !make_map(&tm_ws, sdt, a->wscales, a->N, a->K / 64, a->stride_wsg * 2, BN, 1, CU_TENSOR_MAP_SWIZZLE_NONE))
        return NB_ERR_UNSUPPORTED;
    int dev = 0, sms = 0;
    NB_CUDA_CHECK(cudaGetDevice(&dev));
    NB_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int total = ((a->M + BM - 1) / BM) * ((a->N + BN - 1) / BN);
    const int grid = total < sms ? total : sms;
    auto kern = gemm_tc_kernel<EPI, T, DEBUG_P>;
    NB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    kern<<<grid, NTHREADS, C::SMEM_BYTES, s>>>(tm_a, tm_w, tm_as, tm_ws, p);
    NB_CUDA_CHECK(cudaGetLastError());
    return NB_OK;
}

}  // namespace tc

#ifdef NB_TRACE
extern "C" int nb_debug_set_trace(void* ptr) {
    unsigned long long* v = static_cast<unsigned long long*>(ptr);
    return cudaMemcpyToSymbol(tc::g_trace, &v, sizeof(v)) == cudaSuccess ? 0 : 3;
}
#endif

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
    if (a->bias && (reinterpret_cast<uintptr_t>(a->bias) & 3)) return "bias alignment";
    if (a->R > 0) {
        if (a->R % 16 || !a->lora_act || !a->lora_up) return "rank";
        if (!aligned16(a->lora_act) || a->stride_lam % 4 || !aligned16(a->lora_up) || a->stride_lun % 8) return "LoRA alignment";
    }
    if (epi_kind == NB_EPI_QK_NORM_ROPE) {
        const nb_qk_args* q = static_cast<const nb_qk_args*>(epi);
        if (a->N % 3 || (a->N / 3) % 128) return "N is not three sets of 128-wide heads";
        if ((reinterpret_cast<uintptr_t>(q->norm_q) & 3) || (reinterpret_cast<uintptr_t>(q->norm_k) & 3) ||
            (reinterpret_cast<uintptr_t>(q->rot) & 7) || q->stride_rm % 2)
            return "QK alignment";
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
    if (p_out)
        return bf ? tc::launch_t<NB_EPI_STORE, __nv_bfloat16, true>(a, p, s) : tc::launch_t<NB_EPI_STORE, __half, true>(a, p, s);
    if (epi_kind == NB_EPI_QK_NORM_ROPE)
        return bf ? tc::launch_t<NB_EPI_QK_NORM_ROPE, __nv_bfloat16, false>(a, p, s)
                  : tc::launch_t<NB_EPI_QK_NORM_ROPE, __half, false>(a, p, s);
    return bf ? tc::launch_t<NB_EPI_STORE, __nv_bfloat16, false>(a, p, s) : tc::launch_t<NB_EPI_STORE, __half, false>(a, p, s);
}

}  // namespace nb

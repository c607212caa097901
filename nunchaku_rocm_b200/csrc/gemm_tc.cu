// W4A4 int4 GEMM on the 5th-generation tensor cores (tcgen05.mma kind::f8f6f4 on e4m3-encoded int4 values, exact
// integer-valued fp32 group sums in tensor memory), with the low-rank branch and the fused epilogues.
//
// Arithmetic contract (reference: nunchaku/ops/triton/gemm_w4a4.py:446-488 and :155-209): for every
// 64-wide K group g one EXACT int32 dot p_g[m,n]; acc += float(p_g) * as[g,m] * ws[g,n] in fp32;
// then + T(lora_act) . lora_up^T (16-bit operands, fp32 accumulate), + bias, one rounding to T.
//
// Two launches per call:
//  1. `prepack_kernel` (HBM-bound, a few microseconds): packed nibbles -> one e4m3 byte per value; row scales ->
//     fp32, column scales kept as T, both in the order a drain thread reads them (one 128-bit load for its 4 rows, two
//     for its 16 columns); lora_act -> T.  Measured on B200: widening inside the GEMM
//     through shared memory costs a generic->async proxy fence of ~3000 cycles per K group and competes with
//     the drain for issue slots and shared-memory bandwidth; with the operands pre-widened every byte the
//     tensor core reads is written by TMA and the SM's CUDA cores only do the per-group scaling.
//  2. `gemm_tc_kernel`: one persistent CTA per SM (320 threads) walks a static contiguous range of
//     128 x 128 output tiles.  A stage of the shared-memory ring holds two K groups (128 k):
//       warp 0    TMA producer: A and W rows (128 x 128 B each, 128-byte swizzle) and the two groups' scale
//                 rows (no multicast, no cluster); low-rank chunks of 32 ranks travel through the same ring.
//       warp 1    MMA issuer: per ring stage (two groups) four 128 x 128 x 32 kind::f8f6f4 MMAs into two of FOUR
//                 tensor-memory slots (the first group's pair goes out before the issuer waits for the second slot)
//                 and ONE tcgen05.commit, which publishes both slots and releases the operands:
//                 the issuing thread pays a few hundred cycles per wait and commit, so the work between two of them has
//                 to be large.  The low-rank product is kind::f16 into an fp32 slot of the same ring.
//       warps 2-9 drain: a warp owns 32 rows x 64 columns.  tcgen05.ld.16x256b gives a thread the
//                 accumulator-fragment layout (4 rows x 16 columns), so it needs 4 row scales and 16 column
//                 scales per group, and a packed fp32x2 multiply and FMA per column pair (below).  The loads of the
//                 next half group are in flight while the current half is scaled.  After the last group: bias,
//                 optional per-head RMSNorm + RoPE, rounding, and a coalesced store through a padded per-warp
//                 staging tile.
//
// Exact integers on the floating-point pipe.  Every int4 value (-8..7, or 0..15 for unsigned activations) is exactly
// representable in e4m3, a product is at most 120 in magnitude and a 64-term sum at most 7680, so kind::f8f6f4 with
// e4m3 operands and fp32 accumulation yields the group sum p_g as an exact integer-valued float (checked bit for bit
// against the integer oracle, worst-case patterns included).  It runs at the rate of kind::i8 and the drain needs no
// int -> float conversion: t = p * as (packed multiply), acc = fma(t, ws, acc) (packed FMA), two issues per column pair,
// which is the reference's float(p) * as * ws accumulated in fp32.
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
constexpr int STAGES = 4;
constexpr int NSLOT = 4;            // tensor-memory accumulator slots of BN columns
#ifndef NB_TC_DRAIN_WARPS
#define NB_TC_DRAIN_WARPS 8
#endif
constexpr int DRAIN_WARPS = NB_TC_DRAIN_WARPS;  // warps 2..: four TMEM lane quarters x NCQ column slices
constexpr int NCQ = DRAIN_WARPS / 4;
constexpr int NTHREADS = 64 + DRAIN_WARPS * 32;
constexpr int COLS = BN / NCQ;      // columns one drain warp owns
constexpr int NJ = COLS / 8;        // 8-column blocks per warp
constexpr int NV = 4 * NJ;          // registers of one 16-lane block of a warp's slice
static_assert(DRAIN_WARPS == 8 || DRAIN_WARPS == 16, "drain warps");
struct Cfg {
    static constexpr int ST_A = BM * 128, ST_W = BN * 128;  // two K groups of int8 per row
    static constexpr int ST_AS = 2 * BM * 4;                // per group and row: as, rows permuted per 32-row block
    static constexpr int ST_WS = 1024;                      // per group and column: ws as T, in drain order (512 B used)
    static constexpr int ST_WS_TX = 2 * BN * 2;
    static constexpr int ST_BYTES = ST_A + ST_W + ST_AS + ST_WS;
    static constexpr int STG_PITCH = COLS * 2 + 16;
    static constexpr int STG_BYTES = DRAIN_WARPS * 32 * STG_PITCH;
    static constexpr int XCH_BYTES = 2 * DRAIN_WARPS * 32 * 4;  // per-row partial sums exchanged between column slices, two buffers
    static constexpr int OFF_ST = 0;
    static constexpr int OFF_STG = OFF_ST + STAGES * ST_BYTES;
    static constexpr int OFF_XCH = OFF_STG + STG_BYTES;
    static constexpr int OFF_BAR = OFF_XCH + XCH_BYTES;
    static constexpr int SMEM_BYTES = OFF_BAR + 512 + 1024;  // + slack to align the base to 1 KB
    static constexpr int TMEM_COLS = NSLOT * BN;             // 512
};
static_assert(Cfg::ST_BYTES % 1024 == 0, "stage buffers must stay 1 KB aligned for the 128-byte swizzle");
static_assert(Cfg::SMEM_BYTES <= 232448, "shared memory budget");

enum {  // barrier indices
    B_FULL = 0,
    B_DONE = B_FULL + STAGES,       // tcgen05.commit: the stage's MMAs have completed (operands read, accumulators written)
    B_SCDONE = B_DONE + STAGES,     // one arrival per drain warp: the stage's scales have been read (int8 stages only)
    B_ACC_EMPTY = B_SCDONE + STAGES,// one arrival per drain warp: the accumulator slot has been read out
    B_XCH = B_ACC_EMPTY + NSLOT,    // one per TMEM lane quarter: the two warps that share rows
    B_LR = B_XCH + 4,               // tcgen05.commit: the tile's low-rank accumulator is complete
    B_COUNT = B_LR + 1
};

struct TcParams {
    void* out;
    const void* bias;
    int32_t* p_out;  // debug: (K/64, M, N) group sums
    int M, N, K, actual_m, R;
    int act_unsigned;
    long long stride_om;
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
enum { E_PROD = 0x10, E_MMA = 0x30, E_DRAIN = 0x40 };

// K-major operand, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3fff);
    d |= (uint64_t)1 << 16;              // leading byte offset: unused for swizzled K-major
    d |= (uint64_t)(1024 >> 4) << 32;    // stride byte offset
    d |= (uint64_t)1 << 46;              // descriptor version of sm_100
    d |= (uint64_t)2 << 61;              // SWIZZLE_128B
    return d;
}
// K-major operand, 64-byte swizzle: rows of 64 bytes, 8-row groups 512 bytes apart
__device__ __forceinline__ uint64_t umma_desc_sw64(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3fff);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(512 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)4 << 61;              // SWIZZLE_64B
    return d;
}

template <int EPI, typename T, bool DEBUG_P>
__global__ void __launch_bounds__(NTHREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w,
               const __grid_constant__ CUtensorMap tm_as, const __grid_constant__ CUtensorMap tm_ws,
               const __grid_constant__ CUtensorMap tm_la, const __grid_constant__ CUtensorMap tm_lu,
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
        for (int i = 0; i < STAGES; ++i) { mbar_init(bar(B_FULL + i), 1); mbar_init(bar(B_DONE + i), 1); mbar_init(bar(B_SCDONE + i), DRAIN_WARPS); }
        for (int i = 0; i < NSLOT; ++i) mbar_init(bar(B_ACC_EMPTY + i), DRAIN_WARPS);
        for (int i = 0; i < 4; ++i) mbar_init(bar(B_XCH + i), NCQ);
        mbar_init(bar(B_LR), 1);
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
    const int GS = (G + 1) / 2;       // int8 stages per tile (two K groups each)
    const int LCH = (p.R + 31) / 32;  // low-rank stages per tile (32 ranks each)

    if (warp == 0) {
        // ================================ TMA producer ================================
        if (lane == 0) {
            tma_prefetch_desc(&tm_a); tma_prefetch_desc(&tm_w); tma_prefetch_desc(&tm_as); tma_prefetch_desc(&tm_ws);
            if (LCH) { tma_prefetch_desc(&tm_la); tma_prefetch_desc(&tm_lu); }
            uint32_t it = 0;
            uint32_t sc_uses = 0;  // 8 bits per stage: how many int8 fills the stage has had (mod 256)
            bool ok = true;
            for (int t = t_begin; t < t_end && ok; ++t) {
                const int m0 = (t / NT) * BM, n0 = (t % NT) * BN;
                for (int j = 0; j < GS + LCH; ++j, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(bar(B_DONE + s), ((it / STAGES) & 1) ^ 1, abort_s, E_PROD | 1, 500)) { ok = false; break; }
                    {
                        // the drain must also be done with the scales of the stage's last int8 fill
                        const uint32_t n = (sc_uses >> (8 * s)) & 0xFFu;
                        if (!mbar_wait(bar(B_SCDONE + s), (n & 1) ^ 1, abort_s, E_PROD | 2, 500)) { ok = false; break; }
                        if (j < GS) sc_uses = (sc_uses & ~(0xFFu << (8 * s))) | (((n + 1) & 0xFFu) << (8 * s));
                    }
                    const uint32_t dst = s_base + C::OFF_ST + s * C::ST_BYTES;
                    if (j < GS) {
                        mbar_expect_tx(bar(B_FULL + s), C::ST_A + C::ST_W + C::ST_AS + C::ST_WS_TX);
                        tma_load_2d(dst, &tm_a, bar(B_FULL + s), j * 128, m0);
                        tma_load_2d(dst + C::ST_A, &tm_w, bar(B_FULL + s), j * 128, n0);
                        tma_load_2d(dst + C::ST_A + C::ST_W, &tm_as, bar(B_FULL + s), m0, j * 2);
                        tma_load_2d(dst + C::ST_A + C::ST_W + C::ST_AS, &tm_ws, bar(B_FULL + s), n0, j * 2);
                    } else {
                        // 32 ranks of T(lora_act) rows m0.. and lora_up rows n0..: 128 x 64 B each, 64-byte swizzle
                        mbar_expect_tx(bar(B_FULL + s), 2 * 128 * 64);
                        tma_load_2d(dst, &tm_la, bar(B_FULL + s), (j - GS) * 32, m0);
                        tma_load_2d(dst + C::ST_A, &tm_lu, bar(B_FULL + s), (j - GS) * 32, n0);
                    }
                }
            }
            if (!ok) {
                // let copies already in flight land before the CTA goes away (bounded)
                for (int s = 0; s < STAGES; ++s) {
                    const uint32_t issued = it > (uint32_t)s ? (it - 1 - s) / STAGES + 1 : 0;  // fills of stage s
                    if (issued) {
                        uint64_t t0 = globaltimer_ns();
                        while (!mbar_try_wait(bar(B_FULL + s), (issued - 1) & 1) && globaltimer_ns() - t0 < 200000000ull) {}
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ================================ MMA issuer ================================
        if (lane == 0) {
            const uint32_t idesc_f8 = umma_idesc(1u, 0u, 0u, BN);  // fp32 accumulators, e4m3 x e4m3
            const uint32_t f16fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
            const uint32_t idesc_lr = umma_idesc(1u, f16fmt, f16fmt, BN);
            uint32_t it = 0, ait = 0;
            bool ok = true;
            // One batch per ring stage: both K groups of the stage (four MMAs) and ONE commit.  The issuing thread
            // pays a few hundred cycles per wait / commit, so the work between two of them has to be large.
            for (int t = t_begin; t < t_end && ok; ++t) {
                for (int j = 0; j < GS && ok; ++j, ++it) {
                    const int s = it % STAGES;
                    const int ng = min(2, G - 2 * j);
                    if (!mbar_wait(bar(B_FULL + s), (it / STAGES) & 1, abort_s, E_MMA | 1, 100)) { ok = false; break; }
                    // the first group's slot is released half a stage before the second's: its MMAs go out before the
                    // issuer waits for the second slot
                    if (!mbar_wait(bar(B_ACC_EMPTY + ait % NSLOT), ((ait / NSLOT) & 1) ^ 1, abort_s, E_MMA | 2, 100)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = s_base + C::OFF_ST + s * C::ST_BYTES;
                    const uint64_t da = umma_desc_sw128(a_addr), dw = umma_desc_sw128(a_addr + C::ST_A);
                    // a 32-byte K step advances the descriptor's start address field by 2
                    {
                        const uint32_t d = tmem_base + (ait % NSLOT) * BN;
                        mma_f8(d, da, dw, idesc_f8, 0u);
                        mma_f8(d, da + 2, dw + 2, idesc_f8, 1u);
                    }
                    if (ng == 2) {
                        if (!mbar_wait(bar(B_ACC_EMPTY + (ait + 1) % NSLOT), (((ait + 1) / NSLOT) & 1) ^ 1, abort_s, E_MMA | 2, 100)) { ok = false; break; }
                        tc_fence_after();
                        const uint32_t d = tmem_base + ((ait + 1) % NSLOT) * BN;
                        mma_f8(d, da + 4, dw + 4, idesc_f8, 0u);
                        mma_f8(d, da + 6, dw + 6, idesc_f8, 1u);
                    }
                    tc_commit(bar(B_DONE + s));
                    ait += ng;
                }
                if (ok && LCH > 0) {
                    const int slot = ait % NSLOT;
                    if (!mbar_wait(bar(B_ACC_EMPTY + slot), ((ait / NSLOT) & 1) ^ 1, abort_s, E_MMA | 3, 100)) { ok = false; break; }
                    for (int c = 0; c < LCH && ok; ++c, ++it) {
                        const int s = it % STAGES;
                        if (!mbar_wait(bar(B_FULL + s), (it / STAGES) & 1, abort_s, E_MMA | 4, 100)) { ok = false; break; }
                        tc_fence_after();
                        const uint32_t a_addr = s_base + C::OFF_ST + s * C::ST_BYTES, w_addr = a_addr + C::ST_A;
                        const uint32_t d = tmem_base + slot * BN;
#pragma unroll
                        for (int h = 0; h < 2; ++h)
                            mma_f16(d, umma_desc_sw64(a_addr + h * 32), umma_desc_sw64(w_addr + h * 32), idesc_lr, (c | h) ? 1u : 0u);
                        tc_commit(bar(B_DONE + s));
                    }
                    if (ok) { tc_commit(bar(B_LR)); ++ait; }
                }
            }
        }
    } else {
        // ================================ drain + epilogue ================================
        // A warp owns 32 rows (its TMEM lane quarter) x 64 columns.  tcgen05.ld.16x256b.x8 hands a thread, for one
        // 16-lane block, rows {gid, gid + 8} and the column pairs 8 j + 2 tig + {0, 1}, j = 0..7: register
        // 4 j + 2 rs + e.
        const int dw = warp - 2;
        const int q = warp & 3;     // TMEM lane quarter this warp may read (warp id mod 4)
        const int half = dw >> 2;   // column slice of the tile
        const int pw = half * 4 + q;             // index used for staging / exchange buffers
        const int gid = lane >> 2, tig = lane & 3;
        uint8_t* stg = smem + C::OFF_STG + pw * 32 * C::STG_PITCH;
        float* xch = reinterpret_cast<float*>(smem + C::OFF_XCH);
        const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16) + half * COLS;
        uint32_t it = 0, ait = 0, xph = 0;
        bool ok = true;
        uint64_t acc[NV];  // [lane block lb][j][row select] pairs of fp32
        uint32_t v[2][NV];

        for (int t = t_begin; t < t_end && ok; ++t) {
            const int m0 = (t / NT) * BM, n0 = (t % NT) * BN;
            const int nc0 = n0 + half * COLS;  // first global column of this warp
#pragma unroll
            for (int i = 0; i < NV; ++i) acc[i] = 0ull;
            // Software pipeline over half groups (16 TMEM lanes = 32 registers each): while one half is scaled the
            // loads of the next are in flight.  `v[0]` holds lane block 0, `v[1]` lane block 1 of a group.  The MMA warp
            // completes a ring stage (two groups) at a time, so there is one wait per stage.
            {
                if (!mbar_wait_warp(bar(B_DONE + it % STAGES), (it / STAGES) & 1, abort_s, E_DRAIN | 1, 100)) { ok = false; break; }
                tc_fence_after();
                tmem_ld_16x256b(lane_base + (ait % NSLOT) * BN, v[0]);
            }
            for (int g = 0; g < G; ++g, ++ait) {
                const int slot = ait % NSLOT;
                const uint32_t itg = it + (g >> 1);
                const int s = itg % STAGES, i = g & 1;
                // scales of this group: the thread's 4 rows (fp32) and 2 NJ columns (T, widened here)
                const uint8_t* st = smem + C::OFF_ST + s * C::ST_BYTES + C::ST_A + C::ST_W;
                const uint4 as4 = *reinterpret_cast<const uint4*>(st + (i * BM + q * 32 + gid * 4) * 4);  // rows gid, +8, +16, +24
                uint64_t as2[4] = {pack_u32x2(as4.x, as4.x), pack_u32x2(as4.y, as4.y), pack_u32x2(as4.z, as4.z), pack_u32x2(as4.w, as4.w)};
                const uint4* ws_s = reinterpret_cast<const uint4*>(st + C::ST_AS + (i * BN + half * COLS + tig * NJ * 2) * 2);
                uint32_t w16[NJ];
#pragma unroll
                for (int jj = 0; jj < NJ / 4; ++jj) { const uint4 t4 = ws_s[jj]; w16[4 * jj] = t4.x; w16[4 * jj + 1] = t4.y; w16[4 * jj + 2] = t4.z; w16[4 * jj + 3] = t4.w; }
                ulonglong2 w[NJ / 2];
#pragma unroll
                for (int jj = 0; jj < NJ / 2; ++jj) {
                    const float2 f0 = unpack2<T>(w16[2 * jj]), f1 = unpack2<T>(w16[2 * jj + 1]);
                    w[jj] = make_ulonglong2(pack_f32x2(f0.x, f0.y), pack_f32x2(f1.x, f1.y));
                }
                tmem_wait_ld();  // v[0] has landed
                tmem_ld_16x256b(lane_base + (16u << 16) + slot * BN, v[1]);
#pragma unroll
                for (int lb = 0; lb < 2; ++lb) {
                    uint32_t(&vv)[NV] = v[lb];
                    if (lb == 1) {
                        tmem_wait_ld();  // v[1] has landed: the slot is read out
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar(B_ACC_EMPTY + slot));
                        const bool last_of_stage = i == 1 || g == G - 1;
                        if (last_of_stage) {
                            // This warp holds the stage's scales in registers (the empty asm makes the loads retire first).
                            // Released BEFORE the wait below: the low-rank slot only completes after the producer has
                            // reused ring stages, which it may not do while a drain warp still owes this arrival.
                            asm volatile("" ::"l"(as2[2]), "l"(as2[3]), "l"(w[NJ / 2 - 1].y) : "memory");
                            if (lane == 0) mbar_arrive(bar(B_SCDONE + s));
                        }
                        // next accumulator: the stage's second group, the next stage, or the low-rank slot after the last group
                        if (!last_of_stage) {
                            tmem_ld_16x256b(lane_base + ((ait + 1) % NSLOT) * BN, v[0]);
                        } else if (g + 1 < G || LCH > 0) {
                            // (the low-rank slot has a barrier of its own: its ring stages are not watched here, and waiting for a
                            // later use of a stage barrier while an earlier one is still pending would alias on the parity)
                            const bool more = g + 1 < G;
                            if (!mbar_wait_warp(more ? bar(B_DONE + (itg + 1) % STAGES) : bar(B_LR),
                                                more ? ((itg + 1) / STAGES) & 1 : (uint32_t)(t - t_begin) & 1, abort_s, E_DRAIN | 2, 100)) { ok = false; break; }
                            tc_fence_after();
                            tmem_ld_16x256b(lane_base + ((ait + 1) % NSLOT) * BN, v[0]);
                        }
                    }
                    if (EPI == NB_EPI_QK_NORM_ROPE) {
#pragma unroll
                        for (int jx = 0; jx < NJ; ++jx) {
                            const uint64_t wj = (jx & 1) ? w[jx >> 1].y : w[jx >> 1].x;
#pragma unroll
                            for (int rs = 0; rs < 2; ++rs) {
                                const int vi = 4 * jx + 2 * rs;
                                const uint64_t tt = mul_f32x2(pack_u32x2(vv[vi], vv[vi + 1]), as2[lb * 2 + rs]);
                                uint64_t& a = acc[(lb * NJ + jx) * 2 + rs];
                                a = fma_f32x2(tt, wj, a);
                            }
                        }
                    } else {
                        // All products p * as of the half group first, then the FMAs: measured 4 % faster than the interleaved
                        // order above for the plain epilogue and 5 % slower for the Q/K one (whose instantiation has fewer
                        // registers to spare), hence the two forms.
                        uint64_t tt[NJ][2];
#pragma unroll
                        for (int jx = 0; jx < NJ; ++jx)
#pragma unroll
                            for (int rs = 0; rs < 2; ++rs) {
                                const int vi = 4 * jx + 2 * rs;
                                tt[jx][rs] = mul_f32x2(pack_u32x2(vv[vi], vv[vi + 1]), as2[lb * 2 + rs]);
                            }
                        asm volatile("" ::: "memory");
#pragma unroll
                        for (int jx = 0; jx < NJ; ++jx) {
                            const uint64_t wj = (jx & 1) ? w[jx >> 1].y : w[jx >> 1].x;
#pragma unroll
                            for (int rs = 0; rs < 2; ++rs) {
                                uint64_t& a = acc[(lb * NJ + jx) * 2 + rs];
                                a = fma_f32x2(tt[jx][rs], wj, a);
                            }
                        }
                    }
                    if (DEBUG_P) {
#pragma unroll
                        for (int e = 0; e < NV; ++e) {
                            const int m = m0 + q * 32 + lb * 16 + ((e >> 1) & 1) * 8 + gid;
                            const int n = nc0 + (e >> 2) * 8 + 2 * tig + (e & 1);
                            if (m < p.M && n < p.N)
                                p.p_out[((long long)g * p.M + m) * p.N + n] = (int)__uint_as_float(vv[e]);
                        }
                    }
                }
                if (!ok) break;
            }
            if (!ok) break;
            it += GS;
            // bias and (Q / K tiles) RMSNorm weights of this warp's columns, requested before the low-rank slot is added
            const int qk_part = EPI == NB_EPI_QK_NORM_ROPE ? n0 / (p.N / 3) : 2;
            uint32_t bias_w[NJ], norm_w[NJ];
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                const int col = nc0 + 8 * j + 2 * tig;
                bias_w[j] = (p.bias && col < p.N) ? __ldg(reinterpret_cast<const uint32_t*>(static_cast<const T*>(p.bias) + col)) : 0u;
                norm_w[j] = 0u;
                if (EPI == NB_EPI_QK_NORM_ROPE && qk_part < 2)
                    norm_w[j] = __ldg(reinterpret_cast<const uint32_t*>(static_cast<const T*>(qk_part == 0 ? p.norm_q : p.norm_k) + half * COLS + 8 * j + 2 * tig));
            }
            if (LCH > 0) {
                const int slot = ait % NSLOT;
                tmem_wait_ld();
                tmem_ld_16x256b(lane_base + (16u << 16) + slot * BN, v[1]);
#pragma unroll
                for (int lb = 0; lb < 2; ++lb) {
                    if (lb == 1) {
                        tmem_wait_ld();
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar(B_ACC_EMPTY + slot));
                    }
#pragma unroll
                    for (int jx = 0; jx < NJ; ++jx)
#pragma unroll
                        for (int rs = 0; rs < 2; ++rs) {
                            uint64_t& a = acc[(lb * NJ + jx) * 2 + rs];
                            a = add_f32x2(a, pack_u32x2(v[lb][4 * jx + 2 * rs], v[lb][4 * jx + 2 * rs + 1]));
                        }
                }
                it += LCH;  // the low-rank stages carry nothing for the drain
                ++ait;
            }

            // ---------------- epilogue: bias, optional RMSNorm + RoPE, rounding, staged store ----------------
            // element (lb, j, rs, e): row q*32 + lb*16 + rs*8 + gid, column nc0 + 8j + 2 tig + e
            float sumsq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int lb = 0; lb < 2; ++lb)
#pragma unroll
                for (int j = 0; j < NJ; ++j) {
                    const float2 b = unpack2<T>(bias_w[j]);
#pragma unroll
                    for (int rs = 0; rs < 2; ++rs) {
                        float2 a = unpack_f32x2(acc[(lb * NJ + j) * 2 + rs]);
                        a.x += b.x;
                        a.y += b.y;
                        acc[(lb * NJ + j) * 2 + rs] = pack_f32x2(a.x, a.y);
                        if (EPI == NB_EPI_QK_NORM_ROPE) sumsq[lb * 2 + rs] = fmaf(a.x, a.x, fmaf(a.y, a.y, sumsq[lb * 2 + rs]));
                    }
                }
            if (EPI == NB_EPI_QK_NORM_ROPE && qk_part < 2) {
                // The 128-column tile is one head.  The rotary values of the first 16-lane block are requested before the
                // exchange of the row sums, those of the second while the first is rotated: their L2 latency is hidden.
                const float2* rp[4];
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const int m = m0 + q * 32 + r * 8 + gid;
                    int mr = m < p.actual_m ? m : 0;
                    if (mr >= p.rot_rows) mr %= p.rot_rows;
                    rp[r] = reinterpret_cast<const float2*>(p.rot + (long long)mr * p.stride_rm + half * COLS + 2 * tig);
                }
                float2 sc[2][NJ];
#pragma unroll
                for (int rs = 0; rs < 2; ++rs)
#pragma unroll
                    for (int j = 0; j < NJ; ++j) sc[rs][j] = __ldg(rp[rs] + 4 * j);
                // the 4 lanes of a quad share a row; the other column slices of the same rows are in the warps with the same q
                float* xb = xch + (xph & 1) * (DRAIN_WARPS * 32);
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    float s = sumsq[r];
                    s += __shfl_xor_sync(0xffffffffu, s, 1);
                    s += __shfl_xor_sync(0xffffffffu, s, 2);
                    if (tig == 0) xb[pw * 32 + r * 8 + gid] = s;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(B_XCH + q));
                if (!mbar_wait_warp(bar(B_XCH + q), xph & 1, abort_s, E_DRAIN | 4, 100)) { ok = false; break; }
                // (the buffer of this parity is written again two exchanges later, and no warp gets there before every
                // warp of the quarter has arrived at the exchange in between, i.e. after it has read this one)
                ++xph;
                float rstd[4];
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    float tot = 0.f;  // every slice adds the partial sums in the same order
#pragma unroll
                    for (int c = 0; c < NCQ; ++c) tot += xb[(c * 4 + q) * 32 + r * 8 + gid];
                    rstd[r] = rsqrtf(tot / 128.0f + p.eps);
                }
#pragma unroll
                for (int lb = 0; lb < 2; ++lb) {
                    float2 scn[2][NJ];
                    if (lb == 0) {
#pragma unroll
                        for (int rs = 0; rs < 2; ++rs)
#pragma unroll
                            for (int j = 0; j < NJ; ++j) scn[rs][j] = __ldg(rp[2 + rs] + 4 * j);
                    }
#pragma unroll
                    for (int j = 0; j < NJ; ++j) {
                        const float2 w = unpack2<T>(norm_w[j]);
#pragma unroll
                        for (int rs = 0; rs < 2; ++rs) {
                            const float2 a = unpack_f32x2(acc[(lb * NJ + j) * 2 + rs]);
                            const float xe = a.x * rstd[lb * 2 + rs] * w.x, xo = a.y * rstd[lb * 2 + rs] * w.y;
                            const float2 c = sc[rs][j];
                            acc[(lb * NJ + j) * 2 + rs] = pack_f32x2(xe * c.y - xo * c.x, xe * c.x + xo * c.y);
                        }
                    }
                    if (lb == 0) {
#pragma unroll
                        for (int rs = 0; rs < 2; ++rs)
#pragma unroll
                            for (int j = 0; j < NJ; ++j) sc[rs][j] = scn[rs][j];
                    }
                }
            }
            // round, transpose through the per-warp staging tile, store whole 128-byte row segments
            __syncwarp();
#pragma unroll
            for (int lb = 0; lb < 2; ++lb)
#pragma unroll
                for (int j = 0; j < NJ; ++j)
#pragma unroll
                    for (int rs = 0; rs < 2; ++rs) {
                        const float2 a = unpack_f32x2(acc[(lb * NJ + j) * 2 + rs]);
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
// pre-pass: nibbles -> e4m3 bytes, scales in drain order, lora_act -> T
// ------------------------------------------------------------------------------------------------
struct PrepackParams {
    const uint8_t* act; const uint8_t* wgt;
    const void* ascales; const void* wscales; const float* lora_act;
    int8_t* a8; int8_t* w8; float* asf; void* wsf; void* la16;
    int M, N, K, R, Np, Mp;  // Np, Mp: N, M rounded up to 128
    int act_unsigned;
    int do_act, do_wgt;      // which half of the work this launch does (activation side / weight side)
    long long stride_am, stride_wn, stride_asg, stride_wsg, stride_lam;
};

template <typename T>
__global__ void __launch_bounds__(256) prepack_kernel(const PrepackParams p) {
    const long long tid = (long long)blockIdx.x * 256 + threadIdx.x;
    const int upr = p.K / 32;  // 16-byte packed units per row
    const long long a_units = p.do_act ? (long long)p.M * upr : 0, w_units = p.do_wgt ? (long long)p.N * upr : 0;
    const int G = p.K / 64;
    const long long as_units = p.do_act ? (long long)G * p.Mp : 0, ws_units = p.do_wgt ? (long long)G * p.Np : 0;
    const long long la_units = (p.do_act && p.R) ? (long long)p.M * (p.R / 8) : 0;
    if (tid < a_units + w_units) {
        const bool is_w = tid >= a_units;
        const long long u = is_w ? tid - a_units : tid;
        const long long row = u / upr;
        const int c = (int)(u % upr);
        const uint8_t* src = (is_w ? p.wgt + row * p.stride_wn : p.act + row * p.stride_am) + c * 16;
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(src));
        // one e4m3 byte per nibble, in k order: a 16-entry table looked up with byte permutes
        const bool uns = !is_w && p.act_unsigned;
        const uint32_t in[4] = {v.x, v.y, v.z, v.w};
        uint32_t o[8];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            o[2 * k] = e4m3_of_nibbles(in[k] & 0xFFFFu, uns);
            o[2 * k + 1] = e4m3_of_nibbles(in[k] >> 16, uns);
        }
        const uint4 o0 = make_uint4(o[0], o[1], o[2], o[3]), o1 = make_uint4(o[4], o[5], o[6], o[7]);
        uint4* dst = reinterpret_cast<uint4*>((is_w ? p.w8 : p.a8) + row * p.K + c * 32);
        dst[0] = o0;
        dst[1] = o1;
        return;
    }
    long long u = tid - (a_units + w_units);
    if (u < as_units) {
        const int g = (int)(u / p.Mp), m = (int)(u % p.Mp);
        const float a = m < p.M ? to_f32<T>(static_cast<const T*>(p.ascales)[(long long)g * p.stride_asg + m]) : 0.f;
        const int r32 = m & 31;  // row r * 8 + gid of its 32-row block -> position gid * 4 + r
        p.asf[(long long)g * p.Mp + (m & ~31) + (r32 & 7) * 4 + (r32 >> 3)] = a;
        return;
    }
    u -= as_units;
    if (u < ws_units) {
        // column n of its 128-wide tile -> [tile][warp half][pair of 8-col blocks][tig][4]: one 128-bit load of a drain
        // thread is (cols c, c+1 of block j, cols c, c+1 of block j+1)
        const int g = (int)(u / p.Np), n = (int)(u % p.Np);
        const T w = n < p.N ? static_cast<const T*>(p.wscales)[(long long)g * p.stride_wsg + n] : from_f32<T>(0.f);
        const int tile = n / BN, i = n % BN;
        const int hf = i / COLS, cc = i % COLS;
        const int blk = cc >> 3, tg = (cc >> 1) & 3, e = cc & 1;
        static_cast<T*>(p.wsf)[(long long)g * p.Np + tile * BN + hf * COLS + tg * (COLS / 4) + blk * 2 + e] = w;
        return;
    }
    u -= ws_units;
    if (u < la_units) {
        const int rpr = p.R / 8;
        const long long m = u / rpr;
        const int c = (int)(u % rpr);
        const float4* src = reinterpret_cast<const float4*>(p.lora_act + m * p.stride_lam + c * 8);
        const float4 x = __ldg(src), y = __ldg(src + 1);
        uint4 o;
        o.x = pack2<T>(x.x, x.y); o.y = pack2<T>(x.z, x.w); o.z = pack2<T>(y.x, y.y); o.w = pack2<T>(y.z, y.w);
        reinterpret_cast<uint4*>(static_cast<T*>(p.la16) + m * p.R)[c] = o;
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

static inline size_t up256(size_t x) { return (x + 255) & ~size_t(255); }

// The weight side (w8, wsf) lives in the caller's prepared buffer when there is one, else in the call's scratch after the
// activation side.
static bool has_prepared(const nb_gemm_args* a) { return has_prepared_weights(a); }
struct WeightSide { size_t w8, wsf, total; };
static WeightSide weight_side(const nb_gemm_args* a) {  // the part of the prepared layout this kernel reads
    const PreparedLayout pl = nb::prepared_layout(a->N, a->K);
    return {pl.w8, pl.wsf, pl.wsf2};
}
struct Scratch {
    size_t a8, asf, la16, wside, total;
    int Np, Mp;
};
static Scratch scratch_layout(const nb_gemm_args* a) {
    Scratch s;
    const size_t G = a->K / 64;
    s.Np = (a->N + BN - 1) / BN * BN;
    size_t off = 0;
    s.a8 = off; off += up256((size_t)a->M * a->K);
    s.Mp = (a->M + BM - 1) / BM * BM;
    s.asf = off; off += up256(G * s.Mp * 4);
    s.la16 = off; off += up256((size_t)a->M * a->R * 2);
    s.wside = off;
    if (!has_prepared(a)) off += weight_side(a).total;
    s.total = off;
    return s;
}

static void fill_prepack_params(PrepackParams& pp, const nb_gemm_args* a) {
    pp.act = static_cast<const uint8_t*>(a->act); pp.wgt = static_cast<const uint8_t*>(a->wgt);
    pp.ascales = a->ascales; pp.wscales = a->wscales; pp.lora_act = static_cast<const float*>(a->lora_act);
    pp.act_unsigned = a->act_unsigned;
    pp.M = a->M; pp.N = a->N; pp.K = a->K; pp.R = a->R;
    pp.Np = (a->N + BN - 1) / BN * BN; pp.Mp = (a->M + BM - 1) / BM * BM;
    pp.stride_am = a->stride_am; pp.stride_wn = a->stride_wn; pp.stride_asg = a->stride_asg;
    pp.stride_wsg = a->stride_wsg; pp.stride_lam = a->stride_lam;
}

template <typename T>
static int launch_prepack(const PrepackParams& pp, cudaStream_t s) {
    const long long G = pp.K / 64;
    long long units = 0;
    if (pp.do_act) units += (long long)pp.M * (pp.K / 32) + G * pp.Mp + (pp.R ? (long long)pp.M * (pp.R / 8) : 0);
    if (pp.do_wgt) units += (long long)pp.N * (pp.K / 32) + G * pp.Np;
    if (units == 0) return NB_OK;
    prepack_kernel<T><<<(unsigned)((units + 255) / 256), 256, 0, s>>>(pp);
    NB_CUDA_CHECK(cudaGetLastError());
    return NB_OK;
}

template <int EPI, typename T, bool DEBUG_P>
static int launch_t(const nb_gemm_args* a, const TcParams& p, cudaStream_t s) {
    using C = Cfg;
    const Scratch sc = scratch_layout(a);
    if (!a->scratch || a->scratch_bytes < (int64_t)sc.total || (reinterpret_cast<uintptr_t>(a->scratch) & 255))
        return NB_ERR_INVALID;
    uint8_t* base = static_cast<uint8_t*>(a->scratch);
    const bool prepared = has_prepared(a);
    const WeightSide pl = weight_side(a);
    uint8_t* wbase = prepared ? const_cast<uint8_t*>(static_cast<const uint8_t*>(a->wgt_prepared)) : base + sc.wside;
    PrepackParams pp;
    fill_prepack_params(pp, a);
    pp.a8 = reinterpret_cast<int8_t*>(base + sc.a8); pp.asf = reinterpret_cast<float*>(base + sc.asf);
    pp.la16 = base + sc.la16;
    pp.w8 = reinterpret_cast<int8_t*>(wbase + pl.w8); pp.wsf = wbase + pl.wsf;
    pp.do_act = 1; pp.do_wgt = prepared ? 0 : 1;
    {
        const int st = launch_prepack<T>(pp, s);
        if (st != NB_OK) return st;
    }

    const long long G = a->K / 64;
    CUtensorMap tm_a, tm_w, tm_as, tm_ws, tm_la, tm_lu;
    const CUtensorMapDataType t16 = std::is_same<T, __nv_bfloat16>::value ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                                          : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    bool ok = make_map(&tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, pp.a8, a->K, a->M, a->K, 128, BM, CU_TENSOR_MAP_SWIZZLE_128B) &&
              make_map(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, pp.w8, a->K, a->N, a->K, 128, BN, CU_TENSOR_MAP_SWIZZLE_128B) &&
              make_map(&tm_as, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, pp.asf, (uint64_t)sc.Mp, G, (uint64_t)sc.Mp * 4, BM, 2,
                       CU_TENSOR_MAP_SWIZZLE_NONE) &&
              make_map(&tm_ws, t16, pp.wsf, sc.Np, G, (uint64_t)sc.Np * 2, BN, 2, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (ok && a->R > 0)
        ok = make_map(&tm_la, t16, pp.la16, a->R, a->M, (uint64_t)a->R * 2, 32, BM, CU_TENSOR_MAP_SWIZZLE_64B) &&
             make_map(&tm_lu, t16, a->lora_up, a->R, a->N, (uint64_t)a->stride_lun * 2, 32, BN, CU_TENSOR_MAP_SWIZZLE_64B);
    else if (ok) { tm_la = tm_a; tm_lu = tm_w; }
    if (!ok) return NB_ERR_UNSUPPORTED;
    int dev = 0, sms = 0;
    NB_CUDA_CHECK(cudaGetDevice(&dev));
    NB_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int total = ((a->M + BM - 1) / BM) * ((a->N + BN - 1) / BN);
    const int grid = total < sms ? total : sms;
    auto kern = gemm_tc_kernel<EPI, T, DEBUG_P>;
    NB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    kern<<<grid, NTHREADS, C::SMEM_BYTES, s>>>(tm_a, tm_w, tm_as, tm_ws, tm_la, tm_lu, p);
    NB_CUDA_CHECK(cudaGetLastError());
    return NB_OK;
}

}  // namespace tc


// What a weight must satisfy for the tensor-core kernel, whatever the call around it looks like.
static bool tc_weight_ok(const nb_gemm_args* a) {
    return a && a->wgt && a->wscales && !a->fp4 && a->N > 0 && a->K > 0 && a->K % 64 == 0 && a->N % 8 == 0 &&
           aligned16(a->wgt) && a->stride_wn % 16 == 0 && (a->dtype == NB_DTYPE_BF16 || a->dtype == NB_DTYPE_FP16);
}

int tcp_prepare_scales(const nb_gemm_args* a, void* wsf2, cudaStream_t s);

int64_t tc_prepared_bytes(const nb_gemm_args* a) { return tc_weight_ok(a) ? (int64_t)prepared_layout(a->N, a->K).total : 0; }

// One e4m3 byte per weight value, then the column scales in the order of either tensor-core kernel's drain.
int tc_prepare_weights(const nb_gemm_args* a, void* dst, int64_t dst_bytes, cudaStream_t s) {
    if (!tc_weight_ok(a)) return NB_ERR_UNSUPPORTED;
    const PreparedLayout pl = prepared_layout(a->N, a->K);
    if (!dst || dst_bytes < (int64_t)pl.total || (reinterpret_cast<uintptr_t>(dst) & 255)) return NB_ERR_INVALID;
    tc::PrepackParams pp = {};
    pp.wgt = static_cast<const uint8_t*>(a->wgt); pp.wscales = a->wscales;
    pp.N = a->N; pp.K = a->K; pp.Np = pl.Np128;
    pp.stride_wn = a->stride_wn; pp.stride_wsg = a->stride_wsg;
    pp.w8 = reinterpret_cast<int8_t*>(static_cast<uint8_t*>(dst) + pl.w8); pp.wsf = static_cast<uint8_t*>(dst) + pl.wsf;
    pp.do_act = 0; pp.do_wgt = 1;
    const int st = a->dtype == NB_DTYPE_BF16 ? tc::launch_prepack<__nv_bfloat16>(pp, s) : tc::launch_prepack<__half>(pp, s);
    if (st != NB_OK) return st;
    return tcp_prepare_scales(a, static_cast<uint8_t*>(dst) + pl.wsf2, s);
}

// Why the tcgen05 kernel cannot take this call, or nullptr (the role of `unsupported_reason`,
// nunchaku/ops/triton/native/w4a4.py:164-231).
const char* tc_unsupported_reason(const nb_gemm_args* a, const void* epi, int epi_kind) {
    if (a->fp4) return "NVFP4 (handled by the block-scaled kernel)";
    if (a->wcscales || a->alpha != 1.0f || a->fuse_silu) return "wcscales / alpha / SiLU";
    if (epi_kind != NB_EPI_STORE && epi_kind != NB_EPI_QK_NORM_ROPE) return "epilogue";
    if (a->K % 64 || a->N % 8 || a->M < 1) return "K % 64, N % 8";
    if (!aligned16(a->act) || !aligned16(a->wgt) || a->stride_am % 16 || a->stride_wn % 16) return "act / wgt alignment";
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

int64_t tc_scratch_bytes(const nb_gemm_args* a) { return (int64_t)tc::scratch_layout(a).total; }

int launch_tc(const nb_gemm_args* a, const void* epi, int epi_kind, int32_t* p_out, cudaStream_t s) {
    tc::TcParams p = {};
    p.out = a->out; p.bias = a->bias;
    p.p_out = p_out;
    p.M = a->M; p.N = a->N; p.K = a->K; p.actual_m = a->actual_m; p.R = a->R;
    p.act_unsigned = a->act_unsigned;
    p.stride_om = a->stride_om;
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

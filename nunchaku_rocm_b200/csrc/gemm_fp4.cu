// NVFP4 W4A4 GEMM on the block-scaled 5th-generation tensor cores (tcgen05.mma kind::mxf4nvf4, block 16).
//
// Arithmetic (reference: nunchaku/ops/triton/gemm_w4a4.py:302-350 and :155-209): codes are e2m1, one e4m3 scale per 16
// consecutive k for activations and weights,
//     out = (sum_k (a_k sa_g(k)[m]) (w_k sw_g(k)[n])) * wcscale[n] * alpha + T(lora_act) . lora_up^T + bias.
// The reference emulates the products group by group; here the tensor core applies both scale vectors itself, so the
// whole K loop accumulates into ONE fp32 accumulator in tensor memory and the CUDA cores only run the epilogue.
//
// Data path: the packed e2m1 nibbles are exactly what the tensor core reads (two codes per byte, even k in the low
// nibble, K-major), so A and W go from the caller's buffers to shared memory by TMA (128 rows x 128 bytes = 256 k per
// ring stage, 128-byte swizzle), with no pre-pass.  The scales need the layout the instruction defines: per 128 rows
// and 64 k a 512-byte chunk in which row r = r0 + 32 r1 keeps its four scales at byte 16 r0 + 4 r1.  A small pre-pass
// writes the group-major (K/16, rows) scale tensors in that order (and lora_act as T); the kernel copies a stage's four
// chunks with one bulk copy and moves each chunk into tensor memory with tcgen05.cp (32 x 128 bit, broadcast to the
// four lane quarters) right before the MMA that uses it.
//
// Roles: warp 0 producer, warp 1 MMA issuer and tensor-memory owner, warps 2-5 epilogue (one per lane quarter).
//
// Two tile widths.  The kernel is bound by operand delivery (TMA from L2 reaches about 25 B/clk/SM on B200, the MMAs of a
// 256-k stage need a sixth of the time its 36 KB take to arrive), so the wide variant, 128 x 256, loads the A rows once
// for twice the output columns: 54 KB per stage for twice the work.  Tensor memory, 128 x 128: two accumulator slots (the
// epilogue of tile t overlaps the main loop of tile t + 1), a low-rank slot, 32 columns of scales per ring stage.
// 128 x 256: one accumulator slot of 256 columns (the ring keeps filling during the epilogue, which is shorter than the
// ring is deep), a 128-column low-rank slot that serves the two column halves one after the other (the low-rank K loop
// runs once per half), two buffers of 48 scale columns (tcgen05.cp and tcgen05.mma of one thread execute in issue order).
// Every mbarrier wait is bounded; on expiry the CTA records a code in the status word and unwinds.
#include <cuda.h>

#include <type_traits>

#include "nb_common.cuh"

namespace nb {
namespace fp4 {

constexpr int BM = 128;
constexpr int KSTAGE = 256;                 // k per ring stage = 128 bytes of packed codes per row
constexpr int EPI_WARPS = 4;
constexpr int NTHREADS = 64 + EPI_WARPS * 32;
constexpr int MAX_STAGES = 4;
template <int BN_>
struct Cfg {
    static constexpr int BN = BN_;
    static constexpr int NH = BN / 128;                  // 128-column halves of a tile
    static constexpr int STAGES = 4;
    static constexpr int ST_A = BM * 128, ST_W = BN * 128;
    static constexpr int ST_SFA = 4 * 512, ST_SFB = NH * 4 * 512;  // four 64-k steps per stage
    static constexpr int ST_BYTES = ST_A + ST_W + ST_SFA + ST_SFB;
    static constexpr int OFF_BAR = STAGES * ST_BYTES;
    static constexpr int OFF_EPI = OFF_BAR + 256;           // per epilogue warp: wcscale and bias of the tile's columns, fp32
    static constexpr int EPI_BYTES = EPI_WARPS * 2 * BN * 4;
    static constexpr int SMEM_BYTES = OFF_EPI + EPI_BYTES + 1024;
    static constexpr int ACC_SLOTS = BN == 128 ? 2 : 1;
    static constexpr uint32_t TM_ACC = 0, TM_LORA = 256, TM_SF = 384;  // tensor-memory columns
    static constexpr int SF_STEP = 4 + 4 * NH;           // scale columns of one 64-k step: A, then B per half
    static constexpr int SF_BUFS = BN == 128 ? STAGES : 2;
    static_assert(ST_BYTES % 1024 == 0, "stage buffers must stay 1 KB aligned for the 128-byte swizzle");
    static_assert(TM_SF + SF_BUFS * 4 * SF_STEP <= 512, "tensor memory budget");
    static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

enum { B_FULL = 0, B_EMPTY = B_FULL + MAX_STAGES, B_ACC_FULL = B_EMPTY + MAX_STAGES, B_ACC_EMPTY = B_ACC_FULL + 2,
       B_LR_FULL = B_ACC_EMPTY + 2, B_LR_EMPTY = B_LR_FULL + 1, B_COUNT = B_LR_EMPTY + 1 };
enum { E_PROD = 0x110, E_MMA = 0x130, E_EPI = 0x140 };

struct Params {
    void* out;
    const void* bias;
    const void* wcscales;
    const uint8_t* sfa;  // (ceil(M/128), K/64, 512)
    const uint8_t* sfb;  // (ceil(N/128), K/64, 512)
    int M, N, K, actual_m, R;
    float alpha;
    long long stride_om;
    int* status;
};

__device__ __forceinline__ uint64_t desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3fff);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
__device__ __forceinline__ uint64_t desc_sw64(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3fff);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(512 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)4 << 61;
    return d;
}
// Block-scaled instruction descriptor: e2m1 x e2m1, ue4m3 scales, M = 128, K = 64 per instruction.
__device__ __host__ constexpr uint32_t idesc_mxf4nvf4(uint32_t n) {
    return (1u << 7) | (1u << 10) | ((n >> 3) << 17) | (0u << 23) | ((128u >> 4) << 24);
}
__device__ __forceinline__ void mma_mxf4nvf4(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa,
                                             uint32_t sfb, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc), "r"(sfa), "r"(sfb)
        : "memory");
}
// 32 rows x 16 bytes of shared memory -> 4 columns of tensor memory, replicated in the four lane quarters
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,"
        "%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}

template <typename T, int BN_>
__global__ void __launch_bounds__(NTHREADS, 1)
gemm_fp4_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w,
                const __grid_constant__ CUtensorMap tm_la, const __grid_constant__ CUtensorMap tm_lu, const Params p) {
    using C = Cfg<BN_>;
    constexpr int BN = C::BN, NH = C::NH, STAGES = C::STAGES, ST_BYTES = C::ST_BYTES, ST_A = C::ST_A, ST_W = C::ST_W;
    constexpr int OFF_BAR = C::OFF_BAR, ACC_SLOTS = C::ACC_SLOTS;
    constexpr uint32_t TM_ACC = C::TM_ACC, TM_LORA = C::TM_LORA, TM_SF = C::TM_SF;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t s_base = smem_u32(smem);
    const uint32_t s_bar = s_base + OFF_BAR;
    uint32_t* tmem_ptr_s = reinterpret_cast<uint32_t*>(smem + OFF_BAR + 8 * B_COUNT);
    volatile int* abort_s = reinterpret_cast<volatile int*>(smem + OFF_BAR + 8 * B_COUNT + 8);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    auto bar = [&](int i) { return s_bar + 8u * i; };

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) { mbar_init(bar(B_FULL + i), 1); mbar_init(bar(B_EMPTY + i), 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(bar(B_ACC_FULL + i), 1); mbar_init(bar(B_ACC_EMPTY + i), EPI_WARPS); }
        mbar_init(bar(B_LR_FULL), 1);
        mbar_init(bar(B_LR_EMPTY), EPI_WARPS);
        *abort_s = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_ptr_s), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr_s;

    const int MT = (p.M + BM - 1) / BM, NT = (p.N + BN - 1) / BN;
    const int total = MT * NT;
    const int per = (total + gridDim.x - 1) / gridDim.x;
    const int t_begin = min(total, (int)blockIdx.x * per), t_end = min(total, t_begin + per);
    const int KS = (p.K + KSTAGE - 1) / KSTAGE;  // ring stages of the main loop per tile (the last one may hold fewer than four 64-k steps)
    const int KS4 = p.K / 64;         // 64-k steps (scale chunks) per row block
    const int LCH = (p.R + 31) / 32;  // low-rank stages per tile (32 ranks each)

    if (warp == 0) {
        // ================================ producer ================================
        // (a whole-warp loop with warp-uniform state; one elected lane issues the copies)
        if (lane == 0) {
            tma_prefetch_desc(&tm_a); tma_prefetch_desc(&tm_w);
            if (LCH) { tma_prefetch_desc(&tm_la); tma_prefetch_desc(&tm_lu); }
        }
        uint32_t it = 0;
        bool ok = true;
        for (int t = t_begin; t < t_end && ok; ++t) {
            const int mt = t / NT, nt = t % NT;
            // 128 x 128: the K loop, then the low-rank K loop.  128 x 256: the low-rank K loop of the first 128-column
            // half, the K loop, then the low-rank K loop of the second half (the issuer consumes them in this order)
            for (int jj = 0; jj < KS + NH * LCH; ++jj, ++it) {
                const int s = it % STAGES;
                if (!mbar_wait_warp(bar(B_EMPTY + s), ((it / STAGES) & 1) ^ 1, abort_s, E_PROD | 1)) { ok = false; break; }
                if (!elect_one()) continue;
                const uint32_t dst = s_base + s * ST_BYTES;
                // position in the old order (K loop first): j < KS is a K-loop stage, else low-rank stage j - KS
                const int j = NH == 1 ? jj : (jj < LCH ? KS + jj : (jj < LCH + KS ? jj - LCH : jj));
                if (j < KS) {
                    // codes beyond K are zero-filled by TMA (and never multiplied); scale chunks exist for whole 64-k steps only
                    const uint32_t nst = (uint32_t)min(4, KS4 - 4 * j);
                    mbar_expect_tx(bar(B_FULL + s), ST_A + ST_W + nst * 512u * (1 + NH));
                    tma_load_2d(dst, &tm_a, bar(B_FULL + s), j * 128, mt * BM);
                    tma_load_2d(dst + ST_A, &tm_w, bar(B_FULL + s), j * 128, nt * BN);
                    bulk_load_1d(dst + ST_A + ST_W, p.sfa + ((size_t)mt * KS4 + j * 4) * 512, nst * 512u, bar(B_FULL + s));
#pragma unroll
                    for (int hh = 0; hh < NH; ++hh)
                        bulk_load_1d(dst + ST_A + ST_W + C::ST_SFA + hh * 2048,
                                     p.sfb + ((size_t)(nt * NH + hh) * KS4 + j * 4) * 512, nst * 512u, bar(B_FULL + s));
                } else {
                    const int h = (j - KS) / LCH, c = (j - KS) % LCH;
                    mbar_expect_tx(bar(B_FULL + s), 2 * 128 * 64);
                    tma_load_2d(dst, &tm_la, bar(B_FULL + s), c * 32, mt * BM);
                    tma_load_2d(dst + ST_A, &tm_lu, bar(B_FULL + s), c * 32, nt * BN + h * 128);
                }
            }
        }
        if (!ok && lane == 0) {
            // let copies already in flight land before the CTA goes away (bounded)
            for (int s = 0; s < STAGES; ++s) {
                const uint32_t issued = it > (uint32_t)s ? (it - 1 - s) / STAGES + 1 : 0;
                if (issued) {
                    uint64_t t0 = globaltimer_ns();
                    while (!mbar_try_wait(bar(B_FULL + s), (issued - 1) & 1) && globaltimer_ns() - t0 < 200000000ull) {}
                }
            }
        }
    } else if (warp == 1) {
        // ================================ MMA issuer ================================
        // (the loop runs as a whole warp with warp-uniform state and one elected lane issues; waits carry no suspend-time hint)
        {
            const uint32_t idesc = idesc_mxf4nvf4(BN);
            const uint32_t f16fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
            const uint32_t idesc_lr = umma_idesc(1u, f16fmt, f16fmt, 128);
            uint32_t it = 0, tl = 0, lrn = 0;  // ring stages, tiles, uses of the low-rank slot
            bool ok = true;
            for (int t = t_begin; t < t_end && ok; ++t, ++tl) {
                const int slot = tl % ACC_SLOTS;
                const uint32_t d = tmem_base + TM_ACC + slot * BN;
                // low-rank product of one 128-column half into the single low-rank slot
                auto low_rank_half = [&]() {
                    if (!mbar_wait_warp(bar(B_LR_EMPTY), (lrn & 1) ^ 1, abort_s, E_MMA | 3)) return false;  // previous contents read
                    for (int c = 0; c < LCH; ++c, ++it) {
                        const int s = it % STAGES;
                        if (!mbar_wait_warp(bar(B_FULL + s), (it / STAGES) & 1, abort_s, E_MMA | 4)) return false;
                        tc_fence_after();
                        if (elect_one()) {
                            const uint32_t a_addr = s_base + s * ST_BYTES, w_addr = a_addr + ST_A;
#pragma unroll
                            for (int kk = 0; kk < 2; ++kk)
                                mma_f16(tmem_base + TM_LORA, desc_sw64(a_addr + kk * 32), desc_sw64(w_addr + kk * 32), idesc_lr,
                                        (c | kk) ? 1u : 0u);
                            tc_commit(bar(B_EMPTY + s));
                        }
                    }
                    if (elect_one()) tc_commit(bar(B_LR_FULL));
                    ++lrn;
                    return true;
                };
                // wide tile: the first half's product goes first; its slot and the accumulator were released together
                if (LCH > 0 && NH == 2 && !low_rank_half()) { ok = false; break; }
                if (!mbar_wait_warp(bar(B_ACC_EMPTY + slot), ((tl / ACC_SLOTS) & 1) ^ 1, abort_s, E_MMA | 2)) { ok = false; break; }
                for (int j = 0; j < KS && ok; ++j, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait_warp(bar(B_FULL + s), (it / STAGES) & 1, abort_s, E_MMA | 1)) { ok = false; break; }
                    tc_fence_after();
                    if (elect_one()) {
                        const uint32_t a_addr = s_base + s * ST_BYTES;
                        const uint64_t da = desc_sw128(a_addr), dw = desc_sw128(a_addr + ST_A);
                        const uint32_t sfa_s = a_addr + ST_A + ST_W, sfb_s = sfa_s + C::ST_SFA;
                        const int nst = min(4, KS4 - 4 * j);
#pragma unroll
                        for (int st = 0; st < 4; ++st) {
                            if (st >= nst) break;
                            // this step's scale chunks -> tensor memory, then the MMA that reads them (issue order is kept):
                            // four columns for the 128 rows of A, four per 128 rows of W
                            const uint32_t tsf = tmem_base + TM_SF + (it % C::SF_BUFS) * (4 * C::SF_STEP) + st * C::SF_STEP;
                            tmem_cp_32x128b_warpx4(tsf, umma_desc_kmajor(sfa_s + st * 512, 16, 128));
#pragma unroll
                            for (int hh = 0; hh < NH; ++hh)
                                tmem_cp_32x128b_warpx4(tsf + 4 + 4 * hh, umma_desc_kmajor(sfb_s + (hh * 4 + st) * 512, 16, 128));
                            mma_mxf4nvf4(d, da + 2 * st, dw + 2 * st, idesc, tsf, tsf + 4, (j | st) ? 1u : 0u);
                        }
                        tc_commit(bar(B_EMPTY + s));
                    }
                }
                if (ok && elect_one()) tc_commit(bar(B_ACC_FULL + slot));
                if (ok && LCH > 0 && !low_rank_half()) { ok = false; break; }
            }
        }
    } else {
        // ================================ epilogue ================================
        // a warp reads its lane quarter: lane = row, 32 columns per load
        const int q = warp & 3;
        uint32_t tl = 0, lrn = 0;
        bool ok = true;
        const float alpha = p.alpha;
        for (int t = t_begin; t < t_end && ok; ++t, ++tl) {
            const int m0 = (t / NT) * BM, n0 = (t % NT) * BN;
            const int slot = tl % ACC_SLOTS;
            // the tile's per-column scale and bias, widened once per warp while the K loop runs
            float* epi_s = reinterpret_cast<float*>(smem + C::OFF_EPI) + (warp - 2) * 2 * BN;
            __syncwarp();
            for (int i = lane; i < BN; i += 32) {
                const int n = n0 + i;
                epi_s[i] = (p.wcscales && n < p.N) ? to_f32<T>(__ldg(static_cast<const T*>(p.wcscales) + n)) : 1.0f;
                epi_s[BN + i] = (p.bias && n < p.N) ? to_f32<T>(__ldg(static_cast<const T*>(p.bias) + n)) : 0.0f;
            }
            __syncwarp();
            if (!mbar_wait_warp(bar(B_ACC_FULL + slot), (tl / ACC_SLOTS) & 1, abort_s, E_EPI | 1, 100)) { ok = false; break; }
            tc_fence_after();
            const int m = m0 + q * 32 + lane;
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
            for (int ch = 0; ch < BN / 32; ++ch) {
                if (LCH > 0 && (ch & 3) == 0) {
                    // the low-rank product of this 128-column half
                    if (!mbar_wait_warp(bar(B_LR_FULL), lrn & 1, abort_s, E_EPI | 2, 100)) { ok = false; break; }
                    ++lrn;
                    tc_fence_after();
                }
                uint32_t v[32], lr[32];
                tmem_ld32(lane_addr + TM_ACC + slot * BN + ch * 32, v);
                if (LCH > 0) tmem_ld32(lane_addr + TM_LORA + (ch & 3) * 32, lr);
                tmem_wait_ld();
                if ((ch & 3) == 3) {
                    // this half of the low-rank slot, and after the last half the accumulator slot, are read out
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if (LCH > 0) mbar_arrive(bar(B_LR_EMPTY));
                        if (ch == BN / 32 - 1) mbar_arrive(bar(B_ACC_EMPTY + slot));
                    }
                }
#pragma unroll
                for (int c8 = 0; c8 < 4; ++c8) {
                    const int n = n0 + ch * 32 + c8 * 8;
                    if (n < p.N) {  // N is a multiple of 8
                        float o[8], cs[8], bs[8];
                        *reinterpret_cast<float4*>(&cs[0]) = *reinterpret_cast<const float4*>(epi_s + ch * 32 + c8 * 8);
                        *reinterpret_cast<float4*>(&cs[4]) = *reinterpret_cast<const float4*>(epi_s + ch * 32 + c8 * 8 + 4);
                        *reinterpret_cast<float4*>(&bs[0]) = *reinterpret_cast<const float4*>(epi_s + BN + ch * 32 + c8 * 8);
                        *reinterpret_cast<float4*>(&bs[4]) = *reinterpret_cast<const float4*>(epi_s + BN + ch * 32 + c8 * 8 + 4);
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            float x = __uint_as_float(v[c8 * 8 + e]);
                            if (p.wcscales) x *= cs[e];
                            x *= alpha;
                            if (LCH > 0) x += __uint_as_float(lr[c8 * 8 + e]);
                            if (p.bias) x += bs[e];
                            o[e] = x;
                        }
                        if (m < p.actual_m) {
                            uint4 w;
                            w.x = pack2<T>(o[0], o[1]); w.y = pack2<T>(o[2], o[3]);
                            w.z = pack2<T>(o[4], o[5]); w.w = pack2<T>(o[6], o[7]);
                            *reinterpret_cast<uint4*>(static_cast<T*>(p.out) + (long long)m * p.stride_om + n) = w;
                        }
                    }
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
        tmem_dealloc(tmem_base, 512);
    }
}

// ------------------------------------------------------------------------------------------------
// pre-pass: scales into the instruction's chunk layout, lora_act -> T
// ------------------------------------------------------------------------------------------------
struct PrepackParams {
    const uint8_t* ascales; const uint8_t* wscales; const float* lora_act;
    uint8_t* sfa; uint8_t* sfb; void* la16;
    int M, N, K, R;
    long long stride_asg, stride_wsg, stride_lam;
    int do_a, do_w;  // which of the two scale sides this launch writes (the weight side may have been prepared before)
};

// VEC: both scale arrays have 4-byte-aligned rows of a multiple of four scales, so a thread takes four consecutive rows of
// a 64-k step with four 32-bit loads and turns the 4 x 4 bytes round in registers.
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) prepack_fp4_kernel(const PrepackParams p) {
    const long long tid = (long long)blockIdx.x * 256 + threadIdx.x;
    const int KS4 = p.K / 64;
    const int Mp = (p.M + 127) / 128 * 128, Np = (p.N + 255) / 256 * 256;  // whole 128-row chunks; W: whole wide tiles
    constexpr int RPT = VEC ? 4 : 1;                                        // rows per thread
    const long long a_units = p.do_a ? (long long)KS4 * (Mp / RPT) : 0, w_units = p.do_w ? (long long)KS4 * (Np / RPT) : 0;
    if (tid < a_units + w_units) {
        // one thread per (64-k step, row or four rows): four scales per row -> one 32-bit word of the chunk
        const bool is_w = tid >= a_units;
        const long long u = is_w ? tid - a_units : tid;
        const int rows_p = (is_w ? Np : Mp) / RPT, rows = is_w ? p.N : p.M;
        const int ks = (int)(u / rows_p), r = (int)(u % rows_p) * RPT;
        const uint8_t* src = is_w ? p.wscales : p.ascales;
        const long long sg = is_w ? p.stride_wsg : p.stride_asg;
        uint8_t* dst = (is_w ? p.sfb : p.sfa) + ((size_t)(r / 128) * KS4 + ks) * 512 + (r % 32) * 16 + ((r % 128) / 32) * 4;
        if (VEC) {
            uint32_t k4[4] = {0, 0, 0, 0};  // k4[kb]: rows r .. r + 3 of 16-group kb
            if (r + 3 < rows) {
#pragma unroll
                for (int kb = 0; kb < 4; ++kb)
                    k4[kb] = __ldg(reinterpret_cast<const uint32_t*>(src + (long long)(ks * 4 + kb) * sg + r));
            } else {
#pragma unroll
                for (int kb = 0; kb < 4; ++kb)
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (r + i < rows) k4[kb] |= (uint32_t)__ldg(src + (long long)(ks * 4 + kb) * sg + r + i) << (8 * i);
            }
            // byte i of k4[kb] -> byte kb of row r + i
            const uint32_t lo01 = __byte_perm(k4[0], k4[1], 0x5140), hi01 = __byte_perm(k4[0], k4[1], 0x7362);
            const uint32_t lo23 = __byte_perm(k4[2], k4[3], 0x5140), hi23 = __byte_perm(k4[2], k4[3], 0x7362);
            *reinterpret_cast<uint32_t*>(dst) = __byte_perm(lo01, lo23, 0x5410);
            *reinterpret_cast<uint32_t*>(dst + 16) = __byte_perm(lo01, lo23, 0x7632);
            *reinterpret_cast<uint32_t*>(dst + 32) = __byte_perm(hi01, hi23, 0x5410);
            *reinterpret_cast<uint32_t*>(dst + 48) = __byte_perm(hi01, hi23, 0x7632);
        } else {
            uint32_t w = 0;
            if (r < rows) {
#pragma unroll
                for (int kb = 0; kb < 4; ++kb) w |= (uint32_t)__ldg(src + (long long)(ks * 4 + kb) * sg + r) << (8 * kb);
            }
            *reinterpret_cast<uint32_t*>(dst) = w;
        }
        return;
    }
    const long long u = tid - (a_units + w_units);
    const long long la_units = p.do_a && p.R ? (long long)p.M * (p.R / 8) : 0;
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
struct Scratch { size_t sfa, sfb, la16, total; };
static Scratch scratch_layout(const nb_gemm_args* a) {
    Scratch s;
    const size_t KS4 = a->K / 64;
    size_t off = 0;
    s.sfa = off; off += up256((size_t)((a->M + 127) / 128) * KS4 * 512);
    s.sfb = off; off += up256((size_t)((a->N + 255) / 256 * 2) * KS4 * 512);
    s.la16 = off; off += up256((size_t)a->M * a->R * 2);
    s.total = off;
    return s;
}

template <typename T, int BN_>
static int launch_kernel(const nb_gemm_args* a, const Params& p, const void* la16, cudaStream_t s) {
    using C = Cfg<BN_>;
    CUtensorMap tm_a, tm_w, tm_la, tm_lu;
    const CUtensorMapDataType t16 = std::is_same<T, __nv_bfloat16>::value ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                                          : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    bool ok = make_map(&tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, a->act, a->K / 2, a->M, a->stride_am, 128, BM, CU_TENSOR_MAP_SWIZZLE_128B) &&
              make_map(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, a->wgt, a->K / 2, a->N, a->stride_wn, 128, C::BN, CU_TENSOR_MAP_SWIZZLE_128B);
    // the low-rank operands travel in 128-row boxes for both tile widths (one 128-column half at a time)
    if (ok && a->R > 0)
        ok = make_map(&tm_la, t16, la16, a->R, a->M, (uint64_t)a->R * 2, 32, BM, CU_TENSOR_MAP_SWIZZLE_64B) &&
             make_map(&tm_lu, t16, a->lora_up, a->R, a->N, (uint64_t)a->stride_lun * 2, 32, 128, CU_TENSOR_MAP_SWIZZLE_64B);
    else if (ok) { tm_la = tm_a; tm_lu = tm_w; }
    if (!ok) return NB_ERR_UNSUPPORTED;
    int dev = 0, sms = 0;
    NB_CUDA_CHECK(cudaGetDevice(&dev));
    NB_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int total = ((a->M + BM - 1) / BM) * ((a->N + C::BN - 1) / C::BN);
    const int grid = total < sms ? total : sms;
    auto kern = gemm_fp4_kernel<T, BN_>;
    NB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    kern<<<grid, NTHREADS, C::SMEM_BYTES, s>>>(tm_a, tm_w, tm_la, tm_lu, p);
    NB_CUDA_CHECK(cudaGetLastError());
    return NB_OK;
}

static int64_t prepared_bytes(const nb_gemm_args* a) {
    return (int64_t)((a->N + 255) / 256 * 2) * (a->K / 64) * 512;
}

template <typename T>
static int launch_prepack(const PrepackParams& pp, cudaStream_t s) {
    const long long KS4 = pp.K / 64;
    const bool vec = pp.stride_asg % 4 == 0 && pp.stride_wsg % 4 == 0 && (reinterpret_cast<uintptr_t>(pp.ascales) & 3) == 0 &&
                     (reinterpret_cast<uintptr_t>(pp.wscales) & 3) == 0;
    const int rpt = vec ? 4 : 1;
    const long long units = (pp.do_a ? KS4 * ((pp.M + 127) / 128 * 128 / rpt) : 0) +
                            (pp.do_w ? KS4 * ((pp.N + 255) / 256 * 256 / rpt) : 0) +
                            (pp.do_a && pp.R ? (long long)pp.M * (pp.R / 8) : 0);
    if (units == 0) return NB_OK;
    if (vec) prepack_fp4_kernel<T, true><<<(unsigned)((units + 255) / 256), 256, 0, s>>>(pp);
    else prepack_fp4_kernel<T, false><<<(unsigned)((units + 255) / 256), 256, 0, s>>>(pp);
    NB_CUDA_CHECK(cudaGetLastError());
    return NB_OK;
}

template <typename T>
static int launch_t(const nb_gemm_args* a, cudaStream_t s) {
    const Scratch sc = scratch_layout(a);
    if (!a->scratch || a->scratch_bytes < (int64_t)sc.total || (reinterpret_cast<uintptr_t>(a->scratch) & 255))
        return NB_ERR_INVALID;
    uint8_t* base = static_cast<uint8_t*>(a->scratch);
    PrepackParams pp;
    pp.ascales = static_cast<const uint8_t*>(a->ascales); pp.wscales = static_cast<const uint8_t*>(a->wscales);
    pp.lora_act = static_cast<const float*>(a->lora_act);
    pp.sfa = base + sc.sfa; pp.sfb = base + sc.sfb; pp.la16 = base + sc.la16;
    pp.M = a->M; pp.N = a->N; pp.K = a->K; pp.R = a->R;
    pp.stride_asg = a->stride_asg; pp.stride_wsg = a->stride_wsg; pp.stride_lam = a->stride_lam;
    // the weight side is static: a caller that prepared it once (nb_gemm_w4a4_prepare_weights) passes it in
    const bool prepared = a->wgt_prepared && a->wgt_prepared_bytes >= prepared_bytes(a) &&
                          (reinterpret_cast<uintptr_t>(a->wgt_prepared) & 255) == 0;
    if (prepared) pp.sfb = const_cast<uint8_t*>(static_cast<const uint8_t*>(a->wgt_prepared));
    pp.do_a = 1; pp.do_w = prepared ? 0 : 1;
    const int st = launch_prepack<T>(pp, s);
    if (st != NB_OK) return st;

    Params p = {};
    p.out = a->out; p.bias = a->bias; p.wcscales = a->wcscales;
    p.sfa = pp.sfa; p.sfb = pp.sfb;
    p.M = a->M; p.N = a->N; p.K = a->K; p.actual_m = a->actual_m; p.R = a->R;
    p.alpha = a->alpha; p.stride_om = a->stride_om;
    p.status = static_cast<int*>(a->status);
    // the wide tile when it does not waste columns, or when the matrix is wide enough for the waste not to matter
    const bool wide = a->N % 256 == 0 || a->N >= 2048;
    return wide ? launch_kernel<T, 256>(a, p, pp.la16, s) : launch_kernel<T, 128>(a, p, pp.la16, s);
}

}  // namespace fp4

// Why the block-scaled tensor-core kernel cannot take this NVFP4 call, or nullptr.
const char* tc_fp4_unsupported_reason(const nb_gemm_args* a, const void* epi, int epi_kind) {
    (void)epi;
    if (!a->fp4) return "not NVFP4";
    if (epi_kind != NB_EPI_STORE || a->fuse_silu) return "epilogue";
    if (a->K % 64 || a->N % 8 || a->M < 1) return "K % 64, N % 8";
    if (!aligned16(a->act) || !aligned16(a->wgt) || a->stride_am % 16 || a->stride_wn % 16) return "act / wgt alignment";
    if (!a->out || !aligned16(a->out) || a->stride_om % 8) return "out alignment";
    if (a->bias && (reinterpret_cast<uintptr_t>(a->bias) & 1)) return "bias alignment";
    if (a->R > 0) {
        if (a->R % 16 || !a->lora_act || !a->lora_up) return "rank";
        if (!aligned16(a->lora_act) || a->stride_lam % 4 || !aligned16(a->lora_up) || a->stride_lun % 8) return "LoRA alignment";
    }
    return nullptr;
}

int64_t tc_fp4_scratch_bytes(const nb_gemm_args* a) { return (int64_t)fp4::scratch_layout(a).total; }

// Load-time form of an NVFP4 weight: its block scales in the chunk layout of the block-scaled MMA (the codes are consumed
// as they are).
static bool tc_fp4_weight_ok(const nb_gemm_args* a) {
    return a && a->fp4 && a->wscales && a->N > 0 && a->K > 0 && a->K % 64 == 0 &&
           (a->dtype == NB_DTYPE_BF16 || a->dtype == NB_DTYPE_FP16);
}
int64_t tc_fp4_prepared_bytes(const nb_gemm_args* a) { return tc_fp4_weight_ok(a) ? fp4::prepared_bytes(a) : 0; }
int tc_fp4_prepare_weights(const nb_gemm_args* a, void* dst, int64_t dst_bytes, cudaStream_t s) {
    if (!tc_fp4_weight_ok(a)) return NB_ERR_UNSUPPORTED;
    if (!dst || dst_bytes < fp4::prepared_bytes(a) || (reinterpret_cast<uintptr_t>(dst) & 255)) return NB_ERR_INVALID;
    fp4::PrepackParams pp = {};
    pp.wscales = static_cast<const uint8_t*>(a->wscales); pp.ascales = pp.wscales;
    pp.sfb = static_cast<uint8_t*>(dst);
    pp.M = 0; pp.N = a->N; pp.K = a->K; pp.R = 0;
    pp.stride_wsg = a->stride_wsg; pp.stride_asg = a->stride_wsg;
    pp.do_a = 0; pp.do_w = 1;
    return a->dtype == NB_DTYPE_BF16 ? fp4::launch_prepack<__nv_bfloat16>(pp, s) : fp4::launch_prepack<__half>(pp, s);
}

int launch_tc_fp4(const nb_gemm_args* a, cudaStream_t s) {
    return a->dtype == NB_DTYPE_BF16 ? fp4::launch_t<__nv_bfloat16>(a, s) : fp4::launch_t<__half>(a, s);
}

}  // namespace nb

// Unmasked flash attention on the 5th-generation tensor cores (tcgen05.mma kind::f16, accumulators and the
// probability tile in tensor memory), head dimension 128.
//
// Rounding points follow the reference kernel (nunchaku/ops/triton/attention.py:61-117): q * scale * log2(e) is rounded
// to the input dtype, scores and the running max / sum are fp32 in base 2, the probabilities are rounded to the input
// dtype before P @ V, the accumulator is fp32, one division by the row sum at the end.  One liberty that does not change
// the result beyond fp32 rounding: the running maximum a row subtracts is only raised when the true maximum has grown by
// more than 8 (probabilities stay below 2^8), which makes the rescaling of the output accumulator a rare event.
//
// One launch, no scratch: a CTA owns 128 query rows of one (batch, head) and walks the keys in tiles of 128.
//       warp 0    TMA producer: the Q tile once, K and V tiles through two-stage rings, all straight from the caller's
//                 strided tensors (4-D tensor maps, 128-byte swizzle, no multicast; rows past the end read as zeros).
//                 The softmax warps turn the Q tile into Q' = T(q * scale * log2 e) in place before the first MMA; V is
//                 consumed as it lies (head dimension contiguous) as an MN-major B operand, K as a K-major one.
//       warp 1    MMA issuer for the scores: S_j = Q' K_j^T (8 MMAs, N = 128) into one of two score slots, so the tensor
//                 pipe works on the next scores while the CUDA cores do the softmax of the current tile.
//       warp 10   MMA issuer for O += P_j V_j, with P read from tensor memory as the A operand.
//       warps 2-9 softmax: two warps per 32-row lane quarter, each with one row per thread and half of the 128 columns
//                 (tcgen05.ld 32x32b): partial row max exchanged with the partner through shared memory, exp2, partial
//                 row sum, P -> tensor memory (tcgen05.st), the occasional rescale of O in tensor memory, and the
//                 final O / l store.  Two warps per scheduler hide each other's latencies.
//     Tensor memory: S0 | S1 | O | P0 | P1 = 128 + 128 + 128 + 64 + 64 columns.
// Every mbarrier wait is bounded; on expiry the CTA records a code in the status word and unwinds.
#include <cuda.h>

#include <algorithm>
#include <type_traits>

#include "nb_common.cuh"

namespace nb {
namespace atc {

constexpr int BM = 128, BN = 128, HD = 128;
constexpr int SM_WARPS = 8;
constexpr int NTHREADS = 64 + SM_WARPS * 32 + 32;  // producer, score issuer, softmax warps, P V issuer
constexpr int TILE = 128 * 128 * 2;  // bytes of a 128 x 128 16-bit tile (two 64-wide halves of 16 KB)
constexpr int OFF_Q = 0, OFF_K = TILE, OFF_V = 3 * TILE, OFF_XCH = 5 * TILE;  // exchange: [2 tiles][2 halves][128] max, [2][128] sum
constexpr int OFF_BAR = OFF_XCH + 6 * 128 * 4;
constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
constexpr uint32_t TM_S = 0, TM_O = 256, TM_P = 384;

enum { B_Q = 0, B_KF = 1, B_KE = 3, B_VF = 5, B_VE = 7, B_SF = 9, B_SE = 11, B_PF = 13, B_PV = 15, B_XM = 17, B_QS = 21, B_COUNT = 22 };
enum { E_PROD = 0x210, E_MMA = 0x230, E_SM = 0x240 };

struct Params {
    void* o;
    int Tq, Tkv, H;
    long long stride_ob, stride_om;
    int tq_pad;  // query rows per (batch, head) rounded up to whole tiles
    float qscale;  // softmax scale x log2(e): applied to the Q tile in shared memory, rounded to T (the reference's rounding point)
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
// The same 128-byte-swizzled tile read as an MN-major operand (the 64 values of a 128-byte row run along M / N, the rows
// along K): 8-row groups 1024 bytes apart along K, the two 64-wide halves of the tile half a tile apart along N.
__device__ __forceinline__ uint64_t desc_sw128_mn(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3fff);
    d |= (uint64_t)((TILE / 2) >> 4) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// A operand from tensor memory (row = lane, two 16-bit values per column), B from shared memory
__device__ __forceinline__ void mma_f16_ts(uint32_t d, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(acc)
        : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void* tmap, uint32_t bar, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,"
        "%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,"
        "%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <typename T>
__global__ void __launch_bounds__(NTHREADS, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const int4 kperm, const int4 qperm, const int4 vperm, const Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t s_base = smem_u32(smem);
    const uint32_t s_bar = s_base + OFF_BAR;
    uint32_t* tmem_ptr_s = reinterpret_cast<uint32_t*>(smem + OFF_BAR + 8 * B_COUNT);
    volatile int* abort_s = reinterpret_cast<volatile int*>(smem + OFF_BAR + 8 * B_COUNT + 8);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    auto bar = [&](int i) { return s_bar + 8u * i; };

    if (threadIdx.x == 0) {
        mbar_init(bar(B_Q), 1);
        mbar_init(bar(B_QS), SM_WARPS);
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar(B_KF + i), 1); mbar_init(bar(B_KE + i), 1);
            mbar_init(bar(B_VF + i), 1); mbar_init(bar(B_VE + i), 1);
            mbar_init(bar(B_SF + i), 1); mbar_init(bar(B_SE + i), SM_WARPS);
            mbar_init(bar(B_PF + i), SM_WARPS); mbar_init(bar(B_PV + i), 1);
        }
        for (int i = 0; i < 4; ++i) mbar_init(bar(B_XM + i), 2);  // the two warps that share a lane quarter
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

    const int m0 = blockIdx.x * BM, head = blockIdx.y, batch = blockIdx.z;
    const int bh = batch * p.H + head;
    const int NT = (p.Tkv + BN - 1) / BN;

    if (warp == 0) {
        // ================================ producer ================================
        if (lane == 0) {
            tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v);
            mbar_expect_tx(bar(B_Q), TILE);
            {
                // Q from the caller's strided (B, H, T, D) view, like K below; rows past Tq read as zeros
                int c[4];
                c[0] = 0;
                c[qperm.x] = m0; c[qperm.y] = head; c[qperm.z] = batch;
                tma_load_4d(s_base + OFF_Q, &tm_q, bar(B_Q), 0, c[1], c[2], c[3]);
                tma_load_4d(s_base + OFF_Q + TILE / 2, &tm_q, bar(B_Q), 64, c[1], c[2], c[3]);
            }
            bool ok = true;
            for (int j = 0; j < NT && ok; ++j) {
                const int s = j & 1;
                const uint32_t par = ((j >> 1) & 1) ^ 1;  // parity of the stage's previous use, tile j - 2
                // stage s is free once the MMAs of its previous use have completed: the scores' / the product's own barrier
                if (j >= 2 && !mbar_wait(bar(B_SF + s), par, abort_s, E_PROD | 1, 50)) { ok = false; break; }
                mbar_expect_tx(bar(B_KF + s), TILE);
                {
                    // coordinates (d, key, head, batch) in the order the tensor map sorted the outer dimensions by stride
                    int c[4];
                    c[0] = 0;
                    c[kperm.x] = j * BN; c[kperm.y] = head; c[kperm.z] = batch;
                    tma_load_4d(s_base + OFF_K + s * TILE, &tm_k, bar(B_KF + s), 0, c[1], c[2], c[3]);
                    tma_load_4d(s_base + OFF_K + s * TILE + TILE / 2, &tm_k, bar(B_KF + s), 64, c[1], c[2], c[3]);
                }
                if (j >= 2 && !mbar_wait(bar(B_PV + s), par, abort_s, E_PROD | 2, 50)) { ok = false; break; }
                mbar_expect_tx(bar(B_VF + s), TILE);
                {
                    // V as it lies in the caller's view: 128 keys x (two halves of) 64 head-dimension values
                    int c[4];
                    c[0] = 0;
                    c[vperm.x] = j * BN; c[vperm.y] = head; c[vperm.z] = batch;
                    tma_load_4d(s_base + OFF_V + s * TILE, &tm_v, bar(B_VF + s), 0, c[1], c[2], c[3]);
                    tma_load_4d(s_base + OFF_V + s * TILE + TILE / 2, &tm_v, bar(B_VF + s), 64, c[1], c[2], c[3]);
                }
            }
            if (!ok) {
                // let copies already in flight land before the CTA goes away (bounded)
                uint64_t t0 = globaltimer_ns();
                while (globaltimer_ns() - t0 < 100000000ull) {}
            }
        }
    } else if (warp == 1) {
        // ================================ MMA issuer: scores ================================
        // The issuing thread pays ~100 cycles per tcgen05.mma and more per commit and wait, and a 128 x 128 x 16 MMA is only
        // 64 cycles of tensor work, so the two products have an issuing warp each and every descriptor is one add away
        // from a precomputed base.  A commit doubles as the "stage consumed" signal for the producer.
        // (the loop runs as a whole warp with warp-uniform state and one elected lane issues: a loop run by one lane inside a
        // divergent branch, and waits with a suspend-time hint, cost the issuing warps of the int4 GEMM most of their time)
        {
            const uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
            const uint32_t idesc = umma_idesc(1u, fmt, fmt, 128);
            bool ok = mbar_wait_warp(bar(B_QS), 0, abort_s, E_MMA | 1);  // the Q tile has landed and been scaled
            const uint64_t dq = desc_sw128(s_base + OFF_Q), dk0 = desc_sw128(s_base + OFF_K);
            for (int j = 0; j < NT && ok; ++j) {
                const int b = j & 1;
                const uint32_t par = (j >> 1) & 1;
                if (!mbar_wait_warp(bar(B_KF + b), par, abort_s, E_MMA | 2)) { ok = false; break; }
                if (!mbar_wait_warp(bar(B_SE + b), par ^ 1, abort_s, E_MMA | 3)) { ok = false; break; }
                tc_fence_after();
                if (elect_one()) {
                    const uint64_t dk = dk0 + (uint64_t)(b * (TILE >> 4));
                    const uint32_t d = tmem_base + TM_S + b * 128;
                    // the descriptor's start-address field counts 16-byte units: +2 per 32-byte K step, +1024 per 64-wide half
#pragma unroll
                    for (int dh = 0; dh < 2; ++dh)
#pragma unroll
                        for (int st = 0; st < 4; ++st)
                            mma_f16(d, dq + dh * 1024 + st * 2, dk + dh * 1024 + st * 2, idesc, (dh || st) ? 1u : 0u);
                    tc_commit(bar(B_SF + b));
                }
            }
        }
    } else if (warp == 2 + SM_WARPS) {
        // ================================ MMA issuer: P V ================================
        {
            const uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
            // V is the B operand with its N dimension (the head dimension) contiguous in shared memory: "MN-major"
            const uint32_t idesc = umma_idesc(1u, fmt, fmt, 128) | (1u << 16);
            const uint64_t dv0 = desc_sw128_mn(s_base + OFF_V);
            bool ok = true;
            for (int i = 0; i < NT && ok; ++i) {
                const int b = i & 1;
                const uint32_t par = (i >> 1) & 1;
                if (!mbar_wait_warp(bar(B_PF + b), par, abort_s, E_MMA | 4)) { ok = false; break; }
                if (!mbar_wait_warp(bar(B_VF + b), par, abort_s, E_MMA | 5)) { ok = false; break; }
                tc_fence_after();
                if (elect_one()) {
                    const uint64_t dv = dv0 + (uint64_t)(b * (TILE >> 4));
                    const uint32_t pa = tmem_base + TM_P + b * 64;
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks)  // 16 keys per MMA: 16 rows of 128 bytes further on
                        mma_f16_ts(tmem_base + TM_O, pa + ks * 8, dv + ks * (16 * 128 >> 4), idesc, (i > 0 || ks) ? 1u : 0u);
                    tc_commit(bar(B_PV + b));
                }
            }
        }
    } else {
        // ================================ softmax ================================
        const int q = warp & 3;            // lane quarter this warp may read
        const int hf = (warp - 2) >> 2;    // column half of the score / output tile
        const int row = q * 32 + lane;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
        float* xmax = reinterpret_cast<float*>(smem + OFF_XCH);            // [tile parity][half][128]
        float* xsum = reinterpret_cast<float*>(smem + OFF_XCH) + 4 * 128;  // [half][128]
        float m_used = -INFINITY, l = 0.f;
        uint32_t xph = 0;
        bool ok = mbar_wait_warp(bar(B_Q), 0, abort_s, E_SM | 7);
        if (ok) {
            // Q' = T(q * scale * log2 e), in place on the tile the TMA load put into shared memory (element-wise, so the
            // swizzle does not matter): 2048 16-byte units over the 256 softmax threads
            const int st = (warp - 2) * 32 + lane;
#pragma unroll
            for (int i = 0; i < TILE / 16 / (SM_WARPS * 32); ++i) {
                uint4* u = reinterpret_cast<uint4*>(smem + OFF_Q) + st + i * (SM_WARPS * 32);
                const uint4 raw = *u;
                const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
                uint32_t z[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = unpack2<T>(w[e]);
                    z[e] = pack2<T>(f.x * p.qscale, f.y * p.qscale);
                }
                *u = make_uint4(z[0], z[1], z[2], z[3]);
            }
            // the tensor cores read shared memory through the async proxy: make these generic-proxy writes visible to it
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(B_QS));
        }
        for (int j = 0; j < NT && ok; ++j) {
            const int b = j & 1;
            const uint32_t par = (j >> 1) & 1;
            if (!mbar_wait_warp(bar(B_SF + b), par, abort_s, E_SM | 1, 100)) { ok = false; break; }
            tc_fence_after();
            float s[64];
#pragma unroll
            for (int c = 0; c < 2; ++c)
                tmem_ld32(lane_addr + TM_S + b * 128 + hf * 64 + c * 32, *reinterpret_cast<float(*)[32]>(&s[c * 32]));
            tmem_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(B_SE + b));  // the score slot may be overwritten by tile j + 2
            if (j == NT - 1 && (p.Tkv & (BN - 1))) {
                const int valid = p.Tkv - j * BN - hf * 64;
#pragma unroll
                for (int i = 0; i < 64; ++i)
                    if (i >= valid) s[i] = -INFINITY;
            }
            float m8[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) m8[i] = s[i];
#pragma unroll
            for (int i = 8; i < 64; ++i) m8[i & 7] = fmaxf(m8[i & 7], s[i]);
            float mx = fmaxf(fmaxf(fmaxf(m8[0], m8[1]), fmaxf(m8[2], m8[3])), fmaxf(fmaxf(m8[4], m8[5]), fmaxf(m8[6], m8[7])));
            // the row maximum over both column halves: exchange with the partner warp (buffers alternate with the tile)
            xmax[(b * 2 + hf) * 128 + row] = mx;
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(B_XM + q));
            if (!mbar_wait_warp(bar(B_XM + q), xph & 1, abort_s, E_SM | 5, 100)) { ok = false; break; }
            ++xph;
            mx = fmaxf(mx, xmax[(b * 2 + (hf ^ 1)) * 128 + row]);
            // raise the subtracted maximum only when it lags by more than 8 (or at the first tile); both warps of a row
            // see the same numbers and take the same decision
            const bool need = mx > m_used + 8.0f;
            if (__any_sync(0xffffffffu, need)) {
                const float m_new = fmaxf(m_used, mx);
                if (j > 0) {
                    // O must hold every product issued so far before it is rescaled; this warp scales its column half
                    if (!mbar_wait_warp(bar(B_PV + ((j - 1) & 1)), ((j - 1) >> 1) & 1, abort_s, E_SM | 2, 100)) { ok = false; break; }
                    tc_fence_after();
                    const float alpha = ex2(m_used - m_new);
#pragma unroll 1
                    for (int c = 0; c < 2; ++c) {
                        float o[32];
                        uint32_t w[32];
                        tmem_ld32(lane_addr + TM_O + hf * 64 + c * 32, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) w[i] = __float_as_uint(o[i] * alpha);
                        tmem_st32(lane_addr + TM_O + hf * 64 + c * 32, w);
                    }
                    tmem_wait_st();
                    l *= alpha;
                }
                m_used = m_new;
            }
            // probabilities: fp32 for the (partial) row sum, rounded to T for the product
            uint32_t pk[32];
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const float p0 = ex2(s[2 * i] - m_used), p1 = ex2(s[2 * i + 1] - m_used);
                sum4[i & 3] += p0 + p1;
                pk[i] = pack2<T>(p0, p1);
            }
            l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            // the P slot is free once the product that read it two tiles ago has completed
            if (j >= 2 && !mbar_wait_warp(bar(B_PV + b), ((j - 2) >> 1) & 1, abort_s, E_SM | 3, 100)) { ok = false; break; }
            tc_fence_after();
            tmem_st32(lane_addr + TM_P + b * 64 + hf * 32, pk);
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(B_PF + b));
        }
        if (ok && NT > 0) {
            // total row sum = the two halves' partial sums
            xsum[hf * 128 + row] = l;
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(B_XM + q));
            ok = mbar_wait_warp(bar(B_XM + q), xph & 1, abort_s, E_SM | 6, 100);
            if (ok) l += xsum[(hf ^ 1) * 128 + row];
        }
        if (ok && NT > 0 && mbar_wait_warp(bar(B_PV + ((NT - 1) & 1)), ((NT - 1) >> 1) & 1, abort_s, E_SM | 4, 100)) {
            tc_fence_after();
            const int m = m0 + row;
            const float inv = 1.0f / (l == 0.f ? 1.0f : l);
            T* og = static_cast<T*>(p.o) + (long long)batch * p.stride_ob + (long long)m * p.stride_om + (long long)head * HD + hf * 64;
#pragma unroll 1
            for (int c = 0; c < 2; ++c) {
                float o[32];
                tmem_ld32(lane_addr + TM_O + hf * 64 + c * 32, o);
                tmem_wait_ld();
                if (m < p.Tq) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        uint4 w;
                        w.x = pack2<T>(o[8 * u] * inv, o[8 * u + 1] * inv);
                        w.y = pack2<T>(o[8 * u + 2] * inv, o[8 * u + 3] * inv);
                        w.z = pack2<T>(o[8 * u + 4] * inv, o[8 * u + 5] * inv);
                        w.w = pack2<T>(o[8 * u + 6] * inv, o[8 * u + 7] * inv);
                        *reinterpret_cast<uint4*>(og + c * 32 + u * 8) = w;
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
static bool make_map(CUtensorMap* m, CUtensorMapDataType dt, int rank, const void* base, const cuuint64_t* dims,
                     const cuuint64_t* strides_bytes, const cuuint32_t* box) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    return fn(m, dt, rank, const_cast<void*>(base), dims, strides_bytes, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// A 4-D tensor map over the caller's strided (B, H, T, D) view of Q or K (element strides; D contiguous): the outer
// dimensions sorted by stride, as the encoder wants them; `perm` = the coordinate slot of (row, head, batch).
static bool make_view_map(CUtensorMap* m, int4* perm, CUtensorMapDataType t16, const void* base, int T_, int H, int B,
                          long long stride_t, long long stride_h, long long stride_b, int box_rows) {
    struct Dim { cuuint64_t size, stride; int role; } d[3] = {{(cuuint64_t)T_, (cuuint64_t)stride_t * 2, 0},
                                                               {(cuuint64_t)H, (cuuint64_t)stride_h * 2, 1},
                                                               {(cuuint64_t)B, (cuuint64_t)stride_b * 2, 2}};
    std::stable_sort(d, d + 3, [](const Dim& x, const Dim& y) { return x.stride < y.stride; });
    cuuint64_t dims[4] = {HD, d[0].size, d[1].size, d[2].size};
    cuuint64_t str[3] = {d[0].stride, d[1].stride, d[2].stride};
    cuuint32_t box[4] = {64, 1, 1, 1};
    int pos[3];
    for (int i = 0; i < 3; ++i) {
        pos[d[i].role] = i + 1;
        if (d[i].role == 0) box[i + 1] = (cuuint32_t)box_rows;
    }
    *perm = make_int4(pos[0], pos[1], pos[2], 0);
    // a dimension of size 1 may carry any stride; give it a valid one.  (A zero or unaligned stride on a larger dimension --
    // a view expanded over heads or batch -- never gets here: attn_tc_unsupported_reason refuses it.)
    for (int i = 0; i < 3; ++i)
        if (dims[i + 1] == 1 && (str[i] == 0 || str[i] % 16)) str[i] = 16;
    return make_map(m, t16, 4, base, dims, str, box);
}


template <typename T>
static int launch_t(const nb_attn_args* a, cudaStream_t s) {
    const int tq_pad = (a->Tq + BM - 1) / BM * BM;  // (Q, K and V are read in place: the kernel needs no scratch)

    const CUtensorMapDataType t16 = std::is_same<T, __nv_bfloat16>::value ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                                          : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUtensorMap tm_q, tm_k, tm_v;
    bool ok;
    int4 qperm;
    ok = make_view_map(&tm_q, &qperm, t16, a->q, a->Tq, a->H, a->B, a->stride_qm, a->stride_qh, a->stride_qb, BM);
    int4 vperm;
    ok = ok && make_view_map(&tm_v, &vperm, t16, a->v, a->Tkv, a->H, a->B, a->stride_vn, a->stride_vh, a->stride_vb, BN);
    int4 kperm;
    ok = ok && make_view_map(&tm_k, &kperm, t16, a->k, a->Tkv, a->H, a->B, a->stride_kn, a->stride_kh, a->stride_kb, BN);
    if (!ok) return NB_ERR_UNSUPPORTED;

    Params p = {};
    p.o = a->o; p.Tq = a->Tq; p.Tkv = a->Tkv; p.H = a->H;
    p.stride_ob = a->stride_ob; p.stride_om = a->stride_om;
    p.tq_pad = tq_pad;
    p.qscale = a->scale * 1.4426950408889634f;
    p.status = static_cast<int*>(a->status);
    auto kern = attention_tc_kernel<T>;
    NB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    kern<<<dim3(tq_pad / BM, a->H, a->B), NTHREADS, SMEM_BYTES, s>>>(tm_q, tm_k, tm_v, kperm, qperm, vperm, p);
    NB_CUDA_CHECK(cudaGetLastError());
    return NB_OK;
}

}  // namespace atc

// Why the tcgen05 kernel cannot take this attention call, or nullptr.
const char* attn_tc_unsupported_reason(const nb_attn_args* a) {
    if (a->D != 128) return "head dimension";
    if (a->Tq < 1 || a->Tkv < 1) return "empty";
    if (!aligned16(a->o) || a->stride_om % 8 || a->stride_ob % 8) return "output alignment";
    if (a->B > 65535 || a->H > 65535) return "grid";
    // K is read through a 4-D tensor map on the caller's view: every dimension larger than 1 needs a non-zero stride of
    // whole 16-byte units (a K broadcast over heads or batch by `expand` has stride 0 there)
    const long long ks[3] = {a->stride_kn, a->stride_kh, a->stride_kb};
    const int kn[3] = {a->Tkv, a->H, a->B};
    for (int i = 0; i < 3; ++i)
        if (kn[i] > 1 && (ks[i] <= 0 || ks[i] % 8)) return "K stride (broadcast or unaligned view)";
    if (!aligned16(a->k)) return "K alignment";
    const long long qs[3] = {a->stride_qm, a->stride_qh, a->stride_qb};
    const int qn[3] = {a->Tq, a->H, a->B};
    for (int i = 0; i < 3; ++i)
        if (qn[i] > 1 && (qs[i] <= 0 || qs[i] % 8)) return "Q stride (broadcast or unaligned view)";
    if (!aligned16(a->q)) return "Q alignment";
    const long long vs[3] = {a->stride_vn, a->stride_vh, a->stride_vb};
    for (int i = 0; i < 3; ++i)
        if (kn[i] > 1 && (vs[i] <= 0 || vs[i] % 8)) return "V stride (broadcast or unaligned view)";
    if (!aligned16(a->v)) return "V alignment";
    return nullptr;
}
int64_t attn_tc_scratch_bytes(const nb_attn_args* a) { (void)a; return 0; }
int launch_attention_tc(const nb_attn_args* a, cudaStream_t s) {
    return a->dtype == NB_DTYPE_BF16 ? atc::launch_t<__nv_bfloat16>(a, s) : atc::launch_t<__half>(a, s);
}

}  // namespace nb


// W4A4 int4 GEMM on the 5th-generation tensor cores, CTA-pair form: a cluster of two CTAs owns a 256 x 256 output tile
// (tcgen05.mma.cta_group::2, M = 256, N = 256, kind::f8f6f4 on e4m3-encoded int4 values, exact integer-valued fp32 group
// sums in tensor memory), with the low-rank branch and the fused epilogues.
//
// Arithmetic contract (reference: nunchaku/ops/triton/gemm_w4a4.py:446-488 and :155-209): for every 64-wide K group g one
// EXACT int32 dot p_g[m,n]; acc += float(p_g) * as[g,m] * ws[g,n] in fp32; then + T(lora_act) . lora_up^T (16-bit
// operands, fp32 accumulate), + bias, epilogue, one rounding to T.
//
// Why a pair.  Per 64-group a CTA computes 128 x 256 outputs from its own 128 activation rows (8 KB as e4m3 bytes) and HALF
// of the tile's 256 weight rows (8 KB); the tensor cores of both SMs read both halves of W from the two shared memories.
// That is 16 KB from L2 per 128 x 256 x 64 group -- half of what two independent 128 x 128 tiles pull -- and L2 -> SM operand
// delivery is what bounds the single-CTA kernel right behind its drain (TMA from L2: 25 B/clk/SM measured).  No load is multicast: every CTA issues plain TMA
// loads into its own shared memory; warp 1 of the second CTA relays "my stage has landed" to the first CTA, whose warp 1
// issues the MMAs for both; tcgen05.commit signals the barriers of both CTAs.
//
// Roles (640 threads per CTA; warps 2 and 3 only exist to complete the control warp group):
//   warp 0     TMA producer: per ring stage (two K groups) this CTA's A rows and W rows (128 x 128 B each, 128-byte
//              swizzle) and the two groups' scale rows; low-rank chunks of 32 ranks travel through the same ring.
//   warp 1     first CTA: MMA issuer, per K group two 256 x 256 x 32 MMAs into one of TWO 256-column accumulator slots and
//              one commit ("slot full", both CTAs); after the last group the low-rank product (kind::f16) goes into the next
//              slot like one more group.  Second CTA: relay.
//   warps 4-19 drain: sixteen warps = four per scheduler, so that the tensor-memory load of one warp (the longest latency
//              in the loop) hides behind the arithmetic of the other three.  A warp owns 32 rows x 64 columns = 64 fp32
//              accumulators per thread and reads a group's sums in four chunks (tcgen05.ld.16x256b.x4: 16 lanes x 32 columns,
//              16 registers): t = p * as (packed multiply), acc = fma(t, ws, acc) (packed FMA).  Scales sit in shared
//              memory in the order the threads read them: one 128-bit load gives a thread its two row scales as
//              duplicated pairs, two give it its eight fp32 column scales.  After the last chunk's load the warp frees the
//              slot (arrive on the first CTA's barrier) so the next group's MMAs overlap the arithmetic.
//   Epilogue (same warps, accumulators in registers): bias, optional per-head RMSNorm + RoPE, or GELU + next-layer int4
//              re-quantisation with the LoRA-down product on mma.sync straight from the accumulator registers; rounding and
//              coalesced stores through a per-warp staging tile.
//
// Every wait on an mbarrier is bounded (~2 s); on expiry the CTA records a code in the status word, unwinds without
// touching more data and frees its tensor memory after the pair has met at a cluster barrier.
#include <cuda.h>

#include <type_traits>

#include "nb_common.cuh"

namespace nb {
namespace tcp {

constexpr int BM = 128;   // rows per CTA (256 per pair)
constexpr int BN = 256;   // columns per pair tile; each CTA keeps 128 of its W rows in shared memory
constexpr int STAGES = 4;
constexpr int NSLOT = 2;
constexpr int DRAIN_WARPS = 16;
constexpr int CTRL_WARPS = 4;   // one warp group: TMA producer, MMA issuer / relay, two idle warps
constexpr int NTHREADS = (CTRL_WARPS + DRAIN_WARPS) * 32;
constexpr int LAUNCH_REGS = 96;   // what 640 threads per CTA leave per thread (the compiler's cap under the launch bound)
constexpr int CTRL_REGS = 32, DRAIN_REGS = 112;
// setmaxnreg.inc can only take what setmaxnreg.dec has put into the CTA's pool: it blocks until the pool has enough, for ever
// if it never will.  The control warp group must give back at least what the four drain warp groups ask for.
static_assert((LAUNCH_REGS - CTRL_REGS) * 128 >= (DRAIN_REGS - LAUNCH_REGS) * DRAIN_WARPS * 32, "register pool of the CTA");
constexpr int COLS = 64;  // columns one drain warp owns
constexpr int NJ = COLS / 8;

struct Cfg {
    static constexpr int ST_A = BM * 128, ST_W = 128 * 128;   // two K groups of e4m3 bytes per row
    static constexpr int ST_AS = 2 * BM * 8;                  // per group and row: (as, as), rows in drain order
    static constexpr int ST_WS = 2 * BN * 4;                  // per group and column: ws as fp32, columns in drain order
    static constexpr int ST_BYTES = ST_A + ST_W + ST_AS + ST_WS;
    static constexpr int STG_PITCH = COLS * 2 + 16;
    static constexpr int STG_WARP = 32 * STG_PITCH;           // 4608 B per warp
    static constexpr int STG_BYTES = DRAIN_WARPS * STG_WARP;
    static constexpr int XCH_BYTES = 2 * DRAIN_WARPS * 32 * 4;
    static constexpr int OFF_ST = 0;
    static constexpr int OFF_STG = OFF_ST + STAGES * ST_BYTES;
    static constexpr int OFF_XCH = OFF_STG + STG_BYTES;
    static constexpr int OFF_BAR = OFF_XCH + XCH_BYTES;
    static constexpr int SMEM_BYTES = OFF_BAR + 512 + 1024;
    static constexpr int TMEM_COLS = NSLOT * BN;              // 512
};
static_assert(Cfg::ST_BYTES % 1024 == 0, "stage buffers must stay 1 KB aligned for the 128-byte swizzle");
static_assert(Cfg::SMEM_BYTES <= 232448, "shared memory budget");
static_assert(Cfg::STG_WARP >= 32 * 32 * 4 + 0, "the staging tile also holds a warp's 32 x 32 fp32 LoRA-down partial");

enum {  // barrier indices
    B_FULL = 0,                     // TMA: this CTA's half of the stage has landed
    B_PFULL = B_FULL + STAGES,      // (first CTA) the second CTA's half of the stage has landed
    B_SCDONE = B_PFULL + STAGES,    // one arrival per drain warp: an int8 stage's MMAs are complete and its scales have been read
    B_ACC_FULL = B_SCDONE + STAGES, // tcgen05.commit: the slot's group is complete (signalled in both CTAs)
    B_ACC_EMPTY = B_ACC_FULL + NSLOT,// (first CTA) one arrival per drain warp of the pair: the slot has been read out
    B_XCH = B_ACC_EMPTY + NSLOT,    // 8: exchange between the warps that share rows (lane quarter x head)
    B_LX = B_XCH + 8,               // 4: the four column slices of a lane quarter (LoRA-down partial sums)
    B_LRDONE = B_LX + 4,            // tcgen05.commit: the MMAs of a low-rank stage have read its operands (both CTAs)
    B_COUNT = B_LRDONE + STAGES
};
enum { E_PROD = 0x310, E_MMA = 0x330, E_DRAIN = 0x340, E_RELAY = 0x350 };

struct Params {
    void* out;
    const void* bias;
    int32_t* p_out;  // debug: (K/64, M, N) group sums
    int M, N, K, actual_m, R;
    long long stride_om;
    int* status;
    // QK epilogue
    const void* norm_q;
    const void* norm_k;
    const float* rot;
    long long stride_rm;
    int rot_rows;
    float eps;
    // GELU + re-quantisation epilogue
    uint8_t* qout;
    void* oscales;
    const float* inv_smooth;   // (N) fp32 reciprocals, or null
    const void* lora_down_t;   // (R2, N) T: lora_down transposed, or null
    float* lora_part;          // (N / 256, M, R2) fp32 partial sums, one slab per column tile
    int R2;
    float shift;
    long long stride_qm, stride_osg;
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
// ACC = 0 overwrites the accumulator, 1 adds to it
template <int ACC>
__device__ __forceinline__ void mma2_f8(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "n"(ACC)
        : "memory");
}
template <int ACC>
__device__ __forceinline__ void mma2_f16(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "n"(ACC)
        : "memory");
}
__device__ __forceinline__ uint64_t desc64(uint32_t lo, uint32_t hi) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
    return d;
}
// D (16 x 8, fp32) += A (16 x 16, row) * B (16 x 8, col), 16-bit operands: the legacy warp-level MMA, used for the small
// LoRA-down product whose A operand is already in the accumulator registers in exactly this fragment layout
template <typename T>
__device__ __forceinline__ void mma_sync_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if (std::is_same<T, __nv_bfloat16>::value)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Registers are handed out per warp group (128 threads): 640 threads start with 96 registers each, the control warp group
// gives 64 of them back (setmaxnreg.dec to 32: 8192 registers into the CTA's pool) and the four drain warp groups grow to
// 112 (setmaxnreg.inc: 8192 registers out of that pool).  (576 threads at 112 registers do not launch: the fifth warp
// group is charged in full.)  The host refuses to launch if the compiled kernel does not start with exactly 96 registers.
// 128-bit shared-memory load as two 64-bit registers (pairs of fp32 for the packed operations)
__device__ __forceinline__ void lds2x64(uint32_t addr, uint64_t& a, uint64_t& b) {
    asm volatile("ld.shared.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "r"(addr));
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {  // shared-memory load by 32-bit address: no 64-bit pointer kept live
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

// The control warps run their loops as whole warps, with everything but the issuing instruction itself warp-uniform (stage
// and slot counters, barrier addresses, descriptors), and one elected lane issues.  They share their schedulers and the
// shared-memory pipe with drain warps that keep both busy (measured from the issuer warp inside the running kernel: about
// 12 cycles per instruction issued, 70 per dependent shared-memory access), so what counts is the number of dependent
// operations per K group: a loop run by one lane inside a divergent branch took about 1700 cycles per ring stage.
template <int EPI, typename T, bool DEBUG_P>
__global__ void __launch_bounds__(NTHREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w,
                    const __grid_constant__ CUtensorMap tm_as, const __grid_constant__ CUtensorMap tm_ws,
                    const __grid_constant__ CUtensorMap tm_la, const __grid_constant__ CUtensorMap tm_lu, const Params p) {
    using C = Cfg;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t s_base = smem_u32(smem);
    const uint32_t s_bar = s_base + C::OFF_BAR;
    uint32_t* tmem_ptr_s = reinterpret_cast<uint32_t*>(smem + C::OFF_BAR + 8 * B_COUNT);
    volatile int* abort_s = reinterpret_cast<volatile int*>(smem + C::OFF_BAR + 8 * B_COUNT + 8);

    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;  // (warp-uniform by construction)
    const uint32_t rank = cluster_ctarank();
    auto bar = [&](int i) { return s_bar + 8u * i; };

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) {
            mbar_init(bar(B_FULL + i), 1);
            mbar_init(bar(B_PFULL + i), 1);
            mbar_init(bar(B_SCDONE + i), DRAIN_WARPS);
            mbar_init(bar(B_LRDONE + i), 1);
        }
        for (int i = 0; i < NSLOT; ++i) {
            mbar_init(bar(B_ACC_FULL + i), 1);
            mbar_init(bar(B_ACC_EMPTY + i), 2 * DRAIN_WARPS);  // (used in the first CTA only)
        }
        for (int i = 0; i < 8; ++i) mbar_init(bar(B_XCH + i), 2);
        for (int i = 0; i < 4; ++i) mbar_init(bar(B_LX + i), 4);
        *abort_s = 0;
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc2(smem_u32(tmem_ptr_s), C::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers exist before anything is signalled across
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr_s;

    // static contiguous tile range of this pair; tile t = m_blk * NT + n_blk (256 x 256)
    const int MT = (p.M + 2 * BM - 1) / (2 * BM), NT = (p.N + BN - 1) / BN;
    const int total = MT * NT;
    const int pairs = gridDim.x / 2, pid = blockIdx.x / 2;
    const int per = (total + pairs - 1) / pairs;
    const int t_begin = min(total, pid * per), t_end = min(total, t_begin + per);
    const int G = p.K / 64;
    const int GS = (G + 1) / 2;       // int8 stages per tile (two K groups each)
    const int LCH = (p.R + 31) / 32;  // low-rank stages per tile (32 ranks each)

    if (warp < CTRL_WARPS) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(CTRL_REGS));
    if (warp == 0) {
        // ================================ TMA producer (both CTAs) ================================
        if (lane == 0) {
            tma_prefetch_desc(&tm_a); tma_prefetch_desc(&tm_w); tma_prefetch_desc(&tm_as); tma_prefetch_desc(&tm_ws);
            if (LCH) { tma_prefetch_desc(&tm_la); tma_prefetch_desc(&tm_lu); }
        }
        // per stage (one bit each): the parity of its int8 fills / low-rank fills so far, and what the last fill was.  An int8
        // fill is released by the sixteen drain warps (they read its scales after its MMAs have completed), a low-rank
        // fill by the MMAs' own completion: a rank above 128 needs more stages than the ring has, so those must come
        // free before the drain has seen the low-rank product.
        uint32_t it = 0, s = 0, n_sc = 0, n_lr = 0, last_lr = 0;
        bool ok = true;
        for (int t = t_begin; t < t_end && ok; ++t) {
            const int m0 = (t / NT) * (2 * BM) + (int)rank * BM, n0 = (t % NT) * BN;
            for (int j = 0; j < GS + LCH; ++j, ++it) {
                if (it >= (uint32_t)STAGES) {
                    const bool was_lr = (last_lr >> s) & 1u;
                    const uint32_t n = ((was_lr ? n_lr : n_sc) >> s) & 1u;  // parity of the fills of that kind so far (>= 1 fill)
                    if (!mbar_wait_warp(bar(was_lr ? B_LRDONE : B_SCDONE) + 8u * s, n ^ 1u, abort_s, E_PROD | 1)) { ok = false; break; }
                }
                const uint32_t dst = s_base + C::OFF_ST + s * C::ST_BYTES;
                const uint32_t fb = bar(B_FULL) + 8u * s;
                if (j < GS) {
                    n_sc ^= 1u << s; last_lr &= ~(1u << s);
                    if (elect_one()) {
                        mbar_expect_tx(fb, C::ST_BYTES);
                        tma_load_2d(dst, &tm_a, fb, j * 128, m0);
                        tma_load_2d(dst + C::ST_A, &tm_w, fb, j * 128, n0 + (int)rank * 128);
                        tma_load_2d(dst + C::ST_A + C::ST_W, &tm_as, fb, m0 * 2, j * 2);
                        tma_load_2d(dst + C::ST_A + C::ST_W + C::ST_AS, &tm_ws, fb, n0, j * 2);
                    }
                } else {
                    n_lr ^= 1u << s; last_lr |= 1u << s;
                    if (elect_one()) {
                        // 32 ranks of T(lora_act) rows m0.. and of this CTA's 128 lora_up rows: 128 x 64 B each, 64-byte swizzle
                        mbar_expect_tx(fb, 2 * 128 * 64);
                        tma_load_2d(dst, &tm_la, fb, (j - GS) * 32, m0);
                        tma_load_2d(dst + C::ST_A, &tm_lu, fb, (j - GS) * 32, n0 + (int)rank * 128);
                    }
                }
                if (++s == STAGES) s = 0;
            }
        }
        if (!ok && lane == 0) {
            // let copies already in flight land before the CTA goes away (bounded)
            for (int st = 0; st < STAGES; ++st) {
                const uint32_t issued = it > (uint32_t)st ? (it - 1 - st) / STAGES + 1 : 0;  // fills of stage st
                if (issued) {
                    uint64_t t0 = globaltimer_ns();
                    while (!mbar_try_wait(bar(B_FULL + st), (issued - 1) & 1) && globaltimer_ns() - t0 < 200000000ull) {}
                }
            }
        }
    } else if (warp == 1 && rank == 1) {
        // ================================ relay (second CTA) ================================
        uint32_t s = 0, ph = 0;
        bool ok = true;
        for (int t = t_begin; t < t_end && ok; ++t)
            for (int j = 0; j < GS + LCH; ++j) {
                if (!mbar_wait_warp(bar(B_FULL) + 8u * s, ph, abort_s, E_RELAY | 1)) { ok = false; break; }
                if (lane == 0) mbar_arrive_cluster_release(bar(B_PFULL) + 8u * s, 0);
                if (++s == STAGES) { s = 0; ph ^= 1u; }
            }
    } else if (warp == 1) {
        // ================================ MMA issuer (first CTA, for the pair) ================================
        // fp32 accumulators, e4m3 x e4m3, N = 256, M = 256 (pair)
        const uint32_t idesc_f8 = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((256u >> 4) << 24);
        const uint32_t f16fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
        const uint32_t idesc_lr = (1u << 4) | (f16fmt << 7) | (f16fmt << 10) | ((uint32_t)(BN >> 3) << 17) | ((256u >> 4) << 24);
        // shared-memory matrix descriptors, K-major: low word = (address >> 4) | leading offset 1 << 16; high word = stride
        // between 8-row groups >> 4, descriptor version 1 (bit 46), swizzle mode (bits 61-63: 2 = 128 bytes, 4 = 64 bytes).
        // An operand's address only changes the low word: stage s adds s * ST_BYTES / 16, a 32-byte K step adds 2.
        const uint32_t lo_a0 = (((s_base + C::OFF_ST) >> 4) & 0x3fffu) | (1u << 16), lo_w0 = lo_a0 + (C::ST_A >> 4);
        constexpr uint32_t HI128 = (1024u >> 4) | (1u << 14) | (2u << 29), HI64 = (512u >> 4) | (1u << 14) | (4u << 29);
        uint32_t s = 0, ph = 0;        // ring stage and the parity of its fill
        uint32_t slot = 0, aph = 0;    // accumulator slot of the next group and the parity of its use
        bool ok = true;
        for (int t = t_begin; t < t_end && ok; ++t) {
            for (int j = 0; j < GS && ok; ++j) {
                const int ng = min(2, G - 2 * j);
                if (!mbar_wait_warp(bar(B_FULL) + 8u * s, ph, abort_s, E_MMA | 1) ||
                    !mbar_wait_warp(bar(B_PFULL) + 8u * s, ph, abort_s, E_MMA | 2)) { ok = false; break; }
                const uint32_t so = s * (C::ST_BYTES >> 4);
                for (int i = 0; i < ng; ++i) {
                    if (!mbar_wait_warp(bar(B_ACC_EMPTY) + 8u * slot, aph ^ 1u, abort_s, E_MMA | 3)) { ok = false; break; }
                    tc_fence_after();
                    if (elect_one()) {
                        const uint32_t d = tmem_base + slot * BN;
                        // a 32-byte K step advances the descriptor's start address field by 2; a group is 64 bytes
                        mma2_f8<0>(d, desc64(lo_a0 + so + 4 * i, HI128), desc64(lo_w0 + so + 4 * i, HI128), idesc_f8);
                        mma2_f8<1>(d, desc64(lo_a0 + so + 4 * i + 2, HI128), desc64(lo_w0 + so + 4 * i + 2, HI128), idesc_f8);
                        tc_commit2(bar(B_ACC_FULL) + 8u * slot);
                    }
                    slot ^= 1u;
                    if (slot == 0) aph ^= 1u;
                }
                if (++s == STAGES) { s = 0; ph ^= 1u; }
            }
            if (ok && LCH > 0) {
                if (!mbar_wait_warp(bar(B_ACC_EMPTY) + 8u * slot, aph ^ 1u, abort_s, E_MMA | 4)) { ok = false; break; }
                for (int c = 0; c < LCH; ++c) {
                    if (!mbar_wait_warp(bar(B_FULL) + 8u * s, ph, abort_s, E_MMA | 5) ||
                        !mbar_wait_warp(bar(B_PFULL) + 8u * s, ph, abort_s, E_MMA | 6)) { ok = false; break; }
                    tc_fence_after();
                    if (elect_one()) {
                        const uint32_t so = s * (C::ST_BYTES >> 4);
                        const uint32_t d = tmem_base + slot * BN;
                        if (c == 0) mma2_f16<0>(d, desc64(lo_a0 + so, HI64), desc64(lo_w0 + so, HI64), idesc_lr);
                        else mma2_f16<1>(d, desc64(lo_a0 + so, HI64), desc64(lo_w0 + so, HI64), idesc_lr);
                        mma2_f16<1>(d, desc64(lo_a0 + so + 2, HI64), desc64(lo_w0 + so + 2, HI64), idesc_lr);
                        tc_commit2(bar(B_LRDONE) + 8u * s);
                    }
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
                if (!ok) break;
                if (elect_one()) tc_commit2(bar(B_ACC_FULL) + 8u * slot);
                slot ^= 1u;
                if (slot == 0) aph ^= 1u;
            }
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(DRAIN_REGS));
        // ================================ drain + epilogue (both CTAs, own 128 rows) ================================
        // tcgen05.ld.16x256b.x4 hands a thread, for one 16-lane block and 32 columns, rows {gid, gid + 8} and the column
        // pairs 8 j + 2 tig + {0, 1}, j = 0..3: register 4 j + 2 rs + e.
        // (Everything the K loop does not need is computed after it: the loop runs with 64 accumulators, one 16-register
        // chunk and 16 scale registers out of 112, and a spill inside it costs more than any of this arithmetic.)
        const int q = warp & 3;                    // TMEM lane quarter this warp may read (warp id mod 4)
        const int cq = (warp - CTRL_WARPS) >> 2;   // 64-column slice of the tile
        const int gid = lane >> 2, tig = lane & 3;
        const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16) + cq * COLS;
        // byte offsets of this thread's scales inside a stage's scale block: row-scale entry (quarter, lane block 0, gid),
        // column-scale entry (slice, half 0, tig)
        const uint32_t sc_off = s_base + C::OFF_ST + C::ST_A + C::ST_W;
        const uint32_t as_off = (q * 16 + gid) * 16, ws_off = C::ST_AS + (cq * 8 + tig) * 32;
        // The loop is bound by instruction issue (four drain warps per scheduler), so everything a K group does not strictly
        // need is kept out of it: slot, ring stage and addresses are carried in registers and advanced by additions, the
        // remote barrier address is mapped once, the slot is freed by one predicated instruction.
        const uint32_t is_lane0 = lane == 0 ? 1u : 0u;
        const uint32_t rem_empty = mapa_cluster(bar(B_ACC_EMPTY), 0);  // the first CTA's slot barriers
        uint32_t ds = 0;               // ring stage of the next int8 stage
        uint32_t slot = 0, fph = 0;    // accumulator slot of the next group and the parity of its use
        uint32_t xph = 0, lxph = 0;
        bool ok = true;
        bool ready = false;  // the next group's barrier has already been seen complete
        // acc[(lb * NJ + jx) * 2 + rs]: rows q*32 + lb*16 + rs*8 + gid, columns cq*64 + 8 jx + 2 tig + {0, 1}
        uint64_t acc[2 * NJ * 2];

        for (int t = t_begin; t < t_end && ok; ++t) {
#pragma unroll
            for (int i = 0; i < 2 * NJ * 2; ++i) acc[i] = 0ull;
            // One K group: four chunks of 16 lanes x 32 columns; the slot is freed when the last chunk has landed.  One load is
            // in flight per warp (the registers hold 64 accumulators, one chunk and its scales); what hides the tensor-memory
            // latency is the arithmetic of the other three warps of the scheduler.  (Two loads of 64 columns per group were
            // measured: 8 % faster with the drain alone, slower inside the whole kernel on long K loops.)
            auto drain_group = [&](uint32_t taddr, uint32_t st, uint32_t rem_bar, int g, uint32_t next_bar, uint32_t next_par) {
                uint64_t ap4[4];  // the row scales of both lane blocks: fetched with the first two chunks, used by all four
#pragma unroll
                for (int ch = 0; ch < 2; ++ch) {
                    uint64_t wp[4];
#pragma unroll
                    for (int lb = 0; lb < 2; ++lb) {
                        uint32_t v[16];
                        tmem_ld_16x256b_x4(taddr + ((uint32_t)(lb * 16) << 16) + ch * 32, v);
                        // the scales are fetched while the chunk is on its way (shared memory answers slowly while the tensor
                        // cores read their operands from it), as 64-bit pairs: the form the packed arithmetic takes
                        if (ch == 0) lds2x64(st + as_off + lb * 128, ap4[2 * lb], ap4[2 * lb + 1]);
                        const uint64_t ap[2] = {ap4[2 * lb], ap4[2 * lb + 1]};
                        if (lb == 0) {
                            lds2x64(st + ws_off + ch * 128, wp[0], wp[1]);
                            lds2x64(st + ws_off + ch * 128 + 16, wp[2], wp[3]);
                        }
                        tmem_wait_ld();  // (warp-wide: every lane's values have landed)
                        if (ch == 1 && lb == 1) {
                            // the slot is read out: the next group's MMAs may overwrite it while this warp does its arithmetic
                            tc_fence_before();
                            mbar_arrive_remote_if(rem_bar, is_lane0);
                            // look at the next group's barrier now: the answer comes back while the last chunk is scaled
                            // (asked after that arithmetic, a test that passes at once still cost this warp some 300 cycles)
                            ready = mbar_test_all(next_bar, next_par);
                        }
#pragma unroll
                        for (int j = 0; j < 4; ++j)
#pragma unroll
                            for (int rs = 0; rs < 2; ++rs) {
                                const uint64_t tt = mul_f32x2(pack_u32x2(v[4 * j + 2 * rs], v[4 * j + 2 * rs + 1]), ap[rs]);
                                uint64_t& a = acc[(lb * NJ + ch * 4 + j) * 2 + rs];
                                a = fma_f32x2(tt, wp[j], a);
                            }
                        if (DEBUG_P) {
#pragma unroll
                            for (int e = 0; e < 16; ++e) {
                                const int m = (t / NT) * (2 * BM) + (int)rank * BM + q * 32 + lb * 16 + ((e >> 1) & 1) * 8 + gid;
                                const int n = (t % NT) * BN + cq * COLS + ch * 32 + (e >> 2) * 8 + 2 * tig + (e & 1);
                                if (m < p.M && n < p.N)
                                    p.p_out[((long long)g * p.M + m) * p.N + n] = (int)__uint_as_float(v[e]);
                            }
                        }
                    }
                }
            };
            for (int j = 0; j < GS; ++j) {
                const uint32_t st = sc_off + ds * C::ST_BYTES;  // both scale blocks keep 1 KB per group
                const int ng = min(2, G - 2 * j);
                for (int i = 0; i < ng; ++i) {
                    if (!ready && !mbar_wait_warp(bar(B_ACC_FULL) + 8u * slot, fph, abort_s, E_DRAIN | 1)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t nslot = slot ^ 1u, nph = fph ^ slot;  // (the parity flips when the slot index wraps to 0)
                    drain_group(lane_base + slot * BN, st + i * 1024, rem_empty + 8u * slot, 2 * j + i, bar(B_ACC_FULL) + 8u * nslot, nph);
                    slot = nslot;
                    fph = nph;
                }
                if (!ok) break;
                // the stage's scales are in registers and have been used (the arithmetic above depends on them)
                if (lane == 0) mbar_arrive(bar(B_SCDONE) + 8u * ds);
                if (++ds == STAGES) ds = 0;
            }
            if (!ok) break;
            if (LCH > 0) {
                // the low-rank product arrives like one more group, with unit scales
                if (!ready && !mbar_wait_warp(bar(B_ACC_FULL) + 8u * slot, fph, abort_s, E_DRAIN | 2)) { ok = false; break; }
                ready = false;
                tc_fence_after();
                const uint32_t taddr = lane_base + slot * BN;
#pragma unroll
                for (int ch = 0; ch < 2; ++ch)
#pragma unroll
                    for (int lb = 0; lb < 2; ++lb) {
                        uint32_t v[16];
                        tmem_ld_16x256b_x4(taddr + ((uint32_t)(lb * 16) << 16) + ch * 32, v);
                        tmem_wait_ld();
                        if (ch == 1 && lb == 1) {
                            tc_fence_before();
                            mbar_arrive_remote_if(rem_empty + 8u * slot, is_lane0);
                        }
#pragma unroll
                        for (int j = 0; j < 4; ++j)
#pragma unroll
                            for (int rs = 0; rs < 2; ++rs) {
                                uint64_t& a = acc[(lb * NJ + ch * 4 + j) * 2 + rs];
                                a = add_f32x2(a, pack_u32x2(v[4 * j + 2 * rs], v[4 * j + 2 * rs + 1]));
                            }
                    }
                slot ^= 1u;
                if (slot == 0) fph ^= 1u;
                ds = (ds + LCH) % STAGES;  // the low-rank stages carry nothing for the drain
            }

            // ---------------- epilogue ----------------
            // element (lb, j, rs, e): row q*32 + lb*16 + rs*8 + gid, column nc0 + 8 j + 2 tig + e
            const int m0 = (t / NT) * (2 * BM) + (int)rank * BM, n0 = (t % NT) * BN;
            const int nc0 = n0 + cq * COLS;                   // first global column of this warp
            const int pw = cq * 4 + q;                        // index of this warp's staging / exchange buffers
            uint8_t* stg = smem + C::OFF_STG + pw * C::STG_WARP;
            float* xch = reinterpret_cast<float*>(smem + C::OFF_XCH);
            const int head = cq >> 1;                         // 128-column half of the tile
            const int hc0 = (cq & 1) * COLS;                  // this warp's first column inside its head
            const int qk_part = EPI == NB_EPI_QK_NORM_ROPE ? (n0 + head * 128) / (p.N / 3) : 2;
            float sumsq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                const int col = nc0 + 8 * j + 2 * tig;
                const uint32_t bw = (p.bias && col < p.N) ? __ldg(reinterpret_cast<const uint32_t*>(static_cast<const T*>(p.bias) + col)) : 0u;
                const float2 b = unpack2<T>(bw);
#pragma unroll
                for (int lb = 0; lb < 2; ++lb)
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
                // A 128-column half of the tile is one head; its row sums come from this warp and the neighbouring slice.
                // The rotary values of a row are requested one row ahead (the first row before the exchange), so that their
                // trip to L2 hides behind the exchange and the arithmetic of the row before.
                float2 sc[2][NJ];
                auto load_rot = [&](int r, float2 (&dst)[NJ]) {
                    const int m = m0 + q * 32 + r * 8 + gid;
                    int mr = m < p.actual_m ? m : 0;
                    if (mr >= p.rot_rows) mr %= p.rot_rows;
                    const float2* rp = reinterpret_cast<const float2*>(p.rot + (long long)mr * p.stride_rm + hc0 + 2 * tig);
#pragma unroll
                    for (int j = 0; j < NJ; ++j) dst[j] = __ldg(rp + 4 * j);
                };
                load_rot(0, sc[0]);
                uint32_t nwv[NJ];
                {
                    const T* nw = static_cast<const T*>(qk_part == 0 ? p.norm_q : p.norm_k) + hc0 + 2 * tig;
#pragma unroll
                    for (int j = 0; j < NJ; ++j) nwv[j] = __ldg(reinterpret_cast<const uint32_t*>(nw + 8 * j));
                }
                float* xb = xch + (xph & 1) * (DRAIN_WARPS * 32);
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    float s = sumsq[r];
                    s += __shfl_xor_sync(0xffffffffu, s, 1);
                    s += __shfl_xor_sync(0xffffffffu, s, 2);
                    if (tig == 0) xb[pw * 32 + r * 8 + gid] = s;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(B_XCH + q * 2 + head));
                if (!mbar_wait_warp(bar(B_XCH + q * 2 + head), xph & 1, abort_s, E_DRAIN | 4, 100)) { ok = false; break; }
                // (the buffer of this parity is written again two exchanges later, and no warp gets there before both warps
                // of the pair have arrived at the exchange in between, i.e. after they have read this one)
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    if (r + 1 < 4) load_rot(r + 1, sc[(r + 1) & 1]);
                    // both slices add the two partial sums in the same order
                    const float tot = xb[((head * 2) * 4 + q) * 32 + r * 8 + gid] + xb[((head * 2 + 1) * 4 + q) * 32 + r * 8 + gid];
                    const float rstd = rsqrtf(tot / 128.0f + p.eps);
                    const int lb = r >> 1, rs = r & 1;
#pragma unroll
                    for (int j = 0; j < NJ; ++j) {
                        const float2 w = unpack2<T>(nwv[j]);
                        const float2 a = unpack_f32x2(acc[(lb * NJ + j) * 2 + rs]);
                        const float2 c = sc[r & 1][j];
                        const float xe = a.x * rstd * w.x, xo = a.y * rstd * w.y;
                        acc[(lb * NJ + j) * 2 + rs] = pack_f32x2(xe * c.y - xo * c.x, xe * c.x + xo * c.y);
                    }
                }
                ++xph;
            } else if (EPI == NB_EPI_QK_NORM_ROPE) {
                // V tiles take no part in the exchange; nothing to do
            }

            if (EPI == NB_EPI_STORE || EPI == NB_EPI_QK_NORM_ROPE || (EPI == NB_EPI_GELU_QUANT && p.out)) {
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
                const int ur = lane >> 3, uc = lane & 7;  // 8 16-byte units per row, 4 rows per pass
#pragma unroll
                for (int r = 0; r < 32; r += 4) {
                    const int rr = r + ur;
                    const int mm = m0 + q * 32 + rr, nn = nc0 + uc * 8;
                    const uint4 o = *reinterpret_cast<const uint4*>(stg + rr * C::STG_PITCH + uc * 16);
                    if (mm < p.actual_m && nn < p.N)
                        *reinterpret_cast<uint4*>(static_cast<T*>(p.out) + (long long)mm * p.stride_om + nn) = o;
                }
                __syncwarp();
            }

            if (EPI == NB_EPI_GELU_QUANT || EPI == NB_EPI_SWIGLU_QUANT) {
                // GELU:   x = gelu(acc) on all N columns; unsigned codes, the 64-column group is this warp's slice.
                // SwiGLU: columns come in blocks of 32 = 16 gate + 16 up (the layer's rows were interleaved at load time);
                //         y = silu(gate) * up gives N / 2 output columns, 32 per warp; signed codes, a 64-column output
                //         group spans this warp and its neighbour slice.
                // Both: LoRA-down from T(x) before shift and smoothing; v = (x + shift) / smooth; scale = max / qmax from the
                // unrounded maximum, stored rounded; code = clamp(rint(v * (1 / scale))).
                constexpr bool SWI = EPI == NB_EPI_SWIGLU_QUANT;
                constexpr int KSTEPS = SWI ? 2 : 4;      // 16 output columns per mma k step
                const int Nq = SWI ? p.N / 2 : p.N;
                const int oc0 = SWI ? nc0 / 2 : nc0;     // this warp's first output column
                if (SWI) {
                    // gate block j = 4 b + jj (jj < 2) and up block j + 2 hold the same (tig, e) positions: thread-local
#pragma unroll
                    for (int lb = 0; lb < 2; ++lb)
#pragma unroll
                        for (int b = 0; b < 2; ++b)
#pragma unroll
                            for (int jj = 0; jj < 2; ++jj)
#pragma unroll
                                for (int rs = 0; rs < 2; ++rs) {
                                    const float2 g2 = unpack_f32x2(acc[(lb * NJ + 4 * b + jj) * 2 + rs]);
                                    const float2 u2 = unpack_f32x2(acc[(lb * NJ + 4 * b + jj + 2) * 2 + rs]);
                                    acc[(lb * NJ + 4 * b + jj) * 2 + rs] = pack_f32x2(silu(g2.x) * u2.x, silu(g2.y) * u2.y);
                                }
                } else {
#pragma unroll
                    for (int i = 0; i < 2 * NJ * 2; ++i) {
                        const float2 a = unpack_f32x2(acc[i]);
                        acc[i] = pack_f32x2(gelu_tanh(a.x), gelu_tanh(a.y));
                    }
                }
                // accumulator index of output k-step kk, half h (columns 16 kk + 8 h + 2 tig + {0, 1} of this warp's outputs)
                auto xi = [](int lb, int kk, int h, int rs) { return SWI ? (lb * NJ + 4 * kk + h) * 2 + rs : (lb * NJ + 2 * kk + h) * 2 + rs; };
                const bool have_lora = p.lora_down_t != nullptr && p.R2 > 0;
                if (have_lora) {
                    // Two adjacent 8-column blocks of the accumulator fragment ARE the A fragment of mma.m16n8k16 (rows gid,
                    // gid + 8; k = 2 tig + {0, 1} and + 8), so the activated values go to the tensor cores without leaving the
                    // registers.  B comes from the transposed lora_down: rank gid, columns k .. k + 1 are one 32-bit load.
                    // R2 is handled in slabs of 32 ranks; a slab's 32 x 32 partial of this warp's columns goes through the
                    // staging tile to the first slice's warp of the lane quarter, which adds the four slices in slice order
                    // and stores the tile's partial sum (the column tiles are added up in tile order by a second kernel).
                    const T* ldt = static_cast<const T*>(p.lora_down_t);
                    float* part = p.lora_part + ((long long)(n0 / BN) * p.M) * p.R2;
                    for (int r0 = 0; r0 < p.R2; r0 += 32) {
                        float c[2][4][4];
#pragma unroll
                        for (int lb = 0; lb < 2; ++lb)
#pragma unroll
                            for (int nb = 0; nb < 4; ++nb)
#pragma unroll
                                for (int e = 0; e < 4; ++e) c[lb][nb][e] = 0.f;
#pragma unroll
                        for (int kk = 0; kk < KSTEPS; ++kk) {
                            uint32_t a[2][4];
#pragma unroll
                            for (int lb = 0; lb < 2; ++lb) {
                                const float2 x00 = unpack_f32x2(acc[xi(lb, kk, 0, 0)]), x10 = unpack_f32x2(acc[xi(lb, kk, 0, 1)]);
                                const float2 x01 = unpack_f32x2(acc[xi(lb, kk, 1, 0)]), x11 = unpack_f32x2(acc[xi(lb, kk, 1, 1)]);
                                a[lb][0] = pack2<T>(x00.x, x00.y); a[lb][1] = pack2<T>(x10.x, x10.y);
                                a[lb][2] = pack2<T>(x01.x, x01.y); a[lb][3] = pack2<T>(x11.x, x11.y);
                            }
#pragma unroll
                            for (int nb = 0; nb < 4; ++nb) {
                                const int r = r0 + nb * 8 + gid;
                                const int col = oc0 + kk * 16 + 2 * tig;
                                uint32_t b0 = 0u, b1 = 0u;
                                if (r < p.R2) {
                                    const T* bp = ldt + (long long)r * Nq + col;
                                    if (col < Nq) b0 = __ldg(reinterpret_cast<const uint32_t*>(bp));
                                    if (col + 8 < Nq) b1 = __ldg(reinterpret_cast<const uint32_t*>(bp + 8));
                                }
                                mma_sync_16816<T>(c[0][nb], a[0], b0, b1);
                                mma_sync_16816<T>(c[1][nb], a[1], b0, b1);
                            }
                        }
                        // C fragment: rows gid, gid + 8 (of 16-row block lb), ranks nb*8 + 2 tig + {0, 1}
                        float* cs = reinterpret_cast<float*>(stg);  // [32 rows][32 ranks]
                        __syncwarp();
#pragma unroll
                        for (int lb = 0; lb < 2; ++lb)
#pragma unroll
                            for (int nb = 0; nb < 4; ++nb) {
                                *reinterpret_cast<float2*>(cs + (lb * 16 + gid) * 32 + nb * 8 + 2 * tig) = make_float2(c[lb][nb][0], c[lb][nb][1]);
                                *reinterpret_cast<float2*>(cs + (lb * 16 + 8 + gid) * 32 + nb * 8 + 2 * tig) = make_float2(c[lb][nb][2], c[lb][nb][3]);
                            }
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar(B_LX + q));
                        if (!mbar_wait_warp(bar(B_LX + q), lxph & 1, abort_s, E_DRAIN | 5, 100)) { ok = false; break; }
                        ++lxph;
                        if (cq == 0) {
                            // row `lane`: 32 ranks; slices added in slice order
                            const int m = m0 + q * 32 + lane;
#pragma unroll
                            for (int u = 0; u < 8; ++u) {
                                float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                                for (int sl = 0; sl < 4; ++sl) {
                                    const float4 x = *reinterpret_cast<const float4*>(smem + C::OFF_STG + (sl * 4 + q) * C::STG_WARP + (lane * 32 + ((u + lane) & 7) * 4) * 4);
                                    sum.x += x.x; sum.y += x.y; sum.z += x.z; sum.w += x.w;
                                }
                                const int rr = r0 + ((u + lane) & 7) * 4;
                                if (m < p.M && rr < p.R2) *reinterpret_cast<float4*>(part + (long long)m * p.R2 + rr) = sum;
                            }
                        }
                        // the staging tiles are rewritten (next slab, or the codes below) only after the first slice's warp has read them
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar(B_LX + q));
                        if (!mbar_wait_warp(bar(B_LX + q), lxph & 1, abort_s, E_DRAIN | 6, 100)) { ok = false; break; }
                        ++lxph;
                    }
                    if (!ok) break;
                }
                // ---- quantise: NH output 8-column blocks per (16-lane block, row select)
                constexpr int NH = SWI ? 4 : 8;
                float isw[NH][2];
#pragma unroll
                for (int h = 0; h < NH; ++h) {
                    const int col = oc0 + 8 * h + 2 * tig;
                    float2 is = make_float2(1.f, 1.f);
                    if (p.inv_smooth && col < Nq) is = __ldg(reinterpret_cast<const float2*>(p.inv_smooth + col));
                    isw[h][0] = is.x; isw[h][1] = is.y;
                }
                float vv[4][NH][2], mx[4];
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const int lb = r >> 1, rs = r & 1;
                    mx[r] = 0.f;
#pragma unroll
                    for (int h = 0; h < NH; ++h) {
                        const float2 a = unpack_f32x2(acc[SWI ? (lb * NJ + 4 * (h >> 1) + (h & 1)) * 2 + rs : (lb * NJ + h) * 2 + rs]);
                        vv[r][h][0] = __fmul_rn(__fadd_rn(a.x, p.shift), isw[h][0]);
                        vv[r][h][1] = __fmul_rn(__fadd_rn(a.y, p.shift), isw[h][1]);
                        mx[r] = SWI ? fmaxf(mx[r], fmaxf(fabsf(vv[r][h][0]), fabsf(vv[r][h][1])))
                                    : fmaxf(mx[r], fmaxf(vv[r][h][0], vv[r][h][1]));
                    }
                    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                }
                if (SWI) {
                    // the 64-column output group is shared with the neighbour slice: exchange the row maxima
                    float* xb = xch + (xph & 1) * (DRAIN_WARPS * 32);
#pragma unroll
                    for (int r = 0; r < 4; ++r)
                        if (tig == 0) xb[pw * 32 + r * 8 + gid] = mx[r];
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar(B_XCH + q * 2 + head));
                    if (!mbar_wait_warp(bar(B_XCH + q * 2 + head), xph & 1, abort_s, E_DRAIN | 7, 100)) { ok = false; break; }
#pragma unroll
                    for (int r = 0; r < 4; ++r)
                        mx[r] = fmaxf(xb[((head * 2) * 4 + q) * 32 + r * 8 + gid], xb[((head * 2 + 1) * 4 + q) * 32 + r * 8 + gid]);
                    ++xph;
                }
                const float qmax = SWI ? 7.0f : 15.0f, qlo = SWI ? -8.0f : 0.0f;
                const int grp = oc0 / 64;
                constexpr int RB = SWI ? 16 : 32;   // code bytes per row of this warp
                constexpr int RP = RB + 16;         // staging pitch
                __syncwarp();
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const float scale = __fdiv_rn(mx[r], qmax);
                    const float inv = __fdiv_rn(1.0f, scale == 0.f ? 1.0f : scale);
                    const int m = m0 + q * 32 + r * 8 + gid;
                    if (tig == 0 && m < p.M && oc0 < Nq && (!SWI || (cq & 1) == 0))
                        static_cast<T*>(p.oscales)[(long long)grp * p.stride_osg + m] = from_f32<T>(scale);
#pragma unroll
                    for (int h = 0; h < NH; ++h) {
                        const int q0 = (int)fminf(fmaxf(rint_small(__fmul_rn(vv[r][h][0], inv)), qlo), qmax);
                        const int q1 = (int)fminf(fmaxf(rint_small(__fmul_rn(vv[r][h][1], inv)), qlo), qmax);
                        stg[(r * 8 + gid) * RP + 4 * h + tig] = (uint8_t)((q0 & 0xF) | ((q1 & 0xF) << 4));
                    }
                }
                __syncwarp();
                {
                    // 32 rows x RB bytes in 16-byte units
                    constexpr int UPR = RB / 16;
#pragma unroll
                    for (int u0 = 0; u0 < 32 * UPR; u0 += 32) {
                        const int idx = u0 + lane, rr = idx / UPR, u = idx % UPR;
                        const int mm = m0 + q * 32 + rr;
                        const uint4 o = *reinterpret_cast<const uint4*>(stg + rr * RP + u * 16);
                        if (mm < p.M && oc0 + u * 32 < Nq)
                            *reinterpret_cast<uint4*>(p.qout + (long long)mm * p.stride_qm + oc0 / 2 + u * 16) = o;
                    }
                }
                __syncwarp();
            }
        }
    }

    // ---------------- teardown: nothing of the pair may be in flight when tensor memory goes ----------------
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_s && p.status) atomicCAS(p.status, 0, *abort_s);
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc2(tmem_base, C::TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------------------------
// pre-pass: nibbles -> e4m3 bytes, scales in drain order, lora_act -> T
// ------------------------------------------------------------------------------------------------
struct PrepackParams {
    const uint8_t* act; const uint8_t* wgt;
    const void* ascales; const void* wscales; const float* lora_act;
    uint8_t* a8; uint8_t* w8; float* asf; float* wsf; void* la16;
    int M, N, K, R, Np, Mp;  // Np, Mp: N, M rounded up to 256
    int act_unsigned;
    int do_act, do_w8, do_wsf;
    long long stride_am, stride_wn, stride_asg, stride_wsg, stride_lam;
};

template <typename T>
__global__ void __launch_bounds__(256) prepack_pair_kernel(const PrepackParams p) {
    const long long tid = (long long)blockIdx.x * 256 + threadIdx.x;
    const int upr = p.K / 32;  // 16-byte packed units per row
    const long long a_units = p.do_act ? (long long)p.M * upr : 0, w_units = p.do_w8 ? (long long)p.N * upr : 0;
    const int G = p.K / 64;
    const long long as_units = p.do_act ? (long long)G * p.Mp : 0, ws_units = p.do_wsf ? (long long)G * p.Np : 0;
    const long long la_units = (p.do_act && p.R) ? (long long)p.M * (p.R / 8) : 0;
    if (tid < a_units + w_units) {
        const bool is_w = tid >= a_units;
        const long long u = is_w ? tid - a_units : tid;
        const long long row = u / upr;
        const int c = (int)(u % upr);
        const uint8_t* src = (is_w ? p.wgt + row * p.stride_wn : p.act + row * p.stride_am) + c * 16;
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(src));
        const bool uns = !is_w && p.act_unsigned;
        const uint32_t in[4] = {v.x, v.y, v.z, v.w};
        uint32_t o[8];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            o[2 * k] = e4m3_of_nibbles(in[k] & 0xFFFFu, uns);
            o[2 * k + 1] = e4m3_of_nibbles(in[k] >> 16, uns);
        }
        uint4* dst = reinterpret_cast<uint4*>((is_w ? p.w8 : p.a8) + row * p.K + c * 32);
        dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
        dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
        return;
    }
    long long u = tid - (a_units + w_units);
    if (u < as_units) {
        // row r of its 128-row block -> entry (quarter * 2 + lane block) * 8 + gid, two duplicated pairs (row, row + 8)
        const int g = (int)(u / p.Mp), m = (int)(u % p.Mp);
        const float a = m < p.M ? to_f32<T>(static_cast<const T*>(p.ascales)[(long long)g * p.stride_asg + m]) : 0.f;
        const int r = m & 127;
        const int entry = ((r >> 5) * 2 + ((r >> 4) & 1)) * 8 + (r & 7), rs = (r >> 3) & 1;
        float2* dst = reinterpret_cast<float2*>(p.asf + ((long long)g * p.Mp + (m & ~127)) * 2 + entry * 4 + rs * 2);
        *dst = make_float2(a, a);
        return;
    }
    u -= as_units;
    if (u < ws_units) {
        // column c of its 256-wide tile -> ((slice * 2 + half) * 4 + tig) * 8 + j * 2 + e
        const int g = (int)(u / p.Np), n = (int)(u % p.Np);
        const float w = n < p.N ? to_f32<T>(static_cast<const T*>(p.wscales)[(long long)g * p.stride_wsg + n]) : 0.f;
        const int c = n & 255;
        const int pos = (((c >> 6) * 2 + ((c >> 5) & 1)) * 4 + ((c >> 1) & 3)) * 8 + ((c >> 3) & 3) * 2 + (c & 1);
        p.wsf[(long long)g * p.Np + (n & ~255) + pos] = w;
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

// GELU epilogue inputs in the form the kernel reads: reciprocal smooth factors (fp32) and lora_down transposed to (R2, N)
template <typename T>
__global__ void __launch_bounds__(256) prepack_requant_kernel(const T* smooth, const T* lora_down, long long stride_ld, int N,
                                                              int R2, float* inv_smooth, T* ldt) {
    const long long tid = (long long)blockIdx.x * 256 + threadIdx.x;
    if (tid < N) inv_smooth[tid] = smooth ? __fdiv_rn(1.0f, to_f32<T>(smooth[tid])) : 1.0f;
    if (lora_down && tid < (long long)N * R2) {
        const int n = (int)(tid / R2), r = (int)(tid % R2);
        ldt[(long long)r * N + n] = lora_down[(long long)n * stride_ld + r];
    }
}

// lora_act_out[m, r] = sum over the column tiles, in tile order (deterministic)
__global__ void __launch_bounds__(256) lora_part_sum_kernel(const float* part, int tiles, int M, int R2, float* out,
                                                            long long stride_lom) {
    const long long tid = (long long)blockIdx.x * 256 + threadIdx.x;
    if (tid >= (long long)M * R2) return;
    float s = 0.f;
    for (int t = 0; t < tiles; ++t) s += part[(long long)t * M * R2 + tid];
    out[(tid / R2) * stride_lom + tid % R2] = s;
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

struct Scratch {
    size_t a8, asf, la16, inv_smooth, ldt, lora_part, w8, wsf, total;
    int Np, Mp;
};
static Scratch scratch_layout(const nb_gemm_args* a, const void* epi, int epi_kind) {
    Scratch s = {};
    const size_t G = a->K / 64;
    s.Np = (a->N + BN - 1) / BN * BN;
    s.Mp = (a->M + 2 * BM - 1) / (2 * BM) * (2 * BM);
    size_t off = 0;
    s.a8 = off; off += up256((size_t)a->M * a->K);
    s.asf = off; off += up256(G * s.Mp * 2 * 4);
    s.la16 = off; off += up256((size_t)a->M * a->R * 2);
    if (epi_kind == NB_EPI_GELU_QUANT || epi_kind == NB_EPI_SWIGLU_QUANT) {
        const nb_requant_args* q = static_cast<const nb_requant_args*>(epi);
        const size_t R2 = (q->lora_down && q->lora_act_out) ? q->R2 : 0;
        s.inv_smooth = off; off += up256((size_t)a->N * 4);
        s.ldt = off; off += up256(R2 * a->N * 2);
        s.lora_part = off; off += up256((size_t)(s.Np / BN) * a->M * R2 * 4);
    }
    if (!has_prepared_weights(a)) {
        s.w8 = off; off += up256((size_t)a->N * a->K);
        s.wsf = off; off += up256(G * s.Np * 4);
    }
    s.total = off;
    return s;
}

template <typename T>
static int launch_prepack(const PrepackParams& pp, cudaStream_t s) {
    const long long G = pp.K / 64;
    long long units = 0;
    if (pp.do_act) units += (long long)pp.M * (pp.K / 32) + G * pp.Mp + (pp.R ? (long long)pp.M * (pp.R / 8) : 0);
    if (pp.do_w8) units += (long long)pp.N * (pp.K / 32);
    if (pp.do_wsf) units += G * pp.Np;
    if (units == 0) return NB_OK;
    prepack_pair_kernel<T><<<(unsigned)((units + 255) / 256), 256, 0, s>>>(pp);
    NB_CUDA_CHECK(cudaGetLastError());
    return NB_OK;
}

// How many CTA pairs can be resident at once on the current device (a persistent grid must not exceed it), cached per device.
template <typename K>
static int max_pairs(K kern, int dev) {
    static int cache[64] = {};
    if (dev >= 0 && dev < 64 && cache[dev]) return cache[dev];
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sms / 2 * 2);
    cfg.blockDim = dim3(NTHREADS);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg) != cudaSuccess) {
        // the query is advisory: without it the grid is one pair per two SMs and the launch itself reports a misfit
        (void)cudaGetLastError();
        clusters = sms / 2;
    }
    if (clusters > sms / 2) clusters = sms / 2;
    if (dev >= 0 && dev < 64) cache[dev] = clusters;
    return clusters;
}

template <int EPI, typename T, bool DEBUG_P>
static int launch_t(const nb_gemm_args* a, const void* epi, Params p, cudaStream_t s) {
    using C = Cfg;
    const Scratch sc = scratch_layout(a, epi, EPI);
    if (!a->scratch || a->scratch_bytes < (int64_t)sc.total || (reinterpret_cast<uintptr_t>(a->scratch) & 255))
        return fail_with(NB_ERR_INVALID, "pair kernel: scratch missing, too small or not 256-byte aligned");
    uint8_t* base = static_cast<uint8_t*>(a->scratch);
    const bool prepared = has_prepared_weights(a);
    const PreparedLayout pl = prepared_layout(a->N, a->K);
    const uint8_t* pw = static_cast<const uint8_t*>(a->wgt_prepared);
    PrepackParams pp = {};
    pp.act = static_cast<const uint8_t*>(a->act); pp.wgt = static_cast<const uint8_t*>(a->wgt);
    pp.ascales = a->ascales; pp.wscales = a->wscales; pp.lora_act = static_cast<const float*>(a->lora_act);
    pp.act_unsigned = a->act_unsigned;
    pp.M = a->M; pp.N = a->N; pp.K = a->K; pp.R = a->R; pp.Np = sc.Np; pp.Mp = sc.Mp;
    pp.stride_am = a->stride_am; pp.stride_wn = a->stride_wn; pp.stride_asg = a->stride_asg;
    pp.stride_wsg = a->stride_wsg; pp.stride_lam = a->stride_lam;
    pp.a8 = base + sc.a8; pp.asf = reinterpret_cast<float*>(base + sc.asf); pp.la16 = base + sc.la16;
    pp.w8 = prepared ? const_cast<uint8_t*>(pw + pl.w8) : base + sc.w8;
    pp.wsf = prepared ? reinterpret_cast<float*>(const_cast<uint8_t*>(pw + pl.wsf2)) : reinterpret_cast<float*>(base + sc.wsf);
    pp.do_act = 1; pp.do_w8 = prepared ? 0 : 1; pp.do_wsf = prepared ? 0 : 1;
    {
        const int st = launch_prepack<T>(pp, s);
        if (st != NB_OK) return st;
    }
    if (EPI == NB_EPI_GELU_QUANT || EPI == NB_EPI_SWIGLU_QUANT) {
        const nb_requant_args* q = static_cast<const nb_requant_args*>(epi);
        const bool lora = q->lora_down && q->lora_act_out && q->R2 > 0;
        const int Nq = EPI == NB_EPI_SWIGLU_QUANT ? a->N / 2 : a->N;  // re-quantised columns
        p.inv_smooth = reinterpret_cast<const float*>(base + sc.inv_smooth);
        p.lora_down_t = lora ? base + sc.ldt : nullptr;
        p.lora_part = lora ? reinterpret_cast<float*>(base + sc.lora_part) : nullptr;
        p.R2 = lora ? q->R2 : 0;
        const long long units = (long long)Nq * (lora ? q->R2 : 1);
        prepack_requant_kernel<T><<<(unsigned)((units + 255) / 256), 256, 0, s>>>(
            static_cast<const T*>(q->smooth), lora ? static_cast<const T*>(q->lora_down) : nullptr, q->stride_ld, Nq,
            lora ? q->R2 : 0, reinterpret_cast<float*>(base + sc.inv_smooth), reinterpret_cast<T*>(base + sc.ldt));
        NB_CUDA_CHECK(cudaGetLastError());
    }

    const long long G = a->K / 64;
    CUtensorMap tm_a, tm_w, tm_as, tm_ws, tm_la, tm_lu;
    const CUtensorMapDataType t16 = std::is_same<T, __nv_bfloat16>::value ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                                          : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    bool ok = make_map(&tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, pp.a8, a->K, a->M, a->K, 128, BM, CU_TENSOR_MAP_SWIZZLE_128B) &&
              make_map(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, pp.w8, a->K, a->N, a->K, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B) &&
              make_map(&tm_as, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, pp.asf, (uint64_t)sc.Mp * 2, G, (uint64_t)sc.Mp * 8, BM * 2, 2,
                       CU_TENSOR_MAP_SWIZZLE_NONE) &&
              make_map(&tm_ws, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, pp.wsf, sc.Np, G, (uint64_t)sc.Np * 4, BN, 2,
                       CU_TENSOR_MAP_SWIZZLE_NONE);
    if (ok && a->R > 0)
        ok = make_map(&tm_la, t16, pp.la16, a->R, a->M, (uint64_t)a->R * 2, 32, BM, CU_TENSOR_MAP_SWIZZLE_64B) &&
             make_map(&tm_lu, t16, a->lora_up, a->R, a->N, (uint64_t)a->stride_lun * 2, 32, 128, CU_TENSOR_MAP_SWIZZLE_64B);
    else if (ok) { tm_la = tm_a; tm_lu = tm_w; }
    if (!ok) return fail_with(NB_ERR_UNSUPPORTED, "pair kernel: a tensor map could not be encoded");

    auto kern = gemm_tc_pair_kernel<EPI, T, DEBUG_P>;
    static bool attr_set[64] = {};  // per instantiation and device: the attribute lives in the device's module
    int dev = 0;
    NB_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        NB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    {
        // the register hand-over inside the kernel is balanced for a launch allocation of LAUNCH_REGS per thread
        static int regs[64] = {};
        if (dev < 0 || dev >= 64 || !regs[dev]) {
            cudaFuncAttributes fa;
            NB_CUDA_CHECK(cudaFuncGetAttributes(&fa, kern));
            if (dev >= 0 && dev < 64) regs[dev] = fa.numRegs;
            if (fa.numRegs != LAUNCH_REGS) return fail_with(NB_ERR_UNSUPPORTED, "pair kernel: unexpected register allocation");
        } else if (regs[dev] != LAUNCH_REGS) {
            return fail_with(NB_ERR_UNSUPPORTED, "pair kernel: unexpected register allocation");
        }
    }
    const int limit = max_pairs(kern, dev);
    if (limit < 1) return fail_with(NB_ERR_UNSUPPORTED, "pair kernel: no CTA pair fits on this device");
    const int total = ((a->M + 2 * BM - 1) / (2 * BM)) * ((a->N + BN - 1) / BN);
    const int pairs = total < limit ? total : limit;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(NTHREADS);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    NB_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, tm_a, tm_w, tm_as, tm_ws, tm_la, tm_lu, p));
    if ((EPI == NB_EPI_GELU_QUANT || EPI == NB_EPI_SWIGLU_QUANT) && p.R2 > 0) {
        const nb_requant_args* q = static_cast<const nb_requant_args*>(epi);
        const long long n = (long long)a->M * p.R2;
        lora_part_sum_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(p.lora_part, sc.Np / BN, a->M, p.R2, q->lora_act_out,
                                                                         q->stride_lom);
        NB_CUDA_CHECK(cudaGetLastError());
    }
    return NB_OK;
}

}  // namespace tcp

// Why the CTA-pair tcgen05 kernel cannot take this call, or nullptr.
const char* tcp_unsupported_reason(const nb_gemm_args* a, const void* epi, int epi_kind) {
    if (a->fp4) return "NVFP4 (handled by the block-scaled kernel)";
    if (a->wcscales || a->alpha != 1.0f || a->fuse_silu) return "wcscales / alpha / SiLU";
    const bool requant = epi_kind == NB_EPI_GELU_QUANT || epi_kind == NB_EPI_SWIGLU_QUANT;
    if (epi_kind != NB_EPI_STORE && epi_kind != NB_EPI_QK_NORM_ROPE && !requant) return "epilogue";
    if (a->K % 64 || a->N % 8 || a->M < 1) return "K % 64, N % 8";
    if (!aligned16(a->act) || !aligned16(a->wgt) || a->stride_am % 16 || a->stride_wn % 16) return "act / wgt alignment";
    if (a->out && (!aligned16(a->out) || a->stride_om % 8)) return "out alignment";
    if (!a->out && !requant) return "no 16-bit output";
    if (a->out && epi_kind == NB_EPI_SWIGLU_QUANT) return "SwiGLU writes no 16-bit tile";
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
    if (requant) {
        const nb_requant_args* q = static_cast<const nb_requant_args*>(epi);
        if (a->N % (epi_kind == NB_EPI_SWIGLU_QUANT ? 128 : 64)) return "N % 64 (re-quantisation groups)";
        if (!aligned16(q->qout) || q->stride_qm % 16) return "qout alignment";
        if (q->lora_down && q->lora_act_out && (q->R2 % 16 || q->R2 < 16 || !aligned16(q->lora_act_out) || q->stride_lom % 4))
            return "LoRA-down rank / alignment";
    }
    return nullptr;
}

// Resource figures of the plain-store instantiation as the runtime sees them on the current device:
// {registers per thread, max threads per block, static shared bytes, occupancy query's cluster count, its error code,
//  dynamic shared bytes asked for, threads per block}
int tcp_kernel_info(int* out) {
    auto kern = tcp::gemm_tc_pair_kernel<NB_EPI_STORE, __nv_bfloat16, false>;
    cudaFuncAttributes fa;
    NB_CUDA_CHECK(cudaFuncGetAttributes(&fa, kern));
    NB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, tcp::Cfg::SMEM_BYTES));
    int dev = 0, sms = 0;
    NB_CUDA_CHECK(cudaGetDevice(&dev));
    NB_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sms / 2 * 2);
    cfg.blockDim = dim3(tcp::NTHREADS);
    cfg.dynamicSmemBytes = tcp::Cfg::SMEM_BYTES;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int clusters = -1;
    const cudaError_t e = cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg);
    (void)cudaGetLastError();
    int blocks = -1;
    const cudaError_t e2 = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, kern, tcp::NTHREADS, tcp::Cfg::SMEM_BYTES);
    (void)cudaGetLastError();
    out[0] = fa.numRegs; out[1] = fa.maxThreadsPerBlock; out[2] = (int)fa.sharedSizeBytes; out[3] = clusters; out[4] = (int)e;
    out[5] = tcp::Cfg::SMEM_BYTES; out[6] = tcp::NTHREADS; out[7] = blocks; out[8] = (int)e2; out[9] = (int)fa.localSizeBytes;
    return NB_OK;
}

int64_t tcp_scratch_bytes(const nb_gemm_args* a, const void* epi, int epi_kind) {
    return (int64_t)tcp::scratch_layout(a, epi, epi_kind).total;
}

// The pair kernel's part of the load-time weight form: column scales as fp32 in its drain order.
int tcp_prepare_scales(const nb_gemm_args* a, void* wsf2, cudaStream_t s) {
    tcp::PrepackParams pp = {};
    pp.wscales = a->wscales;
    pp.N = a->N; pp.K = a->K; pp.Np = (a->N + tcp::BN - 1) / tcp::BN * tcp::BN;
    pp.stride_wsg = a->stride_wsg;
    pp.wsf = static_cast<float*>(wsf2);
    pp.do_wsf = 1;
    return a->dtype == NB_DTYPE_BF16 ? tcp::launch_prepack<__nv_bfloat16>(pp, s) : tcp::launch_prepack<__half>(pp, s);
}

int launch_tc_pair(const nb_gemm_args* a, const void* epi, int epi_kind, int32_t* p_out, cudaStream_t s) {
    tcp::Params p = {};
    p.out = a->out; p.bias = a->bias;
    p.p_out = p_out;
    p.M = a->M; p.N = a->N; p.K = a->K; p.actual_m = a->actual_m; p.R = a->R;
    p.stride_om = a->stride_om;
    p.status = static_cast<int*>(a->status);
    if (epi_kind == NB_EPI_QK_NORM_ROPE) {
        const nb_qk_args* q = static_cast<const nb_qk_args*>(epi);
        p.norm_q = q->norm_q; p.norm_k = q->norm_k; p.rot = q->rot; p.stride_rm = q->stride_rm;
        p.rot_rows = q->rot_rows; p.eps = q->eps;
    }
    if (epi_kind == NB_EPI_GELU_QUANT || epi_kind == NB_EPI_SWIGLU_QUANT) {
        const nb_requant_args* q = static_cast<const nb_requant_args*>(epi);
        p.qout = static_cast<uint8_t*>(q->qout); p.oscales = q->oscales; p.shift = q->shift;
        p.stride_qm = q->stride_qm; p.stride_osg = q->stride_osg;
    }
    const bool bf = a->dtype == NB_DTYPE_BF16;
    if (p_out)
        return bf ? tcp::launch_t<NB_EPI_STORE, __nv_bfloat16, true>(a, epi, p, s) : tcp::launch_t<NB_EPI_STORE, __half, true>(a, epi, p, s);
    if (epi_kind == NB_EPI_QK_NORM_ROPE)
        return bf ? tcp::launch_t<NB_EPI_QK_NORM_ROPE, __nv_bfloat16, false>(a, epi, p, s)
                  : tcp::launch_t<NB_EPI_QK_NORM_ROPE, __half, false>(a, epi, p, s);
    if (epi_kind == NB_EPI_GELU_QUANT)
        return bf ? tcp::launch_t<NB_EPI_GELU_QUANT, __nv_bfloat16, false>(a, epi, p, s)
                  : tcp::launch_t<NB_EPI_GELU_QUANT, __half, false>(a, epi, p, s);
    if (epi_kind == NB_EPI_SWIGLU_QUANT)
        return bf ? tcp::launch_t<NB_EPI_SWIGLU_QUANT, __nv_bfloat16, false>(a, epi, p, s)
                  : tcp::launch_t<NB_EPI_SWIGLU_QUANT, __half, false>(a, epi, p, s);
    return bf ? tcp::launch_t<NB_EPI_STORE, __nv_bfloat16, false>(a, epi, p, s) : tcp::launch_t<NB_EPI_STORE, __half, false>(a, epi, p, s);
}

}  // namespace nb

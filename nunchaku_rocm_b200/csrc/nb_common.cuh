// Shared device helpers: 16-bit conversions, the reference's activation functions, and thin
// wrappers over the sm_100a PTX used by the kernels (mbarrier, TMA, tcgen05, TMEM).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/nunchaku_b200.h"

namespace nb {

// --------------------------------------------------------------------------------------------
// host-side launch bookkeeping
// --------------------------------------------------------------------------------------------
int record_cuda_error(cudaError_t e);  // stores e, returns NB_ERR_LAUNCH (api.cu)
int fail_with(int status, const char* detail);  // stores a one-line reason for nb_last_error_detail, returns status

#define NB_CUDA_CHECK(expr)                                     \
    do {                                                        \
        cudaError_t _e = (expr);                                \
        if (_e != cudaSuccess) return nb::record_cuda_error(_e); \
    } while (0)

#define NB_REQUIRE(cond)                    \
    do {                                    \
        if (!(cond)) return NB_ERR_INVALID; \
    } while (0)

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// --------------------------------------------------------------------------------------------
// 16-bit element access: T is __nv_bfloat16 or __half
// --------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
    return __bfloat162float(v);
}
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) {
    return __half2float(v);
}
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) {
    return __float2half_rn(v);
}

// two fp32 -> one packed pair of T (low half = a)
template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}
template <typename T>
__device__ __forceinline__ float2 unpack2(uint32_t w);
template <>
__device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t w) {
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
template <>
__device__ __forceinline__ float2 unpack2<__half>(uint32_t w) {
    return __half22float2(*reinterpret_cast<__half2*>(&w));
}

// e4m3 byte -> fp32 (NVFP4 scales)
__device__ __forceinline__ float e4m3_to_f32(uint8_t b) {
    __half_raw h = __nv_cvt_fp8_to_halfraw(b, __NV_E4M3);
    return __half2float(*reinterpret_cast<__half*>(&h));
}

__device__ __forceinline__ float exp2f_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// --------------------------------------------------------------------------------------------
// the reference's activation functions (nunchaku/ops/triton/_common.py:70-94), fp32
// --------------------------------------------------------------------------------------------
// gelu_tanh(x) = 0.5 x (1 + tanh(u)), u = 0.79788456 (x + 0.044715 x^3); with tanh(u) = 2 / (1 + exp(-2u)) - 1 (the
// reference's form) this is x / (1 + exp(-2u)): one ex2, one reciprocal, five FMA-pipe operations.  exp(-2u) overflows to
// +inf for large negative x and the quotient is then -0, the limit of the function.
__device__ __forceinline__ float gelu_tanh(float x) {
    constexpr float A = -2.0f * 0.79788456f * 1.4426950408889634f;  // -2 * sqrt(2/pi) * log2(e)
    constexpr float B = A * 0.044715f;
    const float e = exp2f_approx(x * fmaf(x * x, B, A));
    return __fdividef(x, 1.0f + e);
}
__device__ __forceinline__ float silu(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

// round-half-even of |x| < 2^22 by the magic-number add (gemm_w4a4.py:1317-1325)
__device__ __forceinline__ float rint_small(float x) { return __fsub_rn(__fadd_rn(x, 12582912.0f), 12582912.0f); }

// e2m1 encode with the reference's thresholds: ties go to the larger magnitude (gemm_w4a4.py:116-135)
__device__ __forceinline__ uint32_t e2m1_encode(float x) {
    float a = fabsf(x);
    uint32_t c = (a >= 0.25f) + (a >= 0.75f) + (a >= 1.25f) + (a >= 1.75f) + (a >= 2.5f) + (a >= 3.5f) + (a >= 5.0f);
    return c | (x < 0.0f ? 8u : 0u);
}
__device__ __forceinline__ float e2m1_decode(uint32_t c) {
    uint32_t m = c & 7u;
    // 0, .5, 1, 1.5, 2, 3, 4, 6
    float v = m < 4 ? 0.5f * (float)m : (m == 4 ? 2.0f : (m == 5 ? 3.0f : (m == 6 ? 4.0f : 6.0f)));
    return (c & 8u) ? -v : v;
}

// --------------------------------------------------------------------------------------------
// PTX: shared-memory addresses, mbarrier, fences
// --------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// one test by every lane of the (converged) warp and the warp's vote on it: a warp-uniform verdict in three instructions
__device__ __forceinline__ bool mbar_try_wait_all(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "vote.sync.all.pred q, p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// the same as a non-blocking probe (test_wait never parks the warp): for looking at a barrier ahead of time
__device__ __forceinline__ bool mbar_test_all(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "vote.sync.all.pred q, p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// try_wait that lets the hardware park the thread for up to `hint_ns` before it reports "not yet"
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait: gives up after ~2 s (or as soon as another thread of the CTA has given up), records
// `code` in *abort_flag and returns false.  The caller must then unwind without touching the data.
// Every poll is one operation on the shared-memory barrier unit, which all warps of the CTA share, so a
// waiter parks in the hardware (`hint_ns`) instead of polling in a tight loop.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code,
                                          unsigned hint_ns = 200, uint64_t limit_ns = 2000000000ull) {
    if (mbar_try_wait(bar, parity)) return true;
    uint64_t t0 = 0;
    for (uint32_t spin = 1;; ++spin) {
        if (mbar_try_wait_hint(bar, parity, hint_ns)) return true;
        if ((spin & 63u) == 0) {
            if (*abort_flag) return false;
            uint64_t now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            if (now - t0 > limit_ns) {
                *abort_flag = code;
                return false;
            }
        }
    }
}
// The same wait by a whole (converged) warp with a warp-uniform verdict.  Every lane tests and the warp votes; between
// tests the hardware may park the warp for its own short limit and resumes it when the phase completes.  (With a
// suspend-time hint a waiter was measured to come back about a hint late, and a chain of such waits - stage landed, slot
// free, MMAs done - set the pace of the whole pipeline, so the latency-critical waits give no hint.)
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code,
                                               unsigned /*hint_ns*/ = 0, uint64_t limit_ns = 2000000000ull) {
    if (mbar_try_wait_all(bar, parity)) return true;
    uint64_t t0 = 0;
    for (uint32_t spin = 1;; ++spin) {
        if (mbar_try_wait_all(bar, parity)) return true;
        if ((spin & 255u) == 0) {
            int give_up = 0;
            if ((threadIdx.x & 31) == 0) {
                if (*abort_flag) give_up = 1;
                const uint64_t now = globaltimer_ns();
                if (t0 == 0) t0 = now;
                if (now - t0 > limit_ns) {
                    *abort_flag = code;
                    give_up = 1;
                }
            }
            if (__shfl_sync(0xffffffffu, give_up, 0)) return false;
        }
    }
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// make generic-proxy writes to shared memory visible to the async proxy (TMA, tcgen05.mma operand reads)
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// --------------------------------------------------------------------------------------------
// PTX: TMA tiled loads (no multicast anywhere)
// --------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(tmap), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// --------------------------------------------------------------------------------------------
// PTX: tcgen05 / tensor memory
// --------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {  // whole warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// kind::f8f6f4: 8-bit (or narrower) floating-point operands, fp32 accumulators, K = 32 per instruction
__device__ __forceinline__ void mma_f8(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
        : "memory");
}
__device__ __forceinline__ void mma_f16(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
        : "memory");
}


// 16 lanes x 64 columns in the accumulator-fragment layout: with gid = lane / 4, tig = lane % 4, register
// 4 j + 2 r + e is TMEM lane (lane field) + 8 r + gid, column 8 j + 2 tig + e
__device__ __forceinline__ void tmem_ld_16x256b_x8(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.16x256b.x8.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
        "%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}

// the same layout, 16 lanes x 32 columns (j = 0..3)
__device__ __forceinline__ void tmem_ld_16x256b_x4(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.16x256b.x4.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_16x256b(uint32_t taddr, uint32_t (&v)[32]) { tmem_ld_16x256b_x8(taddr, v); }
__device__ __forceinline__ void tmem_ld_16x256b(uint32_t taddr, uint32_t (&v)[16]) { tmem_ld_16x256b_x4(taddr, v); }

// packed pairs of fp32 in one 64-bit register (low word = first element) and the sm_100 packed FMA / ADD
__device__ __forceinline__ uint64_t pack_u32x2(uint32_t lo, uint32_t hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
    return pack_u32x2(__float_as_uint(lo), __float_as_uint(hi));
}
__device__ __forceinline__ float2 unpack_f32x2(uint64_t v) {
    uint32_t lo, hi;
    asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(v));
    return make_float2(__uint_as_float(lo), __uint_as_float(hi));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t mul_f32x2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// Shared-memory matrix descriptor, K-major operand without swizzle: 8-row x 16-byte core matrices,
// `lbo` bytes between the core matrices of consecutive 16-byte K chunks, `sbo` bytes between
// consecutive 8-row groups.
__device__ __forceinline__ uint64_t umma_desc_kmajor(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3fff);
    d |= (uint64_t)((lbo >> 4) & 0x3fff) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3fff) << 32;
    d |= (uint64_t)1 << 46;  // descriptor version of sm_100
    return d;
}

// Four nibbles (low 16 bits of `x`, element k in bits 4k..4k+3) -> four e4m3 bytes.  Signed nibbles are two's complement
// -8..7, unsigned 0..15; every value is exact in e4m3.  Entries 0..7 and 8..15 of the table come from two byte permutes on
// the low three bits; a third permute turns bit 3 of every nibble into a byte mask (selector 1 -> 0xFF, 0 -> 0x00).
__device__ __forceinline__ uint32_t e4m3_of_nibbles(uint32_t x, bool uns) {
    // e4m3: 0 1 2 3 4 5 6 7 -> 00 38 40 44 48 4A 4C 4E;  8..15 -> 50 51 52 53 54 55 56 57;  -8..-1 -> D0 CE CC CA C8 C4 C0 B8
    const uint32_t lo0 = 0x44403800u, lo1 = 0x4E4C4A48u;
    const uint32_t hi0 = uns ? 0x53525150u : 0xCACCCED0u, hi1 = uns ? 0x57565554u : 0xB8C0C4C8u;
    const uint32_t sel = x & 0x7777u;
    const uint32_t lo = __byte_perm(lo0, lo1, sel), hi = __byte_perm(hi0, hi1, sel);
    const uint32_t m = __byte_perm(0x0000FF00u, 0u, (x & 0x8888u) >> 3);
    return lo ^ ((lo ^ hi) & m);
}

// Load-time form of an int4 weight for the tensor-core kernels (nb_gemm_w4a4_prepare_weights): one e4m3 byte per value,
// then the column scales in the single-CTA kernel's drain order (T, N rounded up to 128) and in the CTA-pair kernel's
// (fp32, N rounded up to 256).  Offsets in bytes, each region 256-byte aligned.
struct PreparedLayout {
    size_t w8, wsf, wsf2, total;
    int Np128, Np256;
};
static inline PreparedLayout prepared_layout(int N, int K) {
    auto up256 = [](size_t x) { return (x + 255) & ~size_t(255); };
    PreparedLayout s;
    s.Np128 = (N + 127) / 128 * 128;
    s.Np256 = (N + 255) / 256 * 256;
    size_t off = 0;
    s.w8 = off; off += up256((size_t)N * K);
    s.wsf = off; off += up256((size_t)(K / 64) * s.Np128 * 2);
    s.wsf2 = off; off += up256((size_t)(K / 64) * s.Np256 * 4);
    s.total = off;
    return s;
}
static inline bool has_prepared_weights(const nb_gemm_args* a) {
    return a->wgt_prepared && a->wgt_prepared_bytes >= (int64_t)prepared_layout(a->N, a->K).total &&
           (reinterpret_cast<uintptr_t>(a->wgt_prepared) & 255) == 0;
}

// --------------------------------------------------------------------------------------------
// PTX: CTA pairs (cluster of two, tcgen05 cta_group::2)
// --------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on the barrier at the same shared-memory offset in CTA `rank` of the cluster.  What the arrival publishes is
// "this warp's tcgen05.ld of the slot have completed", which tcgen05.wait::ld + tcgen05.fence::before_thread_sync order;
// no generic-memory write is handed over, so the arrival carries no cluster-scope release (that form compiles to a
// memory barrier which, once per warp and K group, was the largest stall of the kernel).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t local_bar, uint32_t rank) {
    asm volatile(
        "{\n\t.reg .b32 ra;\n\tmapa.shared::cluster.u32 ra, %0, %1;\n\t"
        "mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [ra];\n\t}"
        ::"r"(local_bar), "r"(rank)
        : "memory");
}
__device__ __forceinline__ uint32_t mapa_cluster(uint32_t local_addr, uint32_t rank) {
    uint32_t ra;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(local_addr), "r"(rank));
    return ra;
}
// the same arrival on an address mapa_cluster() gave, by the threads whose `pred` is non-zero
__device__ __forceinline__ void mbar_arrive_remote_if(uint32_t remote_bar, uint32_t pred) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %1, 0;\n\t"
        "@p mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];\n\t}"
        ::"r"(remote_bar), "r"(pred)
        : "memory");
}
// The same with release semantics at cluster scope: the relay's "my half of the stage has landed" precedes reads of this
// CTA's shared memory by the other SM's tensor core (one thread, once per ring stage).
__device__ __forceinline__ void mbar_arrive_cluster_release(uint32_t local_bar, uint32_t rank) {
    asm volatile(
        "{\n\t.reg .b32 ra;\n\tmapa.shared::cluster.u32 ra, %0, %1;\n\t"
        "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n\t}"
        ::"r"(local_bar), "r"(rank)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t dst_smem, uint32_t ncols) {  // warp 1 of both CTAs
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// completion of every MMA issued so far -> one arrival on the barrier at this offset in both CTAs
__device__ __forceinline__ void tc_commit2(uint32_t bar) {
    asm volatile(
        "{\n\t.reg .b16 m;\n\tmov.b16 m, 3;\n\t"
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m;\n\t}"
        ::"r"(bar)
        : "memory");
}
// one lane of the (converged) warp
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}
// Instruction descriptor (dense, K-major A and B, M = 128)
__device__ __host__ constexpr uint32_t umma_idesc(uint32_t c_fmt, uint32_t a_fmt, uint32_t b_fmt, uint32_t n) {
    return (c_fmt << 4) | (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}

}  // namespace nb

// Unmasked flash attention, (B, H, T, D) strided inputs -> (B, Tq, H * D).
//
// Rounding points follow the reference kernel (nunchaku/ops/triton/attention.py:61-117): q * scale * log2(e)
// is rounded to the input dtype, scores and the running max / sum are fp32 in base 2, the probabilities are
// rounded to the input dtype before P @ V, the accumulator is fp32, one division by the row sum at the end.
//
// A CTA of 8 warps owns 128 query rows of one (batch, head); each warp owns 16 rows and keeps its Q
// fragments, the 16 x 64 score tile and the 16 x D output accumulator in registers.  K and V tiles of 64
// keys are double-buffered in shared memory with cp.async, in 16-byte units XOR-swizzled by the row so that
// ldmatrix reads are conflict-free.  The matrix products run on mma.sync.m16n8k16.  This kernel takes the calls the
// tcgen05 kernel does not (head dimension 64, unaligned outputs, views broadcast over heads or batch).
#include "nb_common.cuh"

namespace nb {
namespace {

constexpr int AT_BM = 128, AT_BN = 64, AT_THREADS = 256;

__device__ __forceinline__ void cp16(uint32_t dst, const void* src, bool ok) {
    const int sz = ok ? 16 : 0;  // size 0: zero-fill
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <typename T>
__device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// byte offset of (row, 16-byte unit u) in a tile whose rows hold UPR units; units are XOR-swizzled by the row
template <int UPR>
__device__ __forceinline__ uint32_t sw(int row, int u) {
    return (uint32_t)(row * UPR + (u ^ (row & 7))) * 16u;
}

template <typename T, int D>
__global__ void __launch_bounds__(AT_THREADS) attention_kernel(const nb_attn_args p) {
    constexpr int UPR = D / 8;  // 16-byte units per row
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* q_s = smem;                          // AT_BM x D
    uint8_t* k_s = q_s + AT_BM * D * 2;           // 2 x AT_BN x D
    uint8_t* v_s = k_s + 2 * AT_BN * D * 2;       // 2 x AT_BN x D
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
    const int m0 = blockIdx.x * AT_BM, head = blockIdx.y, batch = blockIdx.z;
    const T* qg = static_cast<const T*>(p.q) + (long long)batch * p.stride_qb + (long long)head * p.stride_qh;
    const T* kg = static_cast<const T*>(p.k) + (long long)batch * p.stride_kb + (long long)head * p.stride_kh;
    const T* vg = static_cast<const T*>(p.v) + (long long)batch * p.stride_vb + (long long)head * p.stride_vh;

    auto load_kv = [&](int tile, int buf) {
        const int n0 = tile * AT_BN;
        for (int u = threadIdx.x; u < AT_BN * UPR; u += AT_THREADS) {
            const int r = u / UPR, c = u % UPR;
            const bool ok = n0 + r < p.Tkv;
            const long long rr = ok ? n0 + r : 0;
            cp16(smem_u32(k_s + buf * AT_BN * D * 2) + sw<UPR>(r, c), kg + rr * p.stride_kn + c * 8, ok);
            cp16(smem_u32(v_s + buf * AT_BN * D * 2) + sw<UPR>(r, c), vg + rr * p.stride_vn + c * 8, ok);
        }
    };

    // ---- Q tile: scale by scale * log2(e), round to T, store swizzled
    const float qscale = p.scale * 1.4426950408889634f;
    for (int u = threadIdx.x; u < AT_BM * UPR; u += AT_THREADS) {
        const int r = u / UPR, c = u % UPR;
        uint4 raw = make_uint4(0, 0, 0, 0);
        if (m0 + r < p.Tq) raw = __ldg(reinterpret_cast<const uint4*>(qg + (long long)(m0 + r) * p.stride_qm + c * 8));
        uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = unpack2<T>(w[i]);
            w[i] = pack2<T>(f.x * qscale, f.y * qscale);
        }
        *reinterpret_cast<uint4*>(q_s + sw<UPR>(r, c)) = make_uint4(w[0], w[1], w[2], w[3]);
    }
    const int ntiles = (p.Tkv + AT_BN - 1) / AT_BN;
    load_kv(0, 0);
    cp_commit();
    __syncthreads();

    // ---- Q fragments of this warp's 16 rows: D/16 k-steps
    uint32_t qf[D / 16][4];
    {
        const int r = warp * 16 + (lane & 15);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) ldsm_x4(qf[ks], smem_u32(q_s) + sw<UPR>(r, ks * 2 + (lane >> 4)));
    }

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};

    for (int t = 0; t < ntiles; ++t) {
        if (t + 1 < ntiles) load_kv(t + 1, (t + 1) & 1);
        cp_commit();
        cp_wait<1>();
        __syncthreads();
        const uint32_t kb = smem_u32(k_s + (t & 1) * AT_BN * D * 2), vb = smem_u32(v_s + (t & 1) * AT_BN * D * 2);

        // ---- S = Q K^T : 16 x 64
        float s[AT_BN / 8][4];
#pragma unroll
        for (int i = 0; i < AT_BN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
            for (int nt = 0; nt < AT_BN / 8; nt += 2) {
                // matrices: (keys nt*8.., d ks*16..+7), (same keys, d +8), (keys +8, d ..+7), (keys +8, d +8)
                uint32_t b[4];
                const int r = nt * 8 + (lane & 7) + ((lane >> 4) << 3);
                ldsm_x4(b, kb + sw<UPR>(r, ks * 2 + ((lane >> 3) & 1)));
                mma<T>(s[nt], qf[ks], b[0], b[1]);
                mma<T>(s[nt + 1], qf[ks], b[2], b[3]);
            }
        }
        // ---- mask the key tail, online softmax in base 2
        const int n0 = t * AT_BN;
        if (n0 + AT_BN > p.Tkv) {
#pragma unroll
            for (int nt = 0; nt < AT_BN / 8; ++nt) {
                const int c = n0 + nt * 8 + 2 * tig;
                if (c >= p.Tkv) s[nt][0] = s[nt][2] = -INFINITY;
                if (c + 1 >= p.Tkv) s[nt][1] = s[nt][3] = -INFINITY;
            }
        }
        float mx[2] = {mrow[0], mrow[1]};
#pragma unroll
        for (int nt = 0; nt < AT_BN / 8; ++nt) {
            mx[0] = fmaxf(mx[0], fmaxf(s[nt][0], s[nt][1]));
            mx[1] = fmaxf(mx[1], fmaxf(s[nt][2], s[nt][3]));
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        }
        float alpha[2], msafe[2], psum[2] = {0.f, 0.f};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            msafe[h] = mx[h] == -INFINITY ? 0.f : mx[h];
            alpha[h] = mrow[h] == -INFINITY ? 0.f : exp2f(mrow[h] - msafe[h]);
            mrow[h] = mx[h];
        }
        uint32_t pf[AT_BN / 16][4];  // P as A fragments of the second product
#pragma unroll
        for (int nt = 0; nt < AT_BN / 8; ++nt) {
            const float p0 = exp2f(s[nt][0] - msafe[0]), p1 = exp2f(s[nt][1] - msafe[0]);
            const float p2 = exp2f(s[nt][2] - msafe[1]), p3 = exp2f(s[nt][3] - msafe[1]);
            psum[0] += p0 + p1;
            psum[1] += p2 + p3;
            pf[nt >> 1][(nt & 1) * 2 + 0] = pack2<T>(p0, p1);
            pf[nt >> 1][(nt & 1) * 2 + 1] = pack2<T>(p2, p3);
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            psum[h] += __shfl_xor_sync(0xffffffffu, psum[h], 1);
            psum[h] += __shfl_xor_sync(0xffffffffu, psum[h], 2);
            lrow[h] = lrow[h] * alpha[h] + psum[h];
        }
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
            o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
            o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
        }
        // ---- O += P V : k = keys (4 steps of 16), n = d
#pragma unroll
        for (int ks = 0; ks < AT_BN / 16; ++ks) {
#pragma unroll
            for (int nt = 0; nt < D / 8; nt += 2) {
                // trans matrices: (keys ks*16..+7, d nt*8..), (keys +8, same d), (keys ..+7, d +8), (keys +8, d +8)
                uint32_t b[4];
                const int r = ks * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
                ldsm_x4_t(b, vb + sw<UPR>(r, nt + (lane >> 4)));
                mma<T>(o[nt], pf[ks], b[0], b[1]);
                mma<T>(o[nt + 1], pf[ks], b[2], b[3]);
            }
        }
        __syncthreads();
    }
    cp_wait<0>();

    // ---- O / l -> T, (B, Tq, H * D)
    T* og = static_cast<T*>(p.o) + (long long)batch * p.stride_ob + (long long)head * D;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int m = m0 + warp * 16 + gid + 8 * h;
        if (m >= p.Tq) continue;
        const float inv = 1.0f / (lrow[h] == 0.f ? 1.0f : lrow[h]);
#pragma unroll
        for (int nt = 0; nt < D / 8; ++nt) {
            const uint32_t w = pack2<T>(o[nt][2 * h] * inv, o[nt][2 * h + 1] * inv);
            *reinterpret_cast<uint32_t*>(og + (long long)m * p.stride_om + nt * 8 + 2 * tig) = w;
        }
    }
}

template <typename T, int D>
int launch_attn(const nb_attn_args* a, cudaStream_t s) {
    const size_t smem = (size_t)(AT_BM + 4 * AT_BN) * D * 2;
    auto kern = attention_kernel<T, D>;
    NB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((a->Tq + AT_BM - 1) / AT_BM, a->H, a->B);
    kern<<<grid, AT_THREADS, smem, s>>>(*a);
    NB_CUDA_CHECK(cudaGetLastError());
    return NB_OK;
}

}  // namespace
}  // namespace nb

namespace nb {
const char* attn_tc_unsupported_reason(const nb_attn_args* a);
int64_t attn_tc_scratch_bytes(const nb_attn_args* a);
int launch_attention_tc(const nb_attn_args* a, cudaStream_t s);

static bool attn_common_ok(const nb_attn_args* a) {
    if (!a || !a->q || !a->k || !a->v || !a->o) return false;
    if (a->dtype != NB_DTYPE_BF16 && a->dtype != NB_DTYPE_FP16) return false;
    const long long strides[] = {a->stride_qb, a->stride_qh, a->stride_qm, a->stride_kb, a->stride_kh, a->stride_kn,
                                 a->stride_vb, a->stride_vh, a->stride_vn};
    for (long long st : strides)
        if (st % 8) return false;
    return aligned16(a->q) && aligned16(a->k) && aligned16(a->v);
}
// the call fits the tcgen05 kernel's rules (scratch apart)
static bool attn_fits_tc(const nb_attn_args* a) {
    return a->impl != NB_IMPL_GENERIC && attn_common_ok(a) && attn_tc_unsupported_reason(a) == nullptr;
}
static bool attn_scratch_ok(const nb_attn_args* a) {
    if (attn_tc_scratch_bytes(a) == 0) return true;  // (the kernel reads Q, K and V in place)
    return a->scratch && a->scratch_bytes >= attn_tc_scratch_bytes(a) && (reinterpret_cast<uintptr_t>(a->scratch) & 255) == 0;
}
}  // namespace nb

extern "C" int64_t nb_attention_scratch_bytes(const nb_attn_args* a) {
    if (!a || a->B <= 0 || a->H <= 0) return 0;
    return nb::attn_fits_tc(a) ? nb::attn_tc_scratch_bytes(a) : 0;
}

extern "C" int nb_attention(const nb_attn_args* a, void* stream) {
    using namespace nb;
    NB_REQUIRE(a && a->q && a->k && a->v && a->o);
    // tcgen05 kernel when the call fits it (and brings the scratch it asks for: none at present)
    if (a->B > 0 && a->H > 0 && attn_fits_tc(a) && attn_scratch_ok(a))
        return launch_attention_tc(a, static_cast<cudaStream_t>(stream));
    if (a->impl == NB_IMPL_TCGEN05) return attn_fits_tc(a) ? NB_ERR_INVALID : NB_ERR_UNSUPPORTED;
    NB_REQUIRE(a->B > 0 && a->H > 0 && a->Tq >= 0 && a->Tkv >= 0);
    NB_REQUIRE(a->dtype == NB_DTYPE_BF16 || a->dtype == NB_DTYPE_FP16);
    if (a->D != 64 && a->D != 128) return NB_ERR_UNSUPPORTED;
    const long long strides[] = {a->stride_qb, a->stride_qh, a->stride_qm, a->stride_kb, a->stride_kh, a->stride_kn,
                                 a->stride_vb, a->stride_vh, a->stride_vn};
    for (long long st : strides)
        if (st % 8) return NB_ERR_UNSUPPORTED;
    if (!aligned16(a->q) || !aligned16(a->k) || !aligned16(a->v) || (reinterpret_cast<uintptr_t>(a->o) & 3) ||
        a->stride_ob % 2 || a->stride_om % 2)
        return NB_ERR_UNSUPPORTED;
    if (a->Tq == 0) return NB_OK;
    if (a->B > 65535 || a->H > 65535) return NB_ERR_UNSUPPORTED;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool bf = a->dtype == NB_DTYPE_BF16;
    if (a->D == 128) return bf ? launch_attn<__nv_bfloat16, 128>(a, s) : launch_attn<__half, 128>(a, s);
    return bf ? launch_attn<__nv_bfloat16, 64>(a, s) : launch_attn<__half, 64>(a, s);
}

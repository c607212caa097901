// Entry point of the W4A4 GEMM: argument contract, kernel choice, and the generic path's scratch.
#include "nb_common.cuh"

namespace nb {

struct GenericParams {
    const uint8_t* act;
    const uint8_t* wgt;
    void* out;
    float* acc_out;
    int32_t* p_out;
    const void* ascales;
    const void* wscales;
    const void* bias;
    const float* lora_act;
    const void* lora_up;
    const void* wcscales;
    int M, N, K, actual_m, R;
    int act_unsigned, fp4, fuse_silu;
    float alpha;
    long long stride_am, stride_wn, stride_asg, stride_wsg, stride_om, stride_lam, stride_lun;
};

int launch_generic(const GenericParams& p, int dtype, cudaStream_t s);
int launch_qk_rows(const float* src_f, void* out, long long stride_om, int M, int N, int dtype, const nb_qk_args* qk,
                   cudaStream_t s);
int launch_requant_rows(const float* lin, int M, int N, int mode, int dtype, const nb_requant_args* q, cudaStream_t s);
const char* tc_unsupported_reason(const nb_gemm_args* a, const void* epi, int epi_kind);
int launch_tc(const nb_gemm_args* a, const void* epi, int epi_kind, int32_t* p_out, cudaStream_t s);
int64_t tc_scratch_bytes(const nb_gemm_args* a);
int64_t tc_prepared_bytes(const nb_gemm_args* a);
int64_t tc_fp4_prepared_bytes(const nb_gemm_args* a);
int tc_fp4_prepare_weights(const nb_gemm_args* a, void* dst, int64_t dst_bytes, cudaStream_t s);
int tc_prepare_weights(const nb_gemm_args* a, void* dst, int64_t dst_bytes, cudaStream_t s);
const char* tcp_unsupported_reason(const nb_gemm_args* a, const void* epi, int epi_kind);
int launch_tc_pair(const nb_gemm_args* a, const void* epi, int epi_kind, int32_t* p_out, cudaStream_t s);
int64_t tcp_scratch_bytes(const nb_gemm_args* a, const void* epi, int epi_kind);
const char* tc_fp4_unsupported_reason(const nb_gemm_args* a, const void* epi, int epi_kind);
int launch_tc_fp4(const nb_gemm_args* a, cudaStream_t s);
int64_t tc_fp4_scratch_bytes(const nb_gemm_args* a);

// Which kernel takes the call.  NVFP4 calls go to the block-scaled kind::mxf4nvf4 kernel.  int4 calls go to one of the two
// kind::f8f6f4 kernels: the CTA-pair kernel (256 x 256 tiles, one pair of SMs per tile, the only one with the fused
// re-quantising epilogues) or the single-CTA kernel (128 x 128 tiles).  Both are persistent with a static tile range per
// CTA (pair), so what decides is the number of tiles the busiest unit gets times the measured cost of a tile's K group:
// about 1250 cycles for a pair tile and 800 for a single tile on a B200 (4608 x 3072 x 3072: 0.105 ms against 0.122 ms,
// 512 x 3072 x 3072: 0.039 ms against 0.025 ms).
enum Kernel { K_GENERIC = 0, K_TC_SINGLE, K_TC_PAIR, K_TC_FP4 };
static int sm_count() {
    static int cache[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!cache[dev]) {
        int sms = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 2) sms = 148;
        cache[dev] = sms;
    }
    return cache[dev];
}
static Kernel choose_kernel(const nb_gemm_args* a, const void* epi, int epi_kind, const char** why) {
    *why = nullptr;
    if (a->impl == NB_IMPL_GENERIC) return K_GENERIC;
    if (a->fp4) {
        // The block-scaled kernel stores 16-bit tiles only.  A Q/K epilogue on an NVFP4 call runs as that kernel plus the
        // row kernel in place on the stored tile: the reference's unfused form (gemm_w4a4.py:834-866), i.e. with the
        // tile rounded to the 16-bit dtype before RMSNorm + RoPE.
        *why = tc_fp4_unsupported_reason(a, epi, epi_kind == NB_EPI_QK_NORM_ROPE ? NB_EPI_STORE : epi_kind);
        return *why ? K_GENERIC : K_TC_FP4;
    }
    const char* single = tc_unsupported_reason(a, epi, epi_kind);
    const char* pair = tcp_unsupported_reason(a, epi, epi_kind);
    if (a->impl == NB_IMPL_TCGEN05_PAIR) { *why = pair; return pair ? K_GENERIC : K_TC_PAIR; }
    if (a->impl == NB_IMPL_TCGEN05_SINGLE) { *why = single; return single ? K_GENERIC : K_TC_SINGLE; }
    if (!pair && !single) {
        const long long sms = sm_count();
        const long long pair_tiles = (long long)((a->M + 255) / 256) * ((a->N + 255) / 256);
        const long long single_tiles = (long long)((a->M + 127) / 128) * ((a->N + 127) / 128);
        const long long pair_cost = (pair_tiles + sms / 2 - 1) / (sms / 2) * 1250;
        const long long single_cost = (single_tiles + sms - 1) / sms * 800;
        return pair_cost <= single_cost ? K_TC_PAIR : K_TC_SINGLE;
    }
    if (!pair) return K_TC_PAIR;
    if (!single) return K_TC_SINGLE;
    *why = single;
    return K_GENERIC;
}

static int validate(const nb_gemm_args* a, const void* epi, int epi_kind) {
    NB_REQUIRE(a && a->act && a->wgt && a->ascales && a->wscales);
    NB_REQUIRE(a->dtype == NB_DTYPE_BF16 || a->dtype == NB_DTYPE_FP16);
    NB_REQUIRE(a->M >= 0 && a->N > 0 && a->K > 0 && a->actual_m >= 0 && a->actual_m <= a->M);
    NB_REQUIRE(a->K % (a->fp4 ? 16 : 64) == 0);
    NB_REQUIRE(a->R >= 0 && (a->R == 0 || (a->lora_act && a->lora_up)));
    NB_REQUIRE(epi_kind >= NB_EPI_STORE && epi_kind <= NB_EPI_SWIGLU_QUANT);
    NB_REQUIRE(epi_kind == NB_EPI_STORE || epi != nullptr);
    if (epi_kind == NB_EPI_STORE || epi_kind == NB_EPI_QK_NORM_ROPE) NB_REQUIRE(a->out != nullptr);
    if (epi_kind == NB_EPI_QK_NORM_ROPE) {
        const nb_qk_args* q = static_cast<const nb_qk_args*>(epi);
        NB_REQUIRE(q->norm_q && q->norm_k && q->rot && q->rot_rows > 0);
        NB_REQUIRE(a->N % 3 == 0 && (a->N / 3) % 128 == 0);
        NB_REQUIRE(a->actual_m % q->rot_rows == 0 || q->rot_rows >= a->actual_m);
    }
    if (epi_kind == NB_EPI_GELU_QUANT || epi_kind == NB_EPI_SWIGLU_QUANT) {
        const nb_requant_args* q = static_cast<const nb_requant_args*>(epi);
        NB_REQUIRE(q->qout && q->oscales && !a->fp4);
        NB_REQUIRE(a->N % (epi_kind == NB_EPI_GELU_QUANT ? 64 : 128) == 0);
        NB_REQUIRE((q->lora_down == nullptr) == (q->lora_act_out == nullptr));
    }
    return NB_OK;
}

static bool uses_tc(const nb_gemm_args* a, const void* epi, int epi_kind) {
    const char* why;
    return choose_kernel(a, epi, epi_kind, &why) != K_GENERIC;
}

// The tensor-core kernels keep their operand form (e4m3 bytes, ordered scales, rounded lora_act, epilogue inputs) in
// scratch; the generic kernel keeps the fp32 tile there when a row-wise epilogue follows.
static int64_t scratch_bytes(const nb_gemm_args* a, const void* epi, int epi_kind) {
    const char* why;
    switch (choose_kernel(a, epi, epi_kind, &why)) {
        case K_TC_FP4: return tc_fp4_scratch_bytes(a);
        case K_TC_SINGLE: return tc_scratch_bytes(a);
        case K_TC_PAIR: return tcp_scratch_bytes(a, epi, epi_kind);
        default: return epi_kind == NB_EPI_STORE ? 0 : (int64_t)a->M * a->N * 4;
    }
}

static GenericParams to_generic(const nb_gemm_args* a) {
    GenericParams p = {};
    p.act = static_cast<const uint8_t*>(a->act); p.wgt = static_cast<const uint8_t*>(a->wgt);
    p.ascales = a->ascales; p.wscales = a->wscales; p.bias = a->bias;
    p.lora_act = static_cast<const float*>(a->lora_act); p.lora_up = a->lora_up; p.wcscales = a->wcscales;
    p.M = a->M; p.N = a->N; p.K = a->K; p.actual_m = a->actual_m; p.R = a->R;
    p.act_unsigned = a->act_unsigned; p.fp4 = a->fp4; p.fuse_silu = a->fuse_silu; p.alpha = a->alpha;
    p.stride_am = a->stride_am; p.stride_wn = a->stride_wn; p.stride_asg = a->stride_asg; p.stride_wsg = a->stride_wsg;
    p.stride_om = a->stride_om; p.stride_lam = a->stride_lam; p.stride_lun = a->stride_lun;
    return p;
}

}  // namespace nb

extern "C" int64_t nb_gemm_w4a4_scratch_bytes(const nb_gemm_args* a, const void* epi, int epi_kind) {
    if (!a || nb::validate(a, epi, epi_kind) != NB_OK) return 0;
    if (a->M == 0) return 0;
    return nb::scratch_bytes(a, epi, epi_kind);
}

extern "C" int nb_gemm_w4a4(const nb_gemm_args* a, const void* epi, int epi_kind, void* stream) {
    using namespace nb;
    int st = validate(a, epi, epi_kind);
    if (st != NB_OK) return st;
    if (a->M == 0) return NB_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const char* reason;
    const Kernel k = choose_kernel(a, epi, epi_kind, &reason);
    if (k == K_GENERIC && a->impl != NB_IMPL_AUTO && a->impl != NB_IMPL_GENERIC) return NB_ERR_UNSUPPORTED;
    if (k == K_TC_FP4) {
        st = launch_tc_fp4(a, s);
        if (st == NB_OK && epi_kind == NB_EPI_QK_NORM_ROPE)
            st = launch_qk_rows(nullptr, a->out, a->stride_om, a->actual_m, a->N, a->dtype, static_cast<const nb_qk_args*>(epi), s);
        return st;
    }
    if (k == K_TC_SINGLE) return launch_tc(a, epi, epi_kind, nullptr, s);
    if (k == K_TC_PAIR) return launch_tc_pair(a, epi, epi_kind, nullptr, s);

    GenericParams p = to_generic(a);
    if (epi_kind == NB_EPI_STORE) {
        p.out = a->out;
        return launch_generic(p, a->dtype, s);
    }
    NB_REQUIRE(a->scratch && a->scratch_bytes >= (int64_t)a->M * a->N * 4);
    p.acc_out = static_cast<float*>(a->scratch);
    p.out = epi_kind == NB_EPI_GELU_QUANT ? a->out : nullptr;  // optional pre-GELU 16-bit tile
    st = launch_generic(p, a->dtype, s);
    if (st != NB_OK) return st;
    if (epi_kind == NB_EPI_QK_NORM_ROPE)
        return launch_qk_rows(p.acc_out, a->out, a->stride_om, a->actual_m, a->N, a->dtype,
                              static_cast<const nb_qk_args*>(epi), s);
    return launch_requant_rows(p.acc_out, a->M, a->N, epi_kind == NB_EPI_GELU_QUANT ? 0 : 1, a->dtype,
                               static_cast<const nb_requant_args*>(epi), s);
}

namespace nb { int tcp_kernel_info(int* out); }
// Diagnostics: how the CTA-pair kernel fits the current device (registers, threads, shared memory, resident pairs).
extern "C" int nb_debug_pair_kernel_info(int* out10) { return out10 ? nb::tcp_kernel_info(out10) : NB_ERR_INVALID; }

extern "C" int64_t nb_gemm_w4a4_prepared_bytes(const nb_gemm_args* a) {
    return a && a->fp4 ? nb::tc_fp4_prepared_bytes(a) : nb::tc_prepared_bytes(a);
}

extern "C" int nb_gemm_w4a4_prepare_weights(const nb_gemm_args* a, void* dst, int64_t dst_bytes, void* stream) {
    if (a && a->fp4) return nb::tc_fp4_prepare_weights(a, dst, dst_bytes, static_cast<cudaStream_t>(stream));
    return nb::tc_prepare_weights(a, dst, dst_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" int64_t nb_gemm_w4a4_uses_tcgen05(const nb_gemm_args* a, const void* epi, int epi_kind) {
    if (!a || nb::validate(a, epi, epi_kind) != NB_OK) return 0;
    return nb::uses_tc(a, epi, epi_kind) ? 1 : 0;
}

extern "C" int nb_gemm_w4a4_group_sums(const nb_gemm_args* a, int32_t* p_out, void* stream) {
    using namespace nb;
    int st = validate(a, nullptr, NB_EPI_STORE);
    if (st != NB_OK) return st;
    NB_REQUIRE(p_out && !a->fp4);
    if (a->M == 0) return NB_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const char* reason;
    const Kernel k = choose_kernel(a, nullptr, NB_EPI_STORE, &reason);
    if (k == K_GENERIC && a->impl != NB_IMPL_AUTO && a->impl != NB_IMPL_GENERIC) return NB_ERR_UNSUPPORTED;
    if (k == K_TC_SINGLE) return launch_tc(a, nullptr, NB_EPI_STORE, p_out, s);
    if (k == K_TC_PAIR) return launch_tc_pair(a, nullptr, NB_EPI_STORE, p_out, s);
    GenericParams p = to_generic(a);
    p.out = a->out;
    p.p_out = p_out;
    return launch_generic(p, a->dtype, s);
}

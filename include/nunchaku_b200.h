/*
 * C ABI of libnunchaku_b200.so: hand-written sm_100a kernels for the SVDQuant hot path
 * (W4A4 GEMM + low-rank branch + fused epilogues, activation quantizer, AWQ W4A16, attention).
 *
 * Every entry point takes plain device pointers, sizes and strides (strides in ELEMENTS of the
 * tensor they index unless a field says bytes), launches on the given CUDA stream of the
 * CURRENT device and returns an nb_status.  Nothing here synchronises the device or throws.
 * All tensors use the reference's natural layouts (nunchaku/ops/triton/gemm_w4a4.py:4-19):
 * packed 4-bit rows are (rows, K/2) bytes with element k in the low nibble of byte k/2 when k is
 * even; scales are group-major (K/G, rows).
 *
 * Each declaration names the reference interface it replaces (paths inside the nunchaku-rocm
 * project).
 */
#ifndef NUNCHAKU_B200_H
#define NUNCHAKU_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum nb_status {
    NB_OK = 0,
    NB_ERR_INVALID = 1,     /* argument contract violated (shape, alignment, null pointer) */
    NB_ERR_UNSUPPORTED = 2, /* valid call that no kernel here implements */
    NB_ERR_LAUNCH = 3,      /* CUDA reported an error at launch; nb_last_cuda_error() has the code */
    NB_ERR_DEVICE = 4,      /* a kernel gave up on a bounded wait and set its status word */
    NB_ERR_TOO_LARGE = 5    /* size beyond the limit of a fixed-capacity entry point */
} nb_status;

enum { NB_DTYPE_BF16 = 0, NB_DTYPE_FP16 = 1 };

/* epilogue selector of nb_gemm_w4a4 */
enum {
    NB_EPI_STORE = 0,       /* 16-bit store of the fp32 tile                                  */
    NB_EPI_QK_NORM_ROPE = 1,/* + per-head RMSNorm and RoPE on the Q and K thirds              */
    NB_EPI_GELU_QUANT = 2,  /* + GELU, next-layer LoRA-down, unsigned int4 re-quantisation    */
    NB_EPI_SWIGLU_QUANT = 3 /* + silu(gate)*up on interleaved rows, signed int4 re-quantisation */
};

/* kernel selector (nb_gemm_args.impl) */
enum {
    NB_IMPL_AUTO = 0,    /* a tcgen05 kernel when the call meets its alignment rules, else the generic kernel */
    NB_IMPL_TCGEN05 = 1, /* a tcgen05 kernel (chosen as under AUTO) or NB_ERR_UNSUPPORTED */
    NB_IMPL_GENERIC = 2, /* CUDA-core kernel that takes every shape the op accepts */
    NB_IMPL_TCGEN05_PAIR = 3,  /* int4: the CTA-pair kernel (256 x 256 tiles) or NB_ERR_UNSUPPORTED */
    NB_IMPL_TCGEN05_SINGLE = 4 /* int4: the single-CTA kernel (128 x 128 tiles) or NB_ERR_UNSUPPORTED */
};

/*
 * Mirrors `struct GemmArgs` of nunchaku/ops/triton/native/w4a4_gfx11.hip:69-82 (ctypes twin
 * `_GemmArgs`, nunchaku/ops/triton/native/w4a4.py:80-103) and adds what the Triton entry
 * `gemm_w4a4` takes beyond it (nunchaku/ops/triton/gemm_w4a4.py:1003-1027): wcscales, alpha,
 * fp4, fuse_silu.
 */
typedef struct nb_gemm_args {
    const void* act;      /* (M, K/2) u8                                                     */
    const void* wgt;      /* (N, K/2) u8                                                     */
    void* out;            /* (actual_m, N) T, may be null when the epilogue writes no 16-bit tile */
    const void* ascales;  /* (K/G, >=M) T, or e4m3 when fp4                                   */
    const void* wscales;  /* (K/G, >=N) T, or e4m3 when fp4                                   */
    const void* bias;     /* (N) T or null                                                   */
    const void* lora_act; /* (>=M, R) f32 or null                                            */
    const void* lora_up;  /* (>=N, R) T or null                                              */
    const void* wcscales; /* (N) T or null (NVFP4 per-channel scale)                         */
    int32_t M, N, K;      /* rows of act, rows of wgt, logical K                             */
    int32_t actual_m;     /* rows of out (<= M); rows >= actual_m are computed but not stored */
    int32_t R;            /* LoRA-up rank, multiple of 16, 0 = none                          */
    int32_t dtype;        /* NB_DTYPE_*: T                                                   */
    int32_t act_unsigned; /* activations are 0..15 instead of -8..7 (int4 only)              */
    int32_t fp4;          /* nibbles are e2m1, G = 16, scales e4m3                            */
    int32_t fuse_silu;
    int32_t impl;         /* NB_IMPL_*                                                       */
    float alpha;          /* NVFP4 per-tensor scale                                          */
    int64_t stride_am, stride_wn;   /* row strides of act / wgt in BYTES                      */
    int64_t stride_asg, stride_wsg; /* group strides of ascales / wscales                     */
    int64_t stride_om, stride_lam, stride_lun;
    void* status;         /* device int32 the kernel sets non-zero if a bounded wait expires; may be null */
    void* scratch;        /* device scratch, see nb_gemm_w4a4_scratch_bytes(); may be null when that is 0 */
    int64_t scratch_bytes;
    const void* wgt_prepared;     /* optional: what nb_gemm_w4a4_prepare_weights wrote for this wgt / wscales, or null */
    int64_t wgt_prepared_bytes;
} nb_gemm_args;

/* Mirrors `QKNormRopeEpilogue::Args` (w4a4_gfx11.hip:440-446; ctypes `_QKArgs`, w4a4.py:106-115). */
typedef struct nb_qk_args {
    const void* norm_q;   /* (128) T */
    const void* norm_k;   /* (128) T */
    const float* rot;     /* (rot_rows, 128) f32: (sin, cos) per channel pair */
    int64_t stride_rm;
    int32_t rot_rows;     /* actual_m, or a divisor S of it: row m then reads rot[m % S] (one table for a batch) */
    float eps;
} nb_qk_args;

/* Mirrors `QuantArgs` (w4a4_gfx11.hip:585-594; ctypes `_GQArgs`, w4a4.py:118-124). */
typedef struct nb_requant_args {
    void* qout;            /* (>=M, Nq/2) u8, Nq = N (GELU) or N/2 (SwiGLU)                  */
    void* oscales;         /* (Nq/64, >=M) T                                                 */
    const void* smooth;    /* (Nq) T or null                                                 */
    const void* lora_down; /* (Nq, R2) T or null                                             */
    float* lora_act_out;   /* (>=M, R2) f32 or null                                          */
    int32_t R2;
    float shift;           /* 0.171875 for the GELU path                                     */
    int64_t stride_qm, stride_osg, stride_ld, stride_lom;
} nb_requant_args;

/*
 * W4A4 GEMM.  Replaces `gemm_w4a4` (nunchaku/ops/triton/gemm_w4a4.py:1003-1314) and the native
 * launchers `try_gemm` / `try_gemm_qk` / `try_gemm_gelu_quant` / `try_gemm_swiglu_quant`
 * (nunchaku/ops/triton/native/w4a4.py:969-1060).  `epi` points at nb_qk_args (NB_EPI_QK_NORM_ROPE),
 * nb_requant_args (NB_EPI_GELU_QUANT, NB_EPI_SWIGLU_QUANT) or is null.
 */
int nb_gemm_w4a4(const nb_gemm_args* args, const void* epi, int epi_kind, void* stream);

/*
 * Bytes of device scratch nb_gemm_w4a4 needs for this call: the tensor-core kernel keeps its operand form there (one
 * e4m3 byte per int4 value, the scale rows in the order its drain reads them, lora_act rounded to T), the generic
 * kernel the fp32 tile of a fused row epilogue.
 * The buffer must be 256-byte aligned; its contents are dead when the call's kernels have run.
 */
int64_t nb_gemm_w4a4_scratch_bytes(const nb_gemm_args* args, const void* epi, int epi_kind);

/*
 * Load-time half of the tensor-core paths.  The weights of a layer do not change between calls, so the form the
 * kernel reads (int4: one e4m3 byte per value and the column scales in the drain's order; NVFP4, `fp4` set: the block
 * scales in the chunk layout of the block-scaled MMA, the codes are used as they are) can be written once instead of by
 * every call's pre-pass: the role of the reference's load-time weight packing (`NunchakuWeightPacker`,
 * nunchaku/lora/flux/packer.py:165-517) for its MMA layout.  `args` needs wgt, wscales, N, K, dtype, fp4 and the two
 * strides.  nb_gemm_w4a4_prepared_bytes returns the size of the buffer (0: this weight cannot use a tensor-core kernel,
 * e.g. K % 64 != 0); nb_gemm_w4a4_prepare_weights fills it (256-byte aligned) on `stream`.  A later nb_gemm_w4a4 call
 * with the same wgt / wscales / N / K / dtype may pass it as `wgt_prepared`; it then needs less scratch (ask
 * nb_gemm_w4a4_scratch_bytes with the field set) and skips that part of the pre-pass.  The generic kernel ignores it.
 * The caller must drop the buffer when it changes the weights.
 */
int64_t nb_gemm_w4a4_prepared_bytes(const nb_gemm_args* args);
int nb_gemm_w4a4_prepare_weights(const nb_gemm_args* args, void* dst, int64_t dst_bytes, void* stream);

/* 1 when nb_gemm_w4a4 would run this call on the tcgen05 kernel, 0 when on the generic kernel. */
int64_t nb_gemm_w4a4_uses_tcgen05(const nb_gemm_args* args, const void* epi, int epi_kind);

/*
 * nb_gemm_w4a4 for callers that cannot provide scratch memory.  NO COUNTERPART IN THE REFERENCE: its operators
 * allocate through torch whenever they need to.  Same arguments, kernels and results as nb_gemm_w4a4; `scratch` and
 * `scratch_bytes` of the argument block are ignored and the scratch block lives in a fixed array of
 * NB_NOALLOC_SCRATCH_BYTES inside the library's device module.  The call allocates and frees nothing, on the device
 * or the host.  Meant for hosts that own all device memory themselves and expose no allocator to a plugin (a serving
 * runtime that has carved up the whole HBM in advance, a foreign-language host that only holds raw input and output
 * pointers), and for call sites where an allocation is not allowed or may fail late (inside a latency-critical
 * region where a device allocation would synchronise the device, under memory pressure).
 *   - Limit: a call whose nb_gemm_w4a4_scratch_bytes() exceeds NB_NOALLOC_SCRATCH_BYTES returns NB_ERR_TOO_LARGE and
 *     launches nothing (for the tensor-core kernel the need is about (M + N) * K bytes plus the converted scales).
 *   - First call on a device: the address of the array is looked up once (cudaGetSymbolAddress, which may load the
 *     module).  Make that first call during set-up, outside any stream capture; later calls only launch kernels.
 *     The address is remembered per device for the primary context it was looked up in: a process that destroys
 *     that context (cudaDeviceReset) must not call this entry point on the device again.
 *   - The array is shared by every caller on the device: two calls that can overlap in time (different streams or
 *     threads without ordering between them) race on it.  Order such calls on one stream or with events.
 *   - Nothing in the array has to start at zero and nothing is cleared: each call's first kernel writes every byte its
 *     later kernels read.
 */
#define NB_NOALLOC_SCRATCH_BYTES (16 << 20)
int nb_gemm_w4a4_noalloc(const nb_gemm_args* args, const void* epi, int epi_kind, void* stream);

/*
 * Debug: the exact int32 group sums p_g[m, n] = sum_{k in g} a[m,k] * w[n,k] as the tensor-core
 * kernel accumulates them, (K/64, M, N) int32.  The reference's integer contract
 * (nunchaku/ops/triton/gemm_w4a4.py:477-483) is checked against this.
 */
int nb_gemm_w4a4_group_sums(const nb_gemm_args* args, int32_t* p_out, void* stream);

/*
 * Activation quantizer with fused LoRA-down.  Replaces `quantize_w4a4_act_fuse_lora` /
 * `_launch_quantize` (nunchaku/ops/triton/gemm_w4a4.py:1465-1565).
 */
typedef struct nb_quant_args {
    const void* input;     /* (M, K) T, or (M, 2K) when fuse_glu                            */
    void* output;          /* (>=M, K/2) u8                                                 */
    void* oscales;         /* (K/G, >=M) T, e4m3 when fp4                                   */
    const void* lora_down; /* (K, R) T or null                                              */
    float* lora_act_out;   /* (>=M, R) f32 or null                                          */
    const void* smooth;    /* (K) T or null                                                 */
    int32_t M, K, R;
    int32_t dtype;
    int32_t fuse_glu, fuse_gelu, fp4, is_unsigned;
    float shift;
    int64_t stride_im, stride_om, stride_sg, stride_ld, stride_lam;
} nb_quant_args;
int nb_quantize_w4a4(const nb_quant_args* args, void* stream);

/*
 * Unfused per-head RMSNorm + RoPE on the Q/K thirds of a stored (M, N) tile, in place.
 * Replaces `_apply_rmsnorm_rope_qk` (nunchaku/ops/triton/gemm_w4a4.py:834-866).
 */
int nb_qk_norm_rope(void* out, int32_t M, int32_t N, int64_t stride_om, int32_t dtype, const nb_qk_args* qk,
                    void* stream);

/*
 * AWQ W4A16.  `nb_awq_gemv` replaces `awq_gemv_w4a16` (nunchaku/ops/triton/awq.py:186-229) for
 * group 64; `nb_awq_dequant` replaces `awq_dequantize` (awq.py:83-118); `nb_awq_gemm` replaces
 * `awq_gemm_w4a16` (awq.py:232-251: dequantise, then a dense matmul) with one kernel that widens the
 * weight tile in shared memory (k % 64 == 0, group % 32 == 0, rows of x 16-byte aligned).  `kernel` is
 * the TinyChat int16 (n/4, k) packing (awq.py:8-18).
 */
int nb_awq_gemv(const void* x, const void* kernel, const void* scales, const void* zeros, void* out, int32_t m,
                int32_t n, int32_t k, int64_t stride_xm, int64_t stride_kn, int64_t stride_sg, int64_t stride_om,
                int32_t dtype, void* stream);
int nb_awq_dequant(const void* kernel, const void* scales, const void* zeros, void* out, int32_t n, int32_t k,
                   int32_t group, int64_t stride_kn, int64_t stride_sg, int64_t stride_on, int32_t dtype,
                   void* stream);
int nb_awq_gemm(const void* x, const void* kernel, const void* scales, const void* zeros, void* out, int32_t m,
                int32_t n, int32_t k, int32_t group, int64_t stride_xm, int64_t stride_kn, int64_t stride_sg,
                int64_t stride_om, int32_t dtype, void* stream);

/*
 * The element-wise steps around the quantised linears of a DiT block, one pass over HBM each, rounded to the 16-bit
 * dtype at the points where the reference's operator sequence rounds.  The reference runs them as torch operators (LayerNorm, broadcast multiply, broadcast add):
 * AdaLayerNormZero (nunchaku/models/normalization.py:60-159) and the gated residuals of the blocks
 * (nunchaku/models/transformers/transformer_flux_v2.py:174-343).
 *   nb_layernorm_modulate: out[r] = LayerNorm(x[r]) * (scale[b] + scale_add) + shift[b], b = r / rows_per_batch;
 *                          dim in {1024, 2048, 3072, 4096} (else NB_ERR_UNSUPPORTED)
 *   nb_gated_residual:     out[r] = x[r] + gate[b] * (y[r] + y2[r])   (y2 may be null)
 * Row strides in elements; scale / shift / gate are (batch, dim) views: `stride_*b` elements between batches,
 * `stride_*d` between channels (they are columns of the modulation linear's interleaved output).
 */
int nb_layernorm_modulate(const void* x, const void* scale, const void* shift, void* out, int32_t rows,
                          int32_t rows_per_batch, int32_t dim, int64_t stride_xr, int64_t stride_or, int64_t stride_sb,
                          int64_t stride_sd, float scale_add, float eps, int32_t dtype, void* stream);
int nb_gated_residual(const void* x, const void* gate, const void* y, const void* y2, void* out, int32_t rows,
                      int32_t rows_per_batch, int32_t dim, int64_t stride_xr, int64_t stride_yr, int64_t stride_y2r,
                      int64_t stride_or, int64_t stride_gb, int64_t stride_gd, int32_t dtype, void* stream);

/*
 * Checkpoint layout converter for the 4-bit weight: the stored fragment order of a SVDQuant checkpoint
 * ((n, k/2) bytes viewed as int32 words) -> natural packed nibbles (n, k/2), even k in the low nibble.
 * Replaces `unpack_weight_packed_nibbles` (nunchaku/ops/triton/layout.py:36-118; inverse of
 * NunchakuWeightPacker.pack_weight, nunchaku/lora/flux/packer.py:187-239).  n, k multiples of 128;
 * `stride_on` = bytes between output rows.
 */
int nb_layout_unpack_weight(const void* stored, void* out, int32_t n, int32_t k, int64_t stride_on, void* stream);

/*
 * Unmasked flash attention, (B,H,T,D) strided inputs with unit last stride -> (B,Tq,H*D).
 * Replaces `attention_fp16` (nunchaku/ops/triton/attention.py:120-169).  D in {64, 128}.
 */
typedef struct nb_attn_args {
    const void* q; const void* k; const void* v; void* o;
    int32_t B, H, Tq, Tkv, D, dtype;
    float scale;  /* softmax scale before the log2(e) fold */
    int64_t stride_qb, stride_qh, stride_qm;
    int64_t stride_kb, stride_kh, stride_kn;
    int64_t stride_vb, stride_vh, stride_vn;
    int64_t stride_ob, stride_om;
    void* scratch;         /* device scratch of nb_attention_scratch_bytes() bytes, 256-byte aligned; may be null when that is 0 */
    int64_t scratch_bytes;
    void* status;          /* device int32 a kernel sets non-zero if a bounded wait expires; may be null */
    int32_t impl;          /* NB_IMPL_AUTO: tcgen05 kernel for D = 128, else the mma.sync kernel; NB_IMPL_GENERIC: mma.sync */
} nb_attn_args;
int nb_attention(const nb_attn_args* args, void* stream);
/* Scratch the call needs: 0 for both kernels at present (Q, K and V are read in place from the caller's views); callers still
 * ask, so that a kernel that needs some can be added without touching them. */
int64_t nb_attention_scratch_bytes(const nb_attn_args* args);

/*
 * Self-test on the current device, the role of the reference's native self-test (nunchaku/ops/triton/native/w4a4.py:537-651):
 * a small seeded W4A4 problem with bias and a rank-16 branch runs on the tensor-core kernel and on the generic kernel;
 * the exact integer group sums must be equal and the 16-bit outputs must agree to two rounding steps; the same call with
 * load-time prepared weights must reproduce the tensor-core output bit for bit; an NVFP4 problem (wide tile, per-channel
 * scales, alpha, rank 16) must agree between the block-scaled and the generic kernel.  Allocates and frees its own few MB
 * of device memory and synchronises the device.  Returns NB_OK, or NB_ERR_DEVICE on a mismatch.
 */
int nb_selftest(void);

/*
 * Failure-path check: launches one warp that waits, with the kernels' own bounded wait, on a barrier nothing arrives
 * on.  After `limit_us` microseconds (1 .. 1,000,000) the wait gives up and the kernel stores a non-zero code in the
 * device int32 `status`, as the GEMM and attention kernels do when a wait of theirs expires; the context stays usable.
 * The reference surfaces runtime failures of its native module as exceptions (nunchaku/ops/triton/native/hip.py:110-116);
 * this is the hook that lets a host test that plumbing without faulting or hanging a GPU.
 */
int nb_debug_expire_wait(void* status, int64_t limit_us, void* stream);

/*
 * Diagnostics, the role of the reference's `native.status()` (nunchaku/ops/triton/native/w4a4.py:802-810): resource
 * figures of the CTA-pair GEMM kernel on the current device, ten ints: registers per thread, max threads per block,
 * static shared bytes, resident CTA pairs the occupancy query reports, that query's cudaError_t, dynamic shared bytes
 * requested, threads per block, resident CTAs per SM without clusters, that query's cudaError_t, local-memory bytes.
 */
int nb_debug_pair_kernel_info(int* out10);

/* Diagnostics (the reference's `status()` / error plumbing, nunchaku/ops/triton/native/hip.py:110-116). */
const char* nb_strerror(int status);
int nb_last_cuda_error(void);          /* cudaError_t of the last NB_ERR_LAUNCH, cleared by reading */
const char* nb_last_cuda_error_string(void);
const char* nb_last_error_detail(void); /* which check of the launcher refused the last failed call of this thread ("" if none), cleared by reading */
int nb_version(void);
int nb_num_sms(void);                  /* SM count of the current device, <= 0 on error */

#ifdef __cplusplus
}
#endif
#endif /* NUNCHAKU_B200_H */

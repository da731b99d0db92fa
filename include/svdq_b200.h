/*
 * svdq_b200 - C ABI of the B200 (sm_100a) SVDQuant W4A4 linear hot path.
 *
 * Plain C: raw device pointers, sizes and flags; no C++ or torch types.  Every
 * entry point returns 0 on success or a negative SVDQ_ERR_* code, never throws,
 * aborts or traps; svdq_last_error_string() gives the reason (thread local).
 * Launches are asynchronous on the given stream (a cudaStream_t passed as
 * void*), on the current CUDA device.  The library calls no allocator: all
 * buffers, including scratch, are caller owned.  The one exception is the fixed
 * SVDQ_STATIC_SCRATCH_BYTES array that svdq_gemm_w4a4_static_scratch() uses, which
 * is part of the library image on every GPU that loads it.
 * The first call of any entry point on a device looks up a few per-device facts
 * (SM count, addresses of the library's device symbols) and caches them: make one
 * ordinary call per device before starting a stream capture.  Device ordinals up
 * to 63 are supported.
 *
 * The two compute entry points replace the reference's
 *   nunchaku::ops::quantize_w4a4_act_fuse_lora   (nunchaku/csrc/ops.h:82-110,
 *       src/kernels/zgemm/zgemm.h:36-43, gemm_w4a4.cu:113-125) and
 *   nunchaku::ops::gemm_w4a4                     (nunchaku/csrc/ops.h:10-80,
 *       src/kernels/zgemm/zgemm.h:8-34, gemm_w4a4.cu:34-105).
 */
#ifndef SVDQ_B200_H
#define SVDQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SVDQ_OK 0
#define SVDQ_ERR_INVALID_ARGUMENT (-1) /* null / misaligned pointer, bad shape          */
#define SVDQ_ERR_UNSUPPORTED (-2)      /* valid in the reference, not built here (yet)   */
#define SVDQ_ERR_UNSUPPORTED_ARCH (-3) /* current device is not compute capability 10.x  */
#define SVDQ_ERR_CUDA (-4)             /* a CUDA runtime / driver call failed            */
#define SVDQ_ERR_TIMEOUT (-5)          /* a bounded device-side wait ran out (see status) */

/* Memory order of the activation-side tensors (codes, scales, low-rank activations). */
#define SVDQ_LAYOUT_NATIVE 0    /* row-major codes, 512-byte scale atoms, row-major fp32 low-rank */
#define SVDQ_LAYOUT_REFERENCE 1 /* the reference's mma.sync fragment order (gemm_base.cuh:265-340) */

/* Largest LoRA rank of any low-rank tensor (src/kernels/zgemm/lora.cuh:22); ranks are multiples of 16. */
#define SVDQ_MAX_LORA_RANK 1024

/* The 16-bit floating-point type of activations, smoothing factors, LoRA weights, biases, INT4 group scales and
 * outputs ("bf16" in the comments below): the reference's GEMMConfig_W4A4_BF16 / _FP16 (gemm_w4a4.cu:17-31).   */
#define SVDQ_DTYPE_BF16 0
#define SVDQ_DTYPE_FP16 1

#define SVDQ_ACT_NONE 0
#define SVDQ_ACT_SILU 1 /* fuse_silu  (gemm_w4a4_launch_impl.cuh:407-420) */
#define SVDQ_ACT_GELU 2 /* GELU before next-layer requantisation (launch_impl.cuh:282-309) */

/*
 * Activation quantiser fused with the LoRA down projection.
 * Replaces kernels::quantize_w4a4_act_fuse_lora (zgemm.h:36-43;
 * GEMM_W4A4_Launch::quantize_w4a4_act_fuse_lora, gemm_w4a4_launch_impl.cuh:451-521).
 * `smooth` and `lora_down` are taken in the reference's packed order, exactly as
 * stored in SVDQW4A4Linear.smooth_factor / .proj_down (nunchaku/models/linear.py:56-64).
 */
typedef struct svdq_quantize_args {
    const void* input;     /* bf16 [M, K] row-major ([M, 2K] when fuse_glu)                   */
    void* codes;           /* uint8 [M_pad, K/2]                                              */
    void* scales;          /* NVFP4: e4m3 bytes [K/16, M_pad]; INT4: bf16 [K/64, M_pad]      */
    float* lora_act;       /* fp32 [M_pad, R]; fully written, no zero-fill needed             */
    const void* smooth;    /* bf16 [K], reference-packed                                      */
    const void* lora_down; /* bf16 [K, R], reference-packed                                   */
    int32_t M;             /* valid rows                                                      */
    int32_t M_pad;         /* multiple of 256 (nunchaku/ops/quantize.py:40)                   */
    int32_t K;             /* multiple of 128                                                 */
    int32_t R;             /* multiple of 16, 16..SVDQ_MAX_LORA_RANK (above 128: extra passes)   */
    int32_t fp4;           /* 1: NVFP4 group 16, 0: INT4 group 64                             */
    int32_t fuse_glu;      /* 1: input holds (value, gate) pairs, quantise value*silu(gate)   */
    int32_t layout;        /* SVDQ_LAYOUT_* of codes / scales / lora_act                      */
    int32_t K_in;          /* 0, or the input's real channel count when K is its padding to 128:
                              the input is [M, K_in] ([M, 2 K_in] when fuse_glu), columns [K_in, K) read as
                              zero (the reference's in_features / in_features_pad, src/Linear.cpp:92,452);
                              K - 128 < K_in <= K, multiple of 8                                  */
    int32_t dtype;         /* SVDQ_DTYPE_* of input, smooth, lora_down and the INT4 scales        */
} svdq_quantize_args;

int svdq_quantize_w4a4_act_fuse_lora(const svdq_quantize_args* args, void* stream);

/*
 * One-time re-tiling of a layer's weights from the reference's packed order
 * (NunchakuWeightPacker, nunchaku/lora/flux/packer.py:187-398) into the order
 * the sm_100a GEMM streams with TMA.  Replaces nothing in the reference (its
 * kernels read the packed order directly); it is what lets the checkpoint
 * format stay byte-identical.  Output buffers are caller allocated with the
 * sizes svdq_w4a4_prepared_bytes() reports.
 */
typedef struct svdq_prepared_weights {
    void* wgt;        /* NVFP4: uint8 [N, K/2] row-major codes; INT4: fp16 [N, K] = code * group scale * 2^-e[n]
                         (2 bytes per weight; within each 16-byte chunk the k order is 0,4,1,5,2,6,3,7)      */
    void* wscales;    /* NVFP4: 512-byte e4m3 atoms [N/128][K/64]; INT4: bf16 [K/64, N] (kept for inspection,
                         the GEMM does not read it: the scales are folded into wgt)                          */
    float* lora_up;   /* fp32 [N, R32] (R32 = R rounded up to 32), pre-divided by col_scale */
    float* col_scale; /* fp32 [N] = alpha * wcscales                                       */
    float* col_bias;  /* fp32 [N]                                                          */
} svdq_prepared_weights;

typedef struct svdq_weights_args {
    const void* qweight;  /* int8 [N, K/2], reference-packed (SVDQW4A4Linear.qweight)       */
    const void* wscales;  /* reference-packed: e4m3 [K/16, N] or bf16 [K/64, N]             */
    const void* lora_up;  /* bf16 [N, R] reference-packed, may be NULL when R == 0          */
    const void* bias;     /* bf16 [N] reference-packed, may be NULL                         */
    const void* wcscales; /* bf16 [N] reference-packed, may be NULL (NVFP4 only)            */
    const float* lora_scales; /* host array, one per 16 ranks, may be NULL (all 1.0)        */
    float alpha;          /* NVFP4 per-tensor weight scale (wtscale); must be 1 for INT4    */
    int32_t N, K, R, fp4;
    int32_t dtype;        /* SVDQ_DTYPE_* of wscales (INT4), lora_up, bias, wcscales        */
} svdq_weights_args;

/* bytes[0..4] = sizes of wgt, wscales, lora_up, col_scale, col_bias */
int svdq_w4a4_prepared_bytes(int32_t N, int32_t K, int32_t R, int32_t fp4, size_t bytes[5]);
int svdq_w4a4_prepare_weights(const svdq_weights_args* args, const svdq_prepared_weights* out, void* stream);

/*
 * 4-bit GEMM with the fused epilogue
 *   acc*alpha*wcscale + bias -> + lora_act_in @ lora_up^T -> [SiLU|GELU] ->
 *   { store bf16 `out` } and/or { next layer: LoRA-down, (+shift)/smooth, group-quantise }.
 * Replaces kernels::gemm_w4a4 (zgemm.h:8-34; GEMM_W4A4_Launch::gemm_w4a4,
 * gemm_w4a4_launch_impl.cuh:7-424).
 */
typedef struct svdq_gemm_args {
    const void* act;          /* uint8 [M_pad, K/2]                                          */
    const void* ascales;      /* e4m3 [K/16, M_pad] or bf16 [K/64, M_pad]                    */
    const float* lora_act_in; /* fp32 [M_pad, R] or NULL                                     */
    svdq_prepared_weights w;  /* from svdq_w4a4_prepare_weights                              */
    void* out;                /* bf16 [M, N] or NULL                                         */
    /* next-layer requantisation (all NULL when unused) */
    void* qout;               /* uint8 [M_pad, N/2]                                          */
    void* oscales;            /* e4m3 [N/16, M_pad] or bf16 [N/64, M_pad]                    */
    float* lora_act_out;      /* fp32 [M_pad, R_next]                                        */
    const void* next_smooth;    /* bf16 [N] reference-packed                                 */
    const void* next_lora_down; /* bf16 [N, R_next] reference-packed                         */
    void* workspace;          /* scratch, svdq_gemm_w4a4_workspace_bytes() bytes, 256-aligned: needed by the
                                 requantising epilogue (per-CTA LoRA-down partials) and by every INT4 GEMM
                                 (per-row power-of-two normalisation of the activation scales); else may be NULL */
    size_t workspace_bytes;
    int32_t M, M_pad, N, K, R, R_next; /* R, R_next: multiples of 16 up to SVDQ_MAX_LORA_RANK.  The epilogue computes the
                                 first 64 (32, 16) ranks of the next layer's LoRA-down itself; further ranks are follow-up
                                 launches over the bf16 output (`out`, or a copy of it in the workspace)        */
    int32_t fp4;              /* precision of act / weights                                  */
    int32_t act_unsigned;     /* INT4 only: activations are u4 codes                         */
    int32_t activation;       /* SVDQ_ACT_*; must be SVDQ_ACT_GELU when qout is given        */
    int32_t act_layout;       /* layout of act / ascales / lora_act_in                       */
    int32_t out_layout;       /* layout of qout / oscales / lora_act_out                     */
    int32_t next_fp4;         /* precision of the requantised output                         */
    int32_t N_out;            /* 0, or the real column count of `out` when N is its padding to 128: out is
                                 [M, N_out] and columns [N_out, N) are dropped (the reference's actualN,
                                 gemm_base.cuh:544-548); N - 128 < N_out <= N, multiple of 8      */
    int32_t dtype;            /* SVDQ_DTYPE_* of out, ascales / oscales (INT4), next_smooth, next_lora_down;
                                 the prepared weights do not depend on it beyond what prepare_weights read   */
    /* RMSNorm + rotary embedding of a fused QKV projection inside the epilogue (EpilogueRMSNormRope, epilogues.cuh:269-425):
       set rope_cos to ask for it (NVFP4, no activation, N = 3 * rope_heads * 128 with rope_heads even, M a multiple of
       rope_seq_len, rope_seq_len a multiple of 32; otherwise SVDQ_ERR_UNSUPPORTED: run svdq_gemm_w4a4 and svdq_qk_norm_rope).
       q and k heads are normalised and rotated, v passes through.  The result goes to `out` [M, N], or, when rope_out_q is
       set, to three token-major tensors [M / rope_seq_len, rope_tokens_pad, rope_heads * 128] from token rope_token_offset on
       (rows at or beyond rope_attn_tokens, when > 0, become zeros).                                                      */
    const void* rope_norm_q;  /* bf16 [128]                                                   */
    const void* rope_norm_k;
    const float* rope_cos;    /* fp32 [rope_seq_len, 64]                                      */
    const float* rope_sin;
    void* rope_out_q;
    void* rope_out_k;
    void* rope_out_v;
    float rope_eps;
    int32_t rope_seq_len, rope_heads, rope_tokens_pad, rope_token_offset, rope_attn_tokens;
} svdq_gemm_args;

int svdq_gemm_w4a4_workspace_bytes(const svdq_gemm_args* args, size_t* bytes);
int svdq_gemm_w4a4(const svdq_gemm_args* args, void* stream);

/*
 * The same GEMM for callers that cannot supply `workspace`: a host that divided up its device memory at
 * start-up and has no allocator to call per request, or one that may not make allocation calls once it is
 * serving.  The scratch the requantising epilogue needs (per-CTA partial sums of the next layer's LoRA-down)
 * then comes from an array inside the library: SVDQ_STATIC_SCRATCH_BYTES (8 MiB) of device memory on every GPU
 * that loads the library, kept until the process ends.  args->workspace / workspace_bytes are ignored; inputs
 * and outputs are still the caller's.  No counterpart in the reference, which allocates nothing in this op
 * because its LoRA-down uses atomics.
 *   - Limit: problems that need more than SVDQ_STATIC_SCRATCH_BYTES (see svdq_gemm_w4a4_workspace_bytes) are
 *     refused with SVDQ_ERR_INVALID_ARGUMENT.  Both precisions.
 *   - The first call on each device looks up the array's device address; make that call before starting any
 *     stream capture.  The address is cached per device and is stale after a cudaDeviceReset.
 *   - All calls share the array: do not let two of them run on the same GPU at the same time.
 */
#define SVDQ_STATIC_SCRATCH_BYTES (8u << 20)
int svdq_gemm_w4a4_static_scratch(const svdq_gemm_args* args, void* stream);

/*
 * Activation-side layout conversion (codes, scales, low-rank activations) between
 * SVDQ_LAYOUT_REFERENCE and SVDQ_LAYOUT_NATIVE; no counterpart in the reference,
 * where only one order exists.  NULL pairs are skipped.
 */
typedef struct svdq_relayout_args {
    const void* codes_in;  void* codes_out;   /* uint8 [M_pad, K/2]   */
    const void* scales_in; void* scales_out;  /* see svdq_quantize_args */
    const float* lora_in;  float* lora_out;   /* fp32 [M_pad, R]      */
    int32_t M_pad, K, R, fp4;
    int32_t from_layout, to_layout;
} svdq_relayout_args;
int svdq_w4a4_relayout_act(const svdq_relayout_args* args, void* stream);

/*
 * RMSNorm of q and k per head + rotary embedding, in place on the 16-bit output of a fused QKV projection
 * [rows, 3 * heads * 128] (Q third, K third; V untouched).  What the reference does inside the QKV GEMM's
 * epilogue: EpilogueRMSNormRope, src/kernels/zgemm/epilogues.cuh:269-425, called from
 * nunchaku/ops/fused.py:50-110 (fused_qkv_norm_rottary); same arithmetic (fp32, one rounding), but the rotary table
 * is either two plain fp32 arrays [seq_len, 64] (cos, sin; row = token position, repeated over batches of seq_len rows)
 * or the reference's fragment-packed [1, M, 128] tensor (rotary_packed below).
 */
typedef struct svdq_norm_rope_args {
    void* qkv;                /* bf16 / fp16 (`dtype`) [rows, 3 * heads * 128], modified in place */
    const void* weight_q;     /* [128], qkv's type */
    const void* weight_k;     /* [128], qkv's type */
    const float* cos;         /* fp32 [seq_len, 64] */
    const float* sin;         /* fp32 [seq_len, 64] */
    int64_t rows;
    int32_t seq_len, heads;
    float eps;                /* 1e-6 in the reference */
    /* Optional (all NULL / 0 for the plain in-place form):
     * rotary_packed - the reference's own rotary tensor instead of cos / sin: fp32 [seq_len, 128] in the fragment
     *   order pack_rotemb produces (nunchaku/models/embeddings.py:88-120; seq_len a multiple of 16);
     * out_q / out_k / out_v - write the three thirds head-major, [rows / seq_len, heads, tokens_pad, 128] of qkv's type, instead
     *   of in place (the job of EpiloguePackQKV, epilogues.cuh:427-550; there the destination is the fragment order of
     *   the reference's own fp16 attention kernel with NaN-masked K padding, here it is plain row-major for a
     *   TMA / library attention, and rows at or beyond attn_tokens, when attn_tokens > 0, are written as zeros).
     *   token_offset shifts the destination rows (two streams of a joint block writing one buffer); token_major = 1
     *   selects [rows / seq_len, tokens_pad, heads, 128] instead (what flash-attention style kernels take). */
    const float* rotary_packed;
    void* out_q;
    void* out_k;
    void* out_v;
    int32_t tokens_pad, attn_tokens, token_offset, token_major;
    int32_t dtype;            /* SVDQ_DTYPE_* of qkv, the norm weights and out_q / out_k / out_v */
} svdq_norm_rope_args;
int svdq_qk_norm_rope(const svdq_norm_rope_args* args, void* stream);

/*
 * out = LayerNorm(x) * (1 + scale[b]) + shift[b]: no affine, fp32 statistics, 16-bit in / out, b = row / rows_per_batch.
 * The AdaLN-Zero step in front of each W4A4 projection of a FLUX block.  No counterpart on the reference's W4A4
 * path (its blocks call separate fused norm kernels, src/kernels/layernorm_kernels.cu); provided for the block harness.
 */
typedef struct svdq_ln_modulate_args {
    const void* x;            /* bf16 / fp16 (`dtype`) [rows, cols] */
    const void* scale;        /* [batches, mod_stride], first `cols` entries of a row are used */
    const void* shift;        /* same geometry */
    void* out;                /* [rows, cols] */
    int64_t rows, rows_per_batch, mod_stride;
    int32_t cols;             /* 256, 1024, 2240, 2304 or 3072 */
    float eps;                /* 1e-5 = torch.nn.functional.layer_norm default */
    int32_t dtype;            /* SVDQ_DTYPE_* of all four tensors */
} svdq_ln_modulate_args;
int svdq_layernorm_modulate(const svdq_ln_modulate_args* args, void* stream);

/*
 * Gated residual of a DiT block: out = x + gate[batch] * (y (+ z)), bf16 or fp16, one pass (x, y, z, out: [rows, cols]; gate
 * [batches, gate_stride] with its first `cols` entries used, or NULL for 1; out may be x).  Like svdq_layernorm_modulate
 * it has no counterpart in the reference's W4A4 path; provided for the block harness.
 */
typedef struct svdq_gate_residual_args {
    const void* x;
    const void* gate;         /* or NULL */
    const void* y;
    const void* z;            /* or NULL: a second addend inside the gate */
    void* out;
    int64_t rows, rows_per_batch, gate_stride;
    int32_t cols;             /* multiple of 8 */
    int32_t dtype;            /* SVDQ_DTYPE_* of all tensors */
} svdq_gate_residual_args;
int svdq_gate_residual(const svdq_gate_residual_args* args, void* stream);

/*
 * ReLU linear attention of SANA on the 16-bit output of the fused QKV projection: per (batch, head)
 * vk = [V | 1]^T relu(K) over the tokens (fp32), then out = (relu(Q) vk^T)[:32] / ((relu(Q) vk^T)[32] + eps).
 * What the reference does in the QKV GEMM's epilogue plus a second kernel: EpilogueLiteLA and vk_mul_q_kernel,
 * src/kernels/zgemm/epilogues.cuh:552-761, launched from gemm_w4a4_launch_impl.cuh:311-345,426-448 and called by
 * SanaLinearAttention::forward (src/SanaModel.cpp:25-106).  Column order of qkv as there: Q of all heads in [0, D),
 * then 64 columns [K_h | V_h] per head, D = heads * 32.  Deterministic (no atomics, nothing to zero).
 */
typedef struct svdq_litela_args {
    const void* qkv;          /* bf16 / fp16 (`dtype`) [batches, tokens, 3 * heads * 32] */
    void* out;                /* [batches, tokens, heads * 32], qkv's type */
    float* vk;                /* fp32 [batches, heads, 33, 32] or NULL: the reference's out_vk */
    int32_t batches, tokens, heads;
    float eps;                /* 1e-6 in the reference */
    int32_t mode;             /* 0: all of it.  The reference's two launches on their own: 1 = what EpilogueLiteLA leaves
                                 (vk, and relu(Q) in `out`; vk required); 2 = vk_mul_q_kernel (`out` holds
                                 relu(Q) and is finished in place from vk; qkv is not read and may be NULL)        */
    int32_t dtype;            /* SVDQ_DTYPE_* of qkv and out */
} svdq_litela_args;
int svdq_litela(const svdq_litela_args* args, void* stream);

/*
 * INT4 weight quantiser: a 16-bit weight [N, K] -> signed 4-bit codes with one 16-bit scale per row and group of 64, in the
 * packed layouts svdq_w4a4_prepare_weights reads (qweight as NunchakuWeightPacker.pack_weight lays it out, wscales as
 * pack_scale).  Replaces quantize_w4a4_wgt (src/kernels/zgemm/zgemm.h:48, gemm_w4a4.cu:132-136, kernel
 * gemm_w4a4.cuh:661-689), bit for bit: scale = max|w| / 7 and rscale = 7 / max|w| in the 16-bit type,
 * code = sat_s4(rint(rscale * w)) with the product rounded to 16 bits first.
 */
typedef struct svdq_quantize_wgt_args {
    const void* input;        /* bf16 / fp16 (`dtype`) [N, K] row-major */
    void* qweight;            /* int8 [N, K/2], reference-packed */
    void* wscales;            /* [K/64, N] of the input's type, reference-packed */
    int32_t N, K;             /* multiples of 128 and 64 */
    int32_t dtype;
} svdq_quantize_wgt_args;
int svdq_quantize_w4a4_wgt(const svdq_quantize_wgt_args* args, void* stream);

/*
 * Softmax attention forward, 128-wide heads: out = softmax(scale * Q K^T) V per (batch, head), fp32 accumulation, the
 * probabilities rounded to the 16-bit type before the second product.  Replaces attention_fp16
 * (src/kernels/zgemm/attention.cu:10-96, bound at nunchaku/csrc/pybind.cpp:111, called from
 * nunchaku/models/attention_processors/flux.py:167 and src/FluxModel.cpp:367,618,1063).  Every tensor is addressed as
 * element (b, h, t, c) at b*stride[0] + h*stride[1] + t*stride[2] + c (strides in elements, multiples of 8): the
 * reference's head-major [B, H, T, 128] inputs with its [B, T, H*128] output, or token-major buffers throughout.
 * Token counts need not be multiples of the tile: rows past q_len are not written, keys past kv_len are masked.
 */
typedef struct svdq_attention_args {
    const void* q;
    const void* k;
    const void* v;
    void* out;
    int64_t q_stride[3], k_stride[3], v_stride[3], o_stride[3];   /* batch, head, token */
    int32_t batch, heads, q_len, kv_len;
    int32_t head_dim;         /* 128 */
    float scale;              /* head_dim ** -0.5 in the reference's callers */
    int32_t dtype;            /* SVDQ_DTYPE_BF16 / SVDQ_DTYPE_FP16: q, k, v and out */
} svdq_attention_args;
int svdq_attention(const svdq_attention_args* args, void* stream);

/*
 * Device-side status word of the current device: 0, or the SVDQ_ERR_TIMEOUT code a
 * kernel recorded when one of its bounded waits ran out.  Synchronises the device.
 * `detail` (may be NULL) receives a kernel-specific location code.  Reading clears it.
 */
int svdq_device_status(int32_t* status, int32_t* detail);

const char* svdq_last_error_string(void);
int svdq_version(void);

#ifdef __cplusplus
}
#endif
#endif /* SVDQ_B200_H */

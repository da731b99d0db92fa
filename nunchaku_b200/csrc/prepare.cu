// Layout conversion kernels: reference fragment order <-> the order the sm_100a
// kernels stream.  All of them are word-granular permutations (HBM bound, run once
// per layer for weights), one thread per 32-bit word, fully coalesced on the
// reading side.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "host_common.h"

namespace svdq {

// the 16-bit type of the checkpoint's scales, biases and LoRA weights: bf16 or fp16 (svdq_weights_args.dtype)
__device__ __forceinline__ float tf(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float tf(__half v) { return __half2float(v); }

__device__ __forceinline__ int packed_vec_pos128(int n) {
    return (n & ~15) | (((n >> 1) & 3) << 2) | (((n >> 3) & 1) << 1) | (n & 1);
}

// 4-bit weight codes.  Reference (packer.py:187-239): [N/128][K/64][ntile 8][g 8][t 4][half 2][kh 2] words,
// word = 8 consecutive k of row bn*128 + nt*16 + half*8 + g starting at k = bk*64 + kh*32 + t*8.
// Native: row-major [N][K/2] bytes.
__global__ void retile_wgt_codes_kernel(const uint32_t* __restrict__ src, uint32_t* __restrict__ dst, int N, int K) {
    const size_t total = static_cast<size_t>(N) * K / 8;
    const int KB = K / 64;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        size_t r = i;
        const int kh = r & 1; r >>= 1;
        const int half = r & 1; r >>= 1;
        const int t = r & 3; r >>= 2;
        const int g = r & 7; r >>= 3;
        const int nt = r & 7; r >>= 3;
        const int bk = r % KB;
        const int bn = r / KB;
        const int n = bn * 128 + nt * 16 + half * 8 + g;
        const int k = bk * 64 + kh * 32 + t * 8;
        dst[(static_cast<size_t>(n) * K + k) / 8] = src[i];
    }
}

// INT4 weights.  sm_100 has no 4-bit integer MMA kind, and a kind::i8 GEMM would have to rescale every group of 64 k
// on the SIMT pipes.  Instead each code is multiplied by its group scale once, here, and stored as fp16:
//   w16[n][k'] = fp16( code[n][k] * wscale[n][k/64] / col_scale[n] ),   col_scale[n] = 2^floor(log2(max_g wscale[n][g]))
// code (4 bits) times a bf16 scale (8 bits) is exact in fp16 (11 bits) while the scaled scale is a normal fp16 number;
// the power-of-two column factor keeps the largest scale of a channel in [1, 2) so that only scales more than 2^14
// below it lose bits, and is applied again in the GEMM epilogue.  Within each block of 8 k the order is
// (0, 4, 1, 5, 2, 6, 3, 7): the order in which the GEMM's converter warps produce the activations of a packed word
// (a dot product does not care about the order as long as both operands agree).  Row-major [N][K].
template <typename T>
__global__ void int4_col_scale_kernel(const T* __restrict__ ws, float* __restrict__ col_scale, int N, int KB) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N) return;
    float mx = 0.f;
    for (int g = 0; g < KB; ++g) mx = fmaxf(mx, fabsf(tf(ws[static_cast<size_t>(g) * N + n])));
    int e = 0;
    if (mx > 0.f && mx < 3.0e38f) {
        (void)frexpf(mx, &e);   // mx = f * 2^e, f in [0.5, 1)
        e -= 1;
    }
    e = max(-100, min(100, e));
    col_scale[n] = ldexpf(1.0f, e);
}

template <typename T>
__global__ void retile_wgt_codes_f16_kernel(const uint32_t* __restrict__ src, const T* __restrict__ ws,
                                            const float* __restrict__ col_scale, uint4* __restrict__ dst, int N, int K) {
    const size_t total = static_cast<size_t>(N) * K / 8;
    const int KB = K / 64;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        size_t r = i;
        const int kh = r & 1; r >>= 1;
        const int half = r & 1; r >>= 1;
        const int t = r & 3; r >>= 2;
        const int g = r & 7; r >>= 3;
        const int nt = r & 7; r >>= 3;
        const int bk = r % KB;
        const int bn = r / KB;
        const int n = bn * 128 + nt * 16 + half * 8 + g;
        const int k = bk * 64 + kh * 32 + t * 8;
        const uint32_t w = src[i];
        const float s = tf(ws[static_cast<size_t>(bk) * N + n]) / col_scale[n];
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {   // output pair j = codes j and j + 4
            const int c0 = (static_cast<int>(w << (28 - 4 * j))) >> 28;          // sign-extended nibble j
            const int c1 = (static_cast<int>(w << (12 - 4 * j))) >> 28;          // nibble j + 4
            const __half2 h = __floats2half2_rn(static_cast<float>(c0) * s, static_cast<float>(c1) * s);
            o[j] = *reinterpret_cast<const uint32_t*>(&h);
        }
        dst[(static_cast<size_t>(n) * K + k) / 8] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// NVFP4 weight micro-scales.  Reference (packer.py:303-360): [N/128][K/64][d 8][c 4][s 4] words, word = the 4
// k-group bytes of row bn*128 + s*32 + c*8 + d.  Native: 512-byte atoms [N/128][K/64][r0 32][r1 4] words with
// row = r1*32 + r0.
__global__ void retile_wgt_mscales_kernel(const uint32_t* __restrict__ src, uint32_t* __restrict__ dst, int N, int K) {
    const size_t total = static_cast<size_t>(N) * K / 64;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int s = i & 3, c = (i >> 2) & 3, d = (i >> 4) & 7;
        const size_t atom = i >> 7;
        const int r0 = c * 8 + d;
        dst[atom * 128 + r0 * 4 + s] = src[i];
    }
}

// INT4 weight scales.  Reference (packer.py:241-301): [N/128][K/64][a 8][c 4][b 2][d 2] bf16,
// n = a*16 + b*8 + c*2 + d.  Native: bf16 [K/64][N] (the values are bf16 in the checkpoint; alpha is 1 for INT4).
__global__ void retile_wgt_scales_kernel(const uint16_t* __restrict__ src, uint16_t* __restrict__ dst, int N, int K) {
    const int KB = K / 64;
    const size_t total = static_cast<size_t>(N) * KB;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int pos = i & 127;
        const size_t blk = i >> 7;
        const int bk = blk % KB;
        const int bn = blk / KB;
        const int a = pos >> 4, c = (pos >> 2) & 3, b = (pos >> 1) & 1, d = pos & 1;
        const int n = bn * 128 + a * 16 + b * 8 + c * 2 + d;
        dst[static_cast<size_t>(bk) * N + n] = src[i];
    }
}

// Per-column epilogue constants and the LoRA-up weight.
//   col_scale[n] = alpha * wcscales[n], col_bias[n] = bias[n]
//   lora_up[n][r] = tf32_rn( Wu[n][r] * lora_scale[r/16] / col_scale[n] ), zero padded to R32 columns
// Reference order of Wu (packer.py:362-398): [N/16][R/16][g 8][t 4][nh 2][kh 2][e 2],
// n = cp*16 + nh*8 + g, r = rp*16 + kh*8 + 2t + e.
struct LoraScales {
    float v[SVDQ_MAX_LORA_RANK / 16];
};

template <typename T>
__global__ void prepare_columns_kernel(const T* __restrict__ bias, const T* __restrict__ wcscales,
                                       const T* __restrict__ lora_up, float* __restrict__ col_scale,
                                       float* __restrict__ col_bias, float* __restrict__ lora_out, float alpha, int N,
                                       int R, int R32, LoraScales ls, bool col_scale_given) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N) return;
    const int pos = (n & ~127) + packed_vec_pos128(n & 127);
    const float wc = wcscales ? tf(wcscales[pos]) : 1.0f;
    const float cs = (col_scale_given ? col_scale[n] : 1.0f) * alpha * wc;   // INT4: times the power of two taken out of the weights
    col_scale[n] = cs;
    col_bias[n] = bias ? tf(bias[pos]) : 0.0f;
    if (lora_out == nullptr) return;
    const float inv = cs != 0.0f ? 1.0f / cs : 0.0f;
    const int cp = n >> 4, nh = (n >> 3) & 1, g = n & 7;
    for (int r = 0; r < R32; ++r) {
        float v = 0.0f;
        if (r < R) {
            const int rp = r >> 4, kh = (r >> 3) & 1, t = (r >> 1) & 3, e = r & 1;
            const size_t idx = ((((static_cast<size_t>(cp) * (R / 16) + rp) * 8 + g) * 4 + t) * 2 + nh) * 4 + kh * 2 + e;
            v = tf(lora_up[idx]) * ls.v[rp] * inv;
            uint32_t u;
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v));
            v = __uint_as_float(u);
        }
        lora_out[static_cast<size_t>(n) * R32 + r] = v;
    }
}

// ---------------------------------------------------------------------------
// Activation-side conversions (reference order -> native order and back)
// ---------------------------------------------------------------------------
// codes: reference [M/256][K/64][warp 8][mtile 2][g 8][t 4][kh 2][half 2] words (gemm_w4a4.cuh:163-187)
template <bool TO_NATIVE>
__global__ void relayout_act_codes_kernel(const uint32_t* __restrict__ src, uint32_t* __restrict__ dst, int M, int K) {
    const size_t total = static_cast<size_t>(M) * K / 8;
    const int KB = K / 64;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        size_t r = i;
        const int half = r & 1; r >>= 1;
        const int kh = r & 1; r >>= 1;
        const int t = r & 3; r >>= 2;
        const int g = r & 7; r >>= 3;
        const int mt = r & 1; r >>= 1;
        const int w = r & 7; r >>= 3;
        const int bk = r % KB;
        const int bm = r / KB;
        const int m = bm * 256 + w * 32 + mt * 16 + half * 8 + g;
        const int k = bk * 64 + kh * 32 + t * 8;
        const size_t j = (static_cast<size_t>(m) * K + k) / 8;
        if (TO_NATIVE) dst[j] = src[i]; else dst[i] = src[j];
    }
}

// NVFP4 activation scales: reference [M/256][K/64][warp 8][lane 32] words, row in warp =
// ((l%4)/2)*16 + (l%2)*8 + l/4 (gemm_w4a4.cuh:144-155); native 512-byte atoms [M/128][K/64][r0 32][r1 4].
template <bool TO_NATIVE>
__global__ void relayout_act_mscales_kernel(const uint32_t* __restrict__ src, uint32_t* __restrict__ dst, int M, int K) {
    const size_t total = static_cast<size_t>(M) * K / 64;
    const int KB = K / 64;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int l = i & 31, w = (i >> 5) & 7;
        const size_t blk = i >> 8;
        const int bk = blk % KB;
        const int bm = blk / KB;
        const int m = bm * 256 + w * 32 + ((l & 3) >> 1) * 16 + (l & 1) * 8 + (l >> 2);
        const size_t j = (static_cast<size_t>(m >> 7) * KB + bk) * 128 + (m & 31) * 4 + ((m >> 5) & 3);
        if (TO_NATIVE) dst[j] = src[i]; else dst[i] = src[j];
    }
}

// INT4 activation scales: reference [M/256][K/64][warp 8][q 2][g 8][e 2] bf16 (gemm_base.cuh:452-468);
// native bf16 [K/64][M].
template <bool TO_NATIVE>
__global__ void relayout_act_scales_kernel(const uint16_t* __restrict__ src, uint16_t* __restrict__ dst, int M, int K) {
    const int KB = K / 64;
    const size_t total = static_cast<size_t>(M) * KB;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int e = i & 1, g = (i >> 1) & 7, q = (i >> 4) & 1, w = (i >> 5) & 7;
        const size_t blk = i >> 8;
        const int bk = blk % KB;
        const int bm = blk / KB;
        const int m = bm * 256 + w * 32 + q * 16 + e * 8 + g;
        const size_t j = static_cast<size_t>(bk) * M + m;
        if (TO_NATIVE) dst[j] = src[i]; else dst[i] = src[j];
    }
}

// low-rank activations: reference [M/256][R/16][warp 8][mtile 2][nh 2][half 2][e 2][g 8][t 4] fp32
// (lora.cuh:61-94); native fp32 [M][R].
template <bool TO_NATIVE>
__global__ void relayout_lora_act_kernel(const float* __restrict__ src, float* __restrict__ dst, int M, int R) {
    const size_t total = static_cast<size_t>(M) * R;
    const int RT = R / 16;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        size_t r = i;
        const int t = r & 3; r >>= 2;
        const int g = r & 7; r >>= 3;
        const int e = r & 1; r >>= 1;
        const int half = r & 1; r >>= 1;
        const int nh = r & 1; r >>= 1;
        const int mt = r & 1; r >>= 1;
        const int w = r & 7; r >>= 3;
        const int rt = r % RT;
        const int bm = r / RT;
        const int m = bm * 256 + w * 32 + mt * 16 + half * 8 + g;
        const int rank = rt * 16 + nh * 8 + 2 * t + e;
        const size_t j = static_cast<size_t>(m) * R + rank;
        if (TO_NATIVE) dst[j] = src[i]; else dst[i] = src[j];
    }
}

static inline int grid_for(size_t total) {
    size_t b = (total + 255) / 256;
    return static_cast<int>(b > 148 * 16 ? 148 * 16 : (b == 0 ? 1 : b));
}

int prepared_bytes_impl(int N, int K, int R, int fp4, size_t bytes[5]) {
    SVDQ_CHECK_ARG(N > 0 && N % 128 == 0 && K > 0 && K % 128 == 0 && R >= 0 && R % 16 == 0,
                   "prepared_bytes: need N%%128==0, K%%128==0, R%%16==0 (N=%d K=%d R=%d)", N, K, R);
    const size_t R32 = (static_cast<size_t>(R) + 31) / 32 * 32;
    bytes[0] = fp4 ? static_cast<size_t>(N) * K / 2 : static_cast<size_t>(N) * K * 2;   // INT4: fp16 per code
    bytes[1] = fp4 ? static_cast<size_t>(N) * K / 16 : static_cast<size_t>(N) * (K / 64) * 2;
    bytes[2] = static_cast<size_t>(N) * R32 * 4;
    bytes[3] = static_cast<size_t>(N) * 4;
    bytes[4] = static_cast<size_t>(N) * 4;
    return SVDQ_OK;
}

template <typename T>
static void prepare_typed(const svdq_weights_args* a, const svdq_prepared_weights* o, cudaStream_t stream) {
    const size_t words = static_cast<size_t>(a->N) * a->K / 8;
    if (a->fp4) {
        retile_wgt_codes_kernel<<<grid_for(words), 256, 0, stream>>>(static_cast<const uint32_t*>(a->qweight),
                                                                    static_cast<uint32_t*>(o->wgt), a->N, a->K);
        const size_t sw = static_cast<size_t>(a->N) * a->K / 64;
        retile_wgt_mscales_kernel<<<grid_for(sw), 256, 0, stream>>>(static_cast<const uint32_t*>(a->wscales),
                                                                   static_cast<uint32_t*>(o->wscales), a->N, a->K);
    } else {
        const size_t sw = static_cast<size_t>(a->N) * (a->K / 64);
        retile_wgt_scales_kernel<<<grid_for(sw), 256, 0, stream>>>(static_cast<const uint16_t*>(a->wscales),
                                                                  static_cast<uint16_t*>(o->wscales), a->N, a->K);
        int4_col_scale_kernel<T><<<(a->N + 127) / 128, 128, 0, stream>>>(static_cast<const T*>(o->wscales), o->col_scale,
                                                                     a->N, a->K / 64);
        retile_wgt_codes_f16_kernel<T><<<grid_for(words), 256, 0, stream>>>(static_cast<const uint32_t*>(a->qweight),
                                                                        static_cast<const T*>(o->wscales), o->col_scale,
                                                                        static_cast<uint4*>(o->wgt), a->N, a->K);
    }
    LoraScales ls;
    for (int i = 0; i < SVDQ_MAX_LORA_RANK / 16; ++i) ls.v[i] = (a->lora_scales && i < a->R / 16) ? a->lora_scales[i] : 1.0f;
    const int R32 = (a->R + 31) / 32 * 32;
    prepare_columns_kernel<T><<<(a->N + 127) / 128, 128, 0, stream>>>(
        static_cast<const T*>(a->bias), static_cast<const T*>(a->wcscales),
        static_cast<const T*>(a->lora_up), o->col_scale, o->col_bias, a->R ? o->lora_up : nullptr, a->alpha,
        a->N, a->R, R32, ls, !a->fp4);
}

int prepare_weights_impl(const svdq_weights_args* a, const svdq_prepared_weights* o, cudaStream_t stream) {
    SVDQ_CHECK_ARG(a && o, "prepare_weights: null args");
    SVDQ_CHECK_ARG(a->qweight && a->wscales && o->wgt && o->wscales && o->col_scale && o->col_bias,
                   "prepare_weights: null tensor pointer");
    SVDQ_CHECK_ARG(a->N > 0 && a->N % 128 == 0 && a->K > 0 && a->K % 128 == 0, "prepare_weights: need N%%128==0 and K%%128==0");
    SVDQ_CHECK_ARG(a->R >= 0 && a->R % 16 == 0 && a->R <= SVDQ_MAX_LORA_RANK, "prepare_weights: R (%d) must be a multiple of 16, at most %d", a->R, SVDQ_MAX_LORA_RANK);
    SVDQ_CHECK_ARG(a->R == 0 || (a->lora_up && o->lora_up), "prepare_weights: lora_up missing");
    SVDQ_CHECK_ARG(a->fp4 || a->alpha == 1.0f, "prepare_weights: alpha must be 1 for INT4 (gemm_w4a4_launch_impl.cuh:107)");
    SVDQ_CHECK_ARG(aligned(a->qweight, 16) && aligned(a->wscales, 16) && aligned(o->wgt, 16) && aligned(o->wscales, 16),
                   "prepare_weights: tensors must be 16-byte aligned");
    if (int rc = check_arch()) return rc;
    SVDQ_CHECK_ARG(a->dtype == SVDQ_DTYPE_BF16 || a->dtype == SVDQ_DTYPE_FP16, "prepare_weights: bad dtype %d", a->dtype);
    if (a->dtype == SVDQ_DTYPE_FP16) prepare_typed<__half>(a, o, stream);
    else prepare_typed<__nv_bfloat16>(a, o, stream);
    SVDQ_CUDA(cudaGetLastError());
    return SVDQ_OK;
}

template <bool TO_NATIVE>
static int relayout_dir(const svdq_relayout_args* a, cudaStream_t stream) {
    if (a->codes_in && a->codes_out) {
        const size_t words = static_cast<size_t>(a->M_pad) * a->K / 8;
        relayout_act_codes_kernel<TO_NATIVE><<<grid_for(words), 256, 0, stream>>>(
            static_cast<const uint32_t*>(a->codes_in), static_cast<uint32_t*>(a->codes_out), a->M_pad, a->K);
    }
    if (a->scales_in && a->scales_out) {
        if (a->fp4) {
            const size_t words = static_cast<size_t>(a->M_pad) * a->K / 64;
            relayout_act_mscales_kernel<TO_NATIVE><<<grid_for(words), 256, 0, stream>>>(
                static_cast<const uint32_t*>(a->scales_in), static_cast<uint32_t*>(a->scales_out), a->M_pad, a->K);
        } else {
            const size_t n = static_cast<size_t>(a->M_pad) * (a->K / 64);
            relayout_act_scales_kernel<TO_NATIVE><<<grid_for(n), 256, 0, stream>>>(
                static_cast<const uint16_t*>(a->scales_in), static_cast<uint16_t*>(a->scales_out), a->M_pad, a->K);
        }
    }
    if (a->lora_in && a->lora_out && a->R > 0) {
        const size_t n = static_cast<size_t>(a->M_pad) * a->R;
        relayout_lora_act_kernel<TO_NATIVE><<<grid_for(n), 256, 0, stream>>>(a->lora_in, a->lora_out, a->M_pad, a->R);
    }
    SVDQ_CUDA(cudaGetLastError());
    return SVDQ_OK;
}

int relayout_impl(const svdq_relayout_args* a, cudaStream_t stream) {
    SVDQ_CHECK_ARG(a != nullptr, "relayout: null args");
    SVDQ_CHECK_ARG(a->M_pad > 0 && a->M_pad % 256 == 0 && a->K % 128 == 0 && a->R % 16 == 0,
                   "relayout: need M_pad%%256==0, K%%128==0, R%%16==0");
    SVDQ_CHECK_ARG(a->from_layout != a->to_layout, "relayout: from_layout == to_layout");
    SVDQ_CHECK_ARG(a->codes_in != a->codes_out || !a->codes_in, "relayout: in-place conversion is not supported");
    if (int rc = check_arch()) return rc;
    if (a->to_layout == SVDQ_LAYOUT_NATIVE) return relayout_dir<true>(a, stream);
    return relayout_dir<false>(a, stream);
}

}  // namespace svdq

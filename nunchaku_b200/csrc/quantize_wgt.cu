// INT4 weight quantiser, sm_100a (any CUDA GPU would do: it is a plain streaming kernel).
//
// What it computes (reference: quantize_w4a4_wgt_kernel + quantize_w4a4_warp, src/kernels/zgemm/gemm_w4a4.cuh:661-689 and
// :527-620; launcher GEMM_W4A4_Launch::quantize_w4a4_wgt, gemm_w4a4_launch_impl.cuh:547-570; declared in zgemm.h:48): for a
// 16-bit weight w[N, K], per row n and group of 64 along k, all in the 16-bit type as the reference does it,
//   m      = max |w|                          scale = m / 7            (the stored group scale)
//   rscale = 7 / m                            code  = sat_s4(rint(float(rscale * w)))   (product rounded to 16 bits first)
// A zero group gives scale 0 and, through 7 / 0 = inf and inf * 0 = NaN, codes 0, as there.
// Outputs in the layouts the GEMM (and svdq_w4a4_prepare_weights) read:
//   qweight  int8 [N, K/2]: [N/128][K/64][n-tile 8][g 8][t 4][half 2][kh 2] words of 8 nibbles, row n = 128 bn + 16 nt + 8 half + g,
//            k = 64 bk + 32 kh + 8 t + j (what ldmatrix + the y/z swap of the reference kernel produce; NunchakuWeightPacker.pack_weight,
//            nunchaku/lora/flux/packer.py:187-239);
//   wscales  16-bit [K/64, N]: [N/128][K/64][128], channel a*16 + b*8 + c*2 + d at a*16 + c*4 + b*2 + d (pack_wscales,
//            gemm_base.cuh:474-489; packer.py:241-301).
// The arithmetic uses the same CUDA 16-bit operators as the reference (operator/ and __hmul2 of cuda_bf16.h / cuda_fp16.h),
// so codes and scales are bit-identical to its kernel's in both types.
//
// One thread per (row, group): 128 contiguous bytes in, eight 4-byte words and one scale out; consecutive lanes take
// consecutive groups of a row.  HBM bound: 2 bytes in, 0.53 out per weight.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "host_common.h"

namespace svdq {

template <typename H> struct Half2Of;
template <> struct Half2Of<__nv_bfloat16> { using type = __nv_bfloat162; };
template <> struct Half2Of<__half> { using type = __half2; };

__device__ __forceinline__ float2 to_float2(__nv_bfloat162 v) { return __bfloat1622float2(v); }
__device__ __forceinline__ float2 to_float2(__half2 v) { return __half22float2(v); }
__device__ __forceinline__ __nv_bfloat16 from_int(int v, __nv_bfloat16) { return __int2bfloat16_rn(v); }
__device__ __forceinline__ __half from_int(int v, __half) { return __int2half_rn(v); }

// two floats -> two signed 4-bit codes (x in the low nibble): round to nearest even, saturate to [-8, 7]
__device__ __forceinline__ uint32_t s4x2(float2 v) {
    int a, b;
    uint32_t r;
    asm("cvt.rni.s32.f32 %0, %1;" : "=r"(a) : "f"(v.x));
    asm("cvt.rni.s32.f32 %0, %1;" : "=r"(b) : "f"(v.y));
    asm("cvt.pack.sat.s4.s32.b32 %0, %1, %2, 0;" : "=r"(r) : "r"(b), "r"(a));
    return r;
}

template <typename H>
__global__ void __launch_bounds__(256)
quantize_wgt_int4_kernel(const H* __restrict__ w, uint32_t* __restrict__ qweight, H* __restrict__ wscales, int N, int K) {
    using H2 = typename Half2Of<H>::type;
    const int KB = K / 64;
    const long long total = static_cast<long long>(N) * KB;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int n = static_cast<int>(i / KB), bk = static_cast<int>(i - static_cast<long long>(n) * KB);
        const uint4* src = reinterpret_cast<const uint4*>(w + static_cast<size_t>(n) * K + bk * 64);
        uint4 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = src[j];
        const H2* h2 = reinterpret_cast<const H2*>(v);   // 32 pairs
        H m = __habs(h2[0].x);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            m = __hmax(m, __habs(h2[j].x));
            m = __hmax(m, __habs(h2[j].y));
        }
        const H seven = from_int(7, H());
        const H scale = m / seven;
        const H rscale = seven / m;
        const H2 rs2 = H2(rscale, rscale);
        // words (kh, t): nibble j = column 32 kh + 8 t + j
        const int bn = n >> 7, nt = (n >> 4) & 7, half = (n >> 3) & 1, g = n & 7;
        uint32_t* dst = qweight + ((((static_cast<size_t>(bn) * KB + bk) * 8 + nt) * 8 + g) * 4) * 4 + half * 2;
#pragma unroll
        for (int kh = 0; kh < 2; ++kh)
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                uint32_t word = 0;
#pragma unroll
                for (int p = 0; p < 4; ++p) word |= s4x2(to_float2(__hmul2(rs2, h2[kh * 16 + t * 4 + p]))) << (8 * p);
                dst[t * 4 + kh] = word;
            }
        const int nn = n & 127;
        const int pos = (nn & ~15) | (((nn >> 1) & 3) << 2) | (((nn >> 3) & 1) << 1) | (nn & 1);
        wscales[(static_cast<size_t>(bn) * KB + bk) * 128 + pos] = scale;
    }
}

}  // namespace svdq

extern "C" int svdq_quantize_w4a4_wgt(const svdq_quantize_wgt_args* a, void* stream) {
    using namespace svdq;
    SVDQ_CHECK_ARG(a && a->input && a->qweight && a->wscales, "quantize_w4a4_wgt: null pointer");
    SVDQ_CHECK_ARG(a->N > 0 && a->N % 128 == 0 && a->K > 0 && a->K % 64 == 0,
                   "quantize_w4a4_wgt: N (%d) must be a multiple of 128 and K (%d) of 64 (gemm_w4a4_launch_impl.cuh:565)", a->N, a->K);
    SVDQ_CHECK_ARG(a->dtype == SVDQ_DTYPE_BF16 || a->dtype == SVDQ_DTYPE_FP16, "quantize_w4a4_wgt: bad dtype %d", a->dtype);
    SVDQ_CHECK_ARG(aligned(a->input, 16) && aligned(a->qweight, 16) && aligned(a->wscales, 16),
                   "quantize_w4a4_wgt: tensors must be 16-byte aligned");
    if (int rc = check_arch()) return rc;
    int sms = 0;
    if (int rc = sm_count(&sms)) return rc;
    const long long total = static_cast<long long>(a->N) * (a->K / 64);
    const long long want = (total + 255) / 256;
    const int grid = static_cast<int>(want < 8LL * sms ? want : 8LL * sms);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (a->dtype == SVDQ_DTYPE_FP16)
        quantize_wgt_int4_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(a->input), static_cast<uint32_t*>(a->qweight),
                                                                 static_cast<__half*>(a->wscales), a->N, a->K);
    else
        quantize_wgt_int4_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(a->input),
                                                                        static_cast<uint32_t*>(a->qweight),
                                                                        static_cast<__nv_bfloat16*>(a->wscales), a->N, a->K);
    SVDQ_CUDA(cudaGetLastError());
    return SVDQ_OK;
}

// Device helpers shared by the activation quantiser and the GEMM's requantising epilogue.
// Rounding follows the reference kernels (src/kernels/zgemm/gemm_w4a4.cuh:85-187,429-523 and
// gemm_utils.cuh:206-264): bf16 round-to-nearest for every half_t step, E2M1 / E4M3 / s4 conversions with
// saturation; a group whose absolute maximum is zero gets all-zero codes.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include <cstdint>

namespace svdq {

__device__ __forceinline__ uint32_t e2m1x2(float lo, float hi) {
    uint32_t r;
    asm("{\n\t.reg .b8 t;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\tcvt.u32.u8 %0, t;\n\t}"
        : "=r"(r)
        : "f"(hi), "f"(lo));
    return r;
}

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t saddr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(saddr));
}

// position of channel n (0..127) inside a 128-block of a reference-packed vector
// (gemm_base.cuh:100-112): n = a*16 + b*8 + c*2 + d  ->  a*16 + c*4 + b*2 + d
__device__ __forceinline__ int packed_vec_pos(int n) {
    return (n & ~15) | (((n >> 1) & 3) << 2) | (((n >> 3) & 1) << 1) | (n & 1);
}

// 16 bf16 values (8 packed words, low half = lower column) times their 16 reciprocal smoothing factors
// (fp32, 16-byte aligned), rounded to bf16: q[] and the group's absolute maximum.
// "x * rcp + 0.0f" as one FMA: the reference adds a bf16 zero shift before dividing, which turns -0 into +0.
__device__ __forceinline__ float smooth16(const uint32_t (&xw)[8], const float4* rc, __nv_bfloat162 (&q)[8]) {
    __nv_bfloat162 mx = __floats2bfloat162_rn(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 r4 = rc[i];
        const float a0 = fmaf(__uint_as_float(xw[2 * i] << 16), r4.x, 0.0f);
        const float a1 = fmaf(__uint_as_float(xw[2 * i] & 0xffff0000u), r4.y, 0.0f);
        const float a2 = fmaf(__uint_as_float(xw[2 * i + 1] << 16), r4.z, 0.0f);
        const float a3 = fmaf(__uint_as_float(xw[2 * i + 1] & 0xffff0000u), r4.w, 0.0f);
        q[2 * i] = __floats2bfloat162_rn(a0, a1);
        q[2 * i + 1] = __floats2bfloat162_rn(a2, a3);
        mx = __hmax2(mx, __hmax2(__habs2(q[2 * i]), __habs2(q[2 * i + 1])));
    }
    return fmaxf(__bfloat162float(mx.x), __bfloat162float(mx.y));
}

// NVFP4 group of 16: E4M3 scale byte and two words of E2M1 codes (lowest nibble = lowest column).
__device__ __forceinline__ uint32_t nvfp4_encode16(const __nv_bfloat162 (&q)[8], float amax, uint32_t (&cw)[2]) {
    const float scale = fminf(amax * (1.0f / 6.0f), 448.0f);
    const float rs = scale == 0.f ? 0.f : __frcp_rn(scale);
    cw[0] = cw[1] = 0u;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float2 f = __bfloat1622float2(q[i]);
        cw[i >> 2] |= e2m1x2(f.x * rs, f.y * rs) << ((i & 3) * 8);
    }
    return static_cast<uint32_t>(__nv_cvt_float_to_fp8(scale, __NV_SATFINITE, __NV_E4M3));
}

// INT4 codes of 16 values given the group's (64-wide) absolute maximum; returns the fp32 scale.
template <bool UNSIGNED>
__device__ __forceinline__ float int4_encode16(const __nv_bfloat162 (&q)[8], float amax, uint32_t (&cw)[2]) {
    const float scale = amax * (UNSIGNED ? (1.0f / 15.0f) : (1.0f / 7.0f));
    const float rs = scale == 0.f ? 0.f : __frcp_rn(scale);
    cw[0] = cw[1] = 0u;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float2 f = __bfloat1622float2(q[i]);
        int c0 = __float2int_rn(f.x * rs), c1 = __float2int_rn(f.y * rs);
        if (UNSIGNED) {
            c0 = max(0, min(15, c0));
            c1 = max(0, min(15, c1));
        } else {
            c0 = max(-8, min(7, c0));
            c1 = max(-8, min(7, c1));
        }
        cw[i >> 2] |= static_cast<uint32_t>((c0 & 0xF) | ((c1 & 0xF) << 4)) << ((i & 3) * 8);
    }
    return scale;
}

}  // namespace svdq

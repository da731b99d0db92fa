// Device helpers shared by the activation quantiser and the GEMM's requantising epilogue.
// Rounding follows the reference kernels (src/kernels/zgemm/gemm_w4a4.cuh:85-187,429-523 and
// gemm_utils.cuh:206-264): bf16 round-to-nearest for every half_t step, the group scale's reciprocal with
// rcp.approx.ftz, E2M1 / E4M3 / s4 conversions with saturation; a group whose absolute maximum is zero gets
// all-zero codes.
#pragma once
#include <cuda_fp8.h>

#include <cstdint>

#include "dtype.cuh"

namespace svdq {
namespace SVDQ_DT {

__device__ __forceinline__ uint32_t e2m1x2(float lo, float hi) {
    uint32_t r;
    asm("{\n\t.reg .b8 t;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\tcvt.u32.u8 %0, t;\n\t}"
        : "=r"(r)
        : "f"(hi), "f"(lo));
    return r;
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t saddr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(saddr));
}

// GLU gating of two (value, gate) bf16 pairs -> two bf16 results in one word.  Per pair
// (gemm_base.cuh:612-623, gemm_utils.cuh:291-327): s = bf16(g * sigmoid(g)), sigmoid(g) = rcp.approx(1 + ex2.approx(-log2(e) g)),
// result = bf16(v * s); words hold the value in the low half and the gate in the high half.
__device__ __forceinline__ float glu_one(uint32_t w) {
    const float2 vg = unpack2(w);
    const float v = vg.x, g = vg.y;
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-1.442695041f * g));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(e + 1.0f));
    const float s = h2f(f2h(g * r));
    return v * s;
}
__device__ __forceinline__ uint32_t glu_pair2(uint32_t w0, uint32_t w1) {
    return pack2(make_float2(glu_one(w0), glu_one(w1)));
}

// position of channel n (0..127) inside a 128-block of a reference-packed vector
// (gemm_base.cuh:100-112): n = a*16 + b*8 + c*2 + d  ->  a*16 + c*4 + b*2 + d
__device__ __forceinline__ int packed_vec_pos(int n) {
    return (n & ~15) | (((n >> 1) & 3) << 2) | (((n >> 3) & 1) << 1) | (n & 1);
}

// Eight fp32 values -> eight E2M1 nibbles in one word (lowest nibble = first value).
__device__ __forceinline__ uint32_t e2m1x8(float2 a, float2 b, float2 c, float2 d) {
    uint32_t r;
    asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
        "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
        : "=r"(r)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y), "f"(d.x), "f"(d.y));
    return r;
}

// 16 bf16 values (8 packed words, low half = lower column) times their 16 reciprocal smoothing factors
// (fp32, 16-byte aligned), rounded to bf16: q[] and the group's absolute maximum.
// "x * rcp + 0.0f" as one FMA: the reference adds a bf16 zero shift before dividing, which turns -0 into +0.
// Packed fp32x2 arithmetic (two IEEE operations per instruction on sm_100).
__device__ __forceinline__ float smooth16(const uint32_t (&xw)[8], const float4* rc, uint32_t (&q)[8]) {
    uint32_t mx = 0u;
    const float2 zero = make_float2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 r4 = rc[i];
        const float2 a = __ffma2_rn(unpack2(xw[2 * i]), make_float2(r4.x, r4.y), zero);
        const float2 b = __ffma2_rn(unpack2(xw[2 * i + 1]), make_float2(r4.z, r4.w), zero);
        q[2 * i] = pack2(a);
        q[2 * i + 1] = pack2(b);
        mx = absmax2(mx, q[2 * i]);
        mx = absmax2(mx, q[2 * i + 1]);
    }
    const float2 m = unpack2(mx);
    return fmaxf(fabsf(m.x), fabsf(m.y));
}

// The reciprocal of a group scale as the reference computes it (cuda_frcp, gemm_utils.cuh:259-263): the hardware's
// approximate reciprocal, not the IEEE one.  Scaled values that sit exactly on a rounding tie (frequent: bf16 values have
// 8-bit mantissas) fall to one side or the other depending on the last bit of this reciprocal, so only the same
// instruction reproduces the reference kernel's codes bit for bit.
__device__ __forceinline__ float rcp_approx_ftz(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

// NVFP4 group of 16: E4M3 scale byte and two words of E2M1 codes (lowest nibble = lowest column).
__device__ __forceinline__ uint32_t nvfp4_encode16(const uint32_t (&q)[8], float amax, uint32_t (&cw)[2]) {
    const float scale = fminf(amax * (1.0f / 6.0f), 448.0f);
    const float rs = scale == 0.f ? 0.f : rcp_approx_ftz(scale);
    const float2 rs2 = make_float2(rs, rs);
#pragma unroll
    for (int w = 0; w < 2; ++w)
        cw[w] = e2m1x8(__fmul2_rn(unpack2(q[4 * w]), rs2), __fmul2_rn(unpack2(q[4 * w + 1]), rs2),
                       __fmul2_rn(unpack2(q[4 * w + 2]), rs2), __fmul2_rn(unpack2(q[4 * w + 3]), rs2));
    return static_cast<uint32_t>(__nv_cvt_float_to_fp8(scale, __NV_SATFINITE, __NV_E4M3));
}

// INT4 codes of 16 values given the group's (64-wide) absolute maximum; returns the fp32 scale.
template <bool UNSIGNED>
__device__ __forceinline__ float int4_encode16(const uint32_t (&q)[8], float amax, uint32_t (&cw)[2]) {
    const float scale = amax * (UNSIGNED ? (1.0f / 15.0f) : (1.0f / 7.0f));
    const float rs = scale == 0.f ? 0.f : rcp_approx_ftz(scale);
    cw[0] = cw[1] = 0u;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float2 f = unpack2(q[i]);
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

}  // namespace SVDQ_DT
}  // namespace svdq

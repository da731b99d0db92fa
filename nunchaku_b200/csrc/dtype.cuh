// The 16-bit floating-point type of activations, smoothing factors, LoRA weights, biases, INT4 group scales and outputs:
// bf16 or fp16 (the reference's GEMMConfig_W4A4_BF16 / _FP16, src/kernels/zgemm/gemm_base.cuh:29-54).  The kernels are
// compiled once per type: a translation unit that defines SVDQ_F16 before including the sources gets the fp16 build, in
// namespace svdq::hf; the default is bf16 in svdq::bf.  Everything that depends on the type goes through the few
// functions below.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>

#ifdef SVDQ_F16
#define SVDQ_DT hf
#define SVDQ_TMAP_16 CU_TENSOR_MAP_DATA_TYPE_FLOAT16
#else
#define SVDQ_DT bf
#define SVDQ_TMAP_16 CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
#endif

namespace svdq {
namespace SVDQ_DT {

#ifdef SVDQ_F16
using h16 = __half;
constexpr bool kF16 = true;
__device__ __forceinline__ float h2f(h16 v) { return __half2float(v); }
__device__ __forceinline__ h16 f2h(float v) { return __float2half_rn(v); }
// two packed values (low half = first) <-> two floats; fp16 saturates to +-65504 like the reference's output clamp
// (gemm_base.cuh:686-693)
__device__ __forceinline__ float2 unpack2(uint32_t w) { return __half22float2(*reinterpret_cast<const __half2*>(&w)); }
__device__ __forceinline__ uint32_t pack2(float2 v) {
    uint32_t r;
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(v.y), "f"(v.x));
    return r;
}
// |result| = max(|a|, |b|) per lane (the sign of the result is meaningless)
__device__ __forceinline__ uint32_t absmax2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("max.xorsign.abs.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
#else
using h16 = __nv_bfloat16;
constexpr bool kF16 = false;
__device__ __forceinline__ float h2f(h16 v) { return __bfloat162float(v); }
__device__ __forceinline__ h16 f2h(float v) { return __float2bfloat16_rn(v); }
__device__ __forceinline__ float2 unpack2(uint32_t w) { return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u)); }
__device__ __forceinline__ uint32_t pack2(float2 v) {
    const __nv_bfloat162 p = __float22bfloat162_rn(v);
    return *reinterpret_cast<const uint32_t*>(&p);
}
// |result| = max(|a|, |b|) per lane (the sign of the result is meaningless): one instruction per pair instead of two
// abs and a max
__device__ __forceinline__ uint32_t absmax2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("max.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
#endif

}  // namespace SVDQ_DT
}  // namespace svdq

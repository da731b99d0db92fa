// ReLU linear attention ("LiteLA") on the bf16 output of SANA's fused QKV projection, sm_100a, HBM bound.
//
// What it computes (reference: EpilogueLiteLA inside the QKV GEMM + vk_mul_q_kernel,
// src/kernels/zgemm/epilogues.cuh:552-761; caller SanaLinearAttention::forward, src/SanaModel.cpp:25-106).
// Input qkv [batches, tokens, 3*D], D = heads*32.  Columns [0, D) hold Q of all heads; after them every head h owns
// 64 columns [K_h (32) | V_h (32)] at D + 64*h (epilogues.cuh:588-605).  Per (batch, head):
//   vk[r, c] = sum_tok V[tok, r] * relu(K[tok, c])   r < 32          fp32 accumulation of bf16 values
//   vk[32, c] = sum_tok relu(K[tok, c])
//   o[j] = sum_i relu(Q[tok, i]) * vk[j, i]  (i ascending, fp32 FMA);   out[tok, i] = bf16(o[i] / (o[32] + eps))
// The reference adds per-256-token partial sums of vk with red.add into a zeroed buffer (order not fixed); here one CTA
// owns a (batch, head) pair, its eight warps take interleaved tokens and their partials are added in warp order, so the
// result does not depend on scheduling and nothing has to be zeroed.  `vk` is also written out ([batches, heads, 33, 32]
// fp32, the reference's out_vk) when the caller asks for it.
//
// Traffic: reads 3*D bf16 per token once (K|V as one 128-byte line per token and head, Q as 64 bytes), writes D bf16.
#include <cuda_bf16.h>

#include "host_common.h"

namespace svdq {

constexpr int LA_HD = 32;
constexpr int LA_WARPS = 8;

__global__ void __launch_bounds__(LA_WARPS * 32)
litela_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ out, float* __restrict__ vk_out,
              int tokens, int heads, float eps) {
    __shared__ float part[LA_WARPS][LA_HD + 1][LA_HD];   // 33.8 KB
    __shared__ __align__(16) float vk[LA_HD + 1][LA_HD];
    const int h = blockIdx.x, b = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int D = heads * LA_HD;
    const size_t pitch = static_cast<size_t>(3) * D;
    const __nv_bfloat16* base = qkv + static_cast<size_t>(b) * tokens * pitch;
    const __nv_bfloat16* kv = base + D + 64 * h;

    // phase 1: lane = column c of K; acc[r] = sum over this warp's tokens of V[tok, r] * relu(K[tok, c])
    float acc[LA_HD + 1];
#pragma unroll
    for (int r = 0; r <= LA_HD; ++r) acc[r] = 0.f;
    for (int t0 = warp; t0 < tokens; t0 += 4 * LA_WARPS) {
        float kk[4], vv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {   // four tokens in flight per warp
            const int t = t0 + u * LA_WARPS;
            const bool in = t < tokens;
            const __nv_bfloat16* p = kv + static_cast<size_t>(in ? t : t0) * pitch;
            kk[u] = in ? fmaxf(__bfloat162float(p[lane]), 0.f) : 0.f;
            vv[u] = in ? __bfloat162float(p[LA_HD + lane]) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
#pragma unroll
            for (int r = 0; r < LA_HD; ++r) acc[r] = fmaf(__shfl_sync(0xffffffffu, vv[u], r), kk[u], acc[r]);
            acc[LA_HD] += kk[u];
        }
    }
#pragma unroll
    for (int r = 0; r <= LA_HD; ++r) part[warp][r][lane] = acc[r];
    __syncthreads();
    for (int i = threadIdx.x; i < (LA_HD + 1) * LA_HD; i += LA_WARPS * 32) {
        const int r = i >> 5, c = i & 31;
        float s = part[0][r][c];
#pragma unroll
        for (int w = 1; w < LA_WARPS; ++w) s += part[w][r][c];   // fixed order
        vk[r][c] = s;
        if (vk_out) vk_out[(static_cast<size_t>(b) * heads + h) * (LA_HD + 1) * LA_HD + i] = s;
    }
    __syncthreads();

    // phase 2: one token per thread
    for (int t = threadIdx.x; t < tokens; t += LA_WARPS * 32) {
        const uint4* qp = reinterpret_cast<const uint4*>(base + static_cast<size_t>(t) * pitch + LA_HD * h);
        float q[LA_HD];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint4 w = qp[j];
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                q[8 * j + 2 * i] = fmaxf(__uint_as_float(ww[i] << 16), 0.f);
                q[8 * j + 2 * i + 1] = fmaxf(__uint_as_float(ww[i] & 0xffff0000u), 0.f);
            }
        }
        float den = 0.f;
#pragma unroll
        for (int i = 0; i < LA_HD; ++i) den = fmaf(q[i], vk[LA_HD][i], den);
        den += eps;
        uint4* op = reinterpret_cast<uint4*>(out + (static_cast<size_t>(b) * tokens + t) * D + LA_HD * h);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t o[4];
#pragma unroll
            for (int i2 = 0; i2 < 4; ++i2) {
                float num[2];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float4* row = reinterpret_cast<const float4*>(vk[8 * j + 2 * i2 + e]);
                    float s = 0.f;
#pragma unroll
                    for (int i = 0; i < LA_HD / 4; ++i) {
                        const float4 v4 = row[i];   // same address in every thread: a broadcast
                        s = fmaf(q[4 * i], v4.x, s);
                        s = fmaf(q[4 * i + 1], v4.y, s);
                        s = fmaf(q[4 * i + 2], v4.z, s);
                        s = fmaf(q[4 * i + 3], v4.w, s);
                    }
                    num[e] = __fdividef(s, den);
                }
                const __nv_bfloat162 pr = __floats2bfloat162_rn(num[0], num[1]);
                o[i2] = *reinterpret_cast<const uint32_t*>(&pr);
            }
            op[j] = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
}

}  // namespace svdq

extern "C" int svdq_litela(const svdq_litela_args* a, void* stream) {
    using namespace svdq;
    SVDQ_CHECK_ARG(a && a->qkv && a->out, "litela: null pointer");
    SVDQ_CHECK_ARG(a->batches > 0 && a->batches <= 65535 && a->tokens > 0 && a->heads > 0,
                   "litela: batches (%d, at most 65535), tokens (%d) and heads (%d) must be positive", a->batches, a->tokens, a->heads);
    SVDQ_CHECK_ARG(aligned(a->qkv, 16) && aligned(a->out, 16) && aligned(a->vk, 16), "litela: tensors must be 16-byte aligned");
    if (int rc = check_arch()) return rc;
    litela_kernel<<<dim3(a->heads, a->batches), LA_WARPS * 32, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(a->qkv), static_cast<__nv_bfloat16*>(a->out), a->vk, a->tokens, a->heads, a->eps);
    SVDQ_CUDA(cudaGetLastError());
    return SVDQ_OK;
}

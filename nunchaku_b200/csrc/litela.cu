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
// owns a (batch, head) pair, its eight warps take runs of tokens and their partials are added in warp order, so the
// result does not depend on scheduling and nothing has to be zeroed.  `vk` is also written out ([batches, heads, 33, 32]
// fp32, the reference's out_vk) when the caller asks for it.
//
// Traffic: reads 3*D bf16 per token once (K|V as one 128-byte line per token and head, Q as 64 bytes), writes D bf16.
#include <cuda_bf16.h>

#include "host_common.h"

namespace svdq {

constexpr int LA_HD = 32;
constexpr int LA_WARPS = 8;
constexpr int LA_U = 16;                         // tokens a warp has in flight

__global__ void __launch_bounds__(LA_WARPS * 32)
litela_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ out, float* __restrict__ vk_out,
              int tokens, int heads, float eps) {
    __shared__ __align__(16) float part[LA_WARPS][LA_HD + 1][LA_HD];   // 33.8 KB
    __shared__ __align__(16) float vk[LA_HD + 1][LA_HD];
    const int h = blockIdx.x, b = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int D = heads * LA_HD;
    const size_t pitch = static_cast<size_t>(3) * D;
    const __nv_bfloat16* base = qkv + static_cast<size_t>(b) * tokens * pitch;
    const __nv_bfloat16* kv = base + D + 64 * h;

    // phase 1: a warp takes runs of LA_U consecutive tokens; lane = column c of K;
    // acc[r] = sum over the warp's tokens of V[tok, r] * relu(K[tok, c]).  V goes through a warp-private fp32 slab of
    // shared memory (it aliases the warp's slice of `part`, which is only written after the loop) and comes back as
    // 16-byte broadcasts, four rows per load; LA_U loads per lane are in flight before the first use.
    float acc[LA_HD + 1];
#pragma unroll
    for (int r = 0; r <= LA_HD; ++r) acc[r] = 0.f;
    float (*vs)[LA_HD] = part[warp];   // [LA_U][32]
    for (int t0 = warp * LA_U; t0 < tokens; t0 += LA_WARPS * LA_U) {
        float kk[LA_U];
        __nv_bfloat16 kraw[LA_U], vraw[LA_U];
#pragma unroll
        for (int u = 0; u < LA_U; ++u) {
            const int t = t0 + u;
            const __nv_bfloat16* p = kv + static_cast<size_t>(t < tokens ? t : t0) * pitch;
            kraw[u] = p[lane];
            vraw[u] = p[LA_HD + lane];
        }
#pragma unroll
        for (int u = 0; u < LA_U; ++u) {
            const bool in = t0 + u < tokens;
            kk[u] = in ? fmaxf(__bfloat162float(kraw[u]), 0.f) : 0.f;
            vs[u][lane] = in ? __bfloat162float(vraw[u]) : 0.f;
        }
        __syncwarp();
#pragma unroll
        for (int u = 0; u < LA_U; ++u) {
#pragma unroll
            for (int r4 = 0; r4 < LA_HD / 4; ++r4) {
                const float4 v4 = *reinterpret_cast<const float4*>(&vs[u][4 * r4]);   // same address in every lane
                acc[4 * r4 + 0] = fmaf(v4.x, kk[u], acc[4 * r4 + 0]);
                acc[4 * r4 + 1] = fmaf(v4.y, kk[u], acc[4 * r4 + 1]);
                acc[4 * r4 + 2] = fmaf(v4.z, kk[u], acc[4 * r4 + 2]);
                acc[4 * r4 + 3] = fmaf(v4.w, kk[u], acc[4 * r4 + 3]);
            }
            acc[LA_HD] += kk[u];
        }
        __syncwarp();
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

    // phase 2: one token per thread; q stays in registers, vk rows come as 16-byte broadcasts from shared memory
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
        auto dot = [&](int row) {
            const float4* vr = reinterpret_cast<const float4*>(vk[row]);
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < LA_HD / 4; ++i) {
                const float4 v4 = vr[i];
                s = fmaf(q[4 * i], v4.x, s);
                s = fmaf(q[4 * i + 1], v4.y, s);
                s = fmaf(q[4 * i + 2], v4.z, s);
                s = fmaf(q[4 * i + 3], v4.w, s);
            }
            return s;
        };
        const float den = dot(LA_HD) + eps;
        uint4* op = reinterpret_cast<uint4*>(out + (static_cast<size_t>(b) * tokens + t) * D + LA_HD * h);
#pragma unroll 1
        for (int j = 0; j < 4; ++j) {
            uint32_t o[4];
#pragma unroll
            for (int i2 = 0; i2 < 4; ++i2) {
                const float n0 = __fdividef(dot(8 * j + 2 * i2), den);
                const float n1 = __fdividef(dot(8 * j + 2 * i2 + 1), den);
                const __nv_bfloat162 pr = __floats2bfloat162_rn(n0, n1);
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

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
              int tokens, int heads, float eps, int mode) {
    __shared__ __align__(16) float part[LA_WARPS][LA_HD + 1][LA_HD];   // 33.8 KB
    __shared__ __align__(16) float vk[LA_HD + 1][LA_HD];
    const int h = blockIdx.x, b = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int D = heads * LA_HD;
    const size_t pitch = static_cast<size_t>(3) * D;
    const __nv_bfloat16* base = qkv + static_cast<size_t>(b) * tokens * pitch;
    const __nv_bfloat16* kv = base + D + 64 * h;
    // mode 0: everything.  The reference does it in two launches, and the two halves exist on their own for callers
    // that follow it: mode 1 = what its GEMM epilogue leaves behind (vk, and relu(Q) as bf16 in `out`), mode 2 = its
    // vk_mul_q_kernel (reads relu(Q) from `out` and vk from `vk_out`, finishes `out` in place; qkv is not read).
    if (mode == 2) {
        for (int i = threadIdx.x; i < (LA_HD + 1) * LA_HD; i += LA_WARPS * 32)
            vk[i >> 5][i & 31] = vk_out[(static_cast<size_t>(b) * heads + h) * (LA_HD + 1) * LA_HD + i];
        __syncthreads();
    } else {

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
    }
    if (mode == 1) {   // relu(Q) of this head -> out, 16 bytes per thread and step
        for (int i = threadIdx.x; i < tokens * 4; i += LA_WARPS * 32) {
            const int t = i >> 2, j = i & 3;
            const uint4 w = reinterpret_cast<const uint4*>(base + static_cast<size_t>(t) * pitch + LA_HD * h)[j];
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
            uint32_t o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const __nv_bfloat162 r = __floats2bfloat162_rn(fmaxf(__uint_as_float(ww[e] << 16), 0.f),
                                                               fmaxf(__uint_as_float(ww[e] & 0xffff0000u), 0.f));
                o[e] = *reinterpret_cast<const uint32_t*>(&r);
            }
            reinterpret_cast<uint4*>(out + (static_cast<size_t>(b) * tokens + t) * D + LA_HD * h)[j] = make_uint4(o[0], o[1], o[2], o[3]);
        }
        return;
    }

    // phase 2: two tokens per thread (t and t + 256); q stays in registers, every vk row comes once as 16-byte
    // broadcasts from shared memory and serves both tokens
    auto load_q = [&](int t, float* q) {
        const uint4* qp = mode == 2 ? reinterpret_cast<const uint4*>(out + (static_cast<size_t>(b) * tokens + t) * D + LA_HD * h)
                                    : reinterpret_cast<const uint4*>(base + static_cast<size_t>(t) * pitch + LA_HD * h);
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
    };
    for (int t = threadIdx.x; t < tokens; t += 2 * LA_WARPS * 32) {
        const int t1 = t + LA_WARPS * 32;
        const bool has1 = t1 < tokens;
        float q0[LA_HD], q1[LA_HD];
        load_q(t, q0);
        load_q(has1 ? t1 : t, q1);
        auto dot2 = [&](int row, float& s0, float& s1) {
            const float4* vr = reinterpret_cast<const float4*>(vk[row]);
            s0 = 0.f;
            s1 = 0.f;
#pragma unroll
            for (int i = 0; i < LA_HD / 4; ++i) {
                const float4 v4 = vr[i];
                s0 = fmaf(q0[4 * i], v4.x, s0);
                s1 = fmaf(q1[4 * i], v4.x, s1);
                s0 = fmaf(q0[4 * i + 1], v4.y, s0);
                s1 = fmaf(q1[4 * i + 1], v4.y, s1);
                s0 = fmaf(q0[4 * i + 2], v4.z, s0);
                s1 = fmaf(q1[4 * i + 2], v4.z, s1);
                s0 = fmaf(q0[4 * i + 3], v4.w, s0);
                s1 = fmaf(q1[4 * i + 3], v4.w, s1);
            }
        };
        float den0, den1;
        dot2(LA_HD, den0, den1);
        den0 += eps;
        den1 += eps;
        uint4* op0 = reinterpret_cast<uint4*>(out + (static_cast<size_t>(b) * tokens + t) * D + LA_HD * h);
        uint4* op1 = reinterpret_cast<uint4*>(out + (static_cast<size_t>(b) * tokens + (has1 ? t1 : t)) * D + LA_HD * h);
#pragma unroll 1
        for (int j = 0; j < 4; ++j) {
            uint32_t o0[4], o1[4];
#pragma unroll
            for (int i2 = 0; i2 < 4; ++i2) {
                float a0, a1, b0, b1;
                dot2(8 * j + 2 * i2, a0, a1);
                dot2(8 * j + 2 * i2 + 1, b0, b1);
                const __nv_bfloat162 p0 = __floats2bfloat162_rn(__fdividef(a0, den0), __fdividef(b0, den0));
                const __nv_bfloat162 p1 = __floats2bfloat162_rn(__fdividef(a1, den1), __fdividef(b1, den1));
                o0[i2] = *reinterpret_cast<const uint32_t*>(&p0);
                o1[i2] = *reinterpret_cast<const uint32_t*>(&p1);
            }
            op0[j] = make_uint4(o0[0], o0[1], o0[2], o0[3]);
            if (has1) op1[j] = make_uint4(o1[0], o1[1], o1[2], o1[3]);
        }
    }
}

}  // namespace svdq

extern "C" int svdq_litela(const svdq_litela_args* a, void* stream) {
    using namespace svdq;
    SVDQ_CHECK_ARG(a && a->out && (a->qkv || a->mode == 2) && (a->vk || a->mode == 0), "litela: null pointer");
    SVDQ_CHECK_ARG(a->mode >= 0 && a->mode <= 2, "litela: mode must be 0 (all), 1 (vk and relu(Q) only) or 2 (finish from vk)");
    SVDQ_CHECK_ARG(a->batches > 0 && a->batches <= 65535 && a->tokens > 0 && a->heads > 0,
                   "litela: batches (%d, at most 65535), tokens (%d) and heads (%d) must be positive", a->batches, a->tokens, a->heads);
    SVDQ_CHECK_ARG(aligned(a->qkv, 16) && aligned(a->out, 16) && aligned(a->vk, 16), "litela: tensors must be 16-byte aligned");
    if (int rc = check_arch()) return rc;
    litela_kernel<<<dim3(a->heads, a->batches), LA_WARPS * 32, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(a->qkv), static_cast<__nv_bfloat16*>(a->out), a->vk, a->tokens, a->heads, a->eps, a->mode);
    SVDQ_CUDA(cudaGetLastError());
    return SVDQ_OK;
}

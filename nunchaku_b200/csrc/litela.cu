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
//
// Compiled once per 16-bit type (see dtype.cuh): bf16 here, fp16 from litela_f16.cu; the entry point picks by `dtype`.
#include "dtype.cuh"
#include "host_common.h"

namespace svdq {
namespace SVDQ_DT {

constexpr int LA_HD = 32;
constexpr int LA_WARPS = 8;
constexpr int LA_SLAB = 16;                      // tokens per warp step = the k (phase 1) / m (phase 2) extent of one mma

__device__ __forceinline__ void la_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) { mma_16816(c, a, b0, b1); }
__device__ __forceinline__ void la_ldsm(uint32_t (&r)[4], uint32_t saddr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(saddr));
}
__device__ __forceinline__ void la_ldsm_t(uint32_t (&r)[4], uint32_t saddr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(saddr));
}
// max(x, 0) on two packed 16-bit values
__device__ __forceinline__ uint32_t la_relu2(uint32_t w) {
#ifdef SVDQ_F16
    const __half2 r = __hmax2(*reinterpret_cast<const __half2*>(&w), __float2half2_rn(0.f));
#else
    const __nv_bfloat162 r = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&w), __floats2bfloat162_rn(0.f, 0.f));
#endif
    return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ uint4 la_relu8(uint4 w) { return make_uint4(la_relu2(w.x), la_relu2(w.y), la_relu2(w.z), la_relu2(w.w)); }
__device__ __forceinline__ uint32_t la_pack(float a, float b) { return pack2(make_float2(a, b)); }
constexpr uint32_t kLaOnes2 = kF16 ? 0x3c003c00u : 0x3f803f80u;   // two packed 1.0

// Both contractions run on the tensor cores (mma.sync m16n8k16, bf16 operands, fp32 accumulation):
//   phase 1  vk[r, c] = sum_tok Vx[tok, r] * relu(K)[tok, c]: M = r (Vx = V with a 33rd column of ones, which makes row 32 the
//            column sums of relu(K)), N = c, K = tokens.  A warp walks slabs of 16 tokens; the [K_h | V_h] lines of a slab
//            go through a 128B-swizzled tile of shared memory (relu applied on the way) and come back as fragments with
//            transposed ldmatrix (both operands have the contraction index as their slow one).  Products of bf16 values are
//            exact in fp32, so only the order of additions differs from the scalar formulation.
//   phase 2  o[tok, j] = sum_i relu(Q)[tok, i] * vk[j, i]: M = tokens, N = j (33 -> five 8-column tiles), K = i.  vk is fp32:
//            it enters as a bf16 high part plus a bf16 low part (two mma per tile; the split is exact to 2^-17).
__global__ void __launch_bounds__(LA_WARPS * 32)
litela_kernel(const h16* __restrict__ qkv, h16* __restrict__ out, float* __restrict__ vk_out,
              int tokens, int heads, float eps, int mode) {
    __shared__ __align__(128) float part[LA_WARPS][LA_HD + 1][LA_HD];   // 33.8 KB; a warp's slice doubles as its staging tile
    __shared__ __align__(16) float vk[LA_HD + 1][LA_HD];
    const int h = blockIdx.x, b = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t4 = lane & 3;
    const int D = heads * LA_HD;
    const size_t pitch = static_cast<size_t>(3) * D;
    const h16* base = qkv + static_cast<size_t>(b) * tokens * pitch;
    const h16* kv = base + D + 64 * h;
    uint8_t* tile = reinterpret_cast<uint8_t*>(&part[warp][0][0]);   // 16 tokens x 128 B ([K | V]) or 16 x 64 B (Q)
    const uint32_t tile_s = static_cast<uint32_t>(__cvta_generic_to_shared(tile));
    // mode 0: everything.  The reference does it in two launches, and the two halves exist on their own for callers
    // that follow it: mode 1 = what its GEMM epilogue leaves behind (vk, and relu(Q) as bf16 in `out`), mode 2 = its
    // vk_mul_q_kernel (reads relu(Q) from `out` and vk from `vk_out`, finishes `out` in place; qkv is not read).
    if (mode == 2) {
        for (int i = threadIdx.x; i < (LA_HD + 1) * LA_HD; i += LA_WARPS * 32)
            vk[i >> 5][i & 31] = vk_out[(static_cast<size_t>(b) * heads + h) * (LA_HD + 1) * LA_HD + i];
        __syncthreads();
    } else {
        // ---------------------------------------------------------------- phase 1
        float acc[3][4][4];   // [m-tile: r 0-15, 16-31, row 32 (+ padding)][n-tile: 8 columns c][fragment]
#pragma unroll
        for (int i = 0; i < 3; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;
        // A fragment of the ones row: row g = 0 of the third m-tile is 1 for every token of the slab
        const uint32_t one2 = g == 0 ? kLaOnes2 : 0u;
        const uint32_t ones[4] = {one2, 0u, one2, 0u};
        // a lane brings 16-byte chunk (lane & 7) of the lines of tokens (lane >> 3) + 4 i
        auto load_slab = [&](int t0, uint4 (&w)[4]) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int t = t0 + (lane >> 3) + 4 * i;
                w[i] = t < tokens ? *reinterpret_cast<const uint4*>(kv + static_cast<size_t>(t) * pitch + (lane & 7) * 8) : make_uint4(0, 0, 0, 0);
            }
        };
        uint4 cur[4], nxt[4];
        int t0 = warp * LA_SLAB;
        if (t0 < tokens) load_slab(t0, cur);
        for (; t0 < tokens; t0 += LA_WARPS * LA_SLAB) {
            const int t1 = t0 + LA_WARPS * LA_SLAB;
            if (t1 < tokens) load_slab(t1, nxt);   // in flight while this slab is multiplied
            __syncwarp();                          // the previous slab's fragments have been read
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int tok = (lane >> 3) + 4 * i, c = lane & 7;   // chunks 0-3: K (relu), 4-7: V
                *reinterpret_cast<uint4*>(tile + tok * 128 + ((c ^ (tok & 7)) << 4)) = c < 4 ? la_relu8(cur[i]) : cur[i];
            }
            __syncwarp();
            // B fragments: relu(K) [tok][c], transposed loads: matrices (tok 0-7 | 8-15) x (c 8n..8n+7) for two n-tiles each
            uint32_t bk[2][4];
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int tok = (lane & 7) + ((lane >> 3) & 1) * 8, chunk = 2 * half + (lane >> 4);
                la_ldsm_t(bk[half], tile_s + tok * 128 + ((chunk ^ (tok & 7)) << 4));
            }
            // A fragments: V [tok][r], transposed loads: matrices (tok 0-7, r lo) (tok 0-7, r hi) (tok 8-15, r lo) (tok 8-15, r hi)
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
                uint32_t av[4];
                const int tok = (lane & 7) + (lane >> 4) * 8, chunk = 4 + 2 * mt + ((lane >> 3) & 1);
                la_ldsm_t(av, tile_s + tok * 128 + ((chunk ^ (tok & 7)) << 4));
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) la_mma(acc[mt][nt], av, bk[nt >> 1][2 * (nt & 1)], bk[nt >> 1][2 * (nt & 1) + 1]);
            }
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) la_mma(acc[2][nt], ones, bk[nt >> 1][2 * (nt & 1)], bk[nt >> 1][2 * (nt & 1) + 1]);
#pragma unroll
            for (int i = 0; i < 4; ++i) cur[i] = nxt[i];
        }
        __syncwarp();   // the staging tile is about to become this warp's partial
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                *reinterpret_cast<float2*>(&part[warp][16 * mt + g][8 * nt + 2 * t4]) = make_float2(acc[mt][nt][0], acc[mt][nt][1]);
                *reinterpret_cast<float2*>(&part[warp][16 * mt + g + 8][8 * nt + 2 * t4]) = make_float2(acc[mt][nt][2], acc[mt][nt][3]);
            }
        if (g == 0) {
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
                *reinterpret_cast<float2*>(&part[warp][LA_HD][8 * nt + 2 * t4]) = make_float2(acc[2][nt][0], acc[2][nt][1]);
        }
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
            reinterpret_cast<uint4*>(out + (static_cast<size_t>(b) * tokens + t) * D + LA_HD * h)[j] = la_relu8(w);
        }
        return;
    }

    // -------------------------------------------------------------------- phase 2
    // B fragments of vk^T (column j = 8 n + g, rows i = 16 s + 2 t4 .. and + 8), high and low 16-bit parts; the fifth n-tile
    // holds row 32 (the denominator) in its column 0
    // fp16 has 5 exponent bits: vk (sums over all tokens) is brought to [2^13, 2^14) at its largest entry by a power of two
    // first; numerator and denominator of the quotient below carry the same factor, eps takes it too.
    float vscale = 1.f;
    if constexpr (kF16) {
        float m = 0.f;
        for (int i = lane; i < (LA_HD + 1) * LA_HD; i += 32) m = fmaxf(m, fabsf(vk[i >> 5][i & 31]));
#pragma unroll
        for (int d = 16; d >= 1; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
        if (m > 0.f && m < 3.0e38f) {
            const int e = static_cast<int>((__float_as_uint(m) >> 23) & 0xff) - 127;   // floor(log2 m) for normal m
            int k = 13 - e;
            k = k < -100 ? -100 : (k > 100 ? 100 : k);
            vscale = __uint_as_float(static_cast<uint32_t>(127 + k) << 23);
        }
    }
    uint32_t bh[5][2][2], bl[5][2][2];
#pragma unroll
    for (int nt = 0; nt < 5; ++nt)
#pragma unroll
        for (int ks = 0; ks < 2; ++ks)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int j = 8 * nt + g, i = 16 * ks + 8 * hh + 2 * t4;
                float v0 = 0.f, v1 = 0.f;
                if (j <= LA_HD) {
                    v0 = vk[j][i] * vscale;
                    v1 = vk[j][i + 1] * vscale;
                }
                const float h0 = h2f(f2h(v0)), h1 = h2f(f2h(v1));
                bh[nt][ks][hh] = la_pack(h0, h1);
                bl[nt][ks][hh] = la_pack(v0 - h0, v1 - h1);
            }
    for (int t0 = warp * LA_SLAB; t0 < tokens; t0 += LA_WARPS * LA_SLAB) {
        // relu(Q) of 16 tokens -> 64-byte rows of the staging tile (16-byte chunk c of token tok at c ^ ((tok >> 1) & 3))
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int tok = (lane >> 2) + 8 * i, c = lane & 3, t = t0 + tok;
            uint4 w = make_uint4(0, 0, 0, 0);
            if (t < tokens)
                w = mode == 2 ? reinterpret_cast<const uint4*>(out + (static_cast<size_t>(b) * tokens + t) * D + LA_HD * h)[c]
                              : reinterpret_cast<const uint4*>(base + static_cast<size_t>(t) * pitch + LA_HD * h)[c];
            *reinterpret_cast<uint4*>(tile + tok * 64 + ((c ^ ((tok >> 1) & 3)) << 4)) = la_relu8(w);
        }
        __syncwarp();
        float o[5][4];
#pragma unroll
        for (int nt = 0; nt < 5; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) o[nt][e] = 0.f;
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
            uint32_t aq[4];   // matrices (tok 0-7, i lo) (tok 8-15, i lo) (tok 0-7, i hi) (tok 8-15, i hi) of this k-step
            const int tok = (lane & 7) + ((lane >> 3) & 1) * 8, c = 2 * ks + (lane >> 4);
            la_ldsm(aq, tile_s + tok * 64 + ((c ^ ((tok >> 1) & 3)) << 4));
#pragma unroll
            for (int nt = 0; nt < 5; ++nt) {
                la_mma(o[nt], aq, bh[nt][ks][0], bh[nt][ks][1]);
                la_mma(o[nt], aq, bl[nt][ks][0], bl[nt][ks][1]);
            }
        }
        // the denominators of rows g and g + 8 sit in column 0 of the fifth tile: lanes with t4 == 0
        const float den0 = __shfl_sync(0xffffffffu, o[4][0], lane & ~3) + eps * vscale;
        const float den1 = __shfl_sync(0xffffffffu, o[4][2], lane & ~3) + eps * vscale;
        const int ta = t0 + g, tb = t0 + g + 8;
        // lane t4 of a quad holds columns 8 n + 2 t4 (+1) of every n-tile n; a 4 x 4 transpose of words inside the quad gives
        // it the eight columns of n-tile t4 instead: one 16-byte store per row, 64 contiguous bytes per quad
        uint32_t wa[4], wb[4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            wa[nt] = la_pack(__fdividef(o[nt][0], den0), __fdividef(o[nt][1], den0));
            wb[nt] = la_pack(__fdividef(o[nt][2], den1), __fdividef(o[nt][3], den1));
        }
        auto quad_transpose = [&](uint32_t (&w)[4]) {
#pragma unroll
            for (int d = 1; d <= 2; d <<= 1) {          // exchange across lane bit d
                const bool up = (t4 & d) != 0;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (i & d) continue;                 // pairs (i, i + d)
                    const uint32_t send = up ? w[i] : w[i + d];
                    const uint32_t got = __shfl_xor_sync(0xffffffffu, send, d);
                    if (up) w[i] = got; else w[i + d] = got;
                }
            }
        };
        quad_transpose(wa);
        quad_transpose(wb);
        if (ta < tokens)
            *reinterpret_cast<uint4*>(out + (static_cast<size_t>(b) * tokens + ta) * D + LA_HD * h + 8 * t4) = make_uint4(wa[0], wa[1], wa[2], wa[3]);
        if (tb < tokens)
            *reinterpret_cast<uint4*>(out + (static_cast<size_t>(b) * tokens + tb) * D + LA_HD * h + 8 * t4) = make_uint4(wb[0], wb[1], wb[2], wb[3]);
    }
}

int litela_impl(const svdq_litela_args* a, void* stream) {
    SVDQ_CHECK_ARG(a && a->out && (a->qkv || a->mode == 2) && (a->vk || a->mode == 0), "litela: null pointer");
    SVDQ_CHECK_ARG(a->mode >= 0 && a->mode <= 2, "litela: mode must be 0 (all), 1 (vk and relu(Q) only) or 2 (finish from vk)");
    SVDQ_CHECK_ARG(a->batches > 0 && a->batches <= 65535 && a->tokens > 0 && a->heads > 0,
                   "litela: batches (%d, at most 65535), tokens (%d) and heads (%d) must be positive", a->batches, a->tokens, a->heads);
    SVDQ_CHECK_ARG(aligned(a->qkv, 16) && aligned(a->out, 16) && aligned(a->vk, 16), "litela: tensors must be 16-byte aligned");
    if (int rc = check_arch()) return rc;
    litela_kernel<<<dim3(a->heads, a->batches), LA_WARPS * 32, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const h16*>(a->qkv), static_cast<h16*>(a->out), a->vk, a->tokens, a->heads, a->eps, a->mode);
    SVDQ_CUDA(cudaGetLastError());
    return SVDQ_OK;
}

}  // namespace SVDQ_DT
}  // namespace svdq

#ifndef SVDQ_F16
namespace svdq {
namespace hf {
int litela_impl(const svdq_litela_args* a, void* stream);
}
}  // namespace svdq

extern "C" int svdq_litela(const svdq_litela_args* a, void* stream) {
    if (a && a->dtype == SVDQ_DTYPE_FP16) return svdq::hf::litela_impl(a, stream);
    if (a && a->dtype != SVDQ_DTYPE_BF16) return svdq::fail(SVDQ_ERR_INVALID_ARGUMENT, "litela: bad dtype %d", a->dtype);
    return svdq::bf::litela_impl(a, stream);
}
#endif

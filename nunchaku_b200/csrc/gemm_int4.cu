// INT4 (group 64) W4A4 GEMM with the fused SVDQuant epilogue, sm_100a.
//
// What it computes (reference: gemm_w4a4_kernel, src/kernels/zgemm/gemm_w4a4.cuh:832-928,1046-1095;
// scale application gemm_base.cuh:367-409; epilogue chain gemm_w4a4_launch_impl.cuh:172-420):
//   acc[m, n] = sum_g ascale[m, g] * wscale[n, g] * ( sum_{k in group g} a[m, k] * w[n, k] )     s4|u4 x s4 -> s32
//             + sum_r lora_act[m, r] * Wu[n, r]
//   out[m, n] = act( acc[m, n] + bias[n] )
// The reference accumulates the per-group terms in bf16; here they are accumulated in fp32.
//
// sm_100 has no 4-bit integer MMA kind, so the codes run through tcgen05.mma kind::i8:
//   * weights are expanded to one signed byte per code once, at weight-preparation time (they are static);
//   * activation codes stay packed in HBM (the public tensor) and are unpacked nibble -> byte in shared
//     memory by four converter warps, straight into the 128B-swizzled K-major tile the MMA reads;
//   * a group of 64 k is two K=32 MMAs into its own 128-column int32 TMEM buffer (4 buffers), and eight
//     epilogue warps drain each group: int32 -> fp32 (magic-number add, no I2F), times ascale[m,g] *
//     wscale[n,g], accumulated in registers.  The low-rank branch is one more "group": a kind::tf32 MMA of
//     the fp32 lora_act and LoRA-up tiles whose fp32 result is added as is.
// Requantising epilogue (GELU + next layer, gemm_w4a4_launch_impl.cuh:282-309): an epilogue thread holds one row x 64
// columns, which is exactly one INT4 group of the next layer, so the u4 codes of bf16(bf16(y + 0.171875) / smooth_next)
// and their bf16 scale (max / 15) come out of registers; the staged bf16 tile feeds the next layer's LoRA-down
// (ldmatrix + mma.sync), kept deterministic like in the NVFP4 kernel: contiguous tile runs per CTA, one partial per
// row block, column half and CTA in caller scratch, a second small kernel adds them in a fixed order.
// One persistent CTA per SM, 128 x 128 output tiles, K in steps of 128 (two groups per stage).
//   warp 0       TMA producer      warp 1       MMA issuer       warps 2..5   nibble -> s8 converters
//   warps 6..13  epilogue (lane quadrant = warp % 4, column half = (warp - 6) / 4)
// The rescale work (M*N*K/64 fused multiply-adds on the SIMT pipes) is what bounds this kernel, not the
// tensor pipe: that is the price of group-64 integer scales on a machine whose block-scaled MMA kinds only
// exist for FP4/FP8 with power-of-two or E4M3 scales.
#include <cuda_bf16.h>

#include "host_common.h"
#include "ptx.cuh"
#include "quant_common.cuh"

namespace svdq {

constexpr int I_BM = 128;
constexpr int I_BN = 128;
constexpr int I_PK_STAGES = 4;                      // packed activation staging ring
constexpr int I_PK_BYTES = I_BM * 64;               // 128 rows x 128 codes packed = 8 KB
constexpr int I_U_STAGES = 3;                       // unpacked operand ring
constexpr int I_A_BYTES = I_BM * 128;               // 16 KB (s8, 128 k per row)
constexpr int I_B_BYTES = I_BN * 128;               // 16 KB
constexpr int I_U_BYTES = I_A_BYTES + I_B_BYTES;
constexpr int I_EPI_BUF_BYTES = 32 * 128;           // 32 rows x 64 bf16
constexpr int I_EPI_BYTES = 8 * I_EPI_BUF_BYTES;
constexpr int I_THREADS = 14 * 32;
constexpr int I_TBUFS = 4;                          // TMEM group buffers of 128 columns
constexpr int I_RCP_BYTES = 8 * 64 * 4;             // per epilogue warp: 1 / smooth_next of its 64 columns
constexpr size_t I_SMEM_BYTES =
    1024 + static_cast<size_t>(I_U_STAGES) * I_U_BYTES + I_PK_STAGES * I_PK_BYTES + I_EPI_BYTES + I_RCP_BYTES + 512;

struct Int4Params {
    const __nv_bfloat16* ascales;   // [K/64][M_pad]
    const __nv_bfloat16* wscales;   // [K/64][N]
    const float* col_bias;          // [N]
    int* status;
    int M, M_pad, N, K;
    int lora_chunks;
    int tiles_m, tiles_n;
    int activation;
    int act_unsigned;
    int store_out;            // bf16 `out` is wanted
    // tile schedule: 0: m-fastest, strided by gridDim; 1: n-fastest, each CTA a contiguous run of `run` tiles
    int contiguous;
    int run;
    // requantising epilogue (GELU + next layer's INT4 quantisation + LoRA-down)
    uint8_t* qout;                      // [M_pad][N/2]
    __nv_bfloat16* oscales;             // [N/64][M_pad]
    const __nv_bfloat16* next_smooth;   // [N] reference-packed
    const uint4* next_lora_down;        // reference-packed [N/16][Rn/16][32] x 16 bytes
    float* lora_partial;                // scratch [CTA][slot][column half 2][128][Rn]
    int slots;
    int next_unsigned;                  // u4 codes of (y + 0.171875) / smooth, as the reference's INT4 chain uses
};

struct I4Run {
    int first, stride, count;
};
__device__ __forceinline__ I4Run i4_run(const Int4Params& p) {
    const int num_tiles = p.tiles_m * p.tiles_n;
    I4Run r;
    if (p.contiguous) {
        r.first = blockIdx.x * p.run;
        r.stride = 1;
        r.count = max(0, min(p.run, num_tiles - r.first));
    } else {
        r.first = blockIdx.x;
        r.stride = gridDim.x;
        r.count = num_tiles > r.first ? (num_tiles - r.first + r.stride - 1) / r.stride : 0;
    }
    return r;
}
__device__ __forceinline__ void i4_coords(const Int4Params& p, int tile, int& m0, int& n0) {
    if (p.contiguous) {
        m0 = (tile / p.tiles_n) * I_BM;
        n0 = (tile % p.tiles_n) * I_BN;
    } else {
        m0 = (tile % p.tiles_m) * I_BM;
        n0 = (tile / p.tiles_m) * I_BN;
    }
}

struct Int4Shared {
    uint64_t pk_full[I_PK_STAGES];
    uint64_t pk_empty[I_PK_STAGES];
    uint64_t b_full[I_U_STAGES];    // weights (or both low-rank tiles) of the stage have landed
    uint64_t a_full[I_U_STAGES];    // converters have written the stage's activation tile
    uint64_t u_empty[I_U_STAGES];   // MMAs that read the stage are done
    uint64_t t_full[I_TBUFS];
    uint64_t t_empty[I_TBUFS];
    uint64_t drain;
    uint32_t tmem_base;
    volatile int abort_flag;
};

__device__ __forceinline__ bool i4_wait(uint64_t* bar, uint32_t parity, Int4Shared* sh, int* status, int where) {
#pragma unroll 1
    for (int i = 0; i < 512; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 128; ++i) {
            if (mbar_try_wait(bar, parity)) return true;
        }
        if (sh->abort_flag) return false;
        if (clock64() - t0 > 4000000000ll) {
            sh->abort_flag = 1;
            atomicExch(&status[0], SVDQ_ERR_TIMEOUT);
            atomicExch(&status[1], where);
            return false;
        }
    }
}

__device__ __forceinline__ float i4_act(float v, int activation) {
    if (activation == SVDQ_ACT_SILU) return v / (1.0f + __expf(-v));
    if (activation == SVDQ_ACT_GELU) {
        float t;
        asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.79788456f * (v + 0.044715f * v * v * v)));
        return v * (0.5f + 0.5f * t);
    }
    return v;
}

// RTN: rank tiles (of 16) of the next layer's LoRA-down; 0 = plain epilogue (no requantisation).
template <int RTN>
__global__ void __launch_bounds__(I_THREADS, 1)
gemm_int4_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                 const __grid_constant__ CUtensorMap tm_la, const __grid_constant__ CUtensorMap tm_lu,
                 const __grid_constant__ CUtensorMap tm_out, const Int4Params p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* ubuf = smem;                                           // [I_U_STAGES][A 16K | B 16K]
    uint8_t* epi_smem = ubuf + I_U_STAGES * I_U_BYTES;              // 8 x 4 KB, 1024-aligned
    uint8_t* pkbuf = epi_smem + I_EPI_BYTES;                        // [I_PK_STAGES][8K]
    float* rcp_smem = reinterpret_cast<float*>(pkbuf + I_PK_STAGES * I_PK_BYTES);   // [8 warps][64]
    Int4Shared* sh = reinterpret_cast<Int4Shared*>(pkbuf + I_PK_STAGES * I_PK_BYTES + I_RCP_BYTES);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int kstages = p.K / 128;
    const int per_tile = kstages + p.lora_chunks;       // stages per tile
    const I4Run tr = i4_run(p);

    if (threadIdx.x == 0) {
        for (int s = 0; s < I_PK_STAGES; ++s) {
            mbar_init(&sh->pk_full[s], 1);
            mbar_init(&sh->pk_empty[s], 4);
        }
        for (int s = 0; s < I_U_STAGES; ++s) {
            mbar_init(&sh->b_full[s], 1);
            mbar_init(&sh->a_full[s], 4);
            mbar_init(&sh->u_empty[s], 1);
        }
        for (int i = 0; i < I_TBUFS; ++i) {
            mbar_init(&sh->t_full[i], 1);
            mbar_init(&sh->t_empty[i], 8);
        }
        mbar_init(&sh->drain, 1);
        sh->abort_flag = 0;
        fence_mbar_init();
        prefetch_tmap(&tm_a);
        prefetch_tmap(&tm_b);
        prefetch_tmap(&tm_out);
    }
    if (warp == 1) {
        tmem_alloc(&sh->tmem_base, 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = sh->tmem_base;

    if (warp == 0) {
        // ------------------------------------------------------------------ producer (whole warp, elected lane issues)
        uint32_t it = 0, pk = 0;   // unpacked-ring position, packed-ring position
        bool ok = true;
        for (int ti = 0; ti < tr.count && ok; ++ti) {
            int m0, n0;
            i4_coords(p, tr.first + ti * tr.stride, m0, n0);
            for (int ks = 0; ks < per_tile; ++ks, ++it) {
                const int u = it % I_U_STAGES;
                uint8_t* ub = ubuf + u * I_U_BYTES;
                if (ks < kstages) {
                    // packed activations -> staging ring (independent of the unpacked ring's progress)
                    const int s = pk % I_PK_STAGES;
                    ok = __all_sync(0xffffffffu, i4_wait(&sh->pk_empty[s], ((pk / I_PK_STAGES) & 1) ^ 1, sh, p.status, 10));
                    if (!ok) break;
                    if (elect_one()) {
                        mbar_arrive_expect_tx(&sh->pk_full[s], I_PK_BYTES);
                        tma_load_2d(pkbuf + s * I_PK_BYTES, &tm_a, &sh->pk_full[s], ks * 64, m0);
                    }
                    __syncwarp();
                    ++pk;
                    ok = __all_sync(0xffffffffu, i4_wait(&sh->u_empty[u], ((it / I_U_STAGES) & 1) ^ 1, sh, p.status, 11));
                    if (!ok) break;
                    if (elect_one()) {
                        mbar_arrive_expect_tx(&sh->b_full[u], I_B_BYTES);
                        tma_load_2d(ub + I_A_BYTES, &tm_b, &sh->b_full[u], ks * 128, n0);
                    }
                    __syncwarp();
                } else {
                    const int c = ks - kstages;
                    ok = __all_sync(0xffffffffu, i4_wait(&sh->u_empty[u], ((it / I_U_STAGES) & 1) ^ 1, sh, p.status, 12));
                    if (!ok) break;
                    if (elect_one()) {
                        mbar_arrive_expect_tx(&sh->b_full[u], I_A_BYTES + I_B_BYTES);
                        tma_load_2d(ub, &tm_la, &sh->b_full[u], c * 32, m0);
                        tma_load_2d(ub + I_A_BYTES, &tm_lu, &sh->b_full[u], c * 32, n0);
                    }
                    __syncwarp();
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (whole warp, elected lane issues:
        // descriptors and TMEM addresses stay warp-uniform, see ptx.cuh elect_one)
        const uint32_t idesc_int8 = idesc_i8(I_BM, I_BN, !p.act_unsigned);
        constexpr uint32_t IDESC_TF32 = idesc_tf32(I_BM, I_BN);
        const uint64_t adesc0 = smem_desc_sw128(smem_u32(ubuf));
        uint32_t it = 0, gq = 0;   // stage count, group (TMEM buffer) count
        bool ok = true;
        for (int ti = 0; ti < tr.count && ok; ++ti) {
            for (int ks = 0; ks < per_tile && ok; ++ks, ++it) {
                const int u = it % I_U_STAGES;
                ok = __all_sync(0xffffffffu, i4_wait(&sh->b_full[u], (it / I_U_STAGES) & 1, sh, p.status, 20) &&
                                                 i4_wait(&sh->a_full[u], (it / I_U_STAGES) & 1, sh, p.status, 21));
                if (!ok) break;
                tc_fence_after_sync();
                const uint64_t adesc = adesc0 + static_cast<uint32_t>(u * (I_U_BYTES >> 4));
                const uint64_t bdesc = adesc + (I_A_BYTES >> 4);
                const int ngroups = ks < kstages ? 2 : 1;
                for (int g = 0; g < ngroups; ++g, ++gq) {
                    const uint32_t tb = gq % I_TBUFS;
                    ok = __all_sync(0xffffffffu, i4_wait(&sh->t_empty[tb], ((gq / I_TBUFS) & 1) ^ 1, sh, p.status, 22));
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t d = tmem + tb * 128;
                    if (elect_one()) {
                        if (ks < kstages) {
                            tc_mma_i8(d, adesc + 4 * g, bdesc + 4 * g, idesc_int8, 0);
                            tc_mma_i8(d, adesc + 4 * g + 2, bdesc + 4 * g + 2, idesc_int8, 1);
                        } else {
#pragma unroll
                            for (int j = 0; j < 4; ++j) tc_mma_tf32(d, adesc + 2 * j, bdesc + 2 * j, IDESC_TF32, j ? 1u : 0u);
                        }
                        tc_commit(&sh->t_full[tb]);
                    }
                    __syncwarp();
                }
                if (ok) {
                    if (elect_one()) tc_commit(&sh->u_empty[u]);
                    __syncwarp();
                }
            }
        }
        if (sh->abort_flag) {
            if (lane == 0) {
                tc_commit(&sh->drain);
                mbar_wait(&sh->drain, 0, 400000000ll);
            }
            __syncwarp();
        }
    } else if (warp < 6) {
        // ------------------------------------------------------------------ converters (warps 2..5)
        // 128 rows x 64 packed bytes -> 128 rows x 128 s8 bytes in the 128B-swizzled K-major layout.
        // Task = one 16-byte chunk (32 codes); consecutive lanes take consecutive chunks of the staging tile.
        const int ct = threadIdx.x - 64;   // 0..127
        const bool is_signed = !p.act_unsigned;
        uint32_t it = 0, pk = 0;
        bool ok = true;
        for (int ti = 0; ti < tr.count && ok; ++ti) {
            for (int ks = 0; ks < per_tile; ++ks, ++it) {
                const int u = it % I_U_STAGES;
                if (ks < kstages) {
                    const int s = pk % I_PK_STAGES;
                    if (!i4_wait(&sh->pk_full[s], (pk / I_PK_STAGES) & 1, sh, p.status, 30) ||
                        !i4_wait(&sh->u_empty[u], ((it / I_U_STAGES) & 1) ^ 1, sh, p.status, 31)) { ok = false; break; }
                    const uint8_t* src = pkbuf + s * I_PK_BYTES;
                    uint8_t* dst = ubuf + u * I_U_BYTES;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int idx = i * 128 + ct;
                        const int row = idx >> 2, c = idx & 3;
                        const uint4 w = *reinterpret_cast<const uint4*>(src + idx * 16);
                        const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
                        uint32_t o[8];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint32_t lo = ws[j] & 0x0F0F0F0Fu, hi = (ws[j] >> 4) & 0x0F0F0F0Fu;
                            if (is_signed) {
                                lo |= (lo & 0x08080808u) * 0x1Eu;
                                hi |= (hi & 0x08080808u) * 0x1Eu;
                            }
                            o[2 * j] = __byte_perm(lo, hi, 0x5140);
                            o[2 * j + 1] = __byte_perm(lo, hi, 0x7362);
                        }
                        uint8_t* drow = dst + row * 128;
                        *reinterpret_cast<uint4*>(drow + (((2 * c) ^ (row & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                        *reinterpret_cast<uint4*>(drow + (((2 * c + 1) ^ (row & 7)) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
                    }
                    fence_proxy_async_smem();   // generic-proxy writes -> visible to the tensor core (async proxy)
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(&sh->pk_empty[s]);
                        mbar_arrive(&sh->a_full[u]);
                    }
                    ++pk;
                } else {
                    // low-rank stage: both tiles come by TMA; still wait for the buffer's previous use so that
                    // this barrier never runs a phase ahead of the MMA issuer
                    if (!i4_wait(&sh->u_empty[u], ((it / I_U_STAGES) & 1) ^ 1, sh, p.status, 32)) { ok = false; break; }
                    if (lane == 0) mbar_arrive(&sh->a_full[u]);
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 6..13)
        const int q = warp & 3;            // TMEM lane quadrant
        const int h = (warp - 6) >> 2;     // column half (64 columns)
        uint8_t* buf = epi_smem + (warp - 6) * I_EPI_BUF_BYTES;
        const int KB = p.K / 64;
        uint32_t gq = 0;
        bool ok = true;
        // next layer's LoRA-down partial of this warp's 32 rows x its column half: [m-tile 2][rank tile][8]
        constexpr int RTA = RTN > 0 ? RTN : 1;
        float lacc[2][RTA][8];
        float* rcs = rcp_smem + (warp - 6) * 64;
        int cur_m0 = -1, slot = 0;
        auto lacc_zero = [&]() {
#pragma unroll
            for (int a = 0; a < 2; ++a)
#pragma unroll
                for (int b = 0; b < RTA; ++b)
#pragma unroll
                    for (int c = 0; c < 8; ++c) lacc[a][b][c] = 0.f;
        };
        auto lacc_flush = [&]() {   // partial of row block cur_m0 -> scratch[blockIdx][slot][h][128][Rn]
            if constexpr (RTN > 0) {
                constexpr int RN = RTN * 16;
                float* dst = p.lora_partial + ((static_cast<size_t>(blockIdx.x) * p.slots + slot) * 2 + h) * (I_BM * RN);
                const int gq4 = lane >> 2, t = lane & 3;
#pragma unroll
                for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                    for (int rt = 0; rt < RTN; ++rt)
#pragma unroll
                        for (int nh = 0; nh < 2; ++nh)
#pragma unroll
                            for (int half = 0; half < 2; ++half) {
                                const int row = q * 32 + mt * 16 + gq4 + half * 8;
                                const int rank = rt * 16 + nh * 8 + 2 * t;
                                *reinterpret_cast<float2*>(dst + row * RN + rank) =
                                    make_float2(lacc[mt][rt][nh * 4 + half * 2], lacc[mt][rt][nh * 4 + half * 2 + 1]);
                            }
                ++slot;
            }
        };
        lacc_zero();
        for (int ti = 0; ti < tr.count && ok; ++ti) {
            int m0, n0;
            i4_coords(p, tr.first + ti * tr.stride, m0, n0);
            const int m = m0 + q * 32 + lane;               // < M_pad always
            const int nb = n0 + h * 64;
            if constexpr (RTN > 0) {
                if (m0 != cur_m0) {
                    if (cur_m0 >= 0) {
                        lacc_flush();
                        lacc_zero();
                    }
                    cur_m0 = m0;
                }
                // 1 / smooth_next of this warp's 64 columns (issued before the accumulators are needed)
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int n = nb + lane + 32 * i;
                    float r = 0.f;
                    if (n < p.N) r = __frcp_rn(__bfloat162float(p.next_smooth[(n & ~127) + packed_vec_pos(n & 127)]));
                    rcs[lane + 32 * i] = r;
                }
                __syncwarp();
            }
            __align__(8) float acc[64];
#pragma unroll
            for (int i = 0; i < 64; ++i) acc[i] = 0.f;
            const __nv_bfloat16* asp = p.ascales + m;
            float as_next = __bfloat162float(asp[0]);
            const int groups = KB + p.lora_chunks;
            for (int g = 0; g < groups; ++g, ++gq) {
                const uint32_t tb = gq % I_TBUFS;
                const float as_g = as_next;
                if (g + 1 < KB) as_next = __bfloat162float(asp[static_cast<size_t>(g + 1) * p.M_pad]);
                // this group's 64 weight scales (bf16, the same for every row): in flight while the MMAs finish
                uint4 wsr[8];
                if (g < KB) {
                    const uint4* wsp = reinterpret_cast<const uint4*>(p.wscales + static_cast<size_t>(g) * p.N + nb);
#pragma unroll
                    for (int i = 0; i < 8; ++i) wsr[i] = __ldg(wsp + i);
                }
                if (!i4_wait(&sh->t_full[tb], (gq / I_TBUFS) & 1, sh, p.status, 40)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t taddr = tmem + (static_cast<uint32_t>(q * 32) << 16) + tb * 128 + h * 64;
                if (g < KB) {
#pragma unroll
                    for (int qt = 0; qt < 4; ++qt) {
                        uint32_t r[16];
                        tc_ld_32x32b_x16(taddr + qt * 16, r);
                        tc_wait_ld();
#pragma unroll
                        for (int i = 0; i < 8; ++i) {       // word i of the quarter = columns 2i, 2i+1
                            const uint4 wq = wsr[2 * qt + (i >> 2)];
                            const uint32_t ww = (i & 3) == 0 ? wq.x : (i & 3) == 1 ? wq.y : (i & 3) == 2 ? wq.z : wq.w;
                            const float2 w2 = make_float2(__uint_as_float(ww << 16), __uint_as_float(ww & 0xffff0000u));
                            // int32 -> fp32 without I2F: |partial| <= 64*15*8 < 2^22, so 1.5*2^23 + p is exact;
                            // the rest is packed two-wide fp32 arithmetic (the rescale is instruction bound)
                            float2 x2 = make_float2(__int_as_float(0x4B400000 + static_cast<int>(r[2 * i])),
                                                    __int_as_float(0x4B400000 + static_cast<int>(r[2 * i + 1])));
                            x2 = __fadd2_rn(x2, make_float2(-12582912.0f, -12582912.0f));
                            const float2 s2 = __fmul2_rn(make_float2(as_g, as_g), w2);
                            float2* a2 = reinterpret_cast<float2*>(&acc[qt * 16 + 2 * i]);
                            *a2 = __ffma2_rn(x2, s2, *a2);
                        }
                    }
                } else {
#pragma unroll
                    for (int qt = 0; qt < 4; ++qt) {
                        uint32_t r[16];
                        tc_ld_32x32b_x16(taddr + qt * 16, r);
                        tc_wait_ld();
#pragma unroll
                        for (int i = 0; i < 16; ++i) acc[qt * 16 + i] += __uint_as_float(r[i]);
                    }
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh->t_empty[tb]);
            }
            if (!ok) break;
            // bias + activation -> bf16 -> swizzled staging -> TMA store of this warp's 32 x 64 box
            if (lane == 0) bulk_wait_group_read<0>();
            __syncwarp();
            if (nb < p.N) {
                const float4* cb = reinterpret_cast<const float4*>(p.col_bias + nb);
#pragma unroll
                uint32_t ow[32];   // this thread's 64 bf16 outputs, packed (kept for the requantisation)
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    uint32_t* o = &ow[4 * j];
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const float4 b4 = __ldg(cb + 2 * j + i);
                        const float v0 = i4_act(acc[8 * j + 4 * i + 0] + b4.x, p.activation);
                        const float v1 = i4_act(acc[8 * j + 4 * i + 1] + b4.y, p.activation);
                        const float v2 = i4_act(acc[8 * j + 4 * i + 2] + b4.z, p.activation);
                        const float v3 = i4_act(acc[8 * j + 4 * i + 3] + b4.w, p.activation);
                        __nv_bfloat162 p0 = __floats2bfloat162_rn(v0, v1);
                        __nv_bfloat162 p1 = __floats2bfloat162_rn(v2, v3);
                        o[2 * i] = *reinterpret_cast<uint32_t*>(&p0);
                        o[2 * i + 1] = *reinterpret_cast<uint32_t*>(&p1);
                    }
                    *reinterpret_cast<uint4*>(buf + lane * 128 + ((j ^ (lane & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    if (p.store_out && m0 + q * 32 < p.M) tma_store_2d(&tm_out, buf, nb, m0 + q * 32);
                    bulk_commit_group();
                }
                if constexpr (RTN > 0) {
                    // ---- next layer's LoRA-down on the staged bf16 tile: [32 x 64] x Wd_next[64 x Rn]
                    const int ch_tile0 = nb >> 4;           // 16-channel tile index of the chunk
                    const uint32_t bufa = smem_u32(buf);
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        uint4 bfrag[RTA];
#pragma unroll
                        for (int rt = 0; rt < RTN; ++rt)
                            bfrag[rt] = __ldg(p.next_lora_down + (static_cast<size_t>(ch_tile0 + kk) * RTN + rt) * 32 + lane);
#pragma unroll
                        for (int mt = 0; mt < 2; ++mt) {
                            const int arow = mt * 16 + (lane & 15);
                            uint32_t a[4];
                            ldmatrix_x4(a, bufa + arow * 128 + (((2 * kk + (lane >> 4)) ^ (arow & 7)) << 4));
#pragma unroll
                            for (int rt = 0; rt < RTN; ++rt) {
                                mma_bf16_16816(*reinterpret_cast<float(*)[4]>(&lacc[mt][rt][0]), a, bfrag[rt].x, bfrag[rt].y);
                                mma_bf16_16816(*reinterpret_cast<float(*)[4]>(&lacc[mt][rt][4]), a, bfrag[rt].z, bfrag[rt].w);
                            }
                        }
                    }
                    // ---- INT4 group quantisation: this thread's 64 values are exactly one group
                    // (+0.171875 in bf16 when the codes are unsigned, gemm_w4a4_launch_impl.cuh:282-309) / smooth
                    const float4* rc4 = reinterpret_cast<const float4*>(rcs);
                    uint32_t qv[4][8];
                    float amax = 0.f;
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        uint32_t xw[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            uint32_t w = ow[8 * g + i];
                            if (p.next_unsigned) {
                                const float2 f = bf16x2_to_float2(w);
                                const __nv_bfloat162 sft = __floats2bfloat162_rn(f.x + 0.171875f, f.y + 0.171875f);
                                w = *reinterpret_cast<const uint32_t*>(&sft);
                            }
                            xw[i] = w;
                        }
                        amax = fmaxf(amax, smooth16(xw, rc4 + 4 * g, qv[g]));
                    }
                    uint32_t codes[8];
                    float scale = 0.f;
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        uint32_t cw[2];
                        scale = p.next_unsigned ? int4_encode16<true>(qv[g], amax, cw) : int4_encode16<false>(qv[g], amax, cw);
                        codes[2 * g] = cw[0];
                        codes[2 * g + 1] = cw[1];
                    }
                    uint4* qdst = reinterpret_cast<uint4*>(p.qout + static_cast<size_t>(m) * (p.N >> 1) + (nb >> 1));
                    qdst[0] = make_uint4(codes[0], codes[1], codes[2], codes[3]);
                    qdst[1] = make_uint4(codes[4], codes[5], codes[6], codes[7]);
                    p.oscales[static_cast<size_t>(nb >> 6) * p.M_pad + m] = __float2bfloat16_rn(scale);
                }
            }
        }
        if constexpr (RTN > 0) {
            if (cur_m0 >= 0) lacc_flush();
        }
        if (lane == 0) bulk_wait_group<0>();
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, 512);
    }
}

// lora_act_out[row][r] = sum over the CTAs that touched the row's 128-row block, in CTA order, of the partials of
// their two column halves.  Row block mb holds tiles [mb*tiles_n, (mb+1)*tiles_n); CTA c owns tiles [c*run, (c+1)*run).
__global__ void int4_lora_partial_reduce_kernel(const float* __restrict__ partial, float* __restrict__ out, int rn, int tiles_n,
                                                int run, int slots, int grid_ctas) {
    const int mb = blockIdx.x;
    const int c_lo = (mb * tiles_n) / run;
    const int c_hi = min(grid_ctas - 1, ((mb + 1) * tiles_n - 1) / run);
    for (int i = threadIdx.x; i < I_BM * rn; i += blockDim.x) {
        float s = 0.f;
        for (int c = c_lo; c <= c_hi; ++c) {
            const int first_mb = (c * run) / tiles_n;
            const float* pp = partial + ((static_cast<size_t>(c) * slots + (mb - first_mb)) * 2) * (I_BM * rn);
            s += pp[i];
            s += pp[I_BM * rn + i];
        }
        out[static_cast<size_t>(mb) * I_BM * rn + i] = s;
    }
}

struct Int4Plan {
    int requant, tiles_m, tiles_n, grid, run, slots, rn;
    size_t workspace;
};

static void plan_int4(const svdq_gemm_args* a, int sms, Int4Plan* pl) {
    pl->requant = a->qout != nullptr;
    pl->tiles_n = (a->N + I_BN - 1) / I_BN;
    pl->tiles_m = pl->requant ? a->M_pad / I_BM : (a->M + I_BM - 1) / I_BM;
    const int num_tiles = pl->tiles_m * pl->tiles_n;
    pl->grid = num_tiles < sms ? num_tiles : sms;
    pl->run = (num_tiles + pl->grid - 1) / pl->grid;
    if (pl->requant) pl->grid = (num_tiles + pl->run - 1) / pl->run;
    pl->slots = (pl->run + pl->tiles_n - 2) / pl->tiles_n + 1;
    pl->rn = a->R_next;
    pl->workspace = pl->requant ? static_cast<size_t>(pl->grid) * pl->slots * 2 * I_BM * pl->rn * sizeof(float) : 0;
}

int gemm_int4_workspace_bytes(const svdq_gemm_args* a, size_t* bytes) {
    int dev = 0, sms = 0;
    SVDQ_CUDA(cudaGetDevice(&dev));
    SVDQ_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    Int4Plan pl;
    plan_int4(a, sms, &pl);
    *bytes = pl.workspace;
    return SVDQ_OK;
}

template <int RTN>
static int launch_int4(int grid, cudaStream_t stream, const CUtensorMap& a, const CUtensorMap& b, const CUtensorMap& la,
                       const CUtensorMap& lu, const CUtensorMap& o, const Int4Params& p) {
    static bool attr_done[64] = {};
    int dev = 0;
    SVDQ_CUDA(cudaGetDevice(&dev));
    if (dev < 64 && !attr_done[dev]) {
        SVDQ_CUDA(cudaFuncSetAttribute(gemm_int4_kernel<RTN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(I_SMEM_BYTES)));
        attr_done[dev] = true;
    }
    gemm_int4_kernel<RTN><<<grid, I_THREADS, I_SMEM_BYTES, stream>>>(a, b, la, lu, o, p);
    SVDQ_CUDA(cudaGetLastError());
    return SVDQ_OK;
}

int gemm_int4_impl(const svdq_gemm_args* a, cudaStream_t stream) {
    const bool requant = a->qout != nullptr;
    SVDQ_CHECK_ARG(a->out != nullptr || requant, "gemm(int4): neither `out` nor `qout` given");
    if (requant) {
        SVDQ_CHECK_ARG(a->oscales && a->lora_act_out && a->next_smooth && a->next_lora_down,
                       "gemm(int4): requantisation needs oscales, lora_act_out, next_smooth and next_lora_down");
        SVDQ_CHECK_ARG(!a->next_fp4, "gemm(int4): the requantised output must be INT4 as well");
        SVDQ_CHECK_ARG(a->out_layout == SVDQ_LAYOUT_NATIVE, "gemm(int4): requantised output is written in SVDQ_LAYOUT_NATIVE");
        SVDQ_CHECK_ARG(a->activation == SVDQ_ACT_GELU, "gemm(int4): the requantising epilogue applies GELU "
                                                       "(gemm_w4a4_launch_impl.cuh:282-309); set activation = SVDQ_ACT_GELU");
        SVDQ_CHECK_ARG(aligned(a->qout, 16) && aligned(a->oscales, 16) && aligned(a->lora_act_out, 16) &&
                           aligned(a->next_smooth, 16) && aligned(a->next_lora_down, 16) && aligned(a->workspace, 256),
                       "gemm(int4): requantisation tensors must be 16-byte aligned (workspace: 256)");
        if (a->R_next != 16 && a->R_next != 32 && a->R_next != 64)
            return fail(SVDQ_ERR_UNSUPPORTED, "gemm(int4): fused next-layer LoRA-down is built for rank 16, 32, 64 (got %d)", a->R_next);
    }
    SVDQ_CHECK_ARG(a->act_layout == SVDQ_LAYOUT_NATIVE, "gemm(int4): activations must be in SVDQ_LAYOUT_NATIVE "
                                                        "(convert with svdq_w4a4_relayout_act)");
    SVDQ_CHECK_ARG(a->R % 16 == 0 && a->R >= 0 && a->R <= 128, "gemm: R (%d) must be a multiple of 16, at most 128", a->R);
    SVDQ_CHECK_ARG(a->R == 0 || (a->lora_act_in && a->w.lora_up), "gemm: low-rank tensors missing");

    int dev = 0, sms = 0;
    SVDQ_CUDA(cudaGetDevice(&dev));
    SVDQ_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));

    Int4Params p = {};
    p.ascales = static_cast<const __nv_bfloat16*>(a->ascales);
    p.wscales = static_cast<const __nv_bfloat16*>(a->w.wscales);
    p.col_bias = a->w.col_bias;
    p.M = a->M;
    p.M_pad = a->M_pad;
    p.N = a->N;
    p.K = a->K;
    p.lora_chunks = (a->R + 31) / 32;
    Int4Plan pl;
    plan_int4(a, sms, &pl);
    SVDQ_CHECK_ARG(!requant || (a->workspace && a->workspace_bytes >= pl.workspace),
                   "gemm(int4): workspace of %zu bytes required (svdq_gemm_w4a4_workspace_bytes)", pl.workspace);
    p.tiles_m = pl.tiles_m;
    p.tiles_n = pl.tiles_n;
    p.activation = a->activation;
    p.act_unsigned = a->act_unsigned;
    p.store_out = a->out != nullptr;
    p.contiguous = requant;
    p.run = pl.run;
    p.qout = static_cast<uint8_t*>(a->qout);
    p.oscales = static_cast<__nv_bfloat16*>(a->oscales);
    p.next_smooth = static_cast<const __nv_bfloat16*>(a->next_smooth);
    p.next_lora_down = static_cast<const uint4*>(a->next_lora_down);
    p.lora_partial = static_cast<float*>(a->workspace);
    p.slots = pl.slots;
    p.next_unsigned = 1;   // the reference's INT4 chain always requantises to u4 with the +0.171875 shift (launch_impl.cuh:282-309)
    if (int rc = status_words(&p.status)) return rc;

    CUtensorMap tm_a, tm_b, tm_la, tm_lu, tm_out;
    if (int rc = make_tmap_2d(&tm_a, a->act, CU_TENSOR_MAP_DATA_TYPE_UINT8, a->K / 2, a->M_pad, a->K / 2, 64, I_BM, false)) return rc;
    if (int rc = make_tmap_2d(&tm_b, a->w.wgt, CU_TENSOR_MAP_DATA_TYPE_UINT8, a->K, a->N, a->K, 128, I_BN)) return rc;
    if (a->R > 0) {
        const int R32 = (a->R + 31) / 32 * 32;
        if (int rc = make_tmap_2d(&tm_la, a->lora_act_in, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, a->R, a->M_pad,
                                  static_cast<uint64_t>(a->R) * 4, 32, I_BM))
            return rc;
        if (int rc = make_tmap_2d(&tm_lu, a->w.lora_up, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, R32, a->N,
                                  static_cast<uint64_t>(R32) * 4, 32, I_BN))
            return rc;
    } else {
        tm_la = tm_b;
        tm_lu = tm_b;
    }
    if (a->out) {
        if (int rc = make_tmap_2d(&tm_out, a->out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, a->N, a->M, static_cast<uint64_t>(a->N) * 2, 64, 32))
            return rc;
    } else {
        tm_out = tm_b;
    }
    int rc;
    if (!requant) rc = launch_int4<0>(pl.grid, stream, tm_a, tm_b, tm_la, tm_lu, tm_out, p);
    else if (a->R_next == 16) rc = launch_int4<1>(pl.grid, stream, tm_a, tm_b, tm_la, tm_lu, tm_out, p);
    else if (a->R_next == 32) rc = launch_int4<2>(pl.grid, stream, tm_a, tm_b, tm_la, tm_lu, tm_out, p);
    else rc = launch_int4<4>(pl.grid, stream, tm_a, tm_b, tm_la, tm_lu, tm_out, p);
    if (rc) return rc;
    if (requant) {
        int4_lora_partial_reduce_kernel<<<pl.tiles_m, 256, 0, stream>>>(p.lora_partial, a->lora_act_out, pl.rn, pl.tiles_n, pl.run,
                                                                       pl.slots, pl.grid);
        SVDQ_CUDA(cudaGetLastError());
    }
    return SVDQ_OK;
}

}  // namespace svdq

// W4A4 GEMM (NVFP4 and INT4) with the fused SVDQuant epilogue, sm_100a.
//
// What it computes (reference: gemm_w4a4_fp4_kernel, src/kernels/zgemm/gemm_w4a4.cuh:273-405,
// epilogue chain gemm_w4a4_launch_impl.cuh:172-420):
//   D[m, n]   = sum_k a[m,k]*sa[m,k/16] * w[n,k]*sw[n,k/16]           E2M1 codes, UE4M3 group-16 scales
//             + sum_r lora_act[m,r] * Wu'[n,r]                          low-rank branch, same accumulator
//   y[m, n]   = act( D[m,n] * col_scale[n] + col_bias[n] )             col_scale = alpha * wcscale
// (Wu' is the LoRA-up weight pre-divided by col_scale, so both branches share one fp32 accumulator.)
// Plain epilogue: out = bf16(y).  Requantising epilogue (GELU + next layer, launch_impl.cuh:282-309,
// gemm_w4a4.cuh:930-1043, lora.cuh:243-353): yb = bf16(y);  lora_act_out = yb @ Wd_next^T (fp32);
// codes/scales = group quantisation of bf16(yb / smooth_next);  out (optional) = yb.
// The INT4 variant (template parameter I4; what it computes is stated above gemm_int4_impl) differs only in how the
// operands reach the tensor core and in the group format of the requantised output.
//
// How it maps to a B200.  The two SMs of a CTA pair (cluster of 2) walk 256 x 256 output tiles together with
// tcgen05 cta_group::2: each CTA holds 128 rows of A, 128 rows of the accumulator (its own TMEM) and 128 of the
// tile's 256 weight rows; the even CTA ("leader") issues one 256-row MMA for both.  Per byte loaded the pair
// does 1.5x the math of two independent 128 x 256 CTAs.  Five-stage operand ring.  In each CTA (NVFP4), by warpgroup:
//   warps 0..3  producers, one TMA stream each (the TMA unit retires the copies of one issuing warp one
//               after the other): per stage (256 codes of K) the 128B-swizzled 128 x 128 B box of A, the 128 x 128 B
//               box of B, the 2 KB of scale atoms of the CTA's activation rows and the 4 KB of the two 128-row
//               weight scale atoms; the cta_group::2 form of the load counts all of them on the leader's barrier
//   warps 4..7  epilogue set 0 (TMEM lane quadrant = warp & 3): tcgen05.ld (one row per thread), scale + bias +
//               activation, bf16 into a swizzled staging buffer, TMA store (coalesced, clipped at M and N by the
//               hardware); when requantising, the staged bf16 tile also feeds the next layer's LoRA-down (ldmatrix +
//               mma.sync) and the thread's own row chunk is group-quantised in registers
//   warps 8..11 epilogue set 1 (all variants but next rank 64): the two warps of a lane quadrant take alternate
//               64-column chunks
//   warp 12     (first warp after the epilogue sets) leader only: MMA issuer.  Per k-block three tcgen05.cp (scale
//               atoms, shared memory -> TMEM) and one tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale (M256 N256
//               K64); the low-rank branch is fed through the same ring as fp32 tiles and issued as kind::tf32 into the
//               same accumulator; one multicast tcgen05.commit per stage releases the stage in both CTAs, one per tile
//               publishes the accumulator.  Its loop carries no division and no descriptor rebuild: this one warp's
//               instruction stream, not bandwidth, is what bounds the kernel
//   warps 13..15 take part in the barriers only (registers are re-divided per warpgroup: producers and this group 48,
//               epilogue 200 per thread)
// INT4 (16 warps, six-stage ring of 32 KB): warp 1 issues, warps 2..5 are the epilogue, warp 6 brings the fp16 weights,
// warps 0 and 7..15 read the packed activation codes from global memory and convert them to fp16(code * group scale)
// into the operand ring; the MMAs are kind::f16.
// TMEM per CTA: two 256-column fp32 accumulators (the epilogue of tile i overlaps the main loop of tile i+1) fill all
// 512 columns.  The two 48-column scale-factor buffers of a tile (16 columns for A, 32 for B) therefore live in the first
// 96 columns of the OTHER accumulator, the one being drained: the epilogue warps arrive on `sfree` once those columns are
// in registers and the MMA warp waits for that before the tile's first tcgen05.cp.
// Every loop that issues tcgen05 / TMA instructions is run by a whole warp with one elected lane issuing, so
// that descriptors and coordinates stay warp-uniform.  Every wait is bounded; a wait that runs out raises the
// abort flag of both CTAs, all roles leave their loops, and the status words tell the host.
//
// The next layer's LoRA-down is a sum over all N, i.e. over tiles of different pairs.  It is kept
// deterministic: in requantising mode every pair owns a contiguous run of tiles in n-fastest order, each CTA
// adds up its tiles of one 128-row block in registers, writes one partial per row block it touches to caller
// scratch, and a second small kernel adds the partials in pair order.

#include <cstdlib>
#include <mutex>

#include "host_common.h"
#include "ptx.cuh"
#include "quant_common.cuh"

namespace svdq {
namespace SVDQ_DT {

// quantize.cu: lora_act[:, 16 rt_first :] = input @ lora_down[:, 16 rt_first :] for a bf16 [M, K] input
int lora_down_rank_tiles(const void* input, int M, int M_pad, int K, const void* smooth, const void* lora_down, int RT_total,
                         int rt_first, float* lora_act, cudaStream_t stream);

constexpr int G_BM = 128;
constexpr int G_BN = 256;
constexpr int G_BNH = G_BN / 2;                 // weight rows each CTA of a pair loads
constexpr int G_STAGES = 5;
constexpr int G_A_BYTES = G_BM * 128;           // 16 KB
constexpr int G_B_BYTES = G_BNH * 128;          // 16 KB
constexpr int G_SFA_BYTES = 4 * 512;            // 4 k-blocks x one 128-row atom
constexpr int G_SFB_BYTES = 2 * 4 * 512;        // 4 k-blocks x two 128-row atoms
constexpr int G_STAGE_BYTES = G_A_BYTES + G_B_BYTES + G_SFA_BYTES + G_SFB_BYTES;  // 38912 = 38 * 1024
// NVFP4 warp map, by warpgroup (four warps; registers are re-divided between warpgroups, see reg_dealloc):
//   warps 0..3   producers (A tile, B tile, scale atoms of A, scale atoms of B)
//   warps 4..7   epilogue set 0 (TMEM lane quadrant = warp & 3);  warps 8..11  epilogue set 1 (when there are two sets)
//   first warp of the last warpgroup: MMA issuer; the other three warps of that group only take part in the barriers
//   requantising variants with two epilogue sets: a fifth warpgroup, warps 16..19 = LoRA-down warp of TMEM lane quadrant 0..3
constexpr int G_THREADS = 12 * 32;             // one epilogue set
constexpr int G_THREADS_RQ = 16 * 32;          // two epilogue sets
constexpr int G_THREADS_LW = 20 * 32;          // two epilogue sets and the LoRA-down warpgroup
constexpr int G_REGS_PRODUCER = 48, G_REGS_MMA = 48, G_REGS_EPILOGUE = 200;   // per thread after the re-division (16 warps, 128 at launch)
// 20 warps start with 96 registers each; what the producers, the MMA group and the LoRA-down warps give back
// (2 x 128 x 56 + 128 x 16 = 16384) is exactly what the eight epilogue warps take (256 x 64)
constexpr int L_REGS_PRODUCER = 40, L_REGS_MMA = 40, L_REGS_LORA = 80, L_REGS_EPILOGUE = 160;
constexpr int G_SF_BUFS = 2;                    // scale-factor buffers in TMEM
constexpr int G_TMEM_COLS = 512;
constexpr int G_TM_ACC1 = G_BN;                 // second accumulator: the two fill all 512 columns
constexpr int G_TM_SF_STRIDE = 48;              // per scale-factor buffer: 4 x 4 columns for A, 4 x 8 for B (two 128-row atoms per k-block)
constexpr int G_TM_SF_COLS = G_SF_BUFS * G_TM_SF_STRIDE;   // 96: they live in the first columns of the accumulator that is being drained
constexpr int G_EPI_BUF_BYTES = 32 * 128;       // one warp's 32 rows x 64 bf16 columns, 128B-swizzled
constexpr int G_EPI_BYTES = 4 * 2 * G_EPI_BUF_BYTES;        // 4 warps x 2 buffers
constexpr int G_COLV_FLOATS = 64;                           // INT4, per epilogue warp: 1/smooth_next of the chunk in hand
constexpr int G_COLV_BYTES = 4 * G_COLV_FLOATS * 4;           // INT4: four epilogue warps
// NVFP4: the tile's per-column constants, staged once per tile by a warp of its own: [scale | bias | 1/smooth_next] x G_BN floats
constexpr int G_TILEC_BYTES = 3 * G_BN * 4 + 512;   // ROPE variant: [scale | bias | RMSNorm weights of q, k (16-bit) | sums of squares]
constexpr int G_SHARED_BYTES = 384;                           // barriers and flags (GemmShared)
// INT4 variant (template parameter I4): a stage is 64 k of fp16 operands, the activation half converted from packed
// codes by converter warps; the packed codes come through a small ring of their own.
constexpr int H_A_BYTES = G_BM * 128;           // 128 rows x 64 fp16
constexpr int H_B_BYTES = G_BNH * 128;          // 128 rows x 64 fp16
constexpr int H_STAGE_BYTES = H_A_BYTES + H_B_BYTES;   // 32768
constexpr int H_STAGES = 6;                     // INT4 operand ring (32 KB stages)
constexpr int H_GROUPS = 5;                     // converter groups: stages in conversion at once
constexpr int H_CONV_WARPS = 2 * H_GROUPS;
constexpr int H_CONV_PER_STAGE = 2;             // converter warps that share one stage (64 rows each); four such groups take turns
constexpr int H_THREADS = (6 + H_CONV_WARPS) * 32;   // warps 0 and 7..15 converters, 1 MMA, 2..5 epilogue, 6 weights: 16 warps
template <bool I4>
constexpr int stage_bytes() { return I4 ? H_STAGE_BYTES : G_STAGE_BYTES; }
template <bool I4>
constexpr size_t smem_bytes() {
    return 1024 + static_cast<size_t>(I4 ? H_STAGES : G_STAGES) * stage_bytes<I4>() + G_EPI_BYTES + (I4 ? G_COLV_BYTES : G_TILEC_BYTES) + G_SHARED_BYTES;
}
static_assert(smem_bytes<false>() <= 227 * 1024 && smem_bytes<true>() <= 227 * 1024, "dynamic shared memory of a CTA on sm_100");

struct GemmParams {
    const uint8_t* sfa;       // activation scale atoms [M_pad/128][K/64][512]
    const uint8_t* sfb;       // weight scale atoms     [N/128][K/64][512]
    const h16* ascales_i4;   // INT4: activation group scales [K/64][M_pad]
    const uint8_t* act_i4;             // INT4: packed activation codes [M_pad][K/2], read directly by the converter warps
    const float* row_scale;            // INT4: power of two taken out of each row's group scales [M_pad] (see int4_row_norm_kernel)
    int act_unsigned;                  // INT4: activation codes are u4
    const float* col_scale;   // [N]
    const float* col_bias;    // [N]
    int* status;
    int M, M_pad, N, K;
    int lora_chunks;          // number of 32-rank chunks of the low-rank branch (0 = none)
    int tiles_m, tiles_n;     // in 256 x 256 pair tiles
    int activation;
    int store_out;            // bf16 `out` is wanted
    // tile schedule: 0: m-fastest, strided by gridDim; 1: n-fastest, each CTA a contiguous run of `run` tiles
    int contiguous;
    int run;
    // requantising epilogue
    uint8_t* qout;                      // [M_pad][N/2]
    uint8_t* oscales;                   // scale atoms [M_pad/128][N/64][512]
    const h16* next_smooth;   // [N] reference-packed
    const uint4* next_lora_down;        // reference-packed [N/16][Rn/16][32] x 16 bytes
    int next_rt_total;                  // Rn/16 of that tensor (the epilogue takes its first RTN rank tiles)
    float* lora_partial;                // scratch [CTA][slots][128][Rn]
    int slots;
    // RMSNorm + rotary embedding of a fused QKV projection in the epilogue (ROPE variants)
    const h16* rope_wq;                 // RMSNorm weights of q and k [128]
    const h16* rope_wk;
    const float* rope_cos;              // [rope_seq_len][64]
    const float* rope_sin;
    float rope_eps;
    int rope_seq_len;                   // rows per batch element (row % rope_seq_len = token position)
    int rope_dim;                       // heads * 128: columns of each of q, k, v
    int rope_split;                     // 1: q, k, v go to three token-major tensors [batch * tokens_pad, rope_dim]
    int rope_tokens_pad, rope_token_offset, rope_attn_tokens;
#ifdef SVDQ_ABLATE
    int ablate;   // timing experiments only (results are wrong): bit 0 no epilogue work, 1 no tcgen05.cp, 2 no scale loads,
                  // 3 no MMAs, 4 no operand loads, 5 next layer's LoRA-down without its weight loads, 6 without its mma.sync,
                  // 7 per-column constants always from the same (cached) addresses
#endif
};
#ifdef SVDQ_ABLATE
#define ABLATE(p, bit) ((p).ablate & (1 << (bit)))
// cycle accounting of pair 0 (timing experiments): [0..3] MMA warp total / wait full / wait tempty / stages,
// [4..5] leader's A producer total / wait empty, [6..7] peer's A producer, [8..10] leader's epilogue warp 2 total / wait tfull / tiles,
// [11] MMA warp: issue of cp + mma, [12] commit, [13..15] that epilogue warp: activation + staging / next layer's LoRA-down /
// smoothing + group quantisation
__device__ long long g_prof[16];
#define PROF_T0(v) const long long v = clock64()
#define PROF_ACC(v) long long v = 0
#define PROF_ADD(acc, t0) acc += clock64() - (t0)
#define PROF_OUT(cond, idx, acc) do { if (cond) g_prof[idx] += (acc); } while (0)
#else
#define ABLATE(p, bit) false
#define PROF_T0(v)
#define PROF_ACC(v)
#define PROF_ADD(acc, t0)
#define PROF_OUT(cond, idx, acc)
#endif

struct GemmShared {
    uint64_t full[H_STAGES];        // leader: operand tiles and scale atoms of both CTAs have landed (8 arrivals + bytes)
    uint64_t empty[H_STAGES];       // each CTA: the MMAs of the stage are done (multicast tcgen05.commit)
    uint64_t tfull[2];              // each CTA: accumulator complete (multicast commit)
    uint64_t tempty[2];             // leader: accumulator drained (4 epilogue warps x 2 CTAs)
    uint64_t sfree[2];              // leader: the first G_TM_SF_COLS columns of the accumulator are in registers (all epilogue warps, both CTAs)
    uint64_t lfull[4][2], lempty[4][2];   // LoRA-down warps: staging buffer of (quadrant, epilogue set) holds a chunk / has been read
    uint64_t xsum[4], xread[4];     // ROPE, per lane quadrant: both epilogue warps have written / read their sums of squares
    uint64_t cfull, cempty;         // NVFP4, each CTA: the tile's per-column constants are in shared memory / have been read by all epilogue warps
    uint64_t drain;
    uint32_t tmem_base;
    volatile int abort_flag;
};

struct TileRun {
    int first, stride, count;
};

__device__ __forceinline__ TileRun tile_run(const GemmParams& p) {
    const int num_tiles = p.tiles_m * p.tiles_n;
    TileRun r;
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    if (p.contiguous) {
        r.first = pair * p.run;
        r.stride = 1;
        r.count = max(0, min(p.run, num_tiles - r.first));
    } else {
        r.first = pair;
        r.stride = npairs;
        r.count = num_tiles > r.first ? (num_tiles - r.first + r.stride - 1) / r.stride : 0;
    }
    return r;
}
// first row of THIS CTA's half of the pair tile, first column of the tile
__device__ __forceinline__ void tile_coords(const GemmParams& p, int tile, uint32_t rank, int& m0, int& n0) {
    if (p.contiguous) {
        m0 = (tile / p.tiles_n) * (2 * G_BM);
        n0 = (tile % p.tiles_n) * G_BN;
    } else {
        m0 = (tile % p.tiles_m) * (2 * G_BM);
        n0 = (tile / p.tiles_m) * G_BN;
    }
    m0 += rank * G_BM;
}

__device__ __forceinline__ void raise_abort(GemmShared* sh) {
    sh->abort_flag = 1;
    st_shared_cluster_u32(mapa_shared(smem_u32(const_cast<int*>(&sh->abort_flag)), cluster_ctarank() ^ 1u), 1u);
}

// Bounded wait.  BACKOFF > 0 puts the warp to sleep for that many nanoseconds between polls: a warp that spins on a
// barrier is always eligible and takes issue slots from the working warps of its scheduler, so the roles with slack
// (producers waiting for a free slot, epilogue warps waiting for an accumulator) back off; the MMA warp does not.
template <int BACKOFF_ = 0>
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, GemmShared* sh, int* status, int where) {
#ifdef SVDQ_BACKOFF_OVERRIDE
    constexpr int BACKOFF = BACKOFF_ ? SVDQ_BACKOFF_OVERRIDE : 0;   // timing experiments
#else
    constexpr int BACKOFF = BACKOFF_;
#endif
#pragma unroll 1
    for (int i = 0; i < (BACKOFF ? 2 : 512); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 128; ++i) {
            if (mbar_try_wait(bar, parity)) return true;
            if (BACKOFF) __nanosleep(BACKOFF);
        }
        if (sh->abort_flag) return false;
        if (clock64() - t0 > 4000000000ll) {  // about 2 s
            raise_abort(sh);
            atomicExch(&status[0], SVDQ_ERR_TIMEOUT);
            atomicExch(&status[1], where);
            return false;
        }
    }
}

// Activation of two values at once with packed fp32 arithmetic (the requantising epilogue is instruction bound).
// GELU: x * (0.5 + 0.5 * tanh.approx(0.79788456 * (x + 0.044715 x^3))) (gemm_utils.cuh:305-319), with the argument
// evaluated as x * (c0 + c0*c1 * x^2).
template <int ACT>
__device__ __forceinline__ float2 act2(float2 v) {
    if constexpr (ACT == SVDQ_ACT_SILU) {
        return make_float2(v.x / (1.0f + __expf(-v.x)), v.y / (1.0f + __expf(-v.y)));
    } else if constexpr (ACT == SVDQ_ACT_GELU) {
        const float2 w = __fmul2_rn(v, v);
        const float2 k = __ffma2_rn(w, make_float2(0.79788456f * 0.044715f, 0.79788456f * 0.044715f), make_float2(0.79788456f, 0.79788456f));
        const float2 u = __fmul2_rn(v, k);
        float2 t;
        asm("tanh.approx.f32 %0, %1;" : "=f"(t.x) : "f"(u.x));
        asm("tanh.approx.f32 %0, %1;" : "=f"(t.y) : "f"(u.y));
        const float2 h = __ffma2_rn(t, make_float2(0.5f, 0.5f), make_float2(0.5f, 0.5f));
        return __fmul2_rn(v, h);
    } else {
        return v;
    }
}

// One thread's 64 accumulator columns -> scale, bias, activation -> 64 bf16 (kept in `ow`) -> its row of the
// 128B-swizzled staging tile.  The activation is a template parameter: selected per element at run time it put a
// branch between every two values and kept the compiler from interleaving them.
// ROWSCALE: the accumulator is first multiplied by this row's power of two `rs` (INT4 operands are normalised per row).
// SMEMC: the per-column constants are in shared memory (plain loads) instead of global memory (read-only path).
template <int ACT, bool ROWSCALE = false, bool SMEMC = false>
__device__ __forceinline__ void stage_chunk(const uint32_t (&r0)[32], const uint32_t (&r1)[32], const float4* cs, const float4* cb,
                                            uint32_t (&ow)[32], uint8_t* buf, int lane, float rs = 1.0f) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {   // 16-byte chunk j = columns 8j .. 8j+7 of this 64-column block
        const uint32_t* r = j < 4 ? &r0[8 * j] : &r1[8 * (j - 4)];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float4 s4 = SMEMC ? cs[2 * j + i] : __ldg(cs + 2 * j + i);
            const float4 b4 = SMEMC ? cb[2 * j + i] : __ldg(cb + 2 * j + i);
            float2 a01 = make_float2(__uint_as_float(r[4 * i + 0]), __uint_as_float(r[4 * i + 1]));
            float2 a23 = make_float2(__uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
            if constexpr (ROWSCALE) {   // exact: a power of two
                a01 = __fmul2_rn(a01, make_float2(rs, rs));
                a23 = __fmul2_rn(a23, make_float2(rs, rs));
            }
            const float2 v01 = act2<ACT>(__ffma2_rn(a01, make_float2(s4.x, s4.y), make_float2(b4.x, b4.y)));
            const float2 v23 = act2<ACT>(__ffma2_rn(a23, make_float2(s4.z, s4.w), make_float2(b4.z, b4.w)));
            ow[4 * j + 2 * i] = pack2(v01);
            ow[4 * j + 2 * i + 1] = pack2(v23);
        }
        *reinterpret_cast<uint4*>(buf + lane * 128 + ((j ^ (lane & 7)) << 4)) =
            make_uint4(ow[4 * j], ow[4 * j + 1], ow[4 * j + 2], ow[4 * j + 3]);
    }
}

// One warp's LoRA-down partial (32 rows of lane quadrant q x RT rank tiles, mma.sync C-fragment order) of a 128-row block
// -> scratch[CTA][slot][128][16 RT].
template <int RT>
__device__ __forceinline__ void store_lora_partial(const GemmParams& p, const float (&lacc)[2][RT][8], int slot, int q, int lane) {
    constexpr int RN = RT * 16;
    float* dst = p.lora_partial + (static_cast<size_t>(blockIdx.x) * p.slots + slot) * (G_BM * RN);
    const int gq = lane >> 2, t = lane & 3;
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int rt = 0; rt < RT; ++rt)
#pragma unroll
            for (int nh = 0; nh < 2; ++nh)
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int row = q * 32 + mt * 16 + gq + half * 8;
                    const int rank = rt * 16 + nh * 8 + 2 * t;
                    *reinterpret_cast<float2*>(dst + row * RN + rank) =
                        make_float2(lacc[mt][rt][nh * 4 + half * 2], lacc[mt][rt][nh * 4 + half * 2 + 1]);
                }
}

// RTN: rank tiles (of 16) of the next layer's LoRA-down; 0 = plain epilogue (no requantisation).
// Requantising epilogues do about three times the work of the plain one per chunk; up to rank 32 (where a warp's
// LoRA-down partial fits its 4 KB staging buffer) a second set of four epilogue warps takes every other 64-column chunk.
template <int RTN, bool I4>
constexpr int epi_sets() { return (!I4 && RTN <= 2) ? 2 : 1; }
// The tensor pipe serves mma.sync poorly while tcgen05.mma keeps it busy (a warp stalls ~80 cycles per instruction): in the
// two-set requantising variants the next layer's LoRA-down therefore runs in four warps of its own, fed from the staged bf16
// tiles, so that those stalls no longer delay the activation and quantisation work of the epilogue warps.
template <int RTN, bool I4>
constexpr bool lora_warps() { return !I4 && RTN > 0 && epi_sets<RTN, I4>() == 2; }
template <int RTN, bool I4>
constexpr int cta_threads() {
    return I4 ? H_THREADS : lora_warps<RTN, I4>() ? G_THREADS_LW : (epi_sets<RTN, I4>() == 2 ? G_THREADS_RQ : G_THREADS);
}
template <int RTN, bool I4>
constexpr int mma_warp() { return I4 ? 1 : 4 + 4 * epi_sets<RTN, I4>(); }

// Eight packed s4 / u4 codes -> eight fp16 values code * scale, in the order (0, 4, 1, 5, 2, 6, 3, 7).
// (x & 0x000f000f) | 0x6400 is the fp16 number 1024 + code, (x & 0x00f000f0) | 0x6400 is 1024 + 16 * code; one exact
// subtraction (or fused multiply-add by 1/16) removes the offset, signed codes are biased by 8 first (flip bit 3).
__device__ __forceinline__ uint4 int4x8_to_f16(uint32_t x, uint32_t flip, __half2 off_lo, __half2 off_hi, __half2 s2) {
    x ^= flip;
    const __half2 sixteenth = __float2half2_rn(0.0625f);
    uint32_t h[4];
    h[0] = (x & 0x000f000fu) | 0x64006400u;
    h[1] = (x & 0x00f000f0u) | 0x64006400u;
    const uint32_t y = x >> 8;
    h[2] = (y & 0x000f000fu) | 0x64006400u;
    h[3] = (y & 0x00f000f0u) | 0x64006400u;
    const __half2 v0 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&h[0]), off_lo), s2);
    const __half2 v1 = __hmul2(__hfma2(*reinterpret_cast<__half2*>(&h[1]), sixteenth, off_hi), s2);
    const __half2 v2 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&h[2]), off_lo), s2);
    const __half2 v3 = __hmul2(__hfma2(*reinterpret_cast<__half2*>(&h[3]), sixteenth, off_hi), s2);
    return make_uint4(*reinterpret_cast<const uint32_t*>(&v0), *reinterpret_cast<const uint32_t*>(&v1),
                      *reinterpret_cast<const uint32_t*>(&v2), *reinterpret_cast<const uint32_t*>(&v3));
}

struct RopeMaps {
    CUtensorMap q, k, v;   // token-major outputs of the ROPE variant in split mode; unused otherwise
};

// ROPE (plain NVFP4 epilogue only): the GEMM is a fused QKV projection [.., 3 * heads * 128]; RMSNorm of every 128-column
// head of q and k and the rotary embedding are applied to the tile before it is stored (EpilogueRMSNormRope,
// src/kernels/zgemm/epilogues.cuh:269-425).
template <int RTN, bool I4, bool ROPE = false>
__global__ void __launch_bounds__(cta_threads<RTN, I4>(), 1)
gemm_w4a4_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                  const __grid_constant__ CUtensorMap tm_la, const __grid_constant__ CUtensorMap tm_lu,
                  const __grid_constant__ CUtensorMap tm_out, const __grid_constant__ CUtensorMap tm_sfa,
                  const __grid_constant__ CUtensorMap tm_sfb, const __grid_constant__ RopeMaps tm_rope, const GemmParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int SB = stage_bytes<I4>();
    constexpr int NS = I4 ? H_STAGES : G_STAGES;                              // depth of the operand ring
    uint8_t* epi_smem = smem + NS * SB;
    float* colv = reinterpret_cast<float*>(epi_smem + G_EPI_BYTES);
    GemmShared* sh = reinterpret_cast<GemmShared*>(epi_smem + G_EPI_BYTES + (I4 ? G_COLV_BYTES : G_TILEC_BYTES));
    static_assert(sizeof(GemmShared) <= G_SHARED_BYTES, "barrier block");

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int KB = p.K / 64;                         // 64-code blocks along K
    const int kstages = I4 ? KB : (KB + 3) / 4;      // NVFP4: 256 codes of K per stage; INT4: 64
    const int per_tile = kstages + p.lora_chunks;
    const int NB = p.N / 128;                        // weight scale atoms along N
    const TileRun tr = tile_run(p);

    const uint32_t rank = cluster_ctarank();      // 0 = leader (issues the MMAs), 1 = peer
    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(&sh->full[s], I4 ? 2 * (1 + H_CONV_PER_STAGE) : 8);   // producers (and converter warps) of both CTAs
            mbar_init(&sh->empty[s], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&sh->tfull[i], 1);
            mbar_init(&sh->tempty[i], 8 * epi_sets<RTN, I4>());
            mbar_init(&sh->sfree[i], 8 * epi_sets<RTN, I4>());
        }
        for (int i = 0; i < 8; ++i) {
            mbar_init(&sh->lfull[i >> 1][i & 1], 1);
            mbar_init(&sh->lempty[i >> 1][i & 1], 1);
        }
        for (int i = 0; i < 4; ++i) {
            mbar_init(&sh->xsum[i], 2);
            mbar_init(&sh->xread[i], 2);
        }
        mbar_init(&sh->cfull, 1);
        mbar_init(&sh->cempty, 4 * epi_sets<RTN, I4>());
        mbar_init(&sh->drain, 1);
        sh->abort_flag = 0;
        fence_mbar_init();
        prefetch_tmap(&tm_a);
        prefetch_tmap(&tm_b);
        prefetch_tmap(&tm_out);
        if (!I4) {
            prefetch_tmap(&tm_sfa);
            prefetch_tmap(&tm_sfb);
        }
        if (p.lora_chunks) {
            prefetch_tmap(&tm_la);
            prefetch_tmap(&tm_lu);
        }
    }
    constexpr int MMA_WARP = mma_warp<RTN, I4>();
    if (warp == MMA_WARP) {
        tmem_alloc_pair(&sh->tmem_base, G_TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    cluster_sync_all();   // barriers of both CTAs are initialised before anything remote touches them
    tc_fence_after_sync();
    pdl_launch_dependents();
    pdl_wait();           // nothing above touches global memory; the quantiser's output is this kernel's input
    const uint32_t tmem = sh->tmem_base;
    // 16 warps at 128 registers each fill the register file; the epilogue needs ~180 and the other roles ~50: each role's
    // branch starts by giving registers back or asking for more (inside the branch, so that the compiler can tell which
    // budget applies to which code)
    constexpr bool REGCTL = !I4 && epi_sets<RTN, I4>() == 2;
    constexpr bool LW = lora_warps<RTN, I4>();
    constexpr int REGS_P = LW ? L_REGS_PRODUCER : G_REGS_PRODUCER, REGS_M = LW ? L_REGS_MMA : G_REGS_MMA,
                  REGS_E = LW ? L_REGS_EPILOGUE : G_REGS_EPILOGUE;

    if (I4 && (warp == 0 || warp >= 6)) {
        // ------------------------------------------------------------------ INT4 producers and converter warps
        // warp 6: this CTA's 96 rows of the fp16 weights, or both fp32 tiles (lora_act, LoRA-up) of a
        // low-rank stage; warps 0 and 7..15: packed codes from global memory (prefetched into registers one turn ahead) ->
        // fp16(code * group scale) straight into the 128B-swizzled K-major tile the MMA reads.
        if constexpr (I4) {
            const int cw = warp == 0 ? 0 : warp - 6;   // converter index 0..9
            const int hh = lane & 1;
            const uint32_t flip = p.act_unsigned ? 0u : 0x88888888u;
            const __half2 off_lo = __float2half2_rn(p.act_unsigned ? 1024.f : 1032.f);
            const __half2 off_hi = __float2half2_rn(p.act_unsigned ? -64.f : -72.f);
            uint32_t it = 0;
            bool ok = true;
            if (warp != 6) {
                // converter warps.  Every shared-memory and barrier operation of a SIMT warp queues behind the tensor core's
                // operand reads, so the fixed chain of a stage's hand-shake (two barrier waits, load, stores, proxy fence,
                // arrivals) costs several hundred cycles however little is converted.  The ten warps therefore form five
                // groups that take every fifth stage each, two warps per stage with 64 rows apiece: five of the ring's six
                // stages are in conversion at once.  A lane converts half a row (32 codes) of rows r0, r0 + 16, r0 + 32, r0 + 48: its 16-byte
                // global loads fill whole 32-byte sectors and its swizzled 16-byte stores are free of bank conflicts.
                // The packed codes and group scales of the next stage the warp will convert are fetched while it converts
                // this one, so no shared-memory load and only one barrier wait are left in the chain.
                const int grp = cw >> 1, g2 = cw & 1;
                const int r0 = g2 * 64 + (lane >> 1);
                uint32_t it_base = 0;
                for (int ti = 0; ti < tr.count && ok; ++ti) {
                    int m0, n0;
                    tile_coords(p, tr.first + ti * tr.stride, rank, m0, n0);
                    const h16* asp = p.ascales_i4 + m0 + r0;
                    int ks = (grp + H_GROUPS - static_cast<int>(it_base % H_GROUPS)) % H_GROUPS;   // first stage of this tile that is ours
                    // the lane's 16 bytes (32 codes) of row r0 + 16 i in k-block ks sit at apk + 16 i * pitch + 32 ks
                    const size_t pitch = static_cast<size_t>(p.K) >> 1;
                    const uint8_t* apk = p.act_i4 + static_cast<size_t>(m0 + r0) * pitch + hh * 16;
                    h16 nxt[4];
                    uint4 wnxt[4];
                    float inv[4];   // 1 / (this row's power-of-two normalisation): exact
#pragma unroll
                    for (int i = 0; i < 4; ++i) inv[i] = __frcp_rn(__ldg(p.row_scale + m0 + r0 + 16 * i));
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        nxt[i] = ks < kstages ? __ldg(asp + static_cast<size_t>(ks) * p.M_pad + 16 * i) : f2h(0.f);
                        wnxt[i] = ks < kstages ? __ldg(reinterpret_cast<const uint4*>(apk + 16 * i * pitch + 32 * ks)) : make_uint4(0, 0, 0, 0);
                    }
                    for (; ks < per_tile; ks += H_GROUPS) {
                        const uint32_t it = it_base + ks;
                        const int s = it % NS;
                        uint8_t* st = smem + s * SB;
                        const uint32_t lfull = mapa_shared(smem_u32(&sh->full[s]), 0);   // the leader's barrier
                        ok = __all_sync(0xffffffffu, wait_or_abort(&sh->empty[s], ((it / NS) & 1) ^ 1, sh, p.status, 12));
                        if (!ok) break;
                        if (ks >= kstages) {   // low-rank stage: nothing to convert, but the arrival keeps this warp in step
                            if (lane == 0) mbar_arrive_cluster(lfull);
                            __syncwarp();
                            continue;
                        }
                        h16 cur[4];
                        uint4 w[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            cur[i] = nxt[i];
                            w[i] = wnxt[i];
                            if (ks + H_GROUPS < kstages) {
                                nxt[i] = __ldg(asp + static_cast<size_t>(ks + H_GROUPS) * p.M_pad + 16 * i);
                                wnxt[i] = __ldg(reinterpret_cast<const uint4*>(apk + 16 * i * pitch + 32 * (ks + H_GROUPS)));
                            }
                        }
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            // the row's largest group scale is in [1, 2) after normalisation, so |code * scale| < 30 in fp16
                            const __half2 s2 = __float2half2_rn(h2f(cur[i]) * inv[i]);
                            const int row = r0 + 16 * i;
                            uint8_t* dst = st + row * 128;
                            const int sw = row & 7;
                            *reinterpret_cast<uint4*>(dst + (((hh * 4 + 0) ^ sw) << 4)) = int4x8_to_f16(w[i].x, flip, off_lo, off_hi, s2);
                            *reinterpret_cast<uint4*>(dst + (((hh * 4 + 1) ^ sw) << 4)) = int4x8_to_f16(w[i].y, flip, off_lo, off_hi, s2);
                            *reinterpret_cast<uint4*>(dst + (((hh * 4 + 2) ^ sw) << 4)) = int4x8_to_f16(w[i].z, flip, off_lo, off_hi, s2);
                            *reinterpret_cast<uint4*>(dst + (((hh * 4 + 3) ^ sw) << 4)) = int4x8_to_f16(w[i].w, flip, off_lo, off_hi, s2);
                        }
                        fence_proxy_async_smem();   // the tile is read by the tensor core
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster(lfull);
                    }
                    it_base += per_tile;
                }
            } else {
                for (int ti = 0; ti < tr.count && ok; ++ti) {
                    int m0, n0;
                    tile_coords(p, tr.first + ti * tr.stride, rank, m0, n0);
                    const int nb0 = n0 + rank * G_BNH;
                    for (int ks = 0; ks < per_tile; ++ks, ++it) {
                        const int s = it % NS;
                        uint8_t* st = smem + s * SB;
                        const uint32_t lfull = mapa_shared(smem_u32(&sh->full[s]), 0);   // the leader's barrier
                        const bool lowrank = ks >= kstages;
                        const uint32_t eparity = ((it / NS) & 1) ^ 1;
                        if (warp == 0) {
                            break;   // nothing to bring: the converter warps read the packed codes from global memory themselves
                        } else {
                            ok = __all_sync(0xffffffffu, wait_or_abort<64>(&sh->empty[s], eparity, sh, p.status, 11));
                            if (!ok) break;
                            if (elect_one()) {
                                if (lowrank) {   // both fp32 tiles of the low-rank stage
                                    mbar_arrive_expect_tx_cluster(lfull, H_A_BYTES + H_B_BYTES);
                                    tma_load_2d_pair(st, &tm_la, lfull, (ks - kstages) * 32, m0);
                                    tma_load_2d_pair(st + H_A_BYTES, &tm_lu, lfull, (ks - kstages) * 32, nb0);
                                } else {
                                    mbar_arrive_expect_tx_cluster(lfull, H_B_BYTES);
                                    tma_load_2d_pair(st + H_A_BYTES, &tm_b, lfull, ks * 64, nb0);
                                }
                            }
                        }
                        __syncwarp();
                    }
                }
            }
        }
    } else if (!I4 && warp < 4) {
        if constexpr (REGCTL) reg_dealloc<REGS_P>();
        // ------------------------------------------------------------------ producers (whole warp, elected lane issues)
        // The TMA unit retires the copies of one issuing warp one after the other (about 500 cycles each,
        // almost independent of size), so each stream of a stage has its own warp: 0 = activation tile,
        // 1 = weight tile, 2 = scale atoms of the activation rows, 3 = scale atoms of the 256 weight rows (whole
        // 128-row atoms: two of them).  All are counted on the leader's barrier; a tile past the end of a
        // tensor is filled with zeros by the hardware and still counts its full size.
        const int role = warp;
        uint32_t it = 0;  // ring position, counted over every stage this CTA ever fills
        bool ok = true;
        const bool prof_me = blockIdx.x < (LW ? 1 : 2) && role == 0 && lane == 0;   // with LoRA-down warps their counters take the peer's slots
        PROF_T0(pt_all);
        PROF_ACC(pa_wait);
        for (int ti = 0; ti < tr.count && ok; ++ti) {
            int m0, n0;
            tile_coords(p, tr.first + ti * tr.stride, rank, m0, n0);
            const int nb0 = n0 + rank * G_BNH;   // this CTA's half of the tile's weight rows
            for (int ks = 0; ks < per_tile; ++ks, ++it) {
                const int s = it % NS;
                PROF_T0(pt_w);
                ok = __all_sync(0xffffffffu, wait_or_abort<64>(&sh->empty[s], ((it / NS) & 1) ^ 1, sh, p.status, 10 + role));
                PROF_ADD(pa_wait, pt_w);
                if (!ok) break;
                uint8_t* st = smem + s * G_STAGE_BYTES;
                const uint32_t lfull = mapa_shared(smem_u32(&sh->full[s]), 0);   // the leader's barrier
                const bool lowrank = ks >= kstages;
                const int kx = lowrank ? (ks - kstages) * 32 : ks * 128;
                if ((role < 2 && ABLATE(p, 4)) || (role >= 2 && ABLATE(p, 2))) {
                    if (elect_one()) mbar_arrive_cluster(lfull);
                } else if (elect_one()) {
                    if (role == 0) {
                        mbar_arrive_expect_tx_cluster(lfull, G_A_BYTES);
                        tma_load_2d_pair(st, lowrank ? &tm_la : &tm_a, lfull, kx, m0);
                    } else if (role == 1) {
                        mbar_arrive_expect_tx_cluster(lfull, G_B_BYTES);
                        tma_load_2d_pair(st + G_A_BYTES, lowrank ? &tm_lu : &tm_b, lfull, kx, nb0);
                    } else if (lowrank) {
                        mbar_arrive_cluster(lfull);   // no scale factors in a low-rank stage
                    } else if (role == 2) {
                        mbar_arrive_expect_tx_cluster(lfull, G_SFA_BYTES);
                        tma_load_2d_pair(st + G_A_BYTES + G_B_BYTES, &tm_sfa, lfull, 0, (m0 >> 7) * KB + ks * 4);
                    } else {
                        mbar_arrive_expect_tx_cluster(lfull, G_SFB_BYTES);
                        tma_load_3d_pair(st + G_A_BYTES + G_B_BYTES + G_SFA_BYTES, &tm_sfb, lfull, 0, ks * 4, n0 >> 7);
                    }
                }
                __syncwarp();
            }
        }
        PROF_ACC(pa_all);
        PROF_ADD(pa_all, pt_all);
        PROF_OUT(prof_me, 4 + 2 * blockIdx.x, pa_all);
        PROF_OUT(prof_me, 5 + 2 * blockIdx.x, pa_wait);
    } else if (warp >= MMA_WARP && (I4 ? warp == MMA_WARP : warp < MMA_WARP + 4)) {
        if constexpr (REGCTL) reg_dealloc<REGS_M>();
        // ------------------------------------------------------------------ MMA issuer (leader CTA only; NVFP4: the other
        // warps of its warpgroup only give their registers back)
        // The whole warp runs the loop and one elected lane issues: descriptors, TMEM addresses and barrier
        // addresses then stay warp-uniform.  (With the loop inside `if (lane == 0)` every operand is a
        // per-thread value and the issue rate, not the tensor pipe, bounds the kernel.)
        if (rank == 0 && warp == MMA_WARP) {
            constexpr uint32_t IDESC_FP4 = idesc_nvfp4(2 * G_BM, G_BN);
            constexpr uint32_t IDESC_TF32 = idesc_tf32(2 * G_BM, G_BN);
            constexpr uint32_t IDESC_F16 = idesc_f16(2 * G_BM, G_BN);
            // This warp's instruction stream is the kernel's critical path: it is one warp, so every dependent instruction
            // costs its full latency, and a stage's four MMAs only take ~470 cycles.  So the loop keeps the ring slot, its
            // phase bit and the slot's descriptor offset as running values (no division), and builds each descriptor from a
            // constant upper half and a lower half that moves by small immediates (the start-address field counts 16-byte
            // units and cannot carry out of its 14 bits for addresses below 256 KB).
            const uint64_t adesc0 = smem_desc_sw128(smem_u32(smem));
            const uint64_t sfdesc0 = smem_desc_sf(smem_u32(smem) + G_A_BYTES + G_B_BYTES);
            const uint32_t sw_hi = static_cast<uint32_t>(adesc0 >> 32), sf_hi = static_cast<uint32_t>(sfdesc0 >> 32);
            const uint32_t a_lo0 = static_cast<uint32_t>(adesc0), sf_lo0 = static_cast<uint32_t>(sfdesc0);
            const uint32_t full0 = smem_u32(&sh->full[0]), empty0 = smem_u32(&sh->empty[0]);
            uint32_t slot = 0, phase = 0, slot_off = 0, sq = 0;   // ring slot, its parity, its offset in 16-byte units, scale buffer
            bool ok = true;
            const bool prof_me = blockIdx.x == 0 && lane == 0;
            PROF_T0(pt_all);
            PROF_ACC(pa_full); PROF_ACC(pa_te); PROF_ACC(pa_n); PROF_ACC(pa_issue); PROF_ACC(pa_commit);
            for (int ti = 0; ti < tr.count && ok; ++ti) {
                const uint32_t as = ti & 1;
                PROF_T0(pt_te);
                ok = __all_sync(0xffffffffu, wait_or_abort(&sh->tempty[as], ((ti >> 1) & 1) ^ 1, sh, p.status, 20));
                // The two accumulators fill TMEM, so this tile's scale factors go to the first columns of the OTHER
                // accumulator: the previous tile's, which its epilogue is draining.  They are free once every epilogue warp
                // of both CTAs has its first chunk in registers (the very first tile finds them unused).
                if (!I4 && ti > 0 && ok)
                    ok = __all_sync(0xffffffffu, wait_or_abort(&sh->sfree[as ^ 1], ((ti - 1) >> 1) & 1, sh, p.status, 22));
                PROF_ADD(pa_te, pt_te);
                if (!ok) break;
                const uint32_t d_tmem = tmem + as * G_TM_ACC1;
                const uint32_t sf_tmem = tmem + (as ^ 1) * G_TM_ACC1;
                uint32_t accumulate = 0;
                for (int ks = 0; ks < per_tile; ++ks) {
                    PROF_T0(pt_f);
                    const uint32_t fbar = full0 + 8 * slot;
                    if (!mbar_try_wait_addr(fbar, phase))   // usually there already
                        ok = wait_or_abort(&sh->full[slot], phase, sh, p.status, 21);
                    ok = __all_sync(0xffffffffu, ok);
                    PROF_ADD(pa_full, pt_f);
#ifdef SVDQ_ABLATE
                    pa_n += 1;
#endif
                    PROF_T0(pt_i);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t a_lo = a_lo0 + slot_off, b_lo = a_lo + (G_A_BYTES >> 4);
                    if (I4 && ks < kstages) {
                        // INT4: four K=16 fp16 MMAs over the stage's 64 k (operands already carry their group scales)
                        if (elect_one()) {
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                tc_mma_pair_f16(d_tmem, a_lo + 2 * j, b_lo + 2 * j, sw_hi, IDESC_F16, j == 0 ? accumulate : 1u);
                            tc_commit_pair_addr(empty0 + 8 * slot, 3);
                        }
                    } else if (ks < kstages) {
                        const int nkb = min(4, KB - ks * 4);
                        // Scale factors: shared memory -> TMEM with tcgen05.cp, issued just ahead of the MMA that
                        // reads them (the tensor pipe keeps the order).  Per k-block one 512-byte atom for the 128
                        // activation rows (4 columns) and two for the tile's 256 weight rows (8 columns).  Two TMEM
                        // buffers alternate.
                        const uint32_t t_sfa = sf_tmem + sq * G_TM_SF_STRIDE;
                        const uint32_t t_sfb = t_sfa + 16;
                        const uint32_t sf_lo = sf_lo0 + slot_off;
                        if (elect_one()) {
                            if (nkb == 4) {
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    if (!ABLATE(p, 1)) {
                                        tc_cp_pair_32x128b_warpx4(t_sfa + 4 * j, sf_lo + 32 * j, sf_hi);
                                        tc_cp_pair_32x128b_warpx4(t_sfb + 8 * j, sf_lo + (G_SFA_BYTES >> 4) + 32 * j, sf_hi);
                                        tc_cp_pair_32x128b_warpx4(t_sfb + 8 * j + 4, sf_lo + ((G_SFA_BYTES + 2048) >> 4) + 32 * j, sf_hi);
                                    }
                                    if (!ABLATE(p, 3))
                                        tc_mma_pair_nvfp4(d_tmem, a_lo + 2 * j, b_lo + 2 * j, sw_hi, IDESC_FP4, t_sfa + 4 * j,
                                                          t_sfb + 8 * j, j == 0 ? accumulate : 1u);
                                }
                            } else {
                                for (int j = 0; j < nkb; ++j) {
                                    tc_cp_pair_32x128b_warpx4(t_sfa + 4 * j, sf_lo + 32 * j, sf_hi);
                                    tc_cp_pair_32x128b_warpx4(t_sfb + 8 * j, sf_lo + (G_SFA_BYTES >> 4) + 32 * j, sf_hi);
                                    tc_cp_pair_32x128b_warpx4(t_sfb + 8 * j + 4, sf_lo + ((G_SFA_BYTES + 2048) >> 4) + 32 * j, sf_hi);
                                    tc_mma_pair_nvfp4(d_tmem, a_lo + 2 * j, b_lo + 2 * j, sw_hi, IDESC_FP4, t_sfa + 4 * j,
                                                      t_sfb + 8 * j, j == 0 ? accumulate : 1u);
                                }
                            }
                            PROF_ADD(pa_issue, pt_i);
                            PROF_T0(pt_c);
                            tc_commit_pair_addr(empty0 + 8 * slot, 3);   // frees the stage in both CTAs
                            PROF_ADD(pa_commit, pt_c);
                        }
                        sq ^= 1;
                    } else {
                        if (elect_one()) {
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                tc_mma_pair_tf32(d_tmem, a_lo + 2 * j, b_lo + 2 * j, sw_hi, IDESC_TF32, j == 0 ? accumulate : 1u);
                            tc_commit_pair_addr(empty0 + 8 * slot, 3);
                        }
                    }
                    accumulate = 1;
                    if (++slot == NS) {
                        slot = 0;
                        slot_off = 0;
                        phase ^= 1;
                    } else {
                        slot_off += SB >> 4;
                    }
                    __syncwarp();
                }
                if (ok) {
                    if (elect_one()) tc_commit_pair(&sh->tfull[as], 3);  // accumulator complete, both CTAs
                    __syncwarp();
                }
            }
            PROF_ACC(pa_all);
            PROF_ADD(pa_all, pt_all);
            PROF_OUT(prof_me, 0, pa_all); PROF_OUT(prof_me, 1, pa_full); PROF_OUT(prof_me, 2, pa_te); PROF_OUT(prof_me, 3, pa_n);
            PROF_OUT(prof_me, 11, pa_issue); PROF_OUT(prof_me, 12, pa_commit);
            if (sh->abort_flag) {  // let whatever was issued finish before TMEM is released
                if (lane == 0) {
                    tc_commit_pair(&sh->drain, 1);
                    mbar_wait(&sh->drain, 0, 400000000ll);
                }
                __syncwarp();
            }
        } else if (!I4 && warp == MMA_WARP + 1) {
            // ------------------------------------------------------------------ per-column constants of every tile (NVFP4)
            // alpha * wcscale, bias and the next layer's reciprocal smoothing factors of the tile's G_BN columns go to shared
            // memory once per tile and CTA; the epilogue warps read them from there (from global memory every 64-column
            // chunk of every warp paid an L2 round trip: the L1 left beside 227 KB of shared memory does not hold them).
            // The values of the next tile wait in registers until all epilogue warps are done with the current ones.
            for (int ti = 0; ti < tr.count; ++ti) {
                int m0, n0;
                tile_coords(p, tr.first + ti * tr.stride, rank, m0, n0);
                float cst[3][G_BN / 32];
#pragma unroll
                for (int i = 0; i < G_BN / 32; ++i) {
                    const int n = n0 + lane + 32 * i;
                    const bool in = n < p.N;
                    cst[0][i] = in ? __ldg(p.col_scale + n) : 1.0f;
                    cst[1][i] = in ? __ldg(p.col_bias + n) : 0.0f;
                    if constexpr (RTN > 0)
                        cst[2][i] = in ? __frcp_rn(h2f(p.next_smooth[(n & ~127) + packed_vec_pos(n & 127)])) : 1.0f;
                }
                if (ti > 0 && !wait_or_abort<32>(&sh->cempty, (ti - 1) & 1, sh, p.status, 60)) break;
                if constexpr (ROPE) {   // RMSNorm weights of q and k: the same for every tile
                    if (ti == 0) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            reinterpret_cast<h16*>(colv + 2 * G_BN)[lane + 32 * i] = p.rope_wq[lane + 32 * i];
                            reinterpret_cast<h16*>(colv + 2 * G_BN)[128 + lane + 32 * i] = p.rope_wk[lane + 32 * i];
                        }
                    }
                }
#pragma unroll
                for (int i = 0; i < G_BN / 32; ++i) {
                    colv[lane + 32 * i] = cst[0][i];
                    colv[G_BN + lane + 32 * i] = cst[1][i];
                    if constexpr (RTN > 0) colv[2 * G_BN + lane + 32 * i] = cst[2][i];
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh->cfull);
            }
        }
    } else if (LW && warp >= MMA_WARP + 4) {
        if constexpr (REGCTL) reg_dealloc<L_REGS_LORA>();
        // ------------------------------------------------------------------ next layer's LoRA-down (two-set requantising variants)
        // Warp q of this group takes every chunk of lane quadrant q, from whichever epilogue set staged it, in tile
        // order: [32 rows x 64 columns] of bf16 from the staging buffer times Wd_next[64 x Rn] (B fragments straight from
        // global memory, asked for before the wait for the tile), accumulated over the tiles of one 128-row block.
        constexpr int RTL = RTN > 0 ? RTN : 1;
        const int q = warp & 3;
        float lacc[2][RTL][8];
        auto lacc_zero = [&]() {
#pragma unroll
            for (int a = 0; a < 2; ++a)
#pragma unroll
                for (int b = 0; b < RTL; ++b)
#pragma unroll
                    for (int c = 0; c < 8; ++c) lacc[a][b][c] = 0.f;
        };
        lacc_zero();
        int cur_m0 = -1, slot = 0;
        uint32_t cnt[2] = {0u, 0u};   // chunks taken from each epilogue set's buffer
        bool ok = true;
        const bool prof_me = blockIdx.x == 0 && q == 0 && lane == 0;
        PROF_T0(pt_all);
        PROF_ACC(pa_wait);
        for (int ti = 0; ti < tr.count && ok; ++ti) {
            int m0, n0;
            tile_coords(p, tr.first + ti * tr.stride, rank, m0, n0);
            if (m0 != cur_m0) {
                if (cur_m0 >= 0) {
                    store_lora_partial<RTL>(p, lacc, slot++, q, lane);
                    lacc_zero();
                }
                cur_m0 = m0;
            }
#pragma unroll 1
            for (int h = 0; h < G_BN / 64; ++h) {
                if (n0 + h * 64 >= p.N) break;
                const int e = (h + ti) & 1;
                const int ch_tile0 = (n0 + h * 64) >> 4;
                uint4 bfrag[4][RTL];
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
#pragma unroll
                    for (int rt = 0; rt < RTL; ++rt)
                        bfrag[kk][rt] = __ldg(p.next_lora_down + (static_cast<size_t>(ch_tile0 + kk) * p.next_rt_total + rt) * 32 + lane);
                const uint32_t par = e ? cnt[1] : cnt[0];
                PROF_T0(pt_w);
                if (!wait_or_abort<32>(&sh->lfull[q][e], par & 1, sh, p.status, 70)) {
                    ok = false;
                    break;
                }
                PROF_ADD(pa_wait, pt_w);
                const uint32_t bufa = smem_u32(epi_smem + (q * 2 + e) * G_EPI_BUF_BYTES);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt) {
                        const int arow = mt * 16 + (lane & 15);
                        uint32_t a[4];
                        ldmatrix_x4(a, bufa + arow * 128 + (((2 * kk + (lane >> 4)) ^ (arow & 7)) << 4));
#pragma unroll
                        for (int rt = 0; rt < RTL; ++rt) {
                            mma_16816(*reinterpret_cast<float(*)[4]>(&lacc[mt][rt][0]), a, bfrag[kk][rt].x, bfrag[kk][rt].y);
                            mma_16816(*reinterpret_cast<float(*)[4]>(&lacc[mt][rt][4]), a, bfrag[kk][rt].z, bfrag[kk][rt].w);
                        }
                    }
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh->lempty[q][e]);   // the epilogue warp may stage its next chunk
                if (e) ++cnt[1]; else ++cnt[0];
            }
        }
        if (ok && cur_m0 >= 0) store_lora_partial<RTL>(p, lacc, slot, q, lane);
        PROF_ACC(pa_all);
        PROF_ADD(pa_all, pt_all);
        PROF_OUT(prof_me, 6, pa_all); PROF_OUT(prof_me, 7, pa_wait);
    } else if (I4 ? (warp >= 2 && warp < 6) : (warp >= 4 && warp < MMA_WARP)) {
        if constexpr (REGCTL) reg_alloc<REGS_E>();
        // ------------------------------------------------------------------ epilogue (INT4: warps 2..5; NVFP4: 4..7 and 8..11)
        // One row per thread.  Per 64-column chunk: two tcgen05.ld, scale + bias + activation, bf16 into a
        // 128B-swizzled [32 rows x 128 B] staging buffer of this warp, then one TMA store of that box (the
        // hardware clips rows >= M and columns >= N).  Two staging buffers per warp keep a store in flight.
        constexpr int SETS = epi_sets<RTN, I4>();
        const int q = warp & 3;  // TMEM lane quadrant this warp may read
        const int eset = I4 ? 0 : (warp - 4) >> 2;
        // one set: two staging buffers per warp (a store stays in flight); two sets: one buffer per warp
        uint8_t* my_buf = epi_smem + (q * 2 + (SETS == 2 ? eset : 0)) * G_EPI_BUF_BYTES;
        float* cvs = colv + q * G_COLV_FLOATS;   // INT4 only
        uint32_t nstore = 0;
        // Next layer's LoRA-down partial of this warp's 32 rows: [m-tile 2][rank tile][8].  ELORA: this warp computes it (one
        // epilogue set); otherwise the LoRA-down warps do, from the staged tiles.
        constexpr bool ELORA = RTN > 0 && !LW;
        constexpr int RTA = ELORA ? RTN : 1;
        float lacc[2][RTA][8];
        int cur_m0 = -1, slot = 0;
        auto lacc_zero = [&]() {
#pragma unroll
            for (int a = 0; a < 2; ++a)
#pragma unroll
                for (int b = 0; b < RTA; ++b)
#pragma unroll
                    for (int c = 0; c < 8; ++c) lacc[a][b][c] = 0.f;
        };
        auto lacc_flush = [&]() {   // partial of row block cur_m0 -> scratch[blockIdx][slot][128][Rn]
            if constexpr (ELORA) store_lora_partial<RTN>(p, lacc, slot++, q, lane);
        };
        lacc_zero();
        float4 rc[8], rs[8];   // ROPE: rotary table entries of this thread's row and this warp's 32 column pairs
        int rope_m0 = -1;
        uint32_t nx = 0;       // ROPE: exchanges of sums of squares so far
        const bool prof_me = blockIdx.x == 0 && (warp == (I4 ? 2 : 4)) && lane == 0;
        PROF_T0(pt_all);
        PROF_ACC(pa_tf); PROF_ACC(pa_tiles); PROF_ACC(pa_stage); PROF_ACC(pa_lora); PROF_ACC(pa_quant);

        for (int ti = 0; ti < tr.count; ++ti) {
            int m0, n0;
            tile_coords(p, tr.first + ti * tr.stride, rank, m0, n0);
            const uint32_t as = ti & 1;
            if constexpr (ELORA) {
                if (m0 != cur_m0) {
                    if (cur_m0 >= 0) {
                        lacc_flush();
                        lacc_zero();
                    }
                    cur_m0 = m0;
                }
            }
            // next layer's smoothing factors of the chunks this warp will take: fetched now, so that the loads fly while the
            // warp waits for the accumulator (lane l: columns l and l + 32 of each 64-column chunk)
            h16 nsm[G_BN / 64][2];
            if constexpr (RTN > 0 && I4) {
#pragma unroll
                for (int h = 0; h < G_BN / 64; ++h)
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const int n = n0 + h * 64 + lane + 32 * i;
                        nsm[h][i] = n < p.N ? p.next_smooth[(n & ~127) + packed_vec_pos(n & 127)] : f2h(1.0f);
                    }
            }
            // ROPE: this warp takes columns [64 eset, 64 eset + 64) of both heads of every tile, i.e. always the same 32 column
            // pairs of its rows: their rotary table entries (32 x (cos, sin) per thread, each lane another table row: 32
            // cache lines per load instruction) are fetched once per row block and stay in registers for all its tiles.
            if constexpr (ROPE) {
                if (m0 != rope_m0) {
                    rope_m0 = m0;
                    const int pos = (m0 + q * 32 + lane) % p.rope_seq_len;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        rc[j] = __ldg(reinterpret_cast<const float4*>(p.rope_cos + static_cast<size_t>(pos) * 64) + 8 * eset + j);
                        rs[j] = __ldg(reinterpret_cast<const float4*>(p.rope_sin + static_cast<size_t>(pos) * 64) + 8 * eset + j);
                    }
                }
            }
            PROF_T0(pt_tf);
            if (!wait_or_abort<64>(&sh->tfull[as], (ti >> 1) & 1, sh, p.status, 30)) break;
            PROF_ADD(pa_tf, pt_tf);
#ifdef SVDQ_ABLATE
            pa_tiles += 1;
#endif
            tc_fence_after_sync();
            if constexpr (!I4) {   // the tile's per-column constants are in shared memory
                if (!wait_or_abort<32>(&sh->cfull, ti & 1, sh, p.status, 31)) break;
            }
            const uint32_t taddr = tmem + (static_cast<uint32_t>(q * 32) << 16) + as * G_TM_ACC1;
            const int grow = m0 + q * 32 + lane;   // this thread's row (< M_pad)
            float rowsc = 1.0f;
            if constexpr (I4) rowsc = __ldg(p.row_scale + grow);
            bool sf_cols_free = I4;   // NVFP4: the accumulator's first columns become the next tile's scale-factor buffers
            bool epi_ok = true;
            if constexpr (ROPE) {
                // Both heads of the tile, one after the other; of each, this warp takes 64 columns (chunk `eset`) of its 32 rows,
                // one row per thread.  Values are rounded to the 16-bit type first and the norm and the rotation computed from
                // those, exactly as a separate pass over the stored tile would.  The two warps of a lane quadrant exchange their
                // halves of the row's sum of squares through shared memory (named barrier of the pair).
                const int pos = grow % p.rope_seq_len;          // token position of this thread's row
                const bool zero_row = p.rope_split && p.rope_attn_tokens > 0 && pos >= p.rope_attn_tokens;
                const int srow = m0 + q * 32;                   // first row of the warp's slab
                const int orow = !p.rope_split ? srow
                                               : (srow / p.rope_seq_len) * p.rope_tokens_pad + p.rope_token_offset + srow % p.rope_seq_len;
                float* xss = colv + 2 * G_BN + 128 + q * 64;   // [set 2][lane 32] of this quadrant
#pragma unroll 1
                for (int hd = 0; hd < 2; ++hd) {
                    const int hb = n0 + hd * 128;                   // first column of the head
                    const int which = hb / p.rope_dim;              // 0: q, 1: k, 2: v
                    const int ccol = hb - (p.rope_split ? which * p.rope_dim : 0) + eset * 64;   // output column of the chunk
                    uint32_t y[32];   // the chunk's 64 values of this row, packed
                    {
                        uint32_t r0[32], r1[32];
                        tc_ld_32x32b_x32(taddr + hd * 128 + eset * 64, r0);
                        tc_ld_32x32b_x32(taddr + hd * 128 + eset * 64 + 32, r1);
                        tc_wait_ld();
                        if (hd == 0) {
                            // columns [0, G_TM_SF_COLS) of this accumulator are in registers (this warp's share of them): the
                            // MMA warp may overwrite them with the next tile's scale factors
                            sf_cols_free = true;
                            tc_fence_before_sync();
                            __syncwarp();
                            if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&sh->sfree[as]), 0));
                        }
                        const float4* cs = reinterpret_cast<const float4*>(colv + hd * 128 + eset * 64);
                        const float4* cb = reinterpret_cast<const float4*>(colv + G_BN + hd * 128 + eset * 64);
#pragma unroll
                        for (int j = 0; j < 16; ++j) {   // columns 4j .. 4j+3 of the chunk
                            const uint32_t* rr = j < 8 ? &r0[4 * j] : &r1[4 * (j - 8)];
                            const float4 s4 = cs[j], b4 = cb[j];
                            y[2 * j] = pack2(__ffma2_rn(make_float2(__uint_as_float(rr[0]), __uint_as_float(rr[1])),
                                                        make_float2(s4.x, s4.y), make_float2(b4.x, b4.y)));
                            y[2 * j + 1] = pack2(__ffma2_rn(make_float2(__uint_as_float(rr[2]), __uint_as_float(rr[3])),
                                                            make_float2(s4.z, s4.w), make_float2(b4.z, b4.w)));
                        }
                    }
                    uint32_t o[32];
                    if (which < 2) {   // (uniform over the CTA: a tile lies inside q, k or v)
                        float2 ss = make_float2(0.f, 0.f);   // even and odd columns apart (packed fp32 arithmetic)
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const float2 f = unpack2(y[i]);
                            ss = __ffma2_rn(f, f, ss);
                        }
                        // the two warps of the quadrant exchange their halves of the sum (bounded waits, like everywhere else)
                        if (nx > 0 && !wait_or_abort(&sh->xread[q], (nx - 1) & 1, sh, p.status, 33)) {   // last exchange's values have been read
                            epi_ok = false;
                            break;
                        }
                        xss[eset * 32 + lane] = ss.x + ss.y;
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&sh->xsum[q]);
                        if (!wait_or_abort(&sh->xsum[q], nx & 1, sh, p.status, 34)) {
                            epi_ok = false;
                            break;
                        }
                        const float coef = rsqrtf((xss[lane] + xss[32 + lane]) * (1.0f / 128.0f) + p.rope_eps);
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&sh->xread[q]);
                        ++nx;
                        const float2 coef2 = make_float2(coef, coef);
                        const uint32_t* wn = reinterpret_cast<const uint32_t*>(colv + 2 * G_BN) + which * 64 + eset * 32;   // 16-bit pairs
#pragma unroll
                        for (int j = 0; j < 8; ++j) {   // four pairs = 8 columns per step
                            const float4 c4a = rc[j], s4a = rs[j];
                            const uint4 w4 = *reinterpret_cast<const uint4*>(wn + 4 * j);
                            // (a, b) = y * (coef * w) as packed pairs; (a c - b s, a s + b c) = (a, b) * c + (-b s, a s)
                            const float2 ab0 = __fmul2_rn(unpack2(y[4 * j]), __fmul2_rn(coef2, unpack2(w4.x)));
                            const float2 ab1 = __fmul2_rn(unpack2(y[4 * j + 1]), __fmul2_rn(coef2, unpack2(w4.y)));
                            const float2 ab2 = __fmul2_rn(unpack2(y[4 * j + 2]), __fmul2_rn(coef2, unpack2(w4.z)));
                            const float2 ab3 = __fmul2_rn(unpack2(y[4 * j + 3]), __fmul2_rn(coef2, unpack2(w4.w)));
                            const float2 t0 = __fmul2_rn(ab0, make_float2(c4a.x, c4a.x)), t1 = __fmul2_rn(ab1, make_float2(c4a.y, c4a.y));
                            const float2 t2 = __fmul2_rn(ab2, make_float2(c4a.z, c4a.z)), t3 = __fmul2_rn(ab3, make_float2(c4a.w, c4a.w));
                            o[4 * j] = pack2(make_float2(fmaf(-ab0.y, s4a.x, t0.x), fmaf(ab0.x, s4a.x, t0.y)));
                            o[4 * j + 1] = pack2(make_float2(fmaf(-ab1.y, s4a.y, t1.x), fmaf(ab1.x, s4a.y, t1.y)));
                            o[4 * j + 2] = pack2(make_float2(fmaf(-ab2.y, s4a.z, t2.x), fmaf(ab2.x, s4a.z, t2.y)));
                            o[4 * j + 3] = pack2(make_float2(fmaf(-ab3.y, s4a.w, t3.x), fmaf(ab3.x, s4a.w, t3.y)));
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = y[i];
                    }
                    if (zero_row) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = 0u;
                    }
                    if (lane == 0) bulk_wait_group_read<0>();   // the store that last used this buffer has been read
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        *reinterpret_cast<uint4*>(my_buf + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                            make_uint4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        const CUtensorMap* omap = !p.rope_split ? &tm_out : which == 0 ? &tm_rope.q : which == 1 ? &tm_rope.k : &tm_rope.v;
                        if (srow < p.M) tma_store_2d(omap, my_buf, ccol, orow);
                        bulk_commit_group();
                    }
                }
            }
#pragma unroll 1
            for (int h = 0; h < (ROPE ? 0 : G_BN / 64); ++h) {
                if (n0 + h * 64 >= p.N || ABLATE(p, 0)) break;
                if (SETS == 2 && ((h + ti) & 1) != eset) continue;   // the other warp of this quadrant takes it
                uint32_t r0[32], r1[32];
                tc_ld_32x32b_x32(taddr + h * 64, r0);
                tc_ld_32x32b_x32(taddr + h * 64 + 32, r1);
                if constexpr (RTN > 0 && I4) {   // reciprocal smoothing factors of the chunk's 64 columns (next layer), un-permuted
                    __syncwarp();          // every lane is done with the previous chunk's factors
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        h16 v = nsm[0][i];
#pragma unroll
                        for (int hh = 1; hh < G_BN / 64; ++hh) v = h == hh ? nsm[hh][i] : v;   // registers: no dynamic indexing
                        cvs[lane + 32 * i] = __frcp_rn(h2f(v));
                    }
                }
                uint8_t* buf = SETS == 2 ? my_buf : my_buf + (nstore & 1) * G_EPI_BUF_BYTES;
                if (lane == 0) {   // the store that last used this buffer has been read
                    if (SETS == 2) bulk_wait_group_read<0>(); else bulk_wait_group_read<1>();
                }
                if constexpr (LW) {   // ... and so has the LoRA-down warp of this quadrant
                    PROF_T0(pt_le);
                    if (nstore > 0 && !wait_or_abort<32>(&sh->lempty[q][eset], (nstore - 1) & 1, sh, p.status, 32)) {
                        epi_ok = false;
                        break;
                    }
                    PROF_ADD(pa_lora, pt_le);
                }
                __syncwarp();
                tc_wait_ld();
                if (!sf_cols_free && h >= G_TM_SF_COLS / 64 - (SETS == 2 ? 1 : 0)) {
                    // columns [0, G_TM_SF_COLS) of this accumulator are in registers (this warp's share of them): the MMA
                    // warp may overwrite them with the next tile's scale factors
                    sf_cols_free = true;
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&sh->sfree[as]), 0));
                }
                // per-column scale and bias (the same address in every lane).  NVFP4: staged in shared memory per tile; INT4
                // (every warp has a job there): straight from global memory
                const float4* cs = reinterpret_cast<const float4*>(I4 ? p.col_scale + n0 + h * 64 : colv + h * 64);
                const float4* cb = reinterpret_cast<const float4*>(I4 ? p.col_bias + n0 + h * 64 : colv + G_BN + h * 64);
#ifdef SVDQ_ABLATE
                if (I4 && ABLATE(p, 7)) {   // always the same 256 bytes of per-column constants: they stay in L1
                    cs = reinterpret_cast<const float4*>(p.col_scale);
                    cb = reinterpret_cast<const float4*>(p.col_bias);
                }
#endif
                uint32_t ow[32];   // this thread's 64 bf16 outputs, packed (kept for the requantisation)
                PROF_T0(pt_stage);
                if constexpr (RTN > 0) {
                    // the reference's requantising branch always applies GELU (gemm_w4a4_launch_impl.cuh:282-309)
                    stage_chunk<SVDQ_ACT_GELU, I4, !I4>(r0, r1, cs, cb, ow, buf, lane, rowsc);
                } else {
                    if (p.activation == SVDQ_ACT_GELU) stage_chunk<SVDQ_ACT_GELU, I4, !I4>(r0, r1, cs, cb, ow, buf, lane, rowsc);
                    else if (p.activation == SVDQ_ACT_SILU) stage_chunk<SVDQ_ACT_SILU, I4, !I4>(r0, r1, cs, cb, ow, buf, lane, rowsc);
                    else stage_chunk<SVDQ_ACT_NONE, I4, !I4>(r0, r1, cs, cb, ow, buf, lane, rowsc);
                }
                fence_proxy_async_smem();
                __syncwarp();
                PROF_ADD(pa_stage, pt_stage);
                if (lane == 0) {
                    if constexpr (LW) mbar_arrive(&sh->lfull[q][eset]);   // the staged tile is complete: the LoRA-down warp may read it
                    if (p.store_out && m0 + q * 32 < p.M) tma_store_2d(&tm_out, buf, n0 + h * 64, m0 + q * 32);
                    bulk_commit_group();
                }
                ++nstore;

                if constexpr (RTN > 0) {
                    // The chunk's slice of the next layer's LoRA-down weight (B fragments, from L2) is asked for now and used after
                    // the quantisation below, whose work covers the latency.  Rank 64: half now, half before the products.
                    const int ch_tile0 = (n0 + h * 64) >> 4;           // 16-channel tile index of the chunk
                    constexpr int KPRE = RTN <= 2 ? 4 : 2;
                    uint4 bfrag[4][RTA];
                    auto load_bfrag = [&](int kk) {
                        if constexpr (ELORA) {
#pragma unroll
                        for (int rt = 0; rt < RTN; ++rt) {
#ifdef SVDQ_ABLATE
                            if (ABLATE(p, 5)) { bfrag[kk][rt] = make_uint4(kk, rt, lane, 0); continue; }
#endif
                            bfrag[kk][rt] = __ldg(p.next_lora_down + (static_cast<size_t>(ch_tile0 + kk) * p.next_rt_total + rt) * 32 + lane);
                        }
                        }
                    };
#pragma unroll
                    for (int kk = 0; kk < KPRE; ++kk) load_bfrag(kk);
                    PROF_T0(pt_quant);
                    const float4* rcn = reinterpret_cast<const float4*>(I4 ? cvs : colv + 2 * G_BN + h * 64);
                    uint4* qdst = reinterpret_cast<uint4*>(p.qout + static_cast<size_t>(grow) * (p.N >> 1) + ((n0 + h * 64) >> 1));
                    if constexpr (I4) {
                        // ---- INT4 group quantisation: this thread's 64 values are exactly one group of the next layer;
                        // u4 codes of bf16(bf16(y + 0.171875) / smooth), scale = max / 15 (gemm_w4a4_launch_impl.cuh:282-309)
                        uint32_t qv[4][8];
                        float amax = 0.f;
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            uint32_t xw[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const float2 f = unpack2(ow[8 * g + i]);
                                xw[i] = pack2(make_float2(f.x + 0.171875f, f.y + 0.171875f));
                            }
                            amax = fmaxf(amax, smooth16(xw, rcn + 4 * g, qv[g]));
                        }
                        uint32_t codes[8];
                        float scale = 0.f;
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            uint32_t cw[2];
                            scale = int4_encode16<true>(qv[g], amax, cw);
                            codes[2 * g] = cw[0];
                            codes[2 * g + 1] = cw[1];
                        }
                        qdst[0] = make_uint4(codes[0], codes[1], codes[2], codes[3]);
                        qdst[1] = make_uint4(codes[4], codes[5], codes[6], codes[7]);
                        reinterpret_cast<h16*>(p.oscales)[static_cast<size_t>((n0 + h * 64) >> 6) * p.M_pad + grow] = f2h(scale);
                    } else {
                        // ---- NVFP4 group quantisation of this thread's 64 values (4 groups of 16)
                        uint32_t codes[8];
                        uint32_t sw = 0;
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            const uint32_t xw[8] = {ow[8 * g], ow[8 * g + 1], ow[8 * g + 2], ow[8 * g + 3],
                                                    ow[8 * g + 4], ow[8 * g + 5], ow[8 * g + 6], ow[8 * g + 7]};
                            uint32_t qv[8];
                            const float amax = smooth16(xw, rcn + 4 * g, qv);
                            uint32_t cw[2];
                            sw |= nvfp4_encode16(qv, amax, cw) << (8 * g);
                            codes[2 * g] = cw[0];
                            codes[2 * g + 1] = cw[1];
                        }
                        qdst[0] = make_uint4(codes[0], codes[1], codes[2], codes[3]);
                        qdst[1] = make_uint4(codes[4], codes[5], codes[6], codes[7]);
                        const size_t soff = (static_cast<size_t>(grow >> 7) * (p.N >> 6) + ((n0 + h * 64) >> 6)) * 512 +
                                            (grow & 31) * 16 + ((grow >> 5) & 3) * 4;
                        *reinterpret_cast<uint32_t*>(p.oscales + soff) = sw;
                    }
                    PROF_ADD(pa_quant, pt_quant);
                    // ---- next layer's LoRA-down on the staged bf16 tile: [32 x 64] x Wd_next[64 x Rn]
                    PROF_T0(pt_lora);
#pragma unroll
                    for (int kk = KPRE; kk < 4; ++kk) load_bfrag(kk);
                    const uint32_t bufa = smem_u32(buf);
#pragma unroll
                    for (int kk = 0; kk < (ELORA ? 4 : 0); ++kk) {
#ifdef SVDQ_ABLATE
                        if (ABLATE(p, 6)) {
#pragma unroll
                            for (int rt = 0; rt < RTN; ++rt)
                                lacc[0][rt][0] += __uint_as_float(bfrag[kk][rt].x ^ bfrag[kk][rt].y ^ bfrag[kk][rt].z ^ bfrag[kk][rt].w);
                            continue;
                        }
#endif
#pragma unroll
                        for (int mt = 0; mt < 2; ++mt) {
                            const int arow = mt * 16 + (lane & 15);
                            uint32_t a[4];
                            ldmatrix_x4(a, bufa + arow * 128 + (((2 * kk + (lane >> 4)) ^ (arow & 7)) << 4));
#pragma unroll
                            for (int rt = 0; rt < RTN; ++rt) {
                                mma_16816(*reinterpret_cast<float(*)[4]>(&lacc[mt][rt][0]), a, bfrag[kk][rt].x, bfrag[kk][rt].y);
                                mma_16816(*reinterpret_cast<float(*)[4]>(&lacc[mt][rt][4]), a, bfrag[kk][rt].z, bfrag[kk][rt].w);
                            }
                        }
                    }
                    PROF_ADD(pa_lora, pt_lora);
                }
            }
            if (!epi_ok) break;
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if (!sf_cols_free) mbar_arrive_cluster(mapa_shared(smem_u32(&sh->sfree[as]), 0));
                mbar_arrive_cluster(mapa_shared(smem_u32(&sh->tempty[as]), 0));
                if constexpr (!I4) mbar_arrive(&sh->cempty);   // this warp is done with the tile's constants
            }
        }
        if constexpr (ELORA) {
            if (cur_m0 >= 0) lacc_flush();
        }
        PROF_ACC(pa_all);
        PROF_ADD(pa_all, pt_all);
        PROF_OUT(prof_me, 8, pa_all); PROF_OUT(prof_me, 9, pa_tf); PROF_OUT(prof_me, 10, pa_tiles);
        PROF_OUT(prof_me, 13, pa_stage); PROF_OUT(prof_me, 14, pa_lora); PROF_OUT(prof_me, 15, pa_quant);
        if (lane == 0) bulk_wait_group<0>();  // all stores of this warp have landed
    }

    // Neither CTA may leave (or give up its TMEM) while the other can still signal its barriers or the
    // leader's MMAs can still read its shared memory: both have passed all their tiles here.
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();
    if (warp == MMA_WARP) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem, G_TMEM_COLS);
    }
}

// lora_act_out[row][r] = sum over the pairs that touched the row's 256-row block, in pair order, of the partial
// of the CTA that owns the row's half.  Row block mb2 (256 rows) holds pair tiles [mb2*tiles_n, (mb2+1)*tiles_n);
// pair c owns tiles [c*run, (c+1)*run); CTA 2c + h of the pair owns rows h*128.. of each tile.
__global__ void __launch_bounds__(256)
lora_partial_reduce_kernel(const float* __restrict__ partial, float* __restrict__ out, int rn, int ld, int tiles_n, int run, int slots,
                           int npairs) {
    const int mb = blockIdx.x;   // 128-row block
    const int mb2 = mb >> 1, h = mb & 1;
    const int c_lo = (mb2 * tiles_n) / run;
    const int c_hi = min(npairs - 1, ((mb2 + 1) * tiles_n - 1) / run);
    const int n4 = G_BM * rn / 4;   // float4 elements of one block; gridDim.y CTAs share them
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < n4; i += gridDim.y * blockDim.x) {
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int c = c_lo; c <= c_hi; ++c) {
            const int first_mb2 = (c * run) / tiles_n;
            const float4 v = __ldg(reinterpret_cast<const float4*>(
                                       partial + (static_cast<size_t>(2 * c + h) * slots + (mb2 - first_mb2)) * (G_BM * rn)) + i);
            s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        }
        const int e = 4 * i;   // element (row, rank) of the block; `out` rows are `ld` floats apart
        *reinterpret_cast<float4*>(out + (static_cast<size_t>(mb) * G_BM + e / rn) * ld + e % rn) = s;
    }
}

// INT4 activations reach the tensor core as fp16(code * group scale).  fp16 has 5 exponent bits, bf16 scales have 8: a
// power of two is taken out of every ROW first (2^e with the row's largest group scale / 2^e in [1, 2)), the accumulator
// is multiplied by it again in the epilogue.  So no scale is clamped and only groups more than 2^14 below their row's
// largest lose bits.  The low-rank activations share the accumulator and are divided by the same factor (into scratch).
// One CTA per 128 rows: thread = row for the maximum, then all threads copy the block's low-rank rows.
__global__ void __launch_bounds__(128)
int4_row_norm_kernel(const h16* __restrict__ ascales, int KB, int M_pad, const float* __restrict__ lora_in, int R,
                     float* __restrict__ row_scale, float* __restrict__ lora_out) {
    __shared__ float inv[128];
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x * 128 + threadIdx.x;
    float mx = 0.f;
    for (int g = 0; g < KB; ++g) mx = fmaxf(mx, fabsf(h2f(ascales[static_cast<size_t>(g) * M_pad + row])));
    int e = 0;
    if (mx > 0.f && mx < 3.0e38f) {
        (void)frexpf(mx, &e);   // mx = f * 2^e, f in [0.5, 1)
        e -= 1;
    }
    e = max(-120, min(120, e));
    row_scale[row] = ldexpf(1.0f, e);
    inv[threadIdx.x] = ldexpf(1.0f, -e);
    __syncthreads();
    if (lora_in != nullptr) {
        const size_t base = static_cast<size_t>(blockIdx.x) * 128 * R;
        for (int i = threadIdx.x; i < 128 * R; i += 128) lora_out[base + i] = lora_in[base + i] * inv[i / R];
    }
}

struct NvfpPlan {
    int requant, tiles_m, tiles_n, npairs, run, slots;   // tiles are 256 x 256 pair tiles
    int rn;              // ranks of the next layer's LoRA-down that the epilogue computes: the first 16, 32 or 64
    size_t partials;     // bytes of the per-CTA partials
    size_t workspace;    // partials + (when further ranks are left and the caller wants no `out`) a bf16 copy of the output
};

// The epilogue holds the next layer's LoRA-down accumulators in registers: 16, 32 or 64 ranks.  Any further ranks
// (lora.cuh:22 allows up to 1024) are computed from the bf16 output by follow-up launches of the quantiser's LoRA-down.
static inline int fused_next_rank(int r_next) { return r_next >= 64 ? 64 : r_next >= 32 ? 32 : 16; }

static void plan_nvfp4(const svdq_gemm_args* a, int sms, NvfpPlan* pl) {
    pl->requant = a->qout != nullptr;
    pl->tiles_n = (a->N + G_BN - 1) / G_BN;
    pl->tiles_m = pl->requant ? a->M_pad / (2 * G_BM) : (a->M + 2 * G_BM - 1) / (2 * G_BM);   // M_pad is a multiple of 256
    const int num_tiles = pl->tiles_m * pl->tiles_n;
    const int max_pairs = sms / 2 > 0 ? sms / 2 : 1;
    pl->npairs = num_tiles < max_pairs ? num_tiles : max_pairs;
    pl->run = (num_tiles + pl->npairs - 1) / pl->npairs;
    if (pl->requant) pl->npairs = (num_tiles + pl->run - 1) / pl->run;
    pl->slots = (pl->run + pl->tiles_n - 2) / pl->tiles_n + 1;
    pl->rn = fused_next_rank(a->R_next);
    pl->partials = pl->requant ? static_cast<size_t>(2 * pl->npairs) * pl->slots * G_BM * pl->rn * sizeof(float) : 0;
    const bool out_copy = pl->requant && a->R_next > pl->rn && a->out == nullptr;
    pl->workspace = pl->partials + (out_copy ? ((static_cast<size_t>(a->M) * a->N * 2 + 255) & ~static_cast<size_t>(255)) : 0);
}

// Launch the fused kernel for the plan's rank count, add up the partials, then the ranks the epilogue did not take.
template <bool I4>
static int launch_requant(const svdq_gemm_args* a, const NvfpPlan& pl, cudaStream_t stream, const CUtensorMap& tm_a, const CUtensorMap& tm_b,
                          const CUtensorMap& tm_la, const CUtensorMap& tm_lu, const CUtensorMap& tm_out, const CUtensorMap& tm_sfa,
                          const CUtensorMap& tm_sfb, const GemmParams& p, const void* out_bf16);


// real column count of `out`: the store's tensor map ends there, so the hardware drops the padded columns
static inline int n_out(const svdq_gemm_args* a) { return a->N_out ? a->N_out : a->N; }
static inline bool n_out_ok(const svdq_gemm_args* a) {
    return n_out(a) <= a->N && n_out(a) > a->N - 128 && n_out(a) % 8 == 0;
}

int gemm_nvfp4_workspace_bytes(const svdq_gemm_args* a, size_t* bytes) {
    int sms = 0;
    if (int rc = sm_count(&sms)) return rc;
    NvfpPlan pl;
    plan_nvfp4(a, sms, &pl);
    *bytes = pl.workspace;
    return SVDQ_OK;
}

template <int RTN, bool I4, bool ROPE = false>
static int launch_pair(int grid, cudaStream_t stream, const CUtensorMap& a, const CUtensorMap& b, const CUtensorMap& la,
                        const CUtensorMap& lu, const CUtensorMap& o, const CUtensorMap& sfa, const CUtensorMap& sfb,
                        const GemmParams& p, const RopeMaps* rope = nullptr) {
    static std::atomic<uint64_t> attr_done{0};
    if (int rc = ensure_dynamic_smem(gemm_w4a4_kernel<RTN, I4, ROPE>, smem_bytes<I4>(), attr_done)) return rc;
    RopeMaps rm;
    if (rope) rm = *rope;
    else rm.q = rm.k = rm.v = a;   // unused: any valid map
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);   // 2 CTAs per pair
    cfg.blockDim = dim3(cta_threads<RTN, I4>(), 1, 1);
    cfg.dynamicSmemBytes = smem_bytes<I4>();
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // overlap launch + prologue with the predecessor's tail
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    SVDQ_CUDA(cudaLaunchKernelEx(&cfg, gemm_w4a4_kernel<RTN, I4, ROPE>, a, b, la, lu, o, sfa, sfb, rm, p));
    return SVDQ_OK;
}

int gemm_nvfp4_impl(const svdq_gemm_args* a, cudaStream_t stream) {
    const bool requant = a->qout != nullptr;
    SVDQ_CHECK_ARG(a->out != nullptr || requant || (a->rope_cos && a->rope_out_q), "gemm(nvfp4): neither `out` nor `qout` given");
    SVDQ_CHECK_ARG(a->act_layout == SVDQ_LAYOUT_NATIVE, "gemm(nvfp4): activations must be in SVDQ_LAYOUT_NATIVE "
                                                         "(convert with svdq_w4a4_relayout_act)");
    SVDQ_CHECK_ARG(!a->act_unsigned, "gemm(nvfp4): act_unsigned is INT4 only (gemm_w4a4_launch_impl.cuh:127)");
    SVDQ_CHECK_ARG(a->R % 16 == 0 && a->R >= 0 && a->R <= SVDQ_MAX_LORA_RANK, "gemm: R (%d) must be a multiple of 16, at most %d", a->R, SVDQ_MAX_LORA_RANK);
    SVDQ_CHECK_ARG(n_out_ok(a), "gemm: N_out (%d) must be a multiple of 8 with N - 128 < N_out <= N (%d)", a->N_out, a->N);
    SVDQ_CHECK_ARG(a->R == 0 || (a->lora_act_in && a->w.lora_up), "gemm: low-rank tensors missing");
    if (requant) {
        SVDQ_CHECK_ARG(a->oscales && a->lora_act_out && a->next_smooth && a->next_lora_down,
                       "gemm(nvfp4): requantisation needs oscales, lora_act_out, next_smooth and next_lora_down");
        SVDQ_CHECK_ARG(a->next_fp4, "gemm(nvfp4): the requantised output must be NVFP4 as well");
        SVDQ_CHECK_ARG(a->out_layout == SVDQ_LAYOUT_NATIVE, "gemm(nvfp4): requantised output is written in SVDQ_LAYOUT_NATIVE");
        SVDQ_CHECK_ARG(a->activation == SVDQ_ACT_GELU, "gemm(nvfp4): the requantising epilogue applies GELU "
                                                       "(gemm_w4a4_launch_impl.cuh:282-309); set activation = SVDQ_ACT_GELU");
        SVDQ_CHECK_ARG(aligned(a->qout, 16) && aligned(a->oscales, 16) && aligned(a->lora_act_out, 16) &&
                           aligned(a->next_smooth, 16) && aligned(a->next_lora_down, 16) && aligned(a->workspace, 256),
                       "gemm(nvfp4): requantisation tensors must be 16-byte aligned (workspace: 256)");
        SVDQ_CHECK_ARG(a->R_next >= 16 && a->R_next % 16 == 0 && a->R_next <= SVDQ_MAX_LORA_RANK,
                       "gemm(nvfp4): R_next (%d) must be a multiple of 16 in [16, %d]", a->R_next, SVDQ_MAX_LORA_RANK);
        SVDQ_CHECK_ARG(a->R_next <= 64 || n_out(a) == a->N, "gemm(nvfp4): next-layer ranks above 64 need an unpadded output (N_out == N)");
    }

    int sms = 0;
    if (int rc = sm_count(&sms)) return rc;
    NvfpPlan pl;
    plan_nvfp4(a, sms, &pl);
    SVDQ_CHECK_ARG(!requant || (a->workspace && a->workspace_bytes >= pl.workspace),
                   "gemm(nvfp4): workspace of %zu bytes required (svdq_gemm_w4a4_workspace_bytes)", pl.workspace);

    GemmParams p = {};
    p.sfa = static_cast<const uint8_t*>(a->ascales);
    p.sfb = static_cast<const uint8_t*>(a->w.wscales);
    p.col_scale = a->w.col_scale;
    p.col_bias = a->w.col_bias;
    p.M = a->M;
    p.M_pad = a->M_pad;
    p.N = a->N;
    p.K = a->K;
    p.lora_chunks = (a->R + 31) / 32;
    p.tiles_m = pl.tiles_m;
    p.tiles_n = pl.tiles_n;
    p.activation = a->activation;
    // the bf16 output: the caller's, or (ranks left for the follow-up LoRA-down and no `out` wanted) a copy in the workspace
    void* const out_bf16 = a->out ? a->out : (pl.workspace > pl.partials ? static_cast<uint8_t*>(a->workspace) + pl.partials : nullptr);
    p.store_out = out_bf16 != nullptr;
    p.contiguous = requant;
    p.run = pl.run;
    p.qout = static_cast<uint8_t*>(a->qout);
    p.oscales = static_cast<uint8_t*>(a->oscales);
    p.next_smooth = static_cast<const h16*>(a->next_smooth);
    p.next_lora_down = static_cast<const uint4*>(a->next_lora_down);
    p.next_rt_total = a->R_next / 16;
    p.lora_partial = static_cast<float*>(a->workspace);
    p.slots = pl.slots;
#ifdef SVDQ_ABLATE
    if (const char* e = getenv("SVDQ_ABLATE")) p.ablate = atoi(e);
#endif
    if (int rc = status_words(&p.status)) return rc;

    CUtensorMap tm_a, tm_b, tm_la, tm_lu, tm_out, tm_sfa, tm_sfb;
    if (int rc = make_tmap_2d(&tm_a, a->act, CU_TENSOR_MAP_DATA_TYPE_UINT8, a->K / 2, a->M_pad, a->K / 2, 128, G_BM)) return rc;
    if (int rc = make_tmap_2d(&tm_b, a->w.wgt, CU_TENSOR_MAP_DATA_TYPE_UINT8, a->K / 2, a->N, a->K / 2, 128, G_BNH)) return rc;
    if (a->R > 0) {
        const int R32 = (a->R + 31) / 32 * 32;
        if (int rc = make_tmap_2d(&tm_la, a->lora_act_in, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, a->R, a->M_pad,
                                  static_cast<uint64_t>(a->R) * 4, 32, G_BM))
            return rc;
        if (int rc = make_tmap_2d(&tm_lu, a->w.lora_up, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, R32, a->N,
                                  static_cast<uint64_t>(R32) * 4, 32, G_BNH))
            return rc;
    } else {
        tm_la = tm_a;
        tm_lu = tm_b;
    }
    if (out_bf16) {
        if (int rc = make_tmap_2d(&tm_out, out_bf16, SVDQ_TMAP_16, n_out(a), a->M, static_cast<uint64_t>(n_out(a)) * 2, 64, 32))
            return rc;
    } else {
        tm_out = tm_a;
    }
    {   // scale atoms: [row atom][K/64][512 bytes]; a stage takes 4 k-blocks of one atom (A) / of two atoms (B)
        const uint64_t KB = a->K / 64;
        if (int rc = make_tmap_2d(&tm_sfa, a->ascales, CU_TENSOR_MAP_DATA_TYPE_UINT32, 128, static_cast<uint64_t>(a->M_pad / 128) * KB,
                                  512, 128, 4, /*swizzle128=*/false))
            return rc;
        if (int rc = make_tmap_3d(&tm_sfb, a->w.wscales, CU_TENSOR_MAP_DATA_TYPE_UINT32, 128, KB, a->N / 128, 512, KB * 512, 128, 4, 2))
            return rc;
    }
    int rc;
    if (a->rope_cos != nullptr) {
        // RMSNorm + rotary embedding of a fused QKV projection inside the epilogue
        const int dim = a->rope_heads * 128;
        const bool split = a->rope_out_q != nullptr;
        if (requant || a->activation != SVDQ_ACT_NONE || a->N != 3 * dim || n_out(a) != a->N || dim % G_BN != 0 ||
            a->rope_seq_len <= 0 || a->rope_seq_len % 32 != 0 || a->M % a->rope_seq_len != 0 || (!split && a->out == nullptr))
            return fail(SVDQ_ERR_UNSUPPORTED, "gemm(nvfp4): this fused RMSNorm + RoPE epilogue is built for a plain QKV projection "
                                              "with N = 3 * heads * 128 (heads even), rows = batch * seq_len and seq_len a multiple of 32");
        SVDQ_CHECK_ARG(a->rope_sin && a->rope_norm_q && a->rope_norm_k && aligned(a->rope_cos, 16) && aligned(a->rope_sin, 16),
                       "gemm(nvfp4): rope_sin, rope_norm_q, rope_norm_k are required; the tables must be 16-byte aligned");
        p.rope_wq = static_cast<const h16*>(a->rope_norm_q);
        p.rope_wk = static_cast<const h16*>(a->rope_norm_k);
        p.rope_cos = a->rope_cos;
        p.rope_sin = a->rope_sin;
        p.rope_eps = a->rope_eps;
        p.rope_seq_len = a->rope_seq_len;
        p.rope_dim = dim;
        p.rope_split = split ? 1 : 0;
        p.rope_tokens_pad = a->rope_tokens_pad;
        p.rope_token_offset = a->rope_token_offset;
        p.rope_attn_tokens = a->rope_attn_tokens;
        // n-fastest tile order in contiguous runs: a pair stays on one row block for many tiles, whose rotary table entries
        // its epilogue warps keep in registers
        p.contiguous = 1;
        p.run = pl.run;
        RopeMaps rm;
        rm.q = rm.k = rm.v = tm_a;
        if (split) {
            SVDQ_CHECK_ARG(a->rope_out_k && a->rope_out_v && a->rope_tokens_pad >= a->rope_token_offset + a->rope_seq_len &&
                               a->rope_token_offset >= 0,
                           "gemm(nvfp4): split q / k / v outputs need all three tensors and tokens_pad >= token_offset + seq_len");
            const uint64_t rows = static_cast<uint64_t>(a->M / a->rope_seq_len) * a->rope_tokens_pad;
            void* outs[3] = {a->rope_out_q, a->rope_out_k, a->rope_out_v};
            CUtensorMap* maps[3] = {&rm.q, &rm.k, &rm.v};
            for (int i = 0; i < 3; ++i)
                if (int rc = make_tmap_2d(maps[i], outs[i], SVDQ_TMAP_16, dim, rows, static_cast<uint64_t>(dim) * 2, 64, 32)) return rc;
            p.store_out = 1;
        }
        return launch_pair<0, false, true>(2 * pl.npairs, stream, tm_a, tm_b, tm_la, tm_lu, tm_out, tm_sfa, tm_sfb, p, &rm);
    }
    if (!requant) return launch_pair<0, false>(2 * pl.npairs, stream, tm_a, tm_b, tm_la, tm_lu, tm_out, tm_sfa, tm_sfb, p);
    return launch_requant<false>(a, pl, stream, tm_a, tm_b, tm_la, tm_lu, tm_out, tm_sfa, tm_sfb, p, out_bf16);
}

template <bool I4>
static int launch_requant(const svdq_gemm_args* a, const NvfpPlan& pl, cudaStream_t stream, const CUtensorMap& tm_a, const CUtensorMap& tm_b,
                          const CUtensorMap& tm_la, const CUtensorMap& tm_lu, const CUtensorMap& tm_out, const CUtensorMap& tm_sfa,
                          const CUtensorMap& tm_sfb, const GemmParams& p, const void* out_bf16) {
    int rc;
    if (pl.rn == 16) rc = launch_pair<1, I4>(2 * pl.npairs, stream, tm_a, tm_b, tm_la, tm_lu, tm_out, tm_sfa, tm_sfb, p);
    else if (pl.rn == 32) rc = launch_pair<2, I4>(2 * pl.npairs, stream, tm_a, tm_b, tm_la, tm_lu, tm_out, tm_sfa, tm_sfb, p);
    else rc = launch_pair<4, I4>(2 * pl.npairs, stream, tm_a, tm_b, tm_la, tm_lu, tm_out, tm_sfa, tm_sfb, p);
    if (rc) return rc;
    lora_partial_reduce_kernel<<<dim3(2 * pl.tiles_m, (G_BM * pl.rn / 4 + 255) / 256), 256, 0, stream>>>(
        p.lora_partial, a->lora_act_out, pl.rn, a->R_next, pl.tiles_n, pl.run, pl.slots, pl.npairs);
    SVDQ_CUDA(cudaGetLastError());
    if (a->R_next > pl.rn)
        return lora_down_rank_tiles(out_bf16, a->M, a->M_pad, a->N, a->next_smooth, a->next_lora_down, a->R_next / 16, pl.rn / 16,
                                    a->lora_act_out, stream);
    return SVDQ_OK;
}

// ---------------------------------------------------------------------------------------------------
// INT4 (group 64).  Reference: gemm_w4a4_kernel, src/kernels/zgemm/gemm_w4a4.cuh:832-928,1046-1095; scale application
// gemm_base.cuh:367-409:
//   acc[m, n] = sum_g ascale[m, g] * wscale[n, g] * ( sum_{k in group g} a[m, k] * w[n, k] ) + sum_r lora_act[m, r] * Wu[n, r]
// sm_100 has no 4-bit integer MMA kind and no block-scaled kind with bf16 scales, and rescaling an integer accumulator
// per group on the SIMT pipes costs M*N*K/64 multiply-adds plus as many TMEM reads.  Both operands are therefore turned
// into fp16 numbers that already carry their group scale - the weights once at preparation time, the activations by
// converter warps as the packed codes arrive in shared memory - and the same pair kernel runs kind::f16 MMAs into one
// fp32 accumulator.  A signed code has at most 3 significant bits and a bf16 scale 8, so code * scale is exact in fp16
// (11 bits); an unsigned code (act_unsigned, up to 15) has 4, and an odd code >= 9 times a scale with a full mantissa is
// rounded by at most 2^-12 relative.  Every product of two fp16 operands is exact in fp32, so apart from that rounding the
// only difference to the integer formulation is the order of fp32 additions.  (The reference adds the per-group terms
// in bf16.)  Range: a power of two is taken out of every activation row and every weight column beforehand and put
// back in the epilogue (int4_row_norm_kernel, prepare.cu), so nothing is clamped.
// ---------------------------------------------------------------------------------------------------
// scratch of the INT4 GEMM: [row scales M_pad fp32 | normalised low-rank activations M_pad x R fp32 | LoRA-down partials]
static inline size_t align256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }
static inline size_t int4_rows_bytes(const svdq_gemm_args* a) { return align256(static_cast<size_t>(a->M_pad) * 4); }
static inline size_t int4_lora_bytes(const svdq_gemm_args* a) { return align256(static_cast<size_t>(a->M_pad) * a->R * 4); }

int gemm_int4_workspace_bytes(const svdq_gemm_args* a, size_t* bytes) {
    size_t partials = 0;
    if (a->qout) {
        if (int rc = gemm_nvfp4_workspace_bytes(a, &partials)) return rc;
    }
    *bytes = int4_rows_bytes(a) + int4_lora_bytes(a) + partials;
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
        SVDQ_CHECK_ARG(a->R_next >= 16 && a->R_next % 16 == 0 && a->R_next <= SVDQ_MAX_LORA_RANK,
                       "gemm(int4): R_next (%d) must be a multiple of 16 in [16, %d]", a->R_next, SVDQ_MAX_LORA_RANK);
        SVDQ_CHECK_ARG(a->R_next <= 64 || n_out(a) == a->N, "gemm(int4): next-layer ranks above 64 need an unpadded output (N_out == N)");
    }
    SVDQ_CHECK_ARG(a->act_layout == SVDQ_LAYOUT_NATIVE, "gemm(int4): activations must be in SVDQ_LAYOUT_NATIVE "
                                                        "(convert with svdq_w4a4_relayout_act)");
    SVDQ_CHECK_ARG(a->R % 16 == 0 && a->R >= 0 && a->R <= SVDQ_MAX_LORA_RANK, "gemm: R (%d) must be a multiple of 16, at most %d", a->R, SVDQ_MAX_LORA_RANK);
    SVDQ_CHECK_ARG(n_out_ok(a), "gemm: N_out (%d) must be a multiple of 8 with N - 128 < N_out <= N (%d)", a->N_out, a->N);
    SVDQ_CHECK_ARG(a->R == 0 || (a->lora_act_in && a->w.lora_up), "gemm: low-rank tensors missing");

    int sms = 0;
    if (int rc = sm_count(&sms)) return rc;
    NvfpPlan pl;
    plan_nvfp4(a, sms, &pl);
    const size_t need = int4_rows_bytes(a) + int4_lora_bytes(a) + pl.workspace;
    SVDQ_CHECK_ARG(a->workspace && a->workspace_bytes >= need && aligned(a->workspace, 256),
                   "gemm(int4): a 256-byte aligned workspace of %zu bytes is required (svdq_gemm_w4a4_workspace_bytes)", need);
    float* row_scale = static_cast<float*>(a->workspace);
    float* lora_scaled = reinterpret_cast<float*>(static_cast<uint8_t*>(a->workspace) + int4_rows_bytes(a));
    float* partials = reinterpret_cast<float*>(static_cast<uint8_t*>(a->workspace) + int4_rows_bytes(a) + int4_lora_bytes(a));

    GemmParams p = {};
    p.ascales_i4 = static_cast<const h16*>(a->ascales);
    p.row_scale = row_scale;
    p.act_i4 = static_cast<const uint8_t*>(a->act);
    p.act_unsigned = a->act_unsigned;
    p.col_scale = a->w.col_scale;
    p.col_bias = a->w.col_bias;
    p.M = a->M;
    p.M_pad = a->M_pad;
    p.N = a->N;
    p.K = a->K;
    p.lora_chunks = (a->R + 31) / 32;
    p.tiles_m = pl.tiles_m;
    p.tiles_n = pl.tiles_n;
    p.activation = a->activation;
    void* const out_bf16 = a->out ? a->out : (pl.workspace > pl.partials ? reinterpret_cast<uint8_t*>(partials) + pl.partials : nullptr);
    p.store_out = out_bf16 != nullptr;
    p.contiguous = requant;
    p.run = pl.run;
    p.qout = static_cast<uint8_t*>(a->qout);
    p.oscales = static_cast<uint8_t*>(a->oscales);
    p.next_smooth = static_cast<const h16*>(a->next_smooth);
    p.next_lora_down = static_cast<const uint4*>(a->next_lora_down);
    p.next_rt_total = a->R_next / 16;
    p.lora_partial = partials;
    p.slots = pl.slots;
    if (int rc = status_words(&p.status)) return rc;

    CUtensorMap tm_a, tm_b, tm_la, tm_lu, tm_out;
    // packed codes: 32 bytes (64 codes) x 128 rows per k-block, unswizzled; weights: fp16 [N][K], 64 x 96 boxes
    if (int rc = make_tmap_2d(&tm_a, a->act, CU_TENSOR_MAP_DATA_TYPE_UINT8, a->K / 2, a->M_pad, a->K / 2, 32, G_BM, false)) return rc;
    if (int rc = make_tmap_2d(&tm_b, a->w.wgt, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, a->K, a->N, static_cast<uint64_t>(a->K) * 2, 64, G_BNH))
        return rc;
    if (a->R > 0) {
        const int R32 = (a->R + 31) / 32 * 32;
        if (int rc = make_tmap_2d(&tm_la, lora_scaled, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, a->R, a->M_pad,
                                  static_cast<uint64_t>(a->R) * 4, 32, G_BM))
            return rc;
        if (int rc = make_tmap_2d(&tm_lu, a->w.lora_up, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, R32, a->N,
                                  static_cast<uint64_t>(R32) * 4, 32, G_BNH))
            return rc;
    } else {
        tm_la = tm_b;
        tm_lu = tm_b;
    }
    if (out_bf16) {
        if (int rc = make_tmap_2d(&tm_out, out_bf16, SVDQ_TMAP_16, n_out(a), a->M, static_cast<uint64_t>(n_out(a)) * 2, 64, 32))
            return rc;
    } else {
        tm_out = tm_b;
    }
    {   // per-row normalisation of the activation scales (and of the low-rank activations that share the accumulator)
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(a->M_pad / 128, 1, 1);
        cfg.blockDim = dim3(128, 1, 1);
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        SVDQ_CUDA(cudaLaunchKernelEx(&cfg, int4_row_norm_kernel, p.ascales_i4, a->K / 64, a->M_pad,
                                     a->R > 0 ? a->lora_act_in : static_cast<const float*>(nullptr), a->R, row_scale, lora_scaled));
    }
    if (!requant) return launch_pair<0, true>(2 * pl.npairs, stream, tm_a, tm_b, tm_la, tm_lu, tm_out, tm_a, tm_a, p);
    return launch_requant<true>(a, pl, stream, tm_a, tm_b, tm_la, tm_lu, tm_out, tm_a, tm_a, p, out_bf16);
}

}  // namespace SVDQ_DT
}  // namespace svdq

#ifndef SVDQ_F16   // what follows exists once, in the bf16 build of this file
namespace svdq {
namespace hf {
int gemm_nvfp4_impl(const svdq_gemm_args* a, cudaStream_t stream);
int gemm_int4_impl(const svdq_gemm_args* a, cudaStream_t stream);
}  // namespace hf
}  // namespace svdq

// ---------------------------------------------------------------------------------------------------
// svdq_gemm_w4a4_static_scratch: the requantising GEMM (either precision) for hosts that have no way to hand over a
// workspace.  Think of a C or C++ serving loop that carved up its device memory once at start-up and has no
// allocator to ask per call, of a host whose policy forbids allocation calls after initialisation (they can
// synchronise the device), or of an op layer that is only ever given the operator's tensors.  For them the
// per-CTA LoRA-down partials live in a library-owned array in device memory instead of args->workspace.
//
// The array is a file-scope __device__ symbol: SVDQ_STATIC_SCRATCH_BYTES of device memory on every GPU that
// loads this library, held until the process exits.  On the host its name is only a handle, not an address,
// so the device address is looked up with cudaGetSymbolAddress - once per device, on the first call made with
// that device current.  That first call per device should therefore happen before any stream capture begins.
// (The cached address belongs to the device's context of that moment; it is stale after a cudaDeviceReset.)
// Nothing is allocated or freed, here or in anything this calls.
//
// All calls share the one array.  Every partial a launch reads was written earlier by the same launch, so
// nothing has to be cleared between calls; but two launches that are in flight on the same GPU at the same
// time (different streams) would overwrite each other's partials: callers must not overlap them.
// Problems whose partials do not fit are refused with SVDQ_ERR_INVALID_ARGUMENT.
// ---------------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_static_scratch[SVDQ_STATIC_SCRATCH_BYTES];

namespace svdq {

static int static_scratch_ptr(void** out) {
    static std::mutex mu;
    static void* ptrs[64] = {};
    int dev = 0;
    SVDQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(SVDQ_ERR_UNSUPPORTED, "static scratch: device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (ptrs[dev] == nullptr) {
        void* p = nullptr;
        SVDQ_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));   // device address of the symbol on the current device
        ptrs[dev] = p;
    }
    *out = ptrs[dev];
    return SVDQ_OK;
}

}  // namespace svdq

extern "C" int svdq_gemm_w4a4_static_scratch(const svdq_gemm_args* args, void* stream) {
    using namespace svdq;
    if (int rc = check_gemm_common(args)) return rc;
    size_t need = 0;   // the scratch does not depend on the 16-bit type
    if (!args->fp4) {
        if (int rc = bf::gemm_int4_workspace_bytes(args, &need)) return rc;
    } else if (args->qout) {
        if (int rc = bf::gemm_nvfp4_workspace_bytes(args, &need)) return rc;
    }
    if (need > SVDQ_STATIC_SCRATCH_BYTES)
        return fail(SVDQ_ERR_INVALID_ARGUMENT,
                    "gemm(static scratch): this problem needs %zu bytes of scratch, the built-in array holds %u; "
                    "use svdq_gemm_w4a4 with a caller workspace",
                    need, SVDQ_STATIC_SCRATCH_BYTES);
    void* scratch = nullptr;
    if (int rc = static_scratch_ptr(&scratch)) return rc;
    svdq_gemm_args local = *args;
    local.workspace = scratch;
    local.workspace_bytes = SVDQ_STATIC_SCRATCH_BYTES;
    const cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (local.dtype == SVDQ_DTYPE_FP16) return local.fp4 ? hf::gemm_nvfp4_impl(&local, st) : hf::gemm_int4_impl(&local, st);
    return local.fp4 ? bf::gemm_nvfp4_impl(&local, st) : bf::gemm_int4_impl(&local, st);
}



#ifdef SVDQ_ABLATE
// timing experiments: read and clear the cycle counters of pair 0
extern "C" int svdq_debug_prof(long long* host16) {
    using namespace svdq;
    SVDQ_CUDA(cudaDeviceSynchronize());
    SVDQ_CUDA(cudaMemcpyFromSymbol(host16, bf::g_prof, sizeof(long long) * 16));
    long long zero[16] = {};
    SVDQ_CUDA(cudaMemcpyToSymbol(bf::g_prof, zero, sizeof(zero)));
    return SVDQ_OK;
}
#endif
#endif   // !SVDQ_F16

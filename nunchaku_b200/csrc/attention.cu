// Softmax attention forward for 128-wide heads on the tcgen05 tensor cores, sm_100a.
//
// What it computes (reference: attention_fp16, src/kernels/zgemm/attention.cu:10-96 and attention.cuh:226-330; called
// from nunchaku/models/attention_processors/flux.py:160-185): per (batch, head)
//   S = Q K^T,  P = exp2(S * scale*log2(e) - rowmax),  O = (P V) / rowsum(P)
// with Q, K, V in a 16-bit type, S and O accumulated in fp32, P rounded to the 16-bit type before the second
// product, as the reference does (it runs both products with mma.sync on fp16 fragments).  No mask, no dropout.
// Q / K / V / O are addressed through (batch, head, token) strides with the 128 head channels contiguous, so the
// reference's head-major [B, H, T, 128] inputs with its token-major [B, T, H*128] output and this library's all-token-major
// buffers (written by the QKV projection's epilogue) are both plain cases.
//
// How it is laid out on a B200.  One CTA owns 256 query rows of one (batch, head) as two 128-row tiles and walks
// the keys in blocks of 128:
//   warp 8      producer: TMA loads of Q (once) and of the K / V blocks into a 5-slot ring of 32 KB (128B swizzle);
//   warp 9      MMA issuer: per tile and block S_t = Q_t K_j^T (8 x tcgen05.mma kind::f16 M128 N128 K16, both operands
//               K-major) into TMEM, then O_t += P_t V_j (A = P_t from tensor memory, B = V_j as it lies in memory, i.e.
//               MN-major: no transposed copy of V is ever made), in two halves of 64 keys as they are handed over.
//               The whole warp walks the loop, one elected lane issues, descriptors are a constant upper half plus a
//               lower half moved by immediates: with per-thread 64-bit descriptors the issue took 88 cycles per MMA
//               against the 64 it runs;
//   warps 0-7   two softmax warpgroups (232 registers each, the others give theirs back), one per tile, one query row
//               per thread: tcgen05.ld of the row of S in two halves, running maximum, exp2, row sum, P_t as packed
//               16-bit pairs over the row's own columns of S_t (tcgen05.st), arrive per half.
// The two tiles alternate on the tensor pipe: while one warpgroup is in its exponentials the issuer runs the other
// tile's P V and next Q K^T.  TMEM: S_0, S_1, O_0, O_1, 128 columns each (all 512).
// Two budgets shape this.  Shared-memory bandwidth: a 128 x 128 x 16 MMA with both operands in shared memory reads 8 KB
// in its 64 cycles, all of the 128 bytes per cycle an SM has, so P goes through tensor memory (P V then reads V alone;
// with P in shared memory the kernel ran at 1.06 against 1.19 PFLOP/s).  Latency: a tile's chain S -> exponentials ->
// P -> P V -> next Q K^T -> S is serial (P lies over S, so the next Q K^T follows P V), and two tiles only half fill the
// tensor pipe unless the softmax part is short: the exponentials of the first half are computed with the maximum in
// use while the second half is still being loaded, a quarter of them on the FMA pipe (exp2_fma2), and the first half of
// P is released to the issuer while the second is computed.  (Two threads per row, four softmax warpgroups, was slower:
// the exchange of the half-row maxima through shared memory cost more than the halved chain gained.)
// Running maximum: O lives in TMEM and is only rescaled (tcgen05.ld / multiply / tcgen05.st by the tile's own
// warpgroup, between two P V products) when some row's maximum has grown by more than 8 in the exponent since the
// last rescale; until then the stale maximum is used for P and the row sum alike, which is exact algebra (the final
// division cancels it) and keeps P <= 2^8.  In that rare case the first half's exponentials are redone.
// Per key block and CTA: 4 x 8 MMAs = 2048 tensor-pipe cycles against 32768 exponentials, 16 per cycle on the
// special-function unit.
//
// Every wait is bounded; a role whose wait runs out records SVDQ_ERR_TIMEOUT and leaves its loop.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "host_common.h"
#include "ptx.cuh"

namespace svdq {

constexpr int AT_D = 128;                  // head channels
constexpr int AT_BM = 128;                 // query rows per tile (TMEM lanes)
constexpr int AT_TILES = 2;                // tiles per CTA
constexpr int AT_BN = 128;                 // keys per block
constexpr int AT_HALF_BYTES = 128 * 128;   // one [128 rows x 64 x 16-bit] swizzled box
constexpr int AT_TILE_BYTES = 2 * AT_HALF_BYTES;
constexpr int AT_SLOTS = 5;                // K / V ring
constexpr int AT_PRODUCER_WARP = 8, AT_MMA_WARP = 9;   // warps 10 and 11 only complete the third warpgroup
constexpr int AT_THREADS = 12 * 32;
// setmaxnreg moves registers inside the pool the CTA was launched with (384 threads x 168): 8 x 32 x 232 + 4 x 32 x 40 is
// all of it.  An increase beyond the pool would wait forever.
constexpr int AT_REGS_LAUNCH = 168, AT_REGS_SOFTMAX = 232, AT_REGS_OTHER = 40;
static_assert(8 * AT_REGS_SOFTMAX + 4 * AT_REGS_OTHER <= 12 * AT_REGS_LAUNCH, "register budget");
constexpr int AT_SMEM = 1024 + (AT_TILES + AT_SLOTS) * AT_TILE_BYTES + 256;
constexpr long long AT_WAIT_CYCLES = 600000000ll;   // ~0.3 s
constexpr float AT_RESCALE_STEP = 8.f;

struct AttnShared {
    uint64_t q_full, kv_full[AT_SLOTS], kv_empty[AT_SLOTS], s_full[AT_TILES], p_half[AT_TILES][2], pv_done[AT_TILES];
    uint32_t tmem_base;
};

struct AttnParams {
    void* out;
    long long o_stride_b, o_stride_h, o_stride_t;   // elements
    int q_len, kv_len;
    float scale_log2;
    int* status;
};

__device__ __forceinline__ void tma_load_4d(void* dst, const void* tmap, uint64_t* bar, int x, int y, int z, int w) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
        : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], 16-bit operands, fp32 accumulation, one CTA.
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// The same with A in tensor memory: lane = row, every 32-bit column holds two consecutive K elements (the lower index in
// the lower half), so a K-step of 16 is 8 columns.
__device__ __forceinline__ void tc_mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// The two forms with descriptors given as 32-bit halves: the upper half (strides, swizzle) is a constant of the kernel and
// the lower half (start address in 16-byte units, leading byte offset) moves by small immediates, so that an unrolled
// issue loop needs no 64-bit arithmetic.  A and B share the upper half in the first form.
__device__ __forceinline__ void tc_mma_f16_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc,
                                              uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_mma_f16_ts_lo(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                                 uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Instruction descriptor, kind::f16: fp32 accumulator, A and B of one 16-bit format (0 = fp16, 1 = bf16), A K-major,
// B K-major or MN-major (bit 16).
__host__ __device__ constexpr uint32_t idesc_h16(int M, int N, bool f16, bool b_mn_major) {
    return (1u << 4) | ((f16 ? 0u : 1u) << 7) | ((f16 ? 0u : 1u) << 10) | ((b_mn_major ? 1u : 0u) << 16) |
           (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}

// Shared-memory descriptor of an MN-major operand under the 128-byte swizzle: 64 consecutive MN elements (128 bytes)
// per row, one row per K index, 8-row groups `sbo` bytes apart (stride byte offset), the next 64 MN elements `lbo`
// bytes on (leading byte offset).
__device__ __forceinline__ uint64_t smem_desc_sw128_mn(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFF) >> 4);
    d |= static_cast<uint64_t>(lbo >> 4) << 16;
    d |= static_cast<uint64_t>(sbo >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

template <bool F16>
__device__ __forceinline__ uint32_t pack_h16(float lo, float hi) {
    uint32_t r;
    if constexpr (F16) asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    else asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// 2^x for a pair of values on the FMA pipe instead of the special-function unit: x = n + f with n = rint(x) and f in
// [-0.5, 0.5]; 2^f by a cubic (relative error 7.6e-5, a sixth of fp16's rounding step and a 25th of bf16's), n added to
// the exponent field.  Adding 1.5 * 2^23 rounds x to an integer and leaves it in the low mantissa bits.  x is clamped
// at -125 (the result is then ~2e-38 instead of less).
__device__ __forceinline__ float2 exp2_fma2(float2 x) {
    x.x = fmaxf(x.x, -125.f);
    x.y = fmaxf(x.y, -125.f);
    const float2 t = __fadd2_rn(x, make_float2(12582912.f, 12582912.f));
    const float2 n = __fadd2_rn(t, make_float2(-12582912.f, -12582912.f));
    const float2 f = __ffma2_rn(n, make_float2(-1.f, -1.f), x);
    float2 r = __ffma2_rn(f, make_float2(0.05520550534129143f, 0.05520550534129143f), make_float2(0.24261397123336792f, 0.24261397123336792f));
    r = __ffma2_rn(r, f, make_float2(0.6932547688484192f, 0.6932547688484192f));
    r = __ffma2_rn(r, f, make_float2(0.9999276995658875f, 0.9999276995658875f));
    return make_float2(__int_as_float(__float_as_int(r.x) + (__float_as_int(t.x) << 23)),
                       __int_as_float(__float_as_int(r.y) + (__float_as_int(t.y) << 23)));
}

// Of every four pairs, this many take the FMA-pipe exponential (the rest ex2.approx): with all 32768 exponentials of a
// key block on the special-function unit it is busy for as long as the tensor pipe.  Measured on [8, 24, 4608, 128]:
// 0 -> 1204, 1 -> 1256, 2 -> 1238 TFLOP/s.
#ifndef AT_POLY_PAIRS
#define AT_POLY_PAIRS 1
#endif

#ifdef AT_PROF
__device__ long long at_prof[32];
__device__ long long at_ev[4][12];   // key blocks 8..11 of CTA 0: time stamps of the two tiles' softmax and MMA events
#define AT_EV(j, slot) do { if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0 && (j) >= 8 && (j) < 12) at_ev[(j) - 8][slot] = clock64(); } while (0)
#define AT_T(v) const long long v = clock64()
#define AT_ADD(slot, t0) prof_acc[slot] += clock64() - (t0)
#else
#define AT_T(v)
#define AT_ADD(slot, t0)
#define AT_EV(j, slot)
#endif

template <bool F16>
__global__ void __launch_bounds__(AT_THREADS, 1)
attention_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
    extern __shared__ __align__(1024) uint8_t at_smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(at_smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* q_s = smem;                                   // [tile][half]
    uint8_t* kv_s = q_s + AT_TILES * AT_TILE_BYTES;        // [slot][half]
    AttnShared* sh = reinterpret_cast<AttnShared*>(kv_s + AT_SLOTS * AT_TILE_BYTES);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int q0 = blockIdx.x * (AT_TILES * AT_BM);
    const int head = blockIdx.y, batch = blockIdx.z;
    const int nblocks = (p.kv_len + AT_BN - 1) / AT_BN;

    if (tid == 0) {
        mbar_init(&sh->q_full, 1);
        for (int i = 0; i < AT_SLOTS; ++i) {
            mbar_init(&sh->kv_full[i], 1);
            mbar_init(&sh->kv_empty[i], 1);
        }
        for (int t = 0; t < AT_TILES; ++t) {
            mbar_init(&sh->s_full[t], 1);
            mbar_init(&sh->p_half[t][0], 4);
            mbar_init(&sh->p_half[t][1], 4);
            mbar_init(&sh->pv_done[t], 1);
        }
        fence_mbar_init();
        prefetch_tmap(&tm_q);
        prefetch_tmap(&tm_k);
        prefetch_tmap(&tm_v);
    }
    if (warp == AT_MMA_WARP) {
        tmem_alloc(&sh->tmem_base, 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = sh->tmem_base;

    if (warp == AT_PRODUCER_WARP) {
        reg_dealloc<AT_REGS_OTHER>();
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            mbar_arrive_expect_tx(&sh->q_full, AT_TILES * AT_TILE_BYTES);
            for (int t = 0; t < AT_TILES; ++t)
                for (int h = 0; h < 2; ++h)
                    tma_load_4d(q_s + t * AT_TILE_BYTES + h * AT_HALF_BYTES, &tm_q, &sh->q_full, h * 64, q0 + t * AT_BM, head, batch);
            for (int i = 0; i < 2 * nblocks; ++i) {   // K_0, V_0, K_1, V_1, ...
                const int slot = i % AT_SLOTS, use = i / AT_SLOTS;
                if (!mbar_wait(&sh->kv_empty[slot], (use & 1) ^ 1, AT_WAIT_CYCLES)) {
                    atomicExch(&p.status[0], SVDQ_ERR_TIMEOUT);
                    atomicExch(&p.status[1], 700 + slot);
                    break;
                }
                mbar_arrive_expect_tx(&sh->kv_full[slot], AT_TILE_BYTES);
                const CUtensorMap* tm = (i & 1) ? &tm_v : &tm_k;
                for (int h = 0; h < 2; ++h)
                    tma_load_4d(kv_s + slot * AT_TILE_BYTES + h * AT_HALF_BYTES, tm, &sh->kv_full[slot], h * 64, (i >> 1) * AT_BN, head, batch);
            }
        }
    } else if (warp == AT_MMA_WARP) {
        reg_dealloc<AT_REGS_OTHER>();
        // ------------------------------------------------------------------ MMA issuer (the whole warp walks the loop, lane 0 issues)
        constexpr uint32_t IDESC_QK = idesc_h16(AT_BM, AT_BN, F16, false);
        constexpr uint32_t IDESC_PV = idesc_h16(AT_BM, AT_D, F16, true);
        // The whole warp walks the loop and one elected lane issues (descriptors, TMEM addresses and barrier addresses then
        // stay warp-uniform); descriptors are a constant upper half and a lower half that moves by immediates (16-byte
        // units: a tile or ring slot is 2048, its second 64-channel half 1024, a K-step inside a swizzled row 2, 16 key rows 128).
        const uint64_t qd = smem_desc_sw128(smem_u32(q_s)), kd = smem_desc_sw128(smem_u32(kv_s));
        const uint64_t vd = smem_desc_sw128_mn(smem_u32(kv_s), AT_HALF_BYTES, 1024);
        const uint32_t hi_k = static_cast<uint32_t>(qd >> 32), hi_v = static_cast<uint32_t>(vd >> 32);
        const uint32_t q_lo = static_cast<uint32_t>(qd), k_lo = static_cast<uint32_t>(kd), v_lo = static_cast<uint32_t>(vd);
        constexpr uint32_t UNIT_TILE = AT_TILE_BYTES >> 4, UNIT_HALF = AT_HALF_BYTES >> 4;
        bool ok = true;
#ifdef AT_PROF
        long long prof_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        const long long prof_t0 = clock64();
#endif
        // S_t = Q_t K^T from the ring slot at `slot_off`: 8 k-steps of 16 channels (elected lane only)
        auto issue_qk = [&](int t, uint32_t slot_off) {
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                const uint32_t off = (kk >> 2) * UNIT_HALF + (kk & 3) * 2;
                tc_mma_f16_lo(tmem + t * AT_BN, q_lo + t * UNIT_TILE + off, k_lo + slot_off + off, hi_k, IDESC_QK, kk > 0);
            }
        };
        // O_t (+)= P_t V for the 64 keys of half `hf`: 4 k-steps of 16 keys.  That half of P_t sits in the first 32 columns
        // of the half's 64 columns of S_t (two keys per column); V rows are keys.
        auto issue_pv = [&](int t, uint32_t slot_off, uint32_t acc, int hf) {
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4)
                tc_mma_f16_ts_lo(tmem + 2 * AT_BN + t * AT_D, tmem + t * AT_BN + hf * 64 + k4 * 8,
                                 v_lo + slot_off + (hf * 4 + k4) * 128, hi_v, IDESC_PV, (hf | k4) ? 1u : acc);
        };
        auto wait = [&](uint64_t* bar, uint32_t parity, int code) {
            if (!ok) return false;
            if (!mbar_wait(bar, parity, AT_WAIT_CYCLES)) {
                if (lane == 0) {
                    atomicExch(&p.status[0], SVDQ_ERR_TIMEOUT);
                    atomicExch(&p.status[1], code);
                }
                ok = false;
            }
            return ok;
        };
        // ring item i (K_j: 2j, V_j: 2j + 1): slot i % AT_SLOTS, parity (i / AT_SLOTS) & 1
        if (wait(&sh->q_full, 0, 710) && wait(&sh->kv_full[0], 0, 711)) {
            tc_fence_after_sync();
            if (elect_one()) {
                issue_qk(0, 0);
                tc_commit(&sh->s_full[0]);
                issue_qk(1, 0);
                tc_commit(&sh->s_full[1]);
                tc_commit(&sh->kv_empty[0]);
            }
            __syncwarp();
        }
        for (int j = 0; j < nblocks && ok; ++j) {
            const int iv = 2 * j + 1, ik = 2 * j + 2;
            const int vslot = iv % AT_SLOTS, kslot = ik % AT_SLOTS;
            const uint32_t voff = vslot * UNIT_TILE, koff = kslot * UNIT_TILE;
            const bool more = j + 1 < nblocks;
            AT_T(tv);
            if (!wait(&sh->kv_full[vslot], (iv / AT_SLOTS) & 1, 720)) break;
            AT_ADD(0, tv);
#pragma unroll
            for (int t = 0; t < AT_TILES; ++t) {
                AT_T(tp0);
                if (!wait(&sh->p_half[t][0], j & 1, 730 + t)) break;
                AT_ADD(1 + t, tp0);
                AT_EV(j, 6 + t * 3);
                AT_T(tk);
                if (more && t == 0 && !wait(&sh->kv_full[kslot], (ik / AT_SLOTS) & 1, 740)) break;
                AT_ADD(0, tk);
                tc_fence_after_sync();
                AT_T(ti0);
                if (elect_one()) issue_pv(t, voff, j > 0, 0);
                __syncwarp();
                AT_ADD(5, ti0);
                AT_T(tp1);
                if (!wait(&sh->p_half[t][1], j & 1, 735 + t)) break;
                AT_ADD(3 + t, tp1);
                AT_EV(j, 7 + t * 3);
                tc_fence_after_sync();
                AT_T(ti1);
                if (elect_one()) {
                    issue_pv(t, voff, 1u, 1);
                    tc_commit(&sh->pv_done[t]);
                    if (t == AT_TILES - 1) tc_commit(&sh->kv_empty[vslot]);
                    if (more) {   // overwrites P_t: behind P V in the tensor pipe's order
                        issue_qk(t, koff);
                        tc_commit(&sh->s_full[t]);
                        if (t == AT_TILES - 1) tc_commit(&sh->kv_empty[kslot]);
                    }
                }
                __syncwarp();
                AT_ADD(5, ti1);
                AT_EV(j, 8 + t * 3);
            }
        }
#ifdef AT_PROF
        if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0) {
            for (int i = 0; i < 8; ++i) at_prof[i] = prof_acc[i];
            at_prof[7] = clock64() - prof_t0;
        }
#endif
    } else if (warp > AT_MMA_WARP) {
        reg_dealloc<AT_REGS_OTHER>();
    } else {
        reg_alloc<AT_REGS_SOFTMAX>();
        // ------------------------------------------------------------------ softmax warpgroups: thread = one query row of tile t
        const int t = warp >> 2, quad = warp & 3;
        const int row = quad * 32 + lane;                       // row of the tile = TMEM lane
        const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
        const uint32_t s_tmem = tmem + lane_addr + t * AT_BN;
        const uint32_t o_tmem = tmem + lane_addr + 2 * AT_BN + t * AT_D;
        float m_used = 0.f, l = 0.f;
        bool ok = true;
#ifdef AT_PROF
        long long prof_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        const long long prof_t0 = clock64();
#endif
        const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
        // 64 keys (two 32-column chunks of S) -> 32 columns of packed 16-bit pairs, and their sum
        auto exp_half = [&](const uint32_t (&a)[32], const uint32_t (&b)[32], float m, uint32_t (&w)[32]) {
            const float2 nm2 = make_float2(-m, -m);
            float2 sum2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const int e = (i & 15) * 2;
                const float2 v = i < 16 ? make_float2(__uint_as_float(a[e]), __uint_as_float(a[e + 1]))
                                        : make_float2(__uint_as_float(b[e]), __uint_as_float(b[e + 1]));
                const float2 x = __ffma2_rn(v, sc2, nm2);
                float2 r;
                if ((i & 3) >= 4 - AT_POLY_PAIRS) {
                    r = exp2_fma2(x);
                } else {
                    r.x = ex2(x.x);
                    r.y = ex2(x.y);
                }
                sum2[i & 1] = __fadd2_rn(sum2[i & 1], r);
                w[i] = pack_h16<F16>(r.x, r.y);
            }
            return (sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y);
        };
        auto max_half = [&](const uint32_t (&a)[32], const uint32_t (&b)[32]) {
            float m0 = __uint_as_float(a[0]), m1 = __uint_as_float(b[0]);
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                m0 = max3(m0, __uint_as_float(a[i]), __uint_as_float(a[i + 1]));
                m1 = max3(m1, __uint_as_float(b[i]), __uint_as_float(b[i + 1]));
            }
            return fmaxf(m0, m1);
        };
        auto mask = [&](uint32_t (&a)[32], int first, int valid) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (first + i >= valid) a[i] = 0xff800000u;   // -inf
        };
        // P half `hf` is complete in tensor memory: the issuer may run its four k-steps of P V
        auto publish = [&](int hf, const uint32_t (&w)[32]) {
            tc_st_32x32b_x32(s_tmem + hf * 64, w);   // over this thread's own S values, which are all in registers by now
            tc_wait_st();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh->p_half[t][hf]);
        };
        for (int j = 0; j < nblocks; ++j) {
            AT_T(ts);
            if (!mbar_wait(&sh->s_full[t], j & 1, AT_WAIT_CYCLES)) {
                if (lane == 0) {
                    atomicExch(&p.status[0], SVDQ_ERR_TIMEOUT);
                    atomicExch(&p.status[1], 750 + t);
                }
                ok = false;
                break;
            }
            AT_ADD(0, ts);
            if (quad == 0) AT_EV(j, t * 3 + 0);
            tc_fence_after_sync();
            AT_T(tl);
            // The row of S arrives in two halves; the exponentials of the first are computed with the maximum in use while
            // the second is still on its way, and only its (rare) growth by more than the step makes them be redone.
            const int valid = p.kv_len - j * AT_BN;   // keys of this block that exist
            uint32_t s0[32], s1[32], s2[32], s3[32], w[32];
            tc_ld_32x32b_x32(s_tmem, s0);
            tc_ld_32x32b_x32(s_tmem + 32, s1);
            tc_wait_ld();
            AT_ADD(1, tl);
            AT_T(te);
            tc_ld_32x32b_x32(s_tmem + 64, s2);
            tc_ld_32x32b_x32(s_tmem + 96, s3);
            if (valid < AT_BN) {
                mask(s0, 0, valid);
                mask(s1, 32, valid);
            }
            float mx = max_half(s0, s1);
            float sum_a = exp_half(s0, s1, m_used, w);
            AT_ADD(2, te);
            if (quad == 0) AT_EV(j, t * 3 + 1);
            AT_T(tg);
            tc_wait_ld();
            if (valid < AT_BN) {
                mask(s2, 64, valid);
                mask(s3, 96, valid);
            }
            mx = fmaxf(mx, max_half(s2, s3));
            const float ms = mx * p.scale_log2;
            const bool grow = j == 0 || ms > m_used + AT_RESCALE_STEP;
            if (__any_sync(0xffffffffu, grow)) {
                if (j > 0) {
                    // O_t is written by the previous P V product until it has completed
                    if (!mbar_wait(&sh->pv_done[t], (j - 1) & 1, AT_WAIT_CYCLES)) {
                        if (lane == 0) {
                            atomicExch(&p.status[0], SVDQ_ERR_TIMEOUT);
                            atomicExch(&p.status[1], 760 + t);
                        }
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const float alpha = grow ? ex2(m_used - ms) : 1.f;
                    l *= alpha;
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t o[32];
                        tc_ld_32x32b_x32(o_tmem + c * 32, o);
                        tc_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tc_st_32x32b_x32(o_tmem + c * 32, o);
                    }
                    tc_wait_st();
                }
                if (grow) {
                    m_used = ms;
                    sum_a = exp_half(s0, s1, m_used, w);
                }
            }
            AT_ADD(3, tg);
            AT_T(tp);
            publish(0, w);
            AT_ADD(4, tp);
            AT_T(te2);
            const float sum_b = exp_half(s2, s3, m_used, w);
            AT_ADD(5, te2);
            AT_T(tp2);
            publish(1, w);
            AT_ADD(6, tp2);
            if (quad == 0) AT_EV(j, t * 3 + 2);
            l += sum_a + sum_b;
        }
#ifdef AT_PROF
        if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && warp == 0 && lane == 0) {
            for (int i = 0; i < 7; ++i) at_prof[8 + i] = prof_acc[i];
            at_prof[15] = clock64() - prof_t0;
        }
#endif
        // ---- O_t / l -> global
        if (ok && !mbar_wait(&sh->pv_done[t], (nblocks - 1) & 1, AT_WAIT_CYCLES)) {
            if (lane == 0) {
                atomicExch(&p.status[0], SVDQ_ERR_TIMEOUT);
                atomicExch(&p.status[1], 770 + t);
            }
            ok = false;
        }
        if (ok) {
            tc_fence_after_sync();
            const float inv = 1.f / l;
            const int qrow = q0 + t * AT_BM + row;
            uint8_t* orow = static_cast<uint8_t*>(p.out) +
                            2 * (batch * p.o_stride_b + head * p.o_stride_h + static_cast<long long>(qrow) * p.o_stride_t);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t o[32];
                tc_ld_32x32b_x32(o_tmem + c * 32, o);
                tc_wait_ld();
                if (qrow < p.q_len) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        uint32_t w[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            w[e] = pack_h16<F16>(__uint_as_float(o[u * 8 + 2 * e]) * inv, __uint_as_float(o[u * 8 + 2 * e + 1]) * inv);
                        *reinterpret_cast<uint4*>(orow + c * 64 + u * 16) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == AT_MMA_WARP) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, 512);
    }
}

// 4-D tiled map (channel, token, head, batch) over a 16-bit tensor whose 128 channels are contiguous.
static int attn_tmap(CUtensorMap* map, const void* base, int dtype, int batch, int heads, int tokens, const int64_t* stride) {
    SVDQ_CHECK_ARG(stride[0] >= 0 && stride[1] > 0 && stride[2] >= AT_D && stride[0] % 8 == 0 && stride[1] % 8 == 0 && stride[2] % 8 == 0,
                   "attention: strides must be multiples of 8 elements (16 bytes), the token stride at least 128");
    const uint64_t dims[4] = {AT_D, static_cast<uint64_t>(tokens), static_cast<uint64_t>(heads), static_cast<uint64_t>(batch)};
    const uint64_t strides[3] = {static_cast<uint64_t>(stride[2]) * 2, static_cast<uint64_t>(stride[1]) * 2,
                                 static_cast<uint64_t>(batch > 1 ? stride[0] : stride[1]) * 2};
    const uint32_t box[4] = {64, AT_BN, 1, 1};
    return make_tmap_nd(map, base, dtype == SVDQ_DTYPE_FP16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
                        dims, strides, box, true);
}

template <bool F16>
static int launch_attention(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& p, dim3 grid,
                            cudaStream_t stream) {
    auto kern = attention_fwd_kernel<F16>;
    static std::atomic<uint64_t> attr_done{0};
    if (int rc = ensure_dynamic_smem(kern, AT_SMEM, attr_done)) return rc;
    kern<<<grid, AT_THREADS, AT_SMEM, stream>>>(tq, tk, tv, p);
    SVDQ_CUDA(cudaGetLastError());
    return SVDQ_OK;
}

}  // namespace svdq

#ifdef AT_PROF
extern "C" int svdq_debug_attn_prof(long long* out) {
    return cudaMemcpyFromSymbol(out, svdq::at_prof, sizeof(long long) * 32) == cudaSuccess ? 0 : 1;
}
extern "C" int svdq_debug_attn_events(long long* out) {
    return cudaMemcpyFromSymbol(out, svdq::at_ev, sizeof(long long) * 48) == cudaSuccess ? 0 : 1;
}
#endif

extern "C" int svdq_attention(const svdq_attention_args* a, void* stream) {
    using namespace svdq;
    SVDQ_CHECK_ARG(a != nullptr, "attention: null args");
    SVDQ_CHECK_ARG(a->q && a->k && a->v && a->out, "attention: null tensor pointer");
    SVDQ_CHECK_ARG(a->head_dim == AT_D, "attention: head_dim %d (only 128, as attention.cuh:13)", a->head_dim);
    SVDQ_CHECK_ARG(a->batch > 0 && a->heads > 0 && a->q_len > 0 && a->kv_len > 0 && a->heads <= 65535 && a->batch <= 65535,
                   "attention: bad sizes");
    SVDQ_CHECK_ARG(a->dtype == SVDQ_DTYPE_BF16 || a->dtype == SVDQ_DTYPE_FP16, "attention: bad dtype %d", a->dtype);
    SVDQ_CHECK_ARG(aligned(a->q, 16) && aligned(a->k, 16) && aligned(a->v, 16) && aligned(a->out, 16),
                   "attention: tensors must be 16-byte aligned");
    SVDQ_CHECK_ARG(a->o_stride[0] % 8 == 0 && a->o_stride[1] % 8 == 0 && a->o_stride[2] % 8 == 0,
                   "attention: output strides must be multiples of 8 elements");
    if (int rc = check_arch()) return rc;
    CUtensorMap tq, tk, tv;
    if (int rc = attn_tmap(&tq, a->q, a->dtype, a->batch, a->heads, a->q_len, a->q_stride)) return rc;
    if (int rc = attn_tmap(&tk, a->k, a->dtype, a->batch, a->heads, a->kv_len, a->k_stride)) return rc;
    if (int rc = attn_tmap(&tv, a->v, a->dtype, a->batch, a->heads, a->kv_len, a->v_stride)) return rc;
    AttnParams p = {};
    p.out = a->out;
    p.o_stride_b = a->o_stride[0];
    p.o_stride_h = a->o_stride[1];
    p.o_stride_t = a->o_stride[2];
    p.q_len = a->q_len;
    p.kv_len = a->kv_len;
    p.scale_log2 = a->scale * 1.4426950408889634f;
    if (int rc = status_words(&p.status)) return rc;
    const dim3 grid((a->q_len + AT_TILES * AT_BM - 1) / (AT_TILES * AT_BM), a->heads, a->batch);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return a->dtype == SVDQ_DTYPE_FP16 ? launch_attention<true>(tq, tk, tv, p, grid, st) : launch_attention<false>(tq, tk, tv, p, grid, st);
}

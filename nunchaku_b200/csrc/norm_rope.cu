// Row-wise kernels either side of the W4A4 linears in a FLUX block, sm_100a.  Both are HBM bound.
//
// qk_norm_rope_kernel — what the reference fuses into the QKV GEMM's epilogue (EpilogueRMSNormRope,
// src/kernels/zgemm/epilogues.cuh:269-425; launcher gemm_w4a4_launch_impl.cuh:347-405), here as a kernel of its
// own that works in place on the GEMM's bf16 output [rows, 3*heads*128]:
//   for the Q third and the K third, per (row, head): coef = rsqrt(sum_128 float(y)^2 / 128 + eps);
//   v = float(y) * (coef * float(w_norm[c])); every (even, odd) column pair is rotated by the row's angle,
//   (a, b) -> (a*cos - b*sin, a*sin + b*cos), all in fp32 with one rounding to bf16 at the end.  V is untouched.
//   The rotary table is two fp32 arrays [seq_len, 64] (cos, sin), row = token position, shared by all batches.
// One warp per (row, head, q|k): 4 consecutive columns per lane (two pairs), an 8-byte load and store.
// Algorithmic bytes per row: 2 * heads*128 * 2 (read) + the same (write) + 512 of table.
//
// layernorm_modulate_kernel — the AdaLN-Zero step in front of every W4A4 projection: LayerNorm without affine
// (eps 1e-5) followed by x * (1 + scale[b]) + shift[b], bf16 in and out, fp32 statistics; one warp per row with the
// row held in registers (two passes over registers, one over memory).  Not part of the reference's W4A4 path (the
// reference has its own fused norm kernels); it is here so that the block harness is not bound by library glue.
//
// Compiled once per 16-bit type (see dtype.cuh): bf16 here, fp16 from norm_rope_f16.cu; the entry points pick by `dtype`.
#include "dtype.cuh"
#include "host_common.h"

namespace svdq {
namespace SVDQ_DT {

__device__ __forceinline__ float2 bf2(uint32_t w) { return unpack2(w); }
__device__ __forceinline__ uint32_t pack_bf2(float a, float b) { return pack2(make_float2(a, b)); }
constexpr uint32_t kOnes2 = kF16 ? 0x3c003c00u : 0x3f803f80u;   // two packed 1.0

// PACKED: the rotary table is the reference's fragment-packed fp32 tensor (pack_rotemb, nunchaku/models/embeddings.py:88-120):
// for row m = 16 mb + 8 h + g and column pair p = 4 j + t, {sin, cos} sit at ((((mb*16 + j)*8 + g)*4 + t)*2 + h)*2.
// SPLIT: instead of working in place, write q, k (normalised + rotated) and v (copied) head-major to
// out_q / out_k / out_v [batch, heads, tokens_pad, 128] (token_major: [batch, tokens_pad, heads, 128]) from token
// token_offset on; rows at or beyond attn_tokens (when given) become zeros.
template <bool PACKED, bool SPLIT>
__global__ void __launch_bounds__(256)
qk_norm_rope_kernel(h16* __restrict__ qkv, const h16* __restrict__ wq, const h16* __restrict__ wk,
                    const float* __restrict__ cosp, const float* __restrict__ sinp, long long rows, int seq_len, int heads,
                    float eps, h16* __restrict__ out_q, h16* __restrict__ out_k,
                    h16* __restrict__ out_v, int tokens_pad, int attn_tokens, int token_offset, int token_major) {
    const int lane = threadIdx.x & 31;
    const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
    const int dim = heads * 128;
    constexpr int PARTS = SPLIT ? 3 : 2;
    // A warp's unit of work is one third (q, k or, when splitting, v) of one row: every head of it in turn, four heads'
    // lines asked for before the first is worked on.  Row, position and the lane's rotary entries are found once per unit
    // (with one item = one head per loop turn, the 64-bit divisions that located it cost more than the arithmetic).
    const long long units = rows * PARTS;
    // norm weights of this lane's 4 columns, for q and k
    const uint2 wq2 = *reinterpret_cast<const uint2*>(wq + lane * 4);
    const uint2 wk2 = *reinterpret_cast<const uint2*>(wk + lane * 4);
    for (long long unit = warp; unit < units; unit += nwarps) {
        const long long row = unit / PARTS;
        const int which = static_cast<int>(unit - row * PARTS);
        const long long b = row / seq_len;
        const int pos = static_cast<int>(row - b * seq_len);
        float2 c = make_float2(1.f, 1.f), s = make_float2(0.f, 0.f);
        if (which < 2) {
            if constexpr (PACKED) {
                // pairs 2*lane and 2*lane + 1: j = lane / 2, t = 2 * (lane & 1) + {0, 1}
                const long long mb = pos >> 4;
                const int h = (pos >> 3) & 1, g = pos & 7;
                const float* e = cosp + ((((mb * 16 + (lane >> 1)) * 8 + g) * 4 + 2 * (lane & 1)) * 2 + h) * 2;
                const float2 sc0 = *reinterpret_cast<const float2*>(e);       // {sin, cos} of pair 2*lane
                const float2 sc1 = *reinterpret_cast<const float2*>(e + 4);   // next t
                s = make_float2(sc0.x, sc1.x);
                c = make_float2(sc0.y, sc1.y);
            } else {
                c = *reinterpret_cast<const float2*>(cosp + static_cast<long long>(pos) * 64 + lane * 2);
                s = *reinterpret_cast<const float2*>(sinp + static_cast<long long>(pos) * 64 + lane * 2);
            }
        }
        const uint2 w = which ? wk2 : wq2;
        const float2 w0 = bf2(w.x), w1 = bf2(w.y);
        h16* src = qkv + row * (3LL * dim) + static_cast<long long>(which) * dim + lane * 4;
        const bool zero = SPLIT && attn_tokens > 0 && pos >= attn_tokens;
        h16* dst = src;
        long long dstride = 128;   // elements between heads at the destination
        if constexpr (SPLIT) {
            h16* base = which == 0 ? out_q : which == 1 ? out_k : out_v;
            const long long tok = token_offset + pos;
            dst = base + (token_major ? (b * tokens_pad + tok) * heads * 128 : (b * heads * tokens_pad + tok) * 128) + lane * 4;
            dstride = token_major ? 128 : static_cast<long long>(tokens_pad) * 128;
        }
        for (int h0 = 0; h0 < heads; h0 += 4) {
            uint2 ov[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (h0 + u < heads) ov[u] = *reinterpret_cast<const uint2*>(src + (h0 + u) * 128);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (h0 + u >= heads) break;
                uint2 o = ov[u];
                if (which < 2) {
                    const float2 y0 = bf2(o.x), y1 = bf2(o.y);
                    float ss = y0.x * y0.x + y0.y * y0.y + y1.x * y1.x + y1.y * y1.y;
#pragma unroll
                    for (int m = 16; m >= 1; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
                    const float coef = rsqrtf(ss * (1.0f / 128.0f) + eps);
                    const float a0 = y0.x * (coef * w0.x), b0 = y0.y * (coef * w0.y);
                    const float a1 = y1.x * (coef * w1.x), b1 = y1.y * (coef * w1.y);
                    o.x = pack_bf2(a0 * c.x - b0 * s.x, a0 * s.x + b0 * c.x);
                    o.y = pack_bf2(a1 * c.y - b1 * s.y, a1 * s.y + b1 * c.y);
                }
                if (zero) o = make_uint2(0u, 0u);
                *reinterpret_cast<uint2*>(dst + (h0 + u) * dstride) = o;
            }
        }
    }
}

// C = 8 * (32 * (V - 1) + TAIL) columns: each lane holds V chunks of 8 columns (16 bytes), chunk j at column
// (j*32 + lane) * 8; only the first TAIL lanes hold a last chunk (TAIL = 32: C = 256 V)
template <int V, int TAIL = 32>
__global__ void __launch_bounds__(256, 2)
layernorm_modulate_kernel(const h16* __restrict__ x, const h16* __restrict__ scale,
                          const h16* __restrict__ shift, h16* __restrict__ out, long long rows,
                          long long rows_per_batch, long long mod_stride, float eps) {
    constexpr int C = (V - 1) * 256 + TAIL * 8;
    const int lane = threadIdx.x & 31;
    const bool last = TAIL == 32 || lane < TAIL;   // this lane holds a chunk V - 1
    const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
    for (long long row = warp; row < rows; row += nwarps) {
        // The row stays in registers as it was loaded (16-bit pairs, V x 4 words) and is unpacked again in each of the three
        // passes: as fp32 it took 206 registers per thread, i.e. one block of eight warps per SM and too few loads in flight.
        const uint4* xp = reinterpret_cast<const uint4*>(x + row * C);
        uint4 raw[V];
#pragma unroll
        for (int j = 0; j < V; ++j) raw[j] = (j < V - 1 || last) ? xp[j * 32 + lane] : make_uint4(0, 0, 0, 0);
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < V; ++j) {
            const float2 f0 = bf2(raw[j].x), f1 = bf2(raw[j].y), f2 = bf2(raw[j].z), f3 = bf2(raw[j].w);
            sum += ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
        }
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, m);
        const float mean = sum * (1.0f / C);
        float var = 0.f;
#pragma unroll
        for (int j = 0; j < V; ++j) {
            if (j == V - 1 && !last) break;
            const uint32_t w4[4] = {raw[j].x, raw[j].y, raw[j].z, raw[j].w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = bf2(w4[i]);
                const float d0 = f.x - mean, d1 = f.y - mean;
                var += d0 * d0 + d1 * d1;
            }
        }
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) var += __shfl_xor_sync(0xffffffffu, var, m);
        const float rstd = rsqrtf(var * (1.0f / C) + eps);
        const long long b = row / rows_per_batch;
        const uint4* scp = reinterpret_cast<const uint4*>(scale + b * mod_stride);
        const uint4* shp = reinterpret_cast<const uint4*>(shift + b * mod_stride);
        uint4* op = reinterpret_cast<uint4*>(out + row * C);
#pragma unroll
        for (int j = 0; j < V; ++j) {
            if (j == V - 1 && !last) break;
            const uint4 sc = scp[j * 32 + lane], sh = shp[j * 32 + lane];
            const uint32_t scw[4] = {sc.x, sc.y, sc.z, sc.w}, shw[4] = {sh.x, sh.y, sh.z, sh.w};
            const uint32_t w4[4] = {raw[j].x, raw[j].y, raw[j].z, raw[j].w};
            uint32_t o[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 s2 = bf2(scw[i]), h2 = bf2(shw[i]), f = bf2(w4[i]);
                // the library sequence it replaces rounds the normalised value to the 16-bit type before modulating
                const float n0 = h2f(f2h((f.x - mean) * rstd));
                const float n1 = h2f(f2h((f.y - mean) * rstd));
                o[i] = pack_bf2(n0 * (1.0f + s2.x) + h2.x, n1 * (1.0f + s2.y) + h2.y);
            }
            op[j * 32 + lane] = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
}

static int grid_for(long long warps_needed) {
    int sms = 148;
    (void)sm_count(&sms);
    const long long blocks = (warps_needed + 7) / 8;
    const long long cap = static_cast<long long>(sms) * 8;
    return static_cast<int>(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

// out[row, c] = x[row, c] + gate[batch, c] * (y[row, c] (+ z[row, c])): the gated residual that follows every projection of a
// DiT block, one pass with 16-byte accesses (the library's broadcasting multiply and add are two passes, neither vectorised).
// fp32 arithmetic, one rounding.  `out` may alias x.
__global__ void __launch_bounds__(256)
gate_residual_kernel(const h16* __restrict__ x, const h16* __restrict__ gate, const h16* __restrict__ y,
                     const h16* __restrict__ z, h16* out, long long rows, long long rows_per_batch,
                     long long gate_stride, int cols) {
    const int c8 = cols >> 3;
    const long long total = rows * c8;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long row = i / c8;
        const int c = static_cast<int>(i - row * c8);
        const uint4 xw = reinterpret_cast<const uint4*>(x)[i];
        const uint4 yw = reinterpret_cast<const uint4*>(y)[i];
        const uint4 gw = gate ? *reinterpret_cast<const uint4*>(gate + (row / rows_per_batch) * gate_stride + 8 * c)
                              : make_uint4(kOnes2, kOnes2, kOnes2, kOnes2);
        uint4 zw = make_uint4(0, 0, 0, 0);
        if (z) zw = reinterpret_cast<const uint4*>(z)[i];
        const uint32_t xs[4] = {xw.x, xw.y, xw.z, xw.w}, ys[4] = {yw.x, yw.y, yw.z, yw.w}, gs[4] = {gw.x, gw.y, gw.z, gw.w},
                       zs[4] = {zw.x, zw.y, zw.z, zw.w};
        uint32_t o[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 xf = bf2(xs[k]), yf = bf2(ys[k]), gf = bf2(gs[k]), zf = bf2(zs[k]);
            o[k] = pack_bf2(fmaf(gf.x, yf.x + zf.x, xf.x), fmaf(gf.y, yf.y + zf.y, xf.y));
        }
        reinterpret_cast<uint4*>(out)[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

int qk_norm_rope_impl(const svdq_norm_rope_args* a, void* stream) {
    SVDQ_CHECK_ARG(a && a->qkv && a->weight_q && a->weight_k && ((a->cos && a->sin) || a->rotary_packed), "qk_norm_rope: null pointer");
    SVDQ_CHECK_ARG(a->rows > 0 && a->seq_len > 0 && a->heads > 0 && a->rows % a->seq_len == 0,
                   "qk_norm_rope: rows (%lld) must be a positive multiple of seq_len (%d)", static_cast<long long>(a->rows), a->seq_len);
    SVDQ_CHECK_ARG(aligned(a->qkv, 16) && aligned(a->weight_q, 8) && aligned(a->weight_k, 8) && aligned(a->cos, 8) && aligned(a->sin, 8) &&
                       aligned(a->rotary_packed, 16) && aligned(a->out_q, 16) && aligned(a->out_k, 16) && aligned(a->out_v, 16),
                   "qk_norm_rope: misaligned tensor");
    SVDQ_CHECK_ARG(!a->rotary_packed || a->seq_len % 16 == 0, "qk_norm_rope: a packed rotary table has a multiple of 16 rows (got %d)", a->seq_len);
    const bool split = a->out_q || a->out_k || a->out_v;
    SVDQ_CHECK_ARG(!split || (a->out_q && a->out_k && a->out_v && a->token_offset >= 0 &&
                              a->tokens_pad >= a->token_offset + a->seq_len && a->attn_tokens >= 0 && a->attn_tokens <= a->seq_len),
                   "qk_norm_rope: out_q, out_k and out_v go together, with tokens_pad >= token_offset + seq_len and "
                   "0 <= attn_tokens <= seq_len");
    if (int rc = check_arch()) return rc;
    const long long items = static_cast<long long>(a->rows) * (split ? 3 : 2);   // one warp per third of a row
    const float* tab = a->rotary_packed ? a->rotary_packed : a->cos;
    auto launch = [&](auto kernel) {
        kernel<<<grid_for(items), 256, 0, static_cast<cudaStream_t>(stream)>>>(
            static_cast<h16*>(a->qkv), static_cast<const h16*>(a->weight_q),
            static_cast<const h16*>(a->weight_k), tab, a->sin, a->rows, a->seq_len, a->heads, a->eps,
            static_cast<h16*>(a->out_q), static_cast<h16*>(a->out_k), static_cast<h16*>(a->out_v),
            a->tokens_pad, a->attn_tokens, a->token_offset, a->token_major);
    };
    if (a->rotary_packed) {
        if (split) launch(qk_norm_rope_kernel<true, true>); else launch(qk_norm_rope_kernel<true, false>);
    } else {
        if (split) launch(qk_norm_rope_kernel<false, true>); else launch(qk_norm_rope_kernel<false, false>);
    }
    SVDQ_CUDA(cudaGetLastError());
    return SVDQ_OK;
}

int layernorm_modulate_impl(const svdq_ln_modulate_args* a, void* stream) {
    SVDQ_CHECK_ARG(a && a->x && a->scale && a->shift && a->out, "layernorm_modulate: null pointer");
    SVDQ_CHECK_ARG(a->rows > 0 && a->rows_per_batch > 0 && a->rows % a->rows_per_batch == 0 && a->mod_stride >= a->cols &&
                       a->mod_stride % 8 == 0,
                   "layernorm_modulate: bad row / batch geometry");
    SVDQ_CHECK_ARG(aligned(a->x, 16) && aligned(a->scale, 16) && aligned(a->shift, 16) && aligned(a->out, 16),
                   "layernorm_modulate: tensors must be 16-byte aligned");
    if (int rc = check_arch()) return rc;
    const int grid = grid_for(a->rows);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const h16* x = static_cast<const h16*>(a->x);
    const h16* sc = static_cast<const h16*>(a->scale);
    const h16* sh = static_cast<const h16*>(a->shift);
    h16* o = static_cast<h16*>(a->out);
    switch (a->cols) {
        case 256: layernorm_modulate_kernel<1><<<grid, 256, 0, st>>>(x, sc, sh, o, a->rows, a->rows_per_batch, a->mod_stride, a->eps); break;
        case 1024: layernorm_modulate_kernel<4><<<grid, 256, 0, st>>>(x, sc, sh, o, a->rows, a->rows_per_batch, a->mod_stride, a->eps); break;
        case 2240: layernorm_modulate_kernel<9, 24><<<grid, 256, 0, st>>>(x, sc, sh, o, a->rows, a->rows_per_batch, a->mod_stride, a->eps); break;
        case 2304: layernorm_modulate_kernel<9><<<grid, 256, 0, st>>>(x, sc, sh, o, a->rows, a->rows_per_batch, a->mod_stride, a->eps); break;
        case 3072: layernorm_modulate_kernel<12><<<grid, 256, 0, st>>>(x, sc, sh, o, a->rows, a->rows_per_batch, a->mod_stride, a->eps); break;
        default: return fail(SVDQ_ERR_UNSUPPORTED, "layernorm_modulate: built for 256, 1024, 2240, 2304 and 3072 columns (got %d)", a->cols);
    }
    SVDQ_CUDA(cudaGetLastError());
    return SVDQ_OK;
}

int gate_residual_impl(const svdq_gate_residual_args* a, void* stream) {
    SVDQ_CHECK_ARG(a && a->x && a->y && a->out, "gate_residual: null pointer");
    SVDQ_CHECK_ARG(a->rows > 0 && a->rows_per_batch > 0 && a->rows % a->rows_per_batch == 0 && a->cols > 0 && a->cols % 8 == 0 &&
                       (a->gate == nullptr || (a->gate_stride >= a->cols && a->gate_stride % 8 == 0)),
                   "gate_residual: bad row / batch geometry (cols and the gate's row stride must be multiples of 8)");
    SVDQ_CHECK_ARG(aligned(a->x, 16) && aligned(a->y, 16) && aligned(a->z, 16) && aligned(a->gate, 16) && aligned(a->out, 16),
                   "gate_residual: tensors must be 16-byte aligned");
    if (int rc = check_arch()) return rc;
    const long long total = a->rows * (a->cols / 8);
    int sms = 0;
    if (int rc = sm_count(&sms)) return rc;
    const long long want = (total + 255) / 256;
    const int grid = static_cast<int>(want < 16LL * sms ? want : 16LL * sms);
    gate_residual_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const h16*>(a->x), static_cast<const h16*>(a->gate), static_cast<const h16*>(a->y),
        static_cast<const h16*>(a->z), static_cast<h16*>(a->out), a->rows, a->rows_per_batch, a->gate_stride, a->cols);
    SVDQ_CUDA(cudaGetLastError());
    return SVDQ_OK;
}

}  // namespace SVDQ_DT
}  // namespace svdq

#ifndef SVDQ_F16
namespace svdq {
namespace hf {
int qk_norm_rope_impl(const svdq_norm_rope_args* a, void* stream);
int layernorm_modulate_impl(const svdq_ln_modulate_args* a, void* stream);
int gate_residual_impl(const svdq_gate_residual_args* a, void* stream);
}  // namespace hf
}  // namespace svdq

#define SVDQ_ROWWISE_ENTRY(name, args_t, impl)                                                                       \
    extern "C" int name(const args_t* a, void* stream) {                                                             \
        if (a && a->dtype == SVDQ_DTYPE_FP16) return svdq::hf::impl(a, stream);                                      \
        if (a && a->dtype != SVDQ_DTYPE_BF16) return svdq::fail(SVDQ_ERR_INVALID_ARGUMENT, #name ": bad dtype %d", a->dtype); \
        return svdq::bf::impl(a, stream);                                                                            \
    }
SVDQ_ROWWISE_ENTRY(svdq_qk_norm_rope, svdq_norm_rope_args, qk_norm_rope_impl)
SVDQ_ROWWISE_ENTRY(svdq_layernorm_modulate, svdq_ln_modulate_args, layernorm_modulate_impl)
SVDQ_ROWWISE_ENTRY(svdq_gate_residual, svdq_gate_residual_args, gate_residual_impl)
#endif

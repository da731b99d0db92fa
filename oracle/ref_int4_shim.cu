// TEST INFRASTRUCTURE, not part of the product: a C-ABI door onto the reference's OWN INT4 (bf16 and fp16) W4A4 kernels,
// compiled from the reference sources where they lie (nothing of them is copied here).  Only tests, the smoke check
// and bench.py's reference leg may load the resulting library; the package never does.
//
// The reference has no CPU implementation of this path and its NVFP4 kernels are sm_120a-only (they __trap() on any
// other architecture, src/kernels/zgemm/gemm_w4a4.cuh:28-41,358-405,1039-1041), but its INT4 kernels carry
// MIN_ARCH = 800 (gemm_w4a4.cuh:626,663,1048,1101; arch gate gemm_base.cuh:891-898) and assemble for sm_100a.  This
// file wraps raw device pointers into the reference's Tensor type (src/Tensor.h) and calls
//   GEMM_W4A4_Launch<GEMMConfig_W4A4_BF16, false>::quantize_w4a4_act_fuse_lora   (gemm_w4a4_launch_impl.cuh:451-521)
//   GEMM_W4A4_Launch<GEMMConfig_W4A4_BF16, false>::gemm_w4a4                     (gemm_w4a4_launch_impl.cuh:7-424)
//   GEMM_W4A4_Launch<GEMMConfig_W4A4_BF16, false>::linearattn_vk_mul_q           (gemm_w4a4_launch_impl.cuh:426-448)
// whose explicit instantiation lives in src/kernels/zgemm/gemm_w4a4_launch_bf16_int4.cu (compiled next to this file), and
// the same three members of GEMM_W4A4_Launch<GEMMConfig_W4A4_FP16, false> (gemm_w4a4_launch_fp16_int4.cu) when a call's
// `fp16` flag is set.
// Entry points never pass fp4 = true.  Shape violations hit the reference's live asserts (abort), so callers
// validate shapes first; CUDA errors surface as the reference's exceptions, turned into -1 here.
#include "kernels/zgemm/zgemm.h"
#include "kernels/zgemm/gemm_w4a4_launch.cuh"

namespace {

class BorrowedBuffer : public Buffer {
public:
    BorrowedBuffer(void *p, size_t bytes, int dev) {
        this->ptr    = p;
        this->size   = bytes;
        this->device = Device::cuda(dev);
    }
    bool isAsyncBuffer() override { return true; }
};

Tensor wrap(const void *p, std::vector<int> shape, Tensor::ScalarType type, int dev) {
    Tensor t;
    if (!p) return t;   // invalid tensor = the reference's "argument not given"
    t.shape      = TensorShape(std::move(shape));
    t.scalarType = type;
    t.buffer     = std::make_shared<BorrowedBuffer>(const_cast<void *>(p), t.shape.size() * Tensor::scalarSize.at(type), dev);
    return t;
}

using LaunchBF16 = nunchaku::kernels::GEMM_W4A4_Launch<nunchaku::kernels::GEMMConfig_W4A4_BF16, false>;
using LaunchFP16 = nunchaku::kernels::GEMM_W4A4_Launch<nunchaku::kernels::GEMMConfig_W4A4_FP16, false>;

thread_local std::string g_error;

}  // namespace

extern "C" {

struct ref_int4_quantize_args {
    const void *input;   // bf16 [M, K] ([M, 2K] when fuse_glu)
    void *output;        // int8 [M_pad, K_pad/2], reference fragment order
    void *oscales;       // bf16 [K_pad/64, M_pad], reference order
    const void *lora_down;   // bf16 [K_pad, R] packed
    float *lora_act_out;     // fp32 [M_pad, R] fragment order (zeroed by the reference launcher)
    const void *smooth;      // bf16 [K_pad] packed
    int M, in_cols, M_pad, K_pad, R, fuse_glu, device;
    int fp16;            // the 16-bit tensors are fp16 instead of bf16
};

}  // extern "C"

template <typename Launch>
static void quantize_typed(const ref_int4_quantize_args *a, Tensor::ScalarType H) {
    Launch::quantize_w4a4_act_fuse_lora(
        wrap(a->input, {a->M, a->in_cols}, H, a->device), wrap(a->output, {a->M_pad, a->K_pad / 2}, Tensor::INT8, a->device),
        wrap(a->oscales, {a->K_pad / 64, a->M_pad}, H, a->device), wrap(a->lora_down, {a->K_pad, a->R}, H, a->device),
        wrap(a->lora_act_out, {a->M_pad, a->R}, Tensor::FP32, a->device), wrap(a->smooth, {a->K_pad}, H, a->device),
        a->fuse_glu != 0, false);
}

extern "C" {

int ref_int4_quantize(const ref_int4_quantize_args *a, void *stream) {
    try {
        CUDAStreamContext ctx(static_cast<cudaStream_t>(stream));
        if (a->fp16) quantize_typed<LaunchFP16>(a, Tensor::FP16);
        else quantize_typed<LaunchBF16>(a, Tensor::BF16);
        return 0;
    } catch (const std::exception &e) {
        g_error = e.what();
        return -1;
    }
}

struct ref_int4_gemm_args {
    const void *act, *wgt;            // int8 [M_pad, K/2], [N, K/2]
    void *out;                        // bf16 [M, N_out] or null
    void *qout;                       // int8 [M_pad, N/2] or null
    const void *ascales, *wscales;    // bf16 [K/64, M_pad], [K/64, N]
    void *oscales;                    // bf16 [N/64, M_pad] or null
    const float *lora_act_in;         // fp32 [M_pad, R_up] or null
    const void *lora_up;              // bf16 [N, R_up] or null
    const void *lora_down;            // bf16 [N, R_down] or null
    float *lora_act_out;              // fp32 [M_pad, R_down] or null
    const void *norm_q, *norm_k;      // bf16 [128] or null
    const float *rotary_emb;          // fp32 [1, M_pad, 128] packed or null
    const void *bias, *smooth_factor; // bf16 [N] packed or null
    float *out_vk;                    // fp32 [B, heads, 33, 32] or null
    void *out_linearattn;             // bf16 [B, tokens, N/3] or null
    void *out_q, *out_k, *out_v;      // bf16 [B, heads, tokens_pad, 128] or null
    const float *lora_scales;         // host, n_lora_scales entries
    int M, M_pad, N, N_out, K, R_up, R_down, act_unsigned, fuse_silu, n_lora_scales;
    int batch, heads, tokens, tokens_pad, attn_tokens, device;
    int fp16;                         // the 16-bit tensors are fp16 instead of bf16
};

}  // extern "C"

template <typename Launch>
static void gemm_typed(const ref_int4_gemm_args *a, Tensor::ScalarType H) {
        const int d = a->device;
        std::vector<float> ls(a->lora_scales, a->lora_scales + a->n_lora_scales);
        Launch::gemm_w4a4(
            wrap(a->act, {a->M_pad, a->K / 2}, Tensor::INT8, d), wrap(a->wgt, {a->N, a->K / 2}, Tensor::INT8, d),
            wrap(a->out, {a->M, a->N_out}, H, d), wrap(a->qout, {a->M_pad, a->N / 2}, Tensor::INT8, d),
            wrap(a->ascales, {a->K / 64, a->M_pad}, H, d), wrap(a->wscales, {a->K / 64, a->N}, H, d),
            wrap(a->oscales, {a->N / 64, a->M_pad}, H, d), Tensor{},
            wrap(a->lora_act_in, {a->M_pad, a->R_up}, Tensor::FP32, d), wrap(a->lora_up, {a->N, a->R_up}, H, d),
            wrap(a->lora_down, {a->N, a->R_down}, H, d), wrap(a->lora_act_out, {a->M_pad, a->R_down}, Tensor::FP32, d),
            wrap(a->norm_q, {128}, H, d), wrap(a->norm_k, {128}, H, d),
            wrap(a->rotary_emb, {1, a->M_pad, 128}, Tensor::FP32, d), wrap(a->bias, {a->N}, H, d),
            wrap(a->smooth_factor, {a->N}, H, d), wrap(a->out_vk, {a->batch, a->heads, 33, 32}, Tensor::FP32, d),
            wrap(a->out_linearattn, {a->batch, a->tokens, a->N / 3}, H, d), a->act_unsigned != 0, ls, a->fuse_silu != 0,
            false, 1.0f, Tensor{}, wrap(a->out_q, {a->batch, a->heads, a->tokens_pad, 128}, H, d),
            wrap(a->out_k, {a->batch, a->heads, a->tokens_pad, 128}, H, d),
            wrap(a->out_v, {a->batch, a->heads, a->tokens_pad, 128}, H, d), a->attn_tokens);
}

extern "C" {

int ref_int4_gemm(const ref_int4_gemm_args *a, void *stream) {
    try {
        CUDAStreamContext ctx(static_cast<cudaStream_t>(stream));
        if (a->fp16) gemm_typed<LaunchFP16>(a, Tensor::FP16);
        else gemm_typed<LaunchBF16>(a, Tensor::BF16);
        return 0;
    } catch (const std::exception &e) {
        g_error = e.what();
        return -1;
    }
}

// q: bf16 [B, tokens, heads*32] modified in place; vk: fp32 [B, heads, 33, 32]
int ref_int4_vk_mul_q(void *q, float *vk, int batch, int tokens, int heads, int device, void *stream) {
    try {
        CUDAStreamContext ctx(static_cast<cudaStream_t>(stream));
        LaunchBF16::linearattn_vk_mul_q(wrap(q, {batch, tokens, heads * 32}, Tensor::BF16, device),
                                    wrap(vk, {batch, heads, 33, 32}, Tensor::FP32, device));
        return 0;
    } catch (const std::exception &e) {
        g_error = e.what();
        return -1;
    }
}

const char *ref_int4_last_error(void) { return g_error.c_str(); }

// quantize_w4a4_wgt (src/kernels/zgemm/zgemm.h:48; gemm_w4a4_launch_impl.cuh:547-570): 16-bit weight [N, K] -> packed INT4
// codes [N, K/2] and packed group scales [K/64, N]
int ref_int4_quantize_wgt(const void *input, void *output, void *oscales, int N, int K, int fp16, int device, void *stream) {
    try {
        CUDAStreamContext ctx(static_cast<cudaStream_t>(stream));
        const Tensor::ScalarType H = fp16 ? Tensor::FP16 : Tensor::BF16;
        Tensor in = wrap(input, {N, K}, H, device), out = wrap(output, {N, K / 2}, Tensor::INT8, device),
               sc = wrap(oscales, {K / 64, N}, H, device);
        if (fp16) LaunchFP16::quantize_w4a4_wgt(in, out, sc);
        else LaunchBF16::quantize_w4a4_wgt(in, out, sc);
        return 0;
    } catch (const std::exception &e) {
        g_error = e.what();
        return -1;
    }
}

}  // extern "C"

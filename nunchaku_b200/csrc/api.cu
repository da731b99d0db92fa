// C-ABI entry points of libsvdq_b200 (declared in include/svdq_b200.h) and the
// host-side plumbing they share.
#include <mutex>

#include "host_common.h"

namespace svdq {

int quantize_impl(const svdq_quantize_args* a, cudaStream_t stream);
int prepared_bytes_impl(int N, int K, int R, int fp4, size_t bytes[5]);
int prepare_weights_impl(const svdq_weights_args* a, const svdq_prepared_weights* o, cudaStream_t stream);
int relayout_impl(const svdq_relayout_args* a, cudaStream_t stream);
int gemm_nvfp4_impl(const svdq_gemm_args* a, cudaStream_t stream);
int gemm_nvfp4_workspace_bytes(const svdq_gemm_args* a, size_t* bytes);
int gemm_int4_workspace_bytes(const svdq_gemm_args* a, size_t* bytes);
int gemm_int4_impl(const svdq_gemm_args* a, cudaStream_t stream);

std::string& last_error() {
    static thread_local std::string s;
    return s;
}

// {code, detail}: written by kernels whose bounded waits ran out.
__device__ int g_status_words[2];

int status_words(int** ptr) {
    void* p = nullptr;
    SVDQ_CUDA(cudaGetSymbolAddress(&p, g_status_words));
    *ptr = static_cast<int*>(p);
    return SVDQ_OK;
}

int check_arch() {
    int dev = 0, major = 0;
    SVDQ_CUDA(cudaGetDevice(&dev));
    SVDQ_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    if (major != 10)
        return fail(SVDQ_ERR_UNSUPPORTED_ARCH, "device %d has compute capability %d.x; this library is sm_100a only", dev, major);
    return SVDQ_OK;
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

int make_tmap_2d(CUtensorMap* map, const void* base, int elem, uint64_t inner, uint64_t rows, uint64_t row_bytes,
                 uint32_t box_inner, uint32_t box_rows, bool swizzle128) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return fail(SVDQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    SVDQ_CHECK_ARG(aligned(base, 16) && row_bytes % 16 == 0, "tensor map: base and row pitch must be 16-byte aligned");
    const cuuint64_t dims[2] = {inner, rows};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {box_inner, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, static_cast<CUtensorMapDataType>(elem), 2, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(SVDQ_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
    return SVDQ_OK;
}

int make_tmap_3d(CUtensorMap* map, const void* base, int elem, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_bytes,
                 uint64_t stride2_bytes, uint32_t box0, uint32_t box1, uint32_t box2) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return fail(SVDQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    SVDQ_CHECK_ARG(aligned(base, 16) && stride1_bytes % 16 == 0 && stride2_bytes % 16 == 0,
                   "tensor map: base and strides must be 16-byte aligned");
    const cuuint64_t dims[3] = {d0, d1, d2};
    const cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
    const cuuint32_t box[3] = {box0, box1, box2};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = fn(map, static_cast<CUtensorMapDataType>(elem), 3, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(SVDQ_ERR_CUDA, "cuTensorMapEncodeTiled (3-D) failed with CUresult %d", static_cast<int>(r));
    return SVDQ_OK;
}

int check_gemm_common(const svdq_gemm_args* a) {
    SVDQ_CHECK_ARG(a != nullptr, "gemm: null args");
    SVDQ_CHECK_ARG(a->act && a->ascales && a->w.wgt && a->w.wscales && a->w.col_scale && a->w.col_bias,
                   "gemm: null tensor pointer");
    SVDQ_CHECK_ARG(a->M > 0 && a->M_pad >= a->M && a->M_pad % 256 == 0, "gemm: M_pad (%d) must be a multiple of 256 >= M (%d)",
                   a->M_pad, a->M);
    SVDQ_CHECK_ARG(a->N > 0 && a->N % 128 == 0, "gemm: N (%d) must be a multiple of 128 (gemm_w4a4_launch_impl.cuh:74)", a->N);
    SVDQ_CHECK_ARG(a->K > 0 && a->K % 128 == 0, "gemm: K (%d) must be a multiple of 128", a->K);
    SVDQ_CHECK_ARG(aligned(a->act, 16) && aligned(a->ascales, 16) && aligned(a->w.wgt, 16) && aligned(a->w.wscales, 16) &&
                       aligned(a->out, 16) && aligned(a->lora_act_in, 16) && aligned(a->w.lora_up, 16) &&
                       aligned(a->w.col_scale, 16) && aligned(a->w.col_bias, 16),
                   "gemm: tensors must be 16-byte aligned");
    SVDQ_CHECK_ARG(a->activation >= SVDQ_ACT_NONE && a->activation <= SVDQ_ACT_GELU, "gemm: bad activation %d", a->activation);
    return check_arch();
}

}  // namespace svdq

extern "C" {

int svdq_quantize_w4a4_act_fuse_lora(const svdq_quantize_args* args, void* stream) {
    return svdq::quantize_impl(args, static_cast<cudaStream_t>(stream));
}

int svdq_w4a4_prepared_bytes(int32_t N, int32_t K, int32_t R, int32_t fp4, size_t bytes[5]) {
    if (!bytes) return svdq::fail(SVDQ_ERR_INVALID_ARGUMENT, "prepared_bytes: null output");
    return svdq::prepared_bytes_impl(N, K, R, fp4, bytes);
}

int svdq_w4a4_prepare_weights(const svdq_weights_args* args, const svdq_prepared_weights* out, void* stream) {
    return svdq::prepare_weights_impl(args, out, static_cast<cudaStream_t>(stream));
}

int svdq_gemm_w4a4_workspace_bytes(const svdq_gemm_args* args, size_t* bytes) {
    if (!args || !bytes) return svdq::fail(SVDQ_ERR_INVALID_ARGUMENT, "workspace_bytes: null argument");
    *bytes = 0;
    if (args->fp4 && args->qout) return svdq::gemm_nvfp4_workspace_bytes(args, bytes);
    if (!args->fp4 && args->qout) return svdq::gemm_int4_workspace_bytes(args, bytes);
    return SVDQ_OK;
}

int svdq_gemm_w4a4(const svdq_gemm_args* args, void* stream) {
    if (int rc = svdq::check_gemm_common(args)) return rc;
    if (args->fp4) return svdq::gemm_nvfp4_impl(args, static_cast<cudaStream_t>(stream));
    return svdq::gemm_int4_impl(args, static_cast<cudaStream_t>(stream));
}

int svdq_w4a4_relayout_act(const svdq_relayout_args* args, void* stream) {
    return svdq::relayout_impl(args, static_cast<cudaStream_t>(stream));
}

int svdq_device_status(int32_t* status, int32_t* detail) {
    int* words = nullptr;
    if (int rc = svdq::status_words(&words)) return rc;
    int host[2] = {0, 0};
    SVDQ_CUDA(cudaDeviceSynchronize());
    SVDQ_CUDA(cudaMemcpy(host, words, sizeof(host), cudaMemcpyDeviceToHost));
    if (host[0] != 0) {
        const int zero[2] = {0, 0};
        SVDQ_CUDA(cudaMemcpy(words, zero, sizeof(zero), cudaMemcpyHostToDevice));
    }
    if (status) *status = host[0];
    if (detail) *detail = host[1];
    return SVDQ_OK;
}

const char* svdq_last_error_string(void) { return svdq::last_error().c_str(); }

int svdq_version(void) { return 100; }

}  // extern "C"

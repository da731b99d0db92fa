// C-ABI entry points of libsvdq_b200 (declared in include/svdq_b200.h) and the
// host-side plumbing they share.
#include <atomic>
#include <cstring>
#include <mutex>

#include "host_common.h"

namespace svdq {

#define SVDQ_DECLARE_TYPED(ns)                                                        \
    namespace ns {                                                                    \
    int quantize_impl(const svdq_quantize_args* a, cudaStream_t stream);              \
    int gemm_nvfp4_impl(const svdq_gemm_args* a, cudaStream_t stream);                \
    int gemm_nvfp4_workspace_bytes(const svdq_gemm_args* a, size_t* bytes);           \
    int gemm_int4_workspace_bytes(const svdq_gemm_args* a, size_t* bytes);            \
    int gemm_int4_impl(const svdq_gemm_args* a, cudaStream_t stream);                 \
    }
SVDQ_DECLARE_TYPED(bf)   // kernels compiled for bf16 tensors
SVDQ_DECLARE_TYPED(hf)   // ... and for fp16 (the *_f16.cu translation units)
int prepared_bytes_impl(int N, int K, int R, int fp4, size_t bytes[5]);
int prepare_weights_impl(const svdq_weights_args* a, const svdq_prepared_weights* o, cudaStream_t stream);
int relayout_impl(const svdq_relayout_args* a, cudaStream_t stream);

std::string& last_error() {
    static thread_local std::string s;
    return s;
}

// {code, detail}: written by kernels whose bounded waits ran out.
__device__ int g_status_words[2];

// Per-device facts that every launch needs, looked up once per device (under a mutex) with that device current:
// SM count, compute capability and the device address of the status words.  Entry points that run inside a stream
// capture find them cached, provided one ordinary call was made on the device before the capture began.  The
// cached address belongs to the context that was current at the time: it does not survive a cudaDeviceReset.
struct DeviceState {
    std::atomic<bool> ready{false};
    int sms = 0, cc_major = 0;
    int* status = nullptr;
};
static DeviceState g_dev[SVDQ_MAX_DEVICES];
static std::mutex g_dev_mu;

static int device_state(const DeviceState** out, int* dev_out = nullptr) {
    int dev = 0;
    SVDQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= SVDQ_MAX_DEVICES)
        return fail(SVDQ_ERR_UNSUPPORTED, "device ordinal %d is outside the supported range [0, %d)", dev, SVDQ_MAX_DEVICES);
    DeviceState& d = g_dev[dev];
    if (!d.ready.load(std::memory_order_acquire)) {
        std::lock_guard<std::mutex> lock(g_dev_mu);
        if (!d.ready.load(std::memory_order_relaxed)) {
            SVDQ_CUDA(cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev));
            SVDQ_CUDA(cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
            void* p = nullptr;
            SVDQ_CUDA(cudaGetSymbolAddress(&p, g_status_words));
            d.status = static_cast<int*>(p);
            d.ready.store(true, std::memory_order_release);
        }
    }
    *out = &d;
    if (dev_out) *dev_out = dev;
    return SVDQ_OK;
}

int status_words(int** ptr) {
    const DeviceState* d = nullptr;
    if (int rc = device_state(&d)) return rc;
    *ptr = d->status;
    return SVDQ_OK;
}

int sm_count(int* sms) {
    const DeviceState* d = nullptr;
    if (int rc = device_state(&d)) return rc;
    *sms = d->sms;
    return SVDQ_OK;
}

int current_device(int* dev) {
    const DeviceState* d = nullptr;
    return device_state(&d, dev);
}

int check_arch() {
    const DeviceState* d = nullptr;
    int dev = 0;
    if (int rc = device_state(&d, &dev)) return rc;
    if (d->cc_major != 10)
        return fail(SVDQ_ERR_UNSUPPORTED_ARCH, "device %d has compute capability %d.x; this library is sm_100a only", dev, d->cc_major);
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

// Encoded tensor maps are kept in a small per-thread, direct-mapped table keyed by everything that goes into the
// encoding: a layer called again with the same buffers (the steady state of an inference loop, where the caching
// allocator hands back the same addresses) costs a hash and a compare instead of a driver call per map.
struct TmapKey {
    const void* base;
    uint64_t dims[4], strides[3];
    uint32_t box[4];
    int32_t elem, rank, swizzle;
};
struct alignas(64) TmapEntry {
    CUtensorMap map;
    TmapKey key;
    bool valid;
};
constexpr int TMAP_CACHE_ENTRIES = 1024;

static int cached_tmap(CUtensorMap* out, const TmapKey& k) {
    static thread_local TmapEntry* table = nullptr;
    if (!table) table = new TmapEntry[TMAP_CACHE_ENTRIES]();
    uint64_t h = reinterpret_cast<uintptr_t>(k.base) * 0x9E3779B97F4A7C15ull;
    h ^= (k.dims[0] * 0xC2B2AE3D27D4EB4Full) ^ (k.dims[1] * 0x165667B19E3779F9ull) ^ (k.dims[2] << 17) ^ (k.strides[0] * 31) ^
         (static_cast<uint64_t>(k.box[0]) << 40) ^ (static_cast<uint64_t>(k.box[1]) << 48) ^ (static_cast<uint64_t>(k.elem) << 56) ^
         (k.dims[3] << 29) ^ (k.strides[1] * 131) ^ (k.strides[2] * 8191);
    TmapEntry& e = table[(h >> 20) & (TMAP_CACHE_ENTRIES - 1)];
    if (e.valid && std::memcmp(&e.key, &k, sizeof(TmapKey)) == 0) {
        *out = e.map;
        return SVDQ_OK;
    }
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return fail(SVDQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult r = fn(&e.map, static_cast<CUtensorMapDataType>(k.elem), static_cast<cuuint32_t>(k.rank), const_cast<void*>(k.base),
                          k.dims, k.strides, k.box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          k.swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        e.valid = false;
        return fail(SVDQ_ERR_CUDA, "cuTensorMapEncodeTiled (%d-D) failed with CUresult %d", k.rank, static_cast<int>(r));
    }
    e.key = k;
    e.valid = true;
    *out = e.map;
    return SVDQ_OK;
}

int make_tmap_2d(CUtensorMap* map, const void* base, int elem, uint64_t inner, uint64_t rows, uint64_t row_bytes,
                 uint32_t box_inner, uint32_t box_rows, bool swizzle128) {
    SVDQ_CHECK_ARG(aligned(base, 16) && row_bytes % 16 == 0, "tensor map: base and row pitch must be 16-byte aligned");
    TmapKey k;
    std::memset(&k, 0, sizeof(k));   // padding bytes take part in the compare
    k.base = base;
    k.dims[0] = inner; k.dims[1] = rows;
    k.strides[0] = row_bytes;
    k.box[0] = box_inner; k.box[1] = box_rows;
    k.elem = elem; k.rank = 2; k.swizzle = swizzle128 ? 1 : 0;
    return cached_tmap(map, k);
}

int make_tmap_3d(CUtensorMap* map, const void* base, int elem, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_bytes,
                 uint64_t stride2_bytes, uint32_t box0, uint32_t box1, uint32_t box2) {
    SVDQ_CHECK_ARG(aligned(base, 16) && stride1_bytes % 16 == 0 && stride2_bytes % 16 == 0,
                   "tensor map: base and strides must be 16-byte aligned");
    TmapKey k;
    std::memset(&k, 0, sizeof(k));
    k.base = base;
    k.dims[0] = d0; k.dims[1] = d1; k.dims[2] = d2;
    k.strides[0] = stride1_bytes; k.strides[1] = stride2_bytes;
    k.box[0] = box0; k.box[1] = box1; k.box[2] = box2;
    k.elem = elem; k.rank = 3; k.swizzle = 0;
    return cached_tmap(map, k);
}

int make_tmap_nd(CUtensorMap* map, const void* base, int elem, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                 const uint32_t* box, bool swizzle128) {
    SVDQ_CHECK_ARG(rank >= 2 && rank <= 4 && aligned(base, 16), "tensor map: rank 2..4 and a 16-byte aligned base");
    TmapKey k;
    std::memset(&k, 0, sizeof(k));
    k.base = base;
    for (int i = 0; i < rank; ++i) {
        k.dims[i] = dims[i];
        k.box[i] = box[i];
        if (i + 1 < rank) {
            SVDQ_CHECK_ARG(strides_bytes[i] % 16 == 0 && strides_bytes[i] > 0, "tensor map: strides must be positive multiples of 16 bytes");
            k.strides[i] = strides_bytes[i];
        }
    }
    k.elem = elem; k.rank = rank; k.swizzle = swizzle128 ? 1 : 0;
    return cached_tmap(map, k);
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
    SVDQ_CHECK_ARG(a->dtype == SVDQ_DTYPE_BF16 || a->dtype == SVDQ_DTYPE_FP16, "gemm: bad dtype %d", a->dtype);
    return check_arch();
}

}  // namespace svdq

extern "C" {

int svdq_quantize_w4a4_act_fuse_lora(const svdq_quantize_args* args, void* stream) {
    if (args && args->dtype == SVDQ_DTYPE_FP16) return svdq::hf::quantize_impl(args, static_cast<cudaStream_t>(stream));
    if (args && args->dtype != SVDQ_DTYPE_BF16) return svdq::fail(SVDQ_ERR_INVALID_ARGUMENT, "quantize: bad dtype %d", args->dtype);
    return svdq::bf::quantize_impl(args, static_cast<cudaStream_t>(stream));
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
    // (the scratch does not depend on the 16-bit type)
    if (args->fp4 && args->qout) return svdq::bf::gemm_nvfp4_workspace_bytes(args, bytes);
    if (!args->fp4) return svdq::bf::gemm_int4_workspace_bytes(args, bytes);   // always: per-row normalisation scratch
    return SVDQ_OK;
}

int svdq_gemm_w4a4(const svdq_gemm_args* args, void* stream) {
    if (int rc = svdq::check_gemm_common(args)) return rc;
    if (args->rope_cos && !args->fp4)
        return svdq::fail(SVDQ_ERR_UNSUPPORTED, "gemm(int4): the fused RMSNorm + RoPE epilogue is built for NVFP4");
    const cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (args->dtype == SVDQ_DTYPE_FP16) return args->fp4 ? svdq::hf::gemm_nvfp4_impl(args, st) : svdq::hf::gemm_int4_impl(args, st);
    return args->fp4 ? svdq::bf::gemm_nvfp4_impl(args, st) : svdq::bf::gemm_int4_impl(args, st);
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

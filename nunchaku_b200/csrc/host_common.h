// Host-side helpers shared by the translation units of libsvdq_b200: error
// reporting, argument checks and TMA tensor-map construction.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <mutex>
#include <string>

#include "../../include/svdq_b200.h"

namespace svdq {

// Thread-local text of the last error returned by an entry point.
std::string& last_error();

inline int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    last_error() = buf;
    return code;
}

#define SVDQ_CHECK_ARG(cond, ...)                                             \
    do {                                                                      \
        if (!(cond)) return ::svdq::fail(SVDQ_ERR_INVALID_ARGUMENT, __VA_ARGS__); \
    } while (0)

#define SVDQ_CUDA(call)                                                                     \
    do {                                                                                    \
        cudaError_t e_ = (call);                                                            \
        if (e_ != cudaSuccess)                                                              \
            return ::svdq::fail(SVDQ_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(e_)); \
    } while (0)

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// Checks that the current device is compute capability 10.x (B200 / GB200).
int check_arch();

// Highest device ordinal + 1 the per-device caches cover; beyond it entry points return SVDQ_ERR_UNSUPPORTED.
constexpr int SVDQ_MAX_DEVICES = 64;

// Device pointer to the library's status words {code, detail} on the current device (cached per device).
int status_words(int** ptr);
// SM count / ordinal of the current device (cached per device; the ordinal is checked against SVDQ_MAX_DEVICES).
int sm_count(int* sms);
int current_device(int* dev);

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per (kernel, device): `done` is a function-local static
// bit mask, one bit per device ordinal, guarded by one mutex for all kernels (set-up only happens a few times).
template <typename Kernel>
inline int ensure_dynamic_smem(Kernel kernel, size_t bytes, std::atomic<uint64_t>& done) {
    int dev = 0;
    if (int rc = current_device(&dev)) return rc;
    const uint64_t bit = 1ull << dev;
    if (done.load(std::memory_order_acquire) & bit) return SVDQ_OK;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (done.load(std::memory_order_relaxed) & bit) return SVDQ_OK;
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
    if (e != cudaSuccess) return fail(SVDQ_ERR_CUDA, "cudaFuncSetAttribute(max dynamic shared memory = %zu) failed: %s", bytes, cudaGetErrorString(e));
    done.fetch_or(bit, std::memory_order_release);
    return SVDQ_OK;
}

// 2-D tiled tensor map: inner dimension contiguous, `row_bytes` between rows.
// `elem` is a CUtensorMapDataType, box_inner*elem_size must be <= 128 with 128B swizzle.
int make_tmap_2d(CUtensorMap* map, const void* base, int elem /*CUtensorMapDataType*/, uint64_t inner,
                 uint64_t rows, uint64_t row_bytes, uint32_t box_inner, uint32_t box_rows, bool swizzle128 = true);

// 3-D tiled map without swizzle (dimension 0 innermost and contiguous); out-of-range boxes read zeros.
int make_tmap_3d(CUtensorMap* map, const void* base, int elem, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_bytes,
                 uint64_t stride2_bytes, uint32_t box0, uint32_t box1, uint32_t box2);

// Tiled map of rank 2..4 (dimension 0 innermost and contiguous; `strides_bytes` for dimensions 1..rank-1, in any order of
// magnitude); out-of-range boxes read zeros.
int make_tmap_nd(CUtensorMap* map, const void* base, int elem, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                 const uint32_t* box, bool swizzle128);

// Pointer / shape / alignment / architecture checks shared by the GEMM entry points.
int check_gemm_common(const svdq_gemm_args* a);

}  // namespace svdq

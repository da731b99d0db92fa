// Tensor-pipe rate probe: one CTA per SM issues tcgen05.mma (and optionally the scale-factor
// tcgen05.cp that a block-scaled stage needs) on operands that never leave shared memory / TMEM, and
// reports the cycles it took.  This gives the measured dense peak of a kind/shape on this GPU (the
// denominator a GEMM's tensor-pipe fraction is judged against) and the cost of the copies.
// Operand contents are whatever shared memory holds after zero-filling: only timing is observed.
#include "host_common.h"
#include "ptx.cuh"

namespace svdq {

struct ProbeShared {
    uint64_t done;
    uint32_t tmem_base;
};

// kind: 0 = mxf4nvf4 block-scaled (K=64 per MMA), 1 = tf32 (K=8), 2 = i8 (K=32)
__global__ void __launch_bounds__(64, 1)
mma_rate_kernel(int kind, int n, int iters, int cps_per_group, int sf_buffers, long long* cycles, int* status) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int STAGE = 48 * 1024;
    ProbeShared* sh = reinterpret_cast<ProbeShared*>(smem + 4 * STAGE);
    for (int i = threadIdx.x; i < 4 * STAGE / 16; i += blockDim.x) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
    if (threadIdx.x == 0) {
        mbar_init(&sh->done, 1);
        fence_mbar_init();
    }
    if (threadIdx.x < 32) {
        tmem_alloc(&sh->tmem_base, 512);
        tmem_relinquish();
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = sh->tmem_base;
    if (threadIdx.x == 0) {
        const uint32_t idesc = kind == 0 ? idesc_nvfp4(128, n) : kind == 1 ? idesc_tf32(128, n) : idesc_i8(128, n, true);
        const long long t0 = clock64();
        for (int it = 0; it < iters; ++it) {
            const uint32_t sa = smem_u32(smem + (it & 3) * STAGE);
            const uint64_t adesc = smem_desc_sw128(sa);
            const uint64_t bdesc = smem_desc_sw128(sa + 16384);
            const uint32_t t_sf = tmem + 384 + (sf_buffers > 1 ? (it % sf_buffers) * 48 : 0);
            for (int j = 0; j < cps_per_group; ++j)
                tc_cp_32x128b_warpx4(t_sf + 4 * j, smem_desc_sf(sa + 40960 + j * 512));
            for (int j = 0; j < 4; ++j) {
                if (kind == 0)
                    tc_mma_nvfp4(tmem, adesc + 2 * j, bdesc + 2 * j, idesc, t_sf + 4 * j, t_sf + 16 + 8 * j, 1);
                else if (kind == 1)
                    tc_mma_tf32(tmem, adesc + 2 * j, bdesc + 2 * j, idesc, 1);
                else
                    tc_mma_i8(tmem, adesc + 2 * j, bdesc + 2 * j, idesc, 1);
            }
        }
        const long long t1 = clock64();
        tc_commit(&sh->done);
        if (!mbar_wait(&sh->done, 0)) atomicExch(&status[0], SVDQ_ERR_TIMEOUT);
        const long long t2 = clock64();
        cycles[blockIdx.x * 2] = t1 - t0;      // issue time
        cycles[blockIdx.x * 2 + 1] = t2 - t0;  // until the last MMA completed
    }
    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x < 32) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, 512);
    }
}

}  // namespace svdq

// cycles: device buffer of 2 * grid int64 {issue, complete} per CTA.  No counterpart in the reference.
extern "C" int svdq_probe_mma_rate(int kind, int n, int iters, int cps_per_group, int sf_buffers, int grid,
                                   long long* cycles, void* stream) {
    using namespace svdq;
    SVDQ_CHECK_ARG(cycles && grid > 0 && grid <= 1024 && iters > 0 && n >= 16 && n <= 256 && n % 16 == 0 &&
                       cps_per_group >= 0 && cps_per_group <= 12 && sf_buffers >= 1 && sf_buffers <= 2 && kind >= 0 && kind <= 2,
                   "probe: bad argument");
    if (int rc = check_arch()) return rc;
    int* status = nullptr;
    if (int rc = status_words(&status)) return rc;
    const size_t smem = 1024 + 4 * 48 * 1024 + 64;
    SVDQ_CUDA(cudaFuncSetAttribute(mma_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    mma_rate_kernel<<<grid, 64, smem, static_cast<cudaStream_t>(stream)>>>(kind, n, iters, cps_per_group, sf_buffers, cycles, status);
    SVDQ_CUDA(cudaGetLastError());
    return SVDQ_OK;
}

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
    uint64_t scratch;
    uint64_t never;
    uint32_t tmem_base;
    volatile int finished;
};

// kind: 0 = mxf4nvf4 block-scaled (K=64 per MMA), 1 = tf32 (K=8), 2 = i8 (K=32)
// sfb_step: TMEM column distance between the B scale factors of consecutive K blocks; commit_every: a
// tcgen05.commit to a scratch barrier after every group of 4 MMAs; blockDim beyond 64 threads = extra warps
// that poll an mbarrier until the loop is over (what waiting epilogue / loader warps do in a real kernel).
__global__ void __launch_bounds__(512, 1)
mma_rate_kernel(int kind, int n, int iters, int cps_per_group, int sf_buffers, int sfb_step, int commit_every,
                long long* cycles, int* status) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int STAGE = 48 * 1024;
    ProbeShared* sh = reinterpret_cast<ProbeShared*>(smem + 4 * STAGE);
    for (int i = threadIdx.x; i < 4 * STAGE / 16; i += blockDim.x) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
    if (threadIdx.x == 0) {
        mbar_init(&sh->done, 1);
        mbar_init(&sh->scratch, 1);
        mbar_init(&sh->never, 1);
        sh->finished = 0;
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
    if (threadIdx.x < 32) {
        // the whole warp runs the loop; one elected lane issues
        const uint32_t idesc = kind == 0 ? idesc_nvfp4(128, n) : kind == 1 ? idesc_tf32(128, n) : idesc_i8(128, n, true);
        const long long t0 = clock64();
        for (int it = 0; it < iters; ++it) {
            const uint32_t sa = smem_u32(smem + (it & 3) * STAGE);
            const uint64_t adesc = smem_desc_sw128(sa);
            const uint64_t bdesc = smem_desc_sw128(sa + 16384);
            const uint32_t t_sf = tmem + 384 + (sf_buffers > 1 ? (it % sf_buffers) * 48 : 0);
            if (elect_one()) {
                for (int j = 0; j < cps_per_group; ++j)
                    tc_cp_32x128b_warpx4(t_sf + 4 * j, smem_desc_sf(sa + 40960 + j * 512));
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (kind == 0)
                        tc_mma_nvfp4(tmem, adesc + 2 * j, bdesc + 2 * j, idesc, t_sf + 4 * j, t_sf + 16 + sfb_step * j, 1);
                    else if (kind == 1)
                        tc_mma_tf32(tmem, adesc + 2 * j, bdesc + 2 * j, idesc, 1);
                    else
                        tc_mma_i8(tmem, adesc + 2 * j, bdesc + 2 * j, idesc, 1);
                }
                if (commit_every & 1) tc_commit(&sh->scratch);
            }
            __syncwarp();
        }
        const long long t1 = clock64();
        bool ok = true;
        if (elect_one()) tc_commit(&sh->done);
        __syncwarp();
        ok = mbar_wait(&sh->done, 0);
        const long long t2 = clock64();
        if (threadIdx.x == 0) {
            if (!ok) atomicExch(&status[0], SVDQ_ERR_TIMEOUT);
            cycles[blockIdx.x * 2] = t1 - t0;      // issue time
            cycles[blockIdx.x * 2 + 1] = t2 - t0;  // until the last MMA completed
            sh->finished = 1;
        }
    } else if (threadIdx.x >= 64) {
        while (!sh->finished) {
            for (int i = 0; i < 64; ++i)
                if (mbar_try_wait(&sh->never, 0)) break;
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x < 32) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, 512);
    }
}

// The same loop on a CTA pair: cluster of 2, TMEM allocated with cta_group::2 by both CTAs, the even CTA
// issues 256-row MMAs (each CTA's tensor core does 128 x n), the completion is multicast to both.
__global__ void __launch_bounds__(64, 1)
mma_rate_pair_kernel(int kind, int n, int iters, int cps_per_group, long long* cycles, int* status) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int STAGE = 48 * 1024;
    ProbeShared* sh = reinterpret_cast<ProbeShared*>(smem + 4 * STAGE);
    for (int i = threadIdx.x; i < 4 * STAGE / 16; i += blockDim.x) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
    const uint32_t rank = cluster_ctarank();
    if (threadIdx.x == 0) {
        mbar_init(&sh->done, 1);
        fence_mbar_init();
    }
    if (threadIdx.x < 32) {
        tmem_alloc_pair(&sh->tmem_base, 512);
        tmem_relinquish_pair();
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    cluster_sync_all();
    tc_fence_after_sync();
    const uint32_t tmem = sh->tmem_base;
    if (threadIdx.x < 32) {
        const uint32_t idesc = kind == 0 ? idesc_nvfp4(256, n) : kind == 3 ? idesc_f16(256, n) : idesc_tf32(256, n);
        const long long t0 = clock64();
        if (rank == 0) {
            for (int it = 0; it < iters; ++it) {
                const uint32_t sa = smem_u32(smem + (it & 3) * STAGE);
                const uint64_t adesc = smem_desc_sw128(sa);
                const uint64_t bdesc = smem_desc_sw128(sa + 16384);
                const uint32_t t_sf = tmem + 384;
                if (elect_one()) {
                    // the scale-factor copies a block-scaled stage needs, interleaved with the MMAs as in the GEMM
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        for (int c = 0; c * 4 < cps_per_group; ++c)
                            if (c * 4 + j < cps_per_group) tc_cp_pair_32x128b_warpx4(t_sf + 4 * (c * 4 + j), smem_desc_sf(sa + 40960 + (c * 4 + j) * 512));
                        if (kind == 0)
                            tc_mma_pair_nvfp4(tmem, adesc + 2 * j, bdesc + 2 * j, idesc, t_sf + 4 * j, t_sf + 16 + 8 * j, 1);
                        else if (kind == 3)
                            tc_mma_pair_f16(tmem, adesc + 2 * j, bdesc + 2 * j, idesc, 1);
                        else
                            tc_mma_pair_tf32(tmem, adesc + 2 * j, bdesc + 2 * j, idesc, 1);
                    }
                }
                __syncwarp();
            }
        }
        const long long t1 = clock64();
        if (rank == 0) {
            if (elect_one()) tc_commit_pair(&sh->done, 3);
            __syncwarp();
        }
        bool ok = true;
        for (int i = 0; i < 64 && ok; ++i) {   // bounded, cluster-scope acquire
            const long long w0 = clock64();
            ok = false;
            while (clock64() - w0 < 60000000ll) {
                if (mbar_try_wait_cluster(&sh->done, 0)) { ok = true; break; }
            }
            if (ok) break;
            ok = i < 63;
        }
        const bool completed = mbar_try_wait_cluster(&sh->done, 0);
        const long long t2 = clock64();
        if (threadIdx.x == 0) {
            if (!completed) atomicExch(&status[0], SVDQ_ERR_TIMEOUT);
            cycles[blockIdx.x * 2] = t1 - t0;
            cycles[blockIdx.x * 2 + 1] = t2 - t0;
        }
    }
    tc_fence_before_sync();
    cluster_sync_all();
    if (threadIdx.x < 32) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem, 512);
    }
}

}  // namespace svdq

// kind 0 = mxf4nvf4, 1 = tf32, 3 = f16 (K = 16); grid must be even (CTA pairs).  No counterpart in the reference.
extern "C" int svdq_probe_mma_rate_pair(int kind, int n, int iters, int grid, long long* cycles, void* stream, int cps_per_group) {
    using namespace svdq;
    SVDQ_CHECK_ARG(cycles && grid > 0 && grid <= 1024 && grid % 2 == 0 && iters > 0 && n >= 32 && n <= 256 && n % 32 == 0 &&
                       (kind == 0 || kind == 1 || kind == 3) && cps_per_group >= 0 && cps_per_group <= 12,
                   "pair probe: bad argument");
    if (int rc = check_arch()) return rc;
    int* status = nullptr;
    if (int rc = status_words(&status)) return rc;
    const size_t smem = 1024 + 4 * 48 * 1024 + 64;
    SVDQ_CUDA(cudaFuncSetAttribute(mma_rate_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(64, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    SVDQ_CUDA(cudaLaunchKernelEx(&cfg, mma_rate_pair_kernel, kind, n, iters, cps_per_group, cycles, status));
    return SVDQ_OK;
}

// cycles: device buffer of 2 * grid int64 {issue, complete} per CTA.  No counterpart in the reference.
extern "C" int svdq_probe_mma_rate(int kind, int n, int iters, int cps_per_group, int sf_buffers, int grid,
                                   long long* cycles, void* stream, int sfb_step, int commit_every, int poll_warps) {
    using namespace svdq;
    SVDQ_CHECK_ARG(cycles && grid > 0 && grid <= 1024 && iters > 0 && n >= 16 && n <= 256 && n % 16 == 0 &&
                       cps_per_group >= 0 && cps_per_group <= 12 && sf_buffers >= 1 && sf_buffers <= 2 && kind >= 0 && kind <= 2 &&
                       sfb_step >= 4 && sfb_step <= 8 && poll_warps >= 0 && poll_warps <= 14,
                   "probe: bad argument");
    if (int rc = check_arch()) return rc;
    int* status = nullptr;
    if (int rc = status_words(&status)) return rc;
    const size_t smem = 1024 + 4 * 48 * 1024 + 64;
    SVDQ_CUDA(cudaFuncSetAttribute(mma_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    mma_rate_kernel<<<grid, 64 + 32 * poll_warps, smem, static_cast<cudaStream_t>(stream)>>>(kind, n, iters, cps_per_group, sf_buffers,
                                                                                     sfb_step, commit_every, cycles, status);
    SVDQ_CUDA(cudaGetLastError());
    return SVDQ_OK;
}

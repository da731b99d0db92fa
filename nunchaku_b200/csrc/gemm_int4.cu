// INT4 (group 64) W4A4 GEMM, sm_100a -- placeholder until the kind::i8 kernel lands.
#include "host_common.h"

namespace svdq {

int gemm_int4_impl(const svdq_gemm_args* a, cudaStream_t stream) {
    (void)a;
    (void)stream;
    return fail(SVDQ_ERR_UNSUPPORTED, "gemm(int4): the INT4 tcgen05 kernel is not built yet");
}

}  // namespace svdq

// The fp16 build of the W4A4 GEMM (namespace svdq::hf): the same source with the 16-bit type switched.
#define SVDQ_F16 1
#include "gemm_w4a4.cu"

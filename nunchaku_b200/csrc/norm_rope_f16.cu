// fp16 build of the row-wise kernels (namespace svdq::hf): the bf16 source compiled with the 16-bit type switched.
#define SVDQ_F16 1
#include "norm_rope.cu"

// fp16 build of the linear-attention kernel (namespace svdq::hf): the bf16 source compiled with the 16-bit type switched.
#define SVDQ_F16 1
#include "litela.cu"

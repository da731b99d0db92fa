// The fp16 build of the activation quantiser (namespace svdq::hf): the same source with the 16-bit type switched.
#define SVDQ_F16 1
#include "quantize.cu"

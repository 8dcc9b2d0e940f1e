// The bf16 build of the library: the same sources as capi.cu, compiled with the
// 16-bit element type switched (see common.cuh), exporting the *_bf16 entry points.
#define TCU_BF16 1
#include "capi.cu"

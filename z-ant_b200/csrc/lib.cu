// Single translation unit of libzant_b200.so: the C entry points and the plan share the
// kernels defined in the .cuh headers.
#include "abi.cu"
#include "plan.cu"
#include "noalloc.cu"
#include "multi.cu"

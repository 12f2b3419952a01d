// Single translation unit of libspiral_b200.so: the kernels share one device
// status word and a few launch helpers, so they are compiled together without
// relocatable device code.
#include "runtime.cu"
#include "rowops.cu"
#include "gemm_fp32.cu"
#include "gemm_umma.cu"
#include "api.cu"
#include "mlp.cu"
#include "mlp_fused.cu"
#include "dp.cu"
#include "selftest.cu"

// Single translation unit of libb200moe.so: all kernels and the C ABI.
#include "quantize.cu"
#include "grouped_gemm.cu"
#include "routing.cu"

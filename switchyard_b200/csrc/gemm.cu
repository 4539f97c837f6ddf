// grouped_gemm: tcgen05 / tensor-memory grouped GEMM (prefill path).
#include "common.cuh"

extern "C" int sy_grouped_gemm(const void* A, const int32_t* a_rows, const void* B, const int32_t* offsets,
                               int n_experts, int rows, int n_out, int k_dim, int swiglu, const void* scale, void* C,
                               int dtype, void* stream) {
  return sy::fail(SY_ERR_ARGUMENT, "grouped_gemm: not built yet");
}

// combine: each token's top-k expert rows summed in float32 in ascending expert order, rounded
// once. One block per token; a thread owns 16-byte slices of the hidden dimension and issues
// all k row loads before adding, so a token's k rows stream in parallel.
// Replaces the reference's combine (switchyard/csrc/moe_kernels.cu:417-444); the order of the
// additions (expert id, ties by slot) and the single final rounding are the same, which is what
// makes the expert-parallel layer bit-identical to the single-GPU one.
#include "combine.cuh"

namespace sy {

template <typename T>
__global__ void __launch_bounds__(COMBINE_THREADS)
combine_kernel(const T* __restrict__ y, const int* __restrict__ pos_of, const int* __restrict__ idx, int k, int H,
               T* __restrict__ out, const T* __restrict__ residual) {
  __shared__ int s_row[COMBINE_MAX_K];
  pdl_launch_dependents();
  pdl_wait();  // y comes from the down projection before this kernel
  combine_token<T, false>(y, pos_of, idx, k, H, out, blockIdx.x, s_row, (int)gridDim.x * k, residual);
}

}  // namespace sy

namespace sy {
static int combine_launch(const char* name, const void* y, const int32_t* pos_of, const int32_t* idx, int n_tokens,
                          int top_k, int hidden, const void* residual, bool wants_residual, void* out, int dtype,
                          void* stream) {
  SY_REQUIRE(n_tokens >= 0 && top_k >= 1 && top_k <= COMBINE_MAX_K, "%s: top_k must be 1..8 (got %d)", name, top_k);
  SY_REQUIRE(hidden > 0 && hidden % 8 == 0, "%s: hidden must be a multiple of 8 (got %d)", name, hidden);
  SY_REQUIRE(dtype == SY_DTYPE_F16 || dtype == SY_DTYPE_BF16, "%s: dtype must be f16 or bf16", name);
  if (n_tokens == 0) return SY_OK;
  SY_REQUIRE(y && pos_of && idx && out && (residual || !wants_residual), "%s: null pointer", name);
  SY_REQUIRE(((uintptr_t)y % 16 == 0) && ((uintptr_t)out % 16 == 0) && ((uintptr_t)residual % 16 == 0),
             "%s: y, residual and out must be 16-byte aligned", name);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == SY_DTYPE_F16)
    return launch_kernel(combine_kernel<__half>, n_tokens, COMBINE_THREADS, 0, s, "combine launch",
                         static_cast<const __half*>(y), pos_of, idx, top_k, hidden, static_cast<__half*>(out),
                         static_cast<const __half*>(residual));
  return launch_kernel(combine_kernel<__nv_bfloat16>, n_tokens, COMBINE_THREADS, 0, s, "combine launch",
                       static_cast<const __nv_bfloat16*>(y), pos_of, idx, top_k, hidden,
                       static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(residual));
}
}  // namespace sy

extern "C" int sy_combine(const void* y, const int32_t* pos_of, const int32_t* idx, int n_tokens, int top_k,
                          int hidden, void* out, int dtype, void* stream) {
  return sy::combine_launch("combine", y, pos_of, idx, n_tokens, top_k, hidden, nullptr, false, out, dtype, stream);
}

extern "C" int sy_combine_add(const void* y, const int32_t* pos_of, const int32_t* idx, int n_tokens, int top_k,
                              int hidden, const void* residual, void* out, int dtype, void* stream) {
  return sy::combine_launch("combine_add", y, pos_of, idx, n_tokens, top_k, hidden, residual, true, out, dtype, stream);
}

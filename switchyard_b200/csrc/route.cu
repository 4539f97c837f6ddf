// route: router logits -> float32 softmax -> top-k experts and weights. One warp per token.
//
// The rule and its implementation are in route.cuh; replaces switchyard/csrc/moe_kernels.cu:23-89.
#include "route.cuh"

namespace sy {

constexpr int ROUTE_THREADS = 256;


template <typename T, int PER_LANE>
__global__ void __launch_bounds__(ROUTE_THREADS)
route_kernel(const T* __restrict__ logits, int n_tokens, int E, int k, int norm, int* __restrict__ idx,
             T* __restrict__ w) {
  pdl_launch_dependents();
  pdl_wait();  // the logits come from the kernel before this one
  const int lane = threadIdx.x & 31;
  const int token = (blockIdx.x * ROUTE_THREADS + threadIdx.x) >> 5;
  if (token >= n_tokens) return;
  route_token<T, PER_LANE>(logits + (size_t)token * E, E, k, norm, lane, idx + (size_t)token * k, w + (size_t)token * k);
}

template <typename T>
static int launch_route(const void* logits, int n_tokens, int E, int k, int norm, int32_t* idx, void* w,
                        cudaStream_t stream) {
  int blocks = (n_tokens * 32 + ROUTE_THREADS - 1) / ROUTE_THREADS;
  const T* l = static_cast<const T*>(logits);
  T* wp = static_cast<T*>(w);
  if (E <= 32) return launch_kernel(route_kernel<T, 1>, blocks, ROUTE_THREADS, 0, stream, "route launch", l, n_tokens, E, k, norm, idx, wp);
  if (E <= 64) return launch_kernel(route_kernel<T, 2>, blocks, ROUTE_THREADS, 0, stream, "route launch", l, n_tokens, E, k, norm, idx, wp);
  return launch_kernel(route_kernel<T, 4>, blocks, ROUTE_THREADS, 0, stream, "route launch", l, n_tokens, E, k, norm, idx, wp);
}

}  // namespace sy

extern "C" int sy_route(const void* logits, int n_tokens, int n_experts, int top_k, int norm_topk_prob, int dtype,
                        int32_t* idx_out, void* w_out, void* stream) {
  using namespace sy;
  SY_REQUIRE(n_tokens >= 0, "route: negative token count");
  SY_REQUIRE(n_experts >= 1 && n_experts <= 128 && top_k >= 1 && top_k <= 8 && top_k <= n_experts,
             "route: at most 128 experts and top-8 (got E=%d, k=%d)", n_experts, top_k);
  SY_REQUIRE(dtype == SY_DTYPE_F16 || dtype == SY_DTYPE_BF16, "route: dtype must be f16 or bf16");
  if (n_tokens == 0) return SY_OK;
  SY_REQUIRE(logits && idx_out && w_out, "route: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return dtype == SY_DTYPE_F16
             ? launch_route<__half>(logits, n_tokens, n_experts, top_k, norm_topk_prob, idx_out, w_out, s)
             : launch_route<__nv_bfloat16>(logits, n_tokens, n_experts, top_k, norm_topk_prob, idx_out, w_out, s);
}

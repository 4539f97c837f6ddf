// combine: each token's top-k expert rows summed in float32 in ascending expert order, rounded
// once. One block per token; a thread owns 16-byte slices of the hidden dimension and issues
// all k row loads before adding, so a token's k rows stream in parallel.
// Replaces the reference's combine (switchyard/csrc/moe_kernels.cu:417-444); the order of the
// additions (expert id, ties by slot) and the single final rounding are the same, which is what
// makes the expert-parallel layer bit-identical to the single-GPU one.
#include "common.cuh"

namespace sy {

constexpr int COMBINE_THREADS = 256;
constexpr int COMBINE_MAX_K = 8;

template <typename T>
__global__ void __launch_bounds__(COMBINE_THREADS)
combine_kernel(const T* __restrict__ y, const int* __restrict__ pos_of, const int* __restrict__ idx, int k, int H,
               T* __restrict__ out) {
  __shared__ int s_row[COMBINE_MAX_K];
  const int t = blockIdx.x;
  pdl_launch_dependents();
  pdl_wait();  // y comes from the down projection before this kernel
  if (threadIdx.x < k) {
    // rank of this slot among the token's k choices by (expert id, slot)
    int e = idx[(size_t)t * k + threadIdx.x], rank = 0;
    for (int j = 0; j < k; ++j) {
      int ej = idx[(size_t)t * k + j];
      rank += (ej < e) || (ej == e && j < (int)threadIdx.x);
    }
    s_row[rank] = pos_of[(size_t)t * k + threadIdx.x];
  }
  __syncthreads();
  const int chunks = H >> 3;
  for (int c = threadIdx.x; c < chunks; c += COMBINE_THREADS) {
    uint4 v[COMBINE_MAX_K];
#pragma unroll
    for (int j = 0; j < COMBINE_MAX_K; ++j)
      if (j < k) v[j] = __ldg(reinterpret_cast<const uint4*>(y + (size_t)s_row[j] * H) + c);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < COMBINE_MAX_K; ++j)
      if (j < k) {
        float f[8];
        unpack8<T>(v[j], f);
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[q] += f[q];
      }
    __align__(16) T r[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) r[q] = Elem<T>::from_f(acc[q]);
    reinterpret_cast<uint4*>(out + (size_t)t * H)[c] = *reinterpret_cast<const uint4*>(r);
  }
}

}  // namespace sy

extern "C" int sy_combine(const void* y, const int32_t* pos_of, const int32_t* idx, int n_tokens, int top_k,
                          int hidden, void* out, int dtype, void* stream) {
  using namespace sy;
  SY_REQUIRE(n_tokens >= 0 && top_k >= 1 && top_k <= COMBINE_MAX_K, "combine: top_k must be 1..8 (got %d)", top_k);
  SY_REQUIRE(hidden > 0 && hidden % 8 == 0, "combine: hidden must be a multiple of 8 (got %d)", hidden);
  SY_REQUIRE(dtype == SY_DTYPE_F16 || dtype == SY_DTYPE_BF16, "combine: dtype must be f16 or bf16");
  if (n_tokens == 0) return SY_OK;
  SY_REQUIRE(y && pos_of && idx && out, "combine: null pointer");
  SY_REQUIRE(((uintptr_t)y % 16 == 0) && ((uintptr_t)out % 16 == 0), "combine: y and out must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == SY_DTYPE_F16)
    return launch_kernel(combine_kernel<__half>, n_tokens, COMBINE_THREADS, 0, s, "combine launch",
                         static_cast<const __half*>(y), pos_of, idx, top_k, hidden, static_cast<__half*>(out));
  return launch_kernel(combine_kernel<__nv_bfloat16>, n_tokens, COMBINE_THREADS, 0, s, "combine launch",
                       static_cast<const __nv_bfloat16*>(y), pos_of, idx, top_k, hidden,
                       static_cast<__nv_bfloat16*>(out));
}

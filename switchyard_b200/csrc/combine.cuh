// The per-token body of combine, shared by the plain kernel (csrc/combine.cu) and the
// expert-parallel one that signals and waits first (csrc/ep.cu).
#pragma once
#include "common.cuh"

namespace sy {

constexpr int COMBINE_THREADS = 256;
constexpr int COMBINE_MAX_K = 8;

// Token t's top-k rows of y summed in float32 in ascending expert order (ties by slot), rounded
// once. The whole block works on one token; s_row is COMBINE_MAX_K ints of shared memory.
// COHERENT: read y with L1 bypassed (rows that another GPU stored while this kernel ran).
// A choice without a row (pos_of outside [0, m): the sort skipped an invalid expert id) adds
// nothing. residual (may be null): [tokens, H]; the rounded sum is added to the token's residual
// row in float32 and rounded again, the bits of the caller's own `x + layer(h)` in 16-bit
// arithmetic (switchyard/model.py:135), without that kernel.
template <typename T, bool COHERENT>
__device__ __forceinline__ void combine_token(const T* __restrict__ y, const int* __restrict__ pos_of,
                                              const int* __restrict__ idx, int k, int H, T* __restrict__ out, int t,
                                              int* s_row, int m, const T* __restrict__ residual = nullptr) {
  if (threadIdx.x < k) {
    // rank of this slot among the token's k choices by (expert id, slot)
    int e = idx[(size_t)t * k + threadIdx.x], rank = 0;
    for (int j = 0; j < k; ++j) {
      int ej = idx[(size_t)t * k + j];
      rank += (ej < e) || (ej == e && j < (int)threadIdx.x);
    }
    const int pos = pos_of[(size_t)t * k + threadIdx.x];
    s_row[rank] = pos >= 0 && pos < m ? pos : -1;
  }
  __syncthreads();
  const int chunks = H >> 3;
  for (int c = threadIdx.x; c < chunks; c += COMBINE_THREADS) {
    uint4 v[COMBINE_MAX_K];
#pragma unroll
    for (int j = 0; j < COMBINE_MAX_K; ++j)
      if (j < k) {
        v[j] = make_uint4(0u, 0u, 0u, 0u);  // sixteen-bit zeros: adds nothing
        if (s_row[j] >= 0) {
          const uint4* p = reinterpret_cast<const uint4*>(y + (size_t)s_row[j] * H) + c;
          v[j] = COHERENT ? __ldcg(p) : __ldg(p);
        }
      }
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
    if (residual) {
      float x[8], sum[8];
      unpack8<T>(__ldg(reinterpret_cast<const uint4*>(residual + (size_t)t * H) + c), x);
      unpack8<T>(*reinterpret_cast<const uint4*>(r), sum);
#pragma unroll
      for (int q = 0; q < 8; ++q) r[q] = Elem<T>::from_f(x[q] + sum[q]);
    }
    reinterpret_cast<uint4*>(out + (size_t)t * H)[c] = *reinterpret_cast<const uint4*>(r);
  }
}

}  // namespace sy

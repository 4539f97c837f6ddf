// The routing of one token by one warp, shared by the routing kernel (route.cu) and the fused
// route + sort kernel for decode-sized batches (sort.cu).
#pragma once

#include "common.cuh"

namespace sy {

// One token, one warp: softmax over its E logits, k picks, weights. All 32 lanes take part.
template <typename T, int PER_LANE>
__device__ __forceinline__ void route_token(const T* __restrict__ row, int E, int k, int norm, int lane,
                                            int* __restrict__ idx_out, T* __restrict__ w_out) {
  float v[PER_LANE];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < PER_LANE; ++j) {
    int e = lane + 32 * j;
    v[j] = e < E ? Elem<T>::to_f(row[e]) : -INFINITY;
    mx = fmaxf(mx, v[j]);
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));

  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < PER_LANE; ++j) {
    int e = lane + 32 * j;
    v[j] = e < E ? expf(v[j] - mx) : 0.f;
    sum += v[j];
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);

  // k rounds of warp arg-max; lane r keeps round r's pick so that the stores are coalesced
  float my_w = 0.f, total = 0.f;
  int my_e = 0;
  for (int r = 0; r < k; ++r) {
    float best = -1.f;
    int best_e = 1 << 30;
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j) {
      int e = lane + 32 * j;
      if (e < E && (v[j] > best || (v[j] == best && e < best_e))) {
        best = v[j];
        best_e = e;
      }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      float ob = __shfl_xor_sync(0xffffffffu, best, o);
      int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) {
        best = ob;
        best_e = oe;
      }
    }
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j)
      if (lane + 32 * j == best_e) v[j] = -1.f;  // taken
    float p = best / sum;
    total += p;
    if (lane == r) {
      my_w = p;
      my_e = best_e;
    }
  }
  if (lane < k) {
    idx_out[lane] = my_e;
    w_out[lane] = Elem<T>::from_f(norm ? my_w / total : my_w);
  }
}

// Dispatch on the number of logits per lane (E <= 32, 64, 128).
template <typename T>
__device__ __forceinline__ void route_token_any(const T* __restrict__ row, int E, int k, int norm, int lane,
                                                int* __restrict__ idx_out, T* __restrict__ w_out) {
  if (E <= 32) route_token<T, 1>(row, E, k, norm, lane, idx_out, w_out);
  else if (E <= 64) route_token<T, 2>(row, E, k, norm, lane, idx_out, w_out);
  else route_token<T, 4>(row, E, k, norm, lane, idx_out, w_out);
}

}  // namespace sy

// The routing of one token by one warp, shared by the routing kernel (route.cu) and the
// one-launch routing kernels for decode-sized batches (sort.cu).
//
// What the rule is (it fixes the expert indices bit for bit, and is what the reference's kernel
// computes, switchyard/csrc/moe_kernels.cu:23-71): float32 softmax numerators exp(v - max) with
// the warp's maximum and sum taken as xor butterflies (expert e lives in lane e % 32, a lane adds
// its own experts in index order first); k picks of the largest numerator, the LOWER expert index
// on equal numerators; weight = numerator / sum, divided by the sum of the picked weights (added
// in pick order) when renormalising; one rounding to the 16-bit type.
//
// How it is done here: selection works on one integer key per expert. A non-negative float's
// bit pattern orders like the float, so (bits << 32) | (127 - e) orders by numerator first and by
// the lower index second, and a pick is one 64-bit maximum over the warp; a taken expert's key
// drops to -1. A row of NaNs or of -inf has no valid numerator: its numerators count as zero,
// so the picks are the k lowest experts with weight 0 and no index ever leaves [0, E).
#pragma once

#include "common.cuh"

namespace sy {

constexpr int ROUTE_MAX_E = 128;

__device__ __forceinline__ long long route_key(float numerator, int e) {
  return ((long long)__float_as_int(numerator) << 32) | (long long)(ROUTE_MAX_E - 1 - e);
}
__device__ __forceinline__ int route_key_expert(long long key) { return ROUTE_MAX_E - 1 - (int)(key & 0xffffffffll); }
__device__ __forceinline__ float route_key_value(long long key) { return __int_as_float((int)(key >> 32)); }

template <typename T> __device__ __forceinline__ float route_load(const T* row, int e) { return Elem<T>::to_f(row[e]); }
template <> __device__ __forceinline__ float route_load<float>(const float* row, int e) { return row[e]; }

// One token, one warp. `row` holds the token's E logits (global or shared memory; element type
// L is the 16-bit type or float holding 16-bit-rounded values). Lane r < k ends up with pick r
// and stores it, so the stores of a token are one coalesced segment. All 32 lanes take part.
template <typename T, int PER_LANE, typename L>
__device__ __forceinline__ void route_token(const L* __restrict__ row, int E, int k, int norm, int lane,
                                            int* __restrict__ idx_out, T* __restrict__ w_out) {
  float x[PER_LANE];
  float top = -INFINITY;
#pragma unroll
  for (int j = 0; j < PER_LANE; ++j) {
    const int e = lane + 32 * j;
    x[j] = e < E ? route_load<L>(row, e) : -INFINITY;
    top = fmaxf(top, x[j]);
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));

  long long key[PER_LANE];
  float denom = 0.f;
#pragma unroll
  for (int j = 0; j < PER_LANE; ++j) {
    const int e = lane + 32 * j;
    float p = e < E ? expf(x[j] - top) : 0.f;
    if (!(p >= 0.f)) p = 0.f;  // NaN: no valid numerator
    denom += p;
    key[j] = e < E ? route_key(p, e) : -1ll;
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) denom += __shfl_xor_sync(0xffffffffu, denom, o);

  float mine = 0.f, picked_sum = 0.f;
  int mine_e = 0;
  for (int r = 0; r < k; ++r) {
    long long best = key[0];
#pragma unroll
    for (int j = 1; j < PER_LANE; ++j) best = key[j] > best ? key[j] : best;
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      const long long other = __shfl_xor_sync(0xffffffffu, best, o);
      best = other > best ? other : best;
    }
    const int e = route_key_expert(best);
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j)
      if (lane + 32 * j == e) key[j] = -1ll;
    const float p = denom > 0.f ? route_key_value(best) / denom : 0.f;
    picked_sum += p;
    if (lane == r) {
      mine = p;
      mine_e = e;
    }
  }
  if (lane < k) {
    idx_out[lane] = mine_e;
    w_out[lane] = Elem<T>::from_f(norm ? (picked_sum > 0.f ? mine / picked_sum : 0.f) : mine);
  }
}

// Dispatch on the number of logits per lane (E <= 32, 64, 128).
template <typename T, typename L>
__device__ __forceinline__ void route_token_any(const L* __restrict__ row, int E, int k, int norm, int lane,
                                                int* __restrict__ idx_out, T* __restrict__ w_out) {
  if (E <= 32) route_token<T, 1, L>(row, E, k, norm, lane, idx_out, w_out);
  else if (E <= 64) route_token<T, 2, L>(row, E, k, norm, lane, idx_out, w_out);
  else route_token<T, 4, L>(row, E, k, norm, lane, idx_out, w_out);
}

}  // namespace sy

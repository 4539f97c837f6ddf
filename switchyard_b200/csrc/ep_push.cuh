// The dispatch of an expert-parallel layer as a device function: every sorted row of this rank
// goes to the rank that owns its expert, stored straight into that rank's mailbox (its own
// rows too, locally) together with the router weight; block 0 adds, per destination, the
// rebased per-expert offsets, the segment's first row and its row count. Every block counts what
// it has stored (one system-scope fence and one atomic per block); the block that completes the
// total fences at system scope and stores the layer's epoch into every receiver's arrival flag.
// Used by the stand-alone dispatch kernel (ep.cu) and by the expert kernel's prologue (gemm.cu),
// which saves a launch on the layer's critical path.
#pragma once

#include "common.cuh"

namespace sy {

constexpr int EP_MAX_RANKS = 16;

struct PushArgs {
  const uint4* h;                   // [tokens][vec_per_row] this rank's hidden states; nullptr: nothing to push
  const int* token;                 // [rows] token of each sorted row
  const unsigned short* wsorted;    // [rows] router weight of each sorted row (16-bit)
  const int* offsets;               // [R * per + 1] sorted-row offsets per global expert
  int per, R, self, vec_per_row, cap;
  unsigned char* x[EP_MAX_RANKS];   // receiver d's mailbox rows for this sender
  unsigned char* w[EP_MAX_RANKS];   // ... router weights
  int* meta[EP_MAX_RANKS];          // ... [per+1 rebased offsets | first row | row count]
  int* flag[EP_MAX_RANKS];          // ... arrival flag of this sender
  int block_fence_sys;              // 1: every block fences at system scope before it counts; 0: at GPU scope
  int* counter;                     // [1] units stored so far (rows + one per destination); zero between launches
  long long* stats;                 // nullptr, or [0] += rows sent to other ranks, [1] += rows kept
};

// All threads of every block of the launch call this once (the block size is a multiple of 32).
// s_seg: R + 1 ints of shared memory; s_done: 2 ints. Returns true in the block that completed
// the push (it has published the flags and reset the counter).
__device__ __forceinline__ bool push_rows(const PushArgs& p, int epoch, int* status, int* s_seg, int* s_done) {
  const int R = p.R, per = p.per;
  if ((int)threadIdx.x <= R) s_seg[threadIdx.x] = p.offsets[threadIdx.x * per];
  if (threadIdx.x == 0) s_done[0] = s_done[1] = 0;
  __syncthreads();
  const int rows = s_seg[R];
  int units = 0;
  if (blockIdx.x == 0) {
    const int meta_ints = per + 3;
    for (int t = threadIdx.x; t < R * meta_ints; t += blockDim.x) {
      const int d = t / meta_ints, j = t - d * meta_ints;
      int v;
      if (j <= per) v = p.offsets[d * per + j] - s_seg[d];
      else if (j == per + 1) v = s_seg[d];
      else v = min(s_seg[d + 1] - s_seg[d], p.cap);
      p.meta[d][j] = v;
    }
    units = R;
    if (threadIdx.x == 0 && p.stats) {
      const int kept = s_seg[p.self + 1] - s_seg[p.self];
      p.stats[0] += rows - kept;
      p.stats[1] += kept;
    }
  }
  // A warp per row, rows dealt to the warps of all blocks in turn: a row costs two dependent
  // round trips (its token index, then its data), so what matters is how many rows are in
  // flight, not how many threads copy one row.
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  int mine = 0, d = 0;
  for (int row = blockIdx.x * warps + warp; row < rows; row += gridDim.x * warps) {
    ++mine;
    while (d + 1 < R && s_seg[d + 1] <= row) ++d;
    const int r = row - s_seg[d];
    if (r >= p.cap) {  // cannot happen when the caller respects its capacity; never write past a mailbox
      if (lane == 0) *status = DS_BAD_INDEX;
      continue;
    }
    const uint4* src = p.h + (size_t)p.token[row] * p.vec_per_row;
    uint4* dst = reinterpret_cast<uint4*>(p.x[d]) + (size_t)r * p.vec_per_row;
    for (int i = lane; i < p.vec_per_row; i += 4 * 32) {  // four loads in flight per lane, then their stores
      uint4 v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (i + 32 * j < p.vec_per_row) v[j] = __ldg(src + i + 32 * j);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (i + 32 * j < p.vec_per_row) dst[i + 32 * j] = v[j];
    }
    if (lane == 0) reinterpret_cast<unsigned short*>(p.w[d])[r] = p.wsorted[row];
  }
  if (lane == 0 && mine > 0) atomicAdd(s_done + 1, mine);
  __syncthreads();  // the block's stores have been issued
  units += s_done[1];
  if (threadIdx.x == 0 && units > 0) {
    // Release: this block's stores (ordered before this thread by the barrier) before its count.
    // The count is an atomic in this GPU's memory read by blocks of this GPU only, so GPU scope
    // orders it; the block that completes the total then fences at system scope before it raises
    // the flags in the receivers' memory, which carries every block's stores along (the chain of
    // release/acquire pairs is transitive whatever the scope of each link).
    if (p.block_fence_sys) __threadfence_system();
    else __threadfence();
    if (atomicAdd(p.counter, units) + units == rows + R) {
      __threadfence_system();
      for (int i = 0; i < R; ++i) st_relaxed_sys(p.flag[i], epoch);  // released by the fence above
      *p.counter = 0;
      s_done[0] = 1;
    }
  }
  __syncthreads();
  return s_done[0] != 0;
}

}  // namespace sy

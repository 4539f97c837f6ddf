// sort_by_expert: stable counting sort of the flat (token, choice) list by expert id.
//
// Deterministic and free of atomics. The list is cut into contiguous chunks, one per block,
// and each chunk into contiguous pieces, one per warp; a warp walks its piece 32 choices at a
// time. Inside a 32-wide step, __match_any_sync groups the lanes that hold the same expert, a
// lane's rank in its group is the number of lower lanes in it, and the group's lowest lane
// advances the warp's private per-expert counter in shared memory. Ranks therefore follow
// increasing flat index, which is exactly the order a stable sort gives.
//
//   one block  (m <= SORT_SINGLE_MAX): count, scan and scatter in a single launch;
//   many blocks: launch 1 writes per-block expert counts to scratch [blocks][E]; launch 2
//                re-counts its own chunk per warp, turns the scratch table into its starting
//                row per expert, and scatters. Two reads of 4 bytes per choice in total.
//
// Replaces the reference's one-block-per-expert sort (switchyard/csrc/moe_kernels.cu:94-157),
// which reads the whole list once per expert and calls torch for the prefix sum in between.
#include <atomic>
#include <mutex>

#include "route.cuh"

namespace sy {

constexpr int SORT_THREADS = 512;
constexpr int SORT_WARPS = SORT_THREADS / 32;
constexpr int SORT_MAX_E = 256;
constexpr int SORT_SINGLE_MAX = 8192;       // choices one block sorts by itself
constexpr int SORT_CHUNK = 1024;            // target choices per block when several blocks sort
constexpr int SORT_MAX_BLOCKS = 128;        // scratch table rows that launch 2 keeps in shared memory

struct SortShape {
  int blocks;      // blocks of the grid
  int per_block;   // choices per block (multiple of 32 * SORT_WARPS)
};

static SortShape sort_shape(int m) {
  SortShape s;
  if (m <= SORT_SINGLE_MAX) {
    s.blocks = 1;
    s.per_block = ((m + SORT_THREADS - 1) / SORT_THREADS) * SORT_THREADS;
    return s;
  }
  int blocks = (m + SORT_CHUNK - 1) / SORT_CHUNK;
  if (blocks > SORT_MAX_BLOCKS) blocks = SORT_MAX_BLOCKS;
  int per = (m + blocks - 1) / blocks;
  per = ((per + SORT_THREADS - 1) / SORT_THREADS) * SORT_THREADS;
  s.blocks = (m + per - 1) / per;
  s.per_block = per;
  return s;
}

// idx[i], read through L2 when COHERENT (the entry may have been written by another block of
// the same launch).
template <bool COHERENT> __device__ __forceinline__ int load_choice(const int* idx, int i) {
  return COHERENT ? __ldcg(idx + i) : idx[i];
}

// Per-warp expert counts of this block's chunk into wcount[warp][e] (shared, zeroed here).
template <bool COHERENT = false>
__device__ __forceinline__ void count_chunk(const int* idx, int m, int begin, int per_warp, int E,
                                            int* wcount) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < SORT_WARPS * E; i += SORT_THREADS) wcount[i] = 0;
  __syncthreads();
  int* mine = wcount + warp * E;
  const int start = begin + warp * per_warp;
  for (int base = start; base < start + per_warp && base < m; base += 32) {
    int i = base + lane;
    int e = i < m ? load_choice<COHERENT>(idx, i) : -1;
    bool ok = e >= 0 && e < E;
    unsigned group = __match_any_sync(0xffffffffu, ok ? e : -1);
    if (ok && lane == __ffs(group) - 1) mine[e] += __popc(group);
    __syncwarp();
  }
  __syncthreads();
}

// Exclusive scan of v[0..E) by one warp, result in out[0..E], out[E] = total. E <= SORT_MAX_E.
__device__ __forceinline__ void warp_scan_experts(const int* v, int E, int* out) {
  const int lane = threadIdx.x & 31;
  int carry = 0;
  for (int base = 0; base < E; base += 32) {
    int e = base + lane;
    int x = e < E ? v[e] : 0, inc = x;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int y = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += y;
    }
    if (e < E) out[e] = carry + inc - x;
    carry += __shfl_sync(0xffffffffu, inc, 31);
  }
  if (lane == 0) out[E] = carry;
}

template <typename T, bool COHERENT = false>
__device__ __forceinline__ void scatter_chunk(const int* idx, const T* w, int m, int k,
                                              int begin, int per_warp, int E, int* wbase,
                                              int* __restrict__ token, T* __restrict__ wsorted,
                                              int* __restrict__ pos_of, int* status) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int* mine = wbase + warp * E;
  const int start = begin + warp * per_warp;
  for (int base = start; base < start + per_warp && base < m; base += 32) {
    int i = base + lane;
    int e = i < m ? load_choice<COHERENT>(idx, i) : -1;
    bool ok = e >= 0 && e < E;
    if (i < m && !ok) {  // an expert id outside [0, E): the choice gets no row; combine skips it
      *status = DS_BAD_INDEX;
      pos_of[i] = -1;
    }
    unsigned group = __match_any_sync(0xffffffffu, ok ? e : -1);
    int pos = 0;
    if (ok) pos = mine[e] + __popc(group & ((1u << lane) - 1u));
    __syncwarp();
    if (ok && lane == __ffs(group) - 1) mine[e] += __popc(group);
    __syncwarp();
    if (ok) {
      token[pos] = i / k;
      wsorted[pos] = COHERENT ? ldcg16(w + i) : w[i];
      pos_of[i] = pos;
    }
  }
}

// One block does everything.
template <typename T>
__global__ void __launch_bounds__(SORT_THREADS)
sort_single_kernel(const int* __restrict__ idx, const T* __restrict__ w, int m, int k, int E, int per_block,
                   int* __restrict__ counts, int* __restrict__ offsets, int* __restrict__ token,
                   T* __restrict__ wsorted, int* __restrict__ pos_of, int* status) {
  extern __shared__ int sh[];
  int* wcount = sh;                       // [SORT_WARPS][E]
  int* total = wcount + SORT_WARPS * E;   // [E]
  int* off = total + E;                   // [E + 1]
  const int per_warp = per_block / SORT_WARPS;
  pdl_launch_dependents();
  pdl_wait();  // idx and w come from the routing kernel
  count_chunk(idx, m, 0, per_warp, E, wcount);
  for (int e = threadIdx.x; e < E; e += SORT_THREADS) {
    int s = 0;
    for (int wi = 0; wi < SORT_WARPS; ++wi) s += wcount[wi * E + e];
    total[e] = s;
    counts[e] = s;
  }
  __syncthreads();
  if (threadIdx.x < 32) warp_scan_experts(total, E, off);
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += SORT_THREADS) offsets[e] = off[e];
  // wcount[warp][e] <- first row of warp's rows of expert e
  for (int e = threadIdx.x; e < E; e += SORT_THREADS) {
    int at = off[e];
    for (int wi = 0; wi < SORT_WARPS; ++wi) {
      int c = wcount[wi * E + e];
      wcount[wi * E + e] = at;
      at += c;
    }
  }
  __syncthreads();
  scatter_chunk<T>(idx, w, m, k, 0, per_warp, E, wcount, token, wsorted, pos_of, status);
}

// Decode-sized batches, everything before the experts in ONE launch: the router GEMM (optional:
// with `logits_in` the logits are taken as given and only the routing and the sort run, which is
// sy_route_sort), the routing and the sort. A block owns sixteen tokens. Its sixteen warps each take every
// sixteenth 32-wide slice of the hidden dimension and multiply the sixteen token rows by all
// E router rows over their slices with warp-level MMAs (the operands come straight from global
// memory, 16 bytes per lane and row: a lane's eight consecutive k feed two MMAs, and because
// both operands use the same assignment of k to fragment slots the products that are summed are
// the right ones); the warps' partial sums meet in shared memory and are added in warp order, so
// a token's logits depend on nothing but its own row. The sums are rounded to the 16-bit type
// (what the router GEMM of the unfused path stores), an optional per-expert bias is added in
// that type, every warp routes one token from shared memory, and the block that finishes last
// (a ticket in `ticket`, which it leaves at zero) sorts all choices as sort_single_kernel does.
// The logits are also written out when `logits_out` is given: the routing is the kernel rule of
// route.cuh applied to exactly those values.
// Replaces switchyard/kernels.py:30-32 (cuBLAS GEMM, then route) and moe_kernels.cu:142-157.
constexpr int RF_TOKENS = 16;

template <typename T, bool GEMM>
__global__ void __launch_bounds__(SORT_THREADS)
route_fused_kernel(const T* __restrict__ h, const T* __restrict__ router, const T* __restrict__ bias,
                   const T* __restrict__ logits_in, int n_tokens, int E,
                   int K, int k, int norm, int per_block, T* __restrict__ logits_out, int* idx, T* w, int* __restrict__ counts,
                   int* __restrict__ offsets, int* __restrict__ token, T* __restrict__ wsorted, int* __restrict__ pos_of,
                   int* ticket, int* status) {
  extern __shared__ int sh[];
  float* partial = reinterpret_cast<float*>(sh);  // [SORT_WARPS][RF_TOKENS][E]
  __shared__ int s_last;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  const int t0 = blockIdx.x * RF_TOKENS;
  const int n_tiles = E >> 3;  // eight experts per MMA
  pdl_launch_dependents();
  pdl_wait();  // the hidden states (or the logits) come from the caller's previous kernel

  if constexpr (!GEMM) {
    // the logits are given (sy_route_sort): a warp per token straight from global memory
    if (t0 + warp < n_tokens)
      route_token_any<T>(logits_in + (size_t)(t0 + warp) * E, E, k, norm, lane, idx + (size_t)(t0 + warp) * k,
                         w + (size_t)(t0 + warp) * k);
  } else {
  // ---- router GEMM: this warp's slices of k
  float acc[ROUTE_MAX_E / 8][4];
#pragma unroll
  for (int n = 0; n < ROUTE_MAX_E / 8; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
  const bool row_a = t0 + g < n_tokens, row_b = t0 + g + 8 < n_tokens;
  const uint4* ha = reinterpret_cast<const uint4*>(h + (size_t)(t0 + g) * K) + q;
  const uint4* hb = reinterpret_cast<const uint4*>(h + (size_t)(t0 + g + 8) * K) + q;
  const uint4* rw = reinterpret_cast<const uint4*>(router + (size_t)g * K) + q;
  const size_t tile_stride = (size_t)K;  // uint4 units between expert n and expert n + 8: 8 rows * K / 8
  for (int c = warp; c * 32 < K; c += SORT_WARPS) {
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    const uint4 a = row_a ? __ldg(ha + c * 4) : zero, b = row_b ? __ldg(hb + c * 4) : zero;
#pragma unroll
    for (int n = 0; n < ROUTE_MAX_E / 8; ++n) {
      if (n < n_tiles) {
        const uint4 r = __ldg(rw + n * tile_stride + c * 4);
        mma_16816<T>(acc[n], a.x, b.x, a.y, b.y, r.x, r.y);
        mma_16816<T>(acc[n], a.z, b.z, a.w, b.w, r.z, r.w);
      }
    }
  }
  float* mine = partial + (size_t)warp * RF_TOKENS * E;
#pragma unroll
  for (int n = 0; n < ROUTE_MAX_E / 8; ++n) {
    if (n < n_tiles) {
      const int col = n * 8 + q * 2;
      mine[g * E + col] = acc[n][0];
      mine[g * E + col + 1] = acc[n][1];
      mine[(g + 8) * E + col] = acc[n][2];
      mine[(g + 8) * E + col + 1] = acc[n][3];
    }
  }
  __syncthreads();
  // ---- the warps' partial sums, added in warp order; rounded; bias; kept as float in partial[0]
  float sums[(RF_TOKENS * ROUTE_MAX_E) / SORT_THREADS];
#pragma unroll
  for (int j = 0; j < (RF_TOKENS * ROUTE_MAX_E) / SORT_THREADS; ++j) {
    const int i = threadIdx.x + j * SORT_THREADS;
    float s = 0.f;
    if (i < RF_TOKENS * E)
      for (int wi = 0; wi < SORT_WARPS; ++wi) s += partial[(size_t)wi * RF_TOKENS * E + i];
    sums[j] = s;
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < (RF_TOKENS * ROUTE_MAX_E) / SORT_THREADS; ++j) {
    const int i = threadIdx.x + j * SORT_THREADS;
    if (i < RF_TOKENS * E) {
      T v = Elem<T>::from_f(sums[j]);
      if (bias) v = Elem<T>::from_f(Elem<T>::to_f(v) + Elem<T>::to_f(bias[i % E]));
      partial[i] = Elem<T>::to_f(v);
      const int t = t0 + i / E;
      if (logits_out && t < n_tokens) logits_out[(size_t)t * E + i % E] = v;
    }
  }
  __syncthreads();
  // ---- routing: a warp per token
  if (t0 + warp < n_tokens)
    route_token_any<T>(partial + warp * E, E, k, norm, lane, idx + (size_t)(t0 + warp) * k, w + (size_t)(t0 + warp) * k);
  }
  // ---- the last block to get here sorts every block's choices
  __syncthreads();
  if (threadIdx.x == 0) {
    int last = 1;
    if (gridDim.x > 1) {
      __threadfence();
      last = atomicAdd(ticket, 1) == (int)gridDim.x - 1;
      if (last) *ticket = 0;
      __threadfence();
    }
    s_last = last;
  }
  __syncthreads();
  if (!s_last) return;
  int* wcount = sh;                       // [SORT_WARPS][E]; the partial sums are no longer needed
  int* total = wcount + SORT_WARPS * E;   // [E]
  int* off = total + E;                   // [E + 1]
  const int per_warp = per_block / SORT_WARPS;
  const int m = n_tokens * k;
  count_chunk<true>(idx, m, 0, per_warp, E, wcount);
  for (int e = threadIdx.x; e < E; e += SORT_THREADS) {
    int s = 0;
    for (int wi = 0; wi < SORT_WARPS; ++wi) s += wcount[wi * E + e];
    total[e] = s;
    counts[e] = s;
  }
  __syncthreads();
  if (threadIdx.x < 32) warp_scan_experts(total, E, off);
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += SORT_THREADS) offsets[e] = off[e];
  for (int e = threadIdx.x; e < E; e += SORT_THREADS) {
    int at = off[e];
    for (int wi = 0; wi < SORT_WARPS; ++wi) {
      int c = wcount[wi * E + e];
      wcount[wi * E + e] = at;
      at += c;
    }
  }
  __syncthreads();
  scatter_chunk<T, true>(idx, w, m, k, 0, per_warp, E, wcount, token, wsorted, pos_of, status);
}

// Launch 1 of the multi-block sort: this block's expert counts into table[block][e].
__global__ void __launch_bounds__(SORT_THREADS)
sort_count_kernel(const int* __restrict__ idx, int m, int E, int per_block, int* __restrict__ table) {
  extern __shared__ int sh[];
  int* wcount = sh;
  count_chunk(idx, m, blockIdx.x * per_block, per_block / SORT_WARPS, E, wcount);
  for (int e = threadIdx.x; e < E; e += SORT_THREADS) {
    int s = 0;
    for (int wi = 0; wi < SORT_WARPS; ++wi) s += wcount[wi * E + e];
    table[blockIdx.x * E + e] = s;
  }
}

// Launch 2: starting rows from the table, then the stable scatter of this block's chunk.
template <typename T>
__global__ void __launch_bounds__(SORT_THREADS)
sort_scatter_kernel(const int* __restrict__ idx, const T* __restrict__ w, int m, int k, int E, int per_block,
                    const int* __restrict__ table, int* __restrict__ counts, int* __restrict__ offsets,
                    int* __restrict__ token, T* __restrict__ wsorted, int* __restrict__ pos_of, int* status) {
  extern __shared__ int sh[];
  int* wcount = sh;                       // [SORT_WARPS][E]
  int* total = wcount + SORT_WARPS * E;   // [E]
  int* off = total + E;                   // [E + 1]
  int* before = off + E + 1;              // [E] rows of expert e in earlier blocks
  const int per_warp = per_block / SORT_WARPS;
  count_chunk(idx, m, blockIdx.x * per_block, per_warp, E, wcount);
  for (int e = threadIdx.x; e < E; e += SORT_THREADS) {
    int s = 0, b4 = 0;
    for (int b = 0; b < (int)gridDim.x; ++b) {
      int c = table[b * E + e];
      if (b < (int)blockIdx.x) b4 += c;
      s += c;
    }
    total[e] = s;
    before[e] = b4;
  }
  __syncthreads();
  if (threadIdx.x < 32) warp_scan_experts(total, E, off);
  __syncthreads();
  if (blockIdx.x == 0) {
    for (int e = threadIdx.x; e < E; e += SORT_THREADS) counts[e] = total[e];
    for (int e = threadIdx.x; e <= E; e += SORT_THREADS) offsets[e] = off[e];
  }
  for (int e = threadIdx.x; e < E; e += SORT_THREADS) {
    int at = off[e] + before[e];
    for (int wi = 0; wi < SORT_WARPS; ++wi) {
      int c = wcount[wi * E + e];
      wcount[wi * E + e] = at;
      at += c;
    }
  }
  __syncthreads();
  scatter_chunk<T>(idx, w, m, k, blockIdx.x * per_block, per_warp, E, wcount, token, wsorted, pos_of, status);
}

template <typename T>
static int launch_sort(const int32_t* idx, const void* w, int m, int k, int E, int32_t* counts, int32_t* offsets,
                       int32_t* token, void* wsorted, int32_t* pos_of, void* scratch, cudaStream_t stream) {
  SortShape s = sort_shape(m);
  int* status = device_status_word();
  if (!status) return SY_ERR_CUDA;
  size_t smem = (size_t)(SORT_WARPS * E + 3 * E + 1) * sizeof(int);
  const T* wp = static_cast<const T*>(w);
  T* ws = static_cast<T*>(wsorted);
  if (s.blocks == 1) {
    return launch_kernel(sort_single_kernel<T>, 1, SORT_THREADS, smem, stream, "sort launch", idx, wp, m, k, E,
                         s.per_block, counts, offsets, token, ws, pos_of, status);
  } else {
    int* table = static_cast<int*>(scratch);
    sort_count_kernel<<<s.blocks, SORT_THREADS, (size_t)SORT_WARPS * E * sizeof(int), stream>>>(idx, m, E, s.per_block,
                                                                                             table);
    sort_scatter_kernel<T><<<s.blocks, SORT_THREADS, smem, stream>>>(idx, wp, m, k, E, s.per_block, table, counts,
                                                                    offsets, token, ws, pos_of, status);
  }
  return check_cuda(cudaGetLastError(), "sort launch");
}

}  // namespace sy

extern "C" size_t sy_sort_scratch_bytes(int m, int n_experts) {
  if (m <= sy::SORT_SINGLE_MAX || n_experts <= 0) return 0;
  return (size_t)sy::sort_shape(m).blocks * n_experts * sizeof(int);
}

extern "C" int sy_sort_by_expert(const int32_t* idx, const void* w, int m, int top_k, int n_experts, int dtype,
                                 int32_t* counts, int32_t* offsets, int32_t* token, void* wsorted, int32_t* pos_of,
                                 void* scratch, size_t scratch_bytes, void* stream) {
  using namespace sy;
  SY_REQUIRE(m >= 0 && top_k >= 1, "sort_by_expert: bad sizes (m=%d, k=%d)", m, top_k);
  SY_REQUIRE(n_experts >= 1 && n_experts <= SORT_MAX_E, "sort_by_expert: at most %d experts (got %d)", SORT_MAX_E,
             n_experts);
  SY_REQUIRE(dtype == SY_DTYPE_F16 || dtype == SY_DTYPE_BF16, "sort_by_expert: dtype must be f16 or bf16");
  SY_REQUIRE(counts && offsets, "sort_by_expert: null output");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (m == 0) {
    SY_CUDA(cudaMemsetAsync(counts, 0, sizeof(int32_t) * n_experts, s));
    SY_CUDA(cudaMemsetAsync(offsets, 0, sizeof(int32_t) * (n_experts + 1), s));
    return SY_OK;
  }
  SY_REQUIRE(idx && w && token && wsorted && pos_of, "sort_by_expert: null pointer");
  size_t need = sy_sort_scratch_bytes(m, n_experts);
  SY_REQUIRE(need == 0 || (scratch && scratch_bytes >= need), "sort_by_expert: %zu bytes of scratch needed, %zu given",
             need, scratch_bytes);
  return dtype == SY_DTYPE_F16
             ? launch_sort<__half>(idx, w, m, top_k, n_experts, counts, offsets, token, wsorted, pos_of, scratch, s)
             : launch_sort<__nv_bfloat16>(idx, w, m, top_k, n_experts, counts, offsets, token, wsorted, pos_of, scratch,
                                          s);
}

extern "C" int sy_route_sort_max_choices(void) { return sy::SORT_SINGLE_MAX; }

namespace sy {
// Shared launch of sy_route_sort (logits given) and sy_route_fused (router GEMM inside).
static int launch_route_fused(const void* h, const void* router, const void* bias, const void* logits_in, int n_tokens,
                              int n_experts, int hidden, int top_k, int norm, int dtype, void* logits_out, int32_t* idx,
                              void* w, int32_t* counts, int32_t* offsets, int32_t* token, void* wsorted, int32_t* pos_of,
                              int32_t* ticket, void* stream) {
  int* status = device_status_word();
  if (!status) return SY_ERR_CUDA;
  const int m = n_tokens * top_k;
  const SortShape sh = sort_shape(m);
  const size_t sort_smem = (size_t)(SORT_WARPS * n_experts + 3 * n_experts + 1) * sizeof(int);
  const size_t gemm_smem = logits_in ? 0 : (size_t)SORT_WARPS * RF_TOKENS * n_experts * sizeof(float);
  const size_t smem = sort_smem > gemm_smem ? sort_smem : gemm_smem;
  const int blocks = (n_tokens + RF_TOKENS - 1) / RF_TOKENS;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // only the form with the GEMM inside needs more than the default 48 KB of dynamic shared memory
  static std::atomic<int> configured[MAX_DEVICES][2];
  int dev = 0;
  SY_CUDA(cudaGetDevice(&dev));
  const int which = dtype == SY_DTYPE_F16 ? 0 : 1;
  if (!logits_in && !configured[dev][which].load(std::memory_order_acquire)) {
    const size_t most = (size_t)SORT_WARPS * RF_TOKENS * ROUTE_MAX_E * sizeof(float);
    if (which == 0)
      SY_CUDA(cudaFuncSetAttribute(route_fused_kernel<__half, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)most));
    else
      SY_CUDA(cudaFuncSetAttribute(route_fused_kernel<__nv_bfloat16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)most));
    configured[dev][which].store(1, std::memory_order_release);
  }
#define SY_RF_LAUNCH(TYPE, GEMM)                                                                                         \
  launch_kernel(route_fused_kernel<TYPE, GEMM>, blocks, SORT_THREADS, smem, s, "route_fused launch",                      \
                static_cast<const TYPE*>(h), static_cast<const TYPE*>(router), static_cast<const TYPE*>(bias),            \
                static_cast<const TYPE*>(logits_in), n_tokens, n_experts, hidden, top_k, norm, sh.per_block,              \
                static_cast<TYPE*>(logits_out), idx, static_cast<TYPE*>(w), counts, offsets, token,                       \
                static_cast<TYPE*>(wsorted), pos_of, ticket, status)
  if (dtype == SY_DTYPE_F16) return logits_in ? SY_RF_LAUNCH(__half, false) : SY_RF_LAUNCH(__half, true);
  return logits_in ? SY_RF_LAUNCH(__nv_bfloat16, false) : SY_RF_LAUNCH(__nv_bfloat16, true);
#undef SY_RF_LAUNCH
}
}  // namespace sy

extern "C" int sy_route_sort(const void* logits, int n_tokens, int n_experts, int top_k, int norm_topk_prob, int dtype,
                             int32_t* idx, void* w, int32_t* counts, int32_t* offsets, int32_t* token, void* wsorted,
                             int32_t* pos_of, int32_t* ticket, void* stream) {
  using namespace sy;
  SY_REQUIRE(n_tokens >= 1 && n_experts >= 1 && n_experts <= 128 && top_k >= 1 && top_k <= 8 && top_k <= n_experts,
             "route_sort: 1..128 experts, top-8, at least one token (got N=%d, E=%d, k=%d)", n_tokens, n_experts, top_k);
  SY_REQUIRE((long long)n_tokens * top_k <= SORT_SINGLE_MAX, "route_sort: at most %d choices (got %lld)",
             SORT_SINGLE_MAX, (long long)n_tokens * top_k);
  SY_REQUIRE(dtype == SY_DTYPE_F16 || dtype == SY_DTYPE_BF16, "route_sort: dtype must be f16 or bf16");
  SY_REQUIRE(logits && idx && w && counts && offsets && token && wsorted && pos_of, "route_sort: null pointer");
  SY_REQUIRE(ticket || n_tokens <= RF_TOKENS, "route_sort: more than %d tokens need a ticket", RF_TOKENS);
  return launch_route_fused(nullptr, nullptr, nullptr, logits, n_tokens, n_experts, 0, top_k, norm_topk_prob, dtype,
                            nullptr, idx, w, counts, offsets, token, wsorted, pos_of, ticket, stream);
}

extern "C" int sy_route_fused_max_tokens(void) { return sy::SORT_SINGLE_MAX / 8; }

extern "C" int sy_route_fused(const void* h, const void* router, const void* bias, int n_tokens, int n_experts, int hidden,
                              int top_k, int norm_topk_prob, int dtype, void* logits_out, int32_t* idx, void* w,
                              int32_t* counts, int32_t* offsets, int32_t* token, void* wsorted, int32_t* pos_of,
                              int32_t* ticket, void* stream) {
  using namespace sy;
  SY_REQUIRE(n_tokens >= 1 && n_experts >= 8 && n_experts <= ROUTE_MAX_E && n_experts % 8 == 0 && top_k >= 1 &&
                 top_k <= 8 && top_k <= n_experts,
             "route_fused: 8..128 experts in multiples of 8, top-8, at least one token (got N=%d, E=%d, k=%d)", n_tokens,
             n_experts, top_k);
  SY_REQUIRE((long long)n_tokens * top_k <= SORT_SINGLE_MAX, "route_fused: at most %d choices (got %lld)",
             SORT_SINGLE_MAX, (long long)n_tokens * top_k);
  SY_REQUIRE(hidden >= 32 && hidden % 32 == 0, "route_fused: hidden must be a multiple of 32 (got %d)", hidden);
  SY_REQUIRE(dtype == SY_DTYPE_F16 || dtype == SY_DTYPE_BF16, "route_fused: dtype must be f16 or bf16");
  SY_REQUIRE(h && router && idx && w && counts && offsets && token && wsorted && pos_of && ticket,
             "route_fused: null pointer");
  SY_REQUIRE(((uintptr_t)h % 16 == 0) && ((uintptr_t)router % 16 == 0), "route_fused: h and router must be 16-byte aligned");
  return launch_route_fused(h, router, bias, nullptr, n_tokens, n_experts, hidden, top_k, norm_topk_prob, dtype, logits_out,
                            idx, w, counts, offsets, token, wsorted, pos_of, ticket, stream);
}

// ---- sort_by_expert_static: the same sort for callers that cannot hand over scratch ----------
// Some hosts of this library must not allocate device memory once they are running: a serving
// process that has given every free byte of HBM to its own cache arena (a later cudaMalloc
// simply fails), or a plugin whose host forbids allocation calls on the request path. For them
// the multi-block sort's table of per-block expert counts lives in the library image itself.
namespace sy {

constexpr int SORT_STATIC_MAX_M = 1 << 20;  // choices per call (131 072 tokens x top-8)

// [SORT_MAX_BLOCKS][SORT_MAX_E] ints = 128 KiB, held by every GPU that loads the library until
// the process exits. In host code this name is only a handle for cudaGetSymbolAddress.
static __device__ __align__(256) int g_sort_static_table[SORT_MAX_BLOCKS * SORT_MAX_E];

static int* g_sort_static_ptr[MAX_DEVICES];
static std::mutex g_sort_static_mutex;

// Device address of the table on the CURRENT device, looked up once per device.
static int sort_static_table(int** out) {
  int dev = -1;
  SY_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= MAX_DEVICES) return fail(SY_ERR_ARGUMENT, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_sort_static_mutex);
  if (!g_sort_static_ptr[dev]) {
    void* p = nullptr;
    SY_CUDA(cudaGetSymbolAddress(&p, g_sort_static_table));
    g_sort_static_ptr[dev] = static_cast<int*>(p);
  }
  *out = g_sort_static_ptr[dev];
  return SY_OK;
}

}  // namespace sy

extern "C" int sy_sort_by_expert_static(const int32_t* idx, const void* w, int m, int top_k, int n_experts,
                                        int dtype, int32_t* counts, int32_t* offsets, int32_t* token, void* wsorted,
                                        int32_t* pos_of, void* stream) {
  using namespace sy;
  SY_REQUIRE(m >= 0 && top_k >= 1, "sort_by_expert_static: bad sizes (m=%d, k=%d)", m, top_k);
  SY_REQUIRE(m <= SORT_STATIC_MAX_M, "sort_by_expert_static: at most %d choices per call (got %d); use "
             "sy_sort_by_expert with caller-provided scratch beyond that", SORT_STATIC_MAX_M, m);
  SY_REQUIRE(n_experts >= 1 && n_experts <= SORT_MAX_E, "sort_by_expert_static: at most %d experts (got %d)",
             SORT_MAX_E, n_experts);
  SY_REQUIRE(dtype == SY_DTYPE_F16 || dtype == SY_DTYPE_BF16, "sort_by_expert_static: dtype must be f16 or bf16");
  SY_REQUIRE(counts && offsets, "sort_by_expert_static: null output");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (m == 0) {
    SY_CUDA(cudaMemsetAsync(counts, 0, sizeof(int32_t) * n_experts, s));
    SY_CUDA(cudaMemsetAsync(offsets, 0, sizeof(int32_t) * (n_experts + 1), s));
    return SY_OK;
  }
  SY_REQUIRE(idx && w && token && wsorted && pos_of, "sort_by_expert_static: null pointer");
  int* table = nullptr;
  int rc = sort_static_table(&table);  // first call on a device: symbol look-up (keep it out of stream capture)
  if (rc != SY_OK) return rc;
  // Nothing in the table has to start at zero: launch 1 writes every [block][expert] entry that
  // launch 2 reads. What is left from the previous call is overwritten or never looked at.
  return dtype == SY_DTYPE_F16
             ? launch_sort<__half>(idx, w, m, top_k, n_experts, counts, offsets, token, wsorted, pos_of, table, s)
             : launch_sort<__nv_bfloat16>(idx, w, m, top_k, n_experts, counts, offsets, token, wsorted, pos_of, table, s);
}

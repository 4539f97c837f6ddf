// grouped_gemv: the decode path. When every expert has only a few rows the layer is a stream
// over expert weights, so this kernel is built around keeping HBM busy:
//
//   * persistent grid, one block per SM. The work is the list of (used expert, 8-column group)
//     units in expert order; experts without rows are skipped entirely, and every block takes
//     an equal contiguous share of the list, so a block changes expert at most a few times;
//   * one producer warp streams each unit's weight rows into a ring of shared-memory stages
//     with 1-D bulk async copies (a unit's rows are contiguous in nn.Linear layout), completion
//     counted in bytes on an mbarrier; the ring is as deep as shared memory allows, and it
//     keeps filling across unit, pass and expert boundaries;
//   * eight consumer warps each own one output column of the stage (its gate row and its up
//     row when SwiGLU is fused). A lane reads 16-byte slices of the weight row and of up to 8
//     activation rows from shared memory, accumulates in float32, and the warp reduces with a
//     xor butterfly. Experts with more than 8 rows take further passes over the same units.
//
// A row's arithmetic (slice order per lane, butterfly, epilogue rounding) does not depend on
// how many rows share its expert or where the expert's units fall among the blocks, so the
// same row gives the same bits on one GPU and inside an expert-parallel segment.
//
// Replaces switchyard/csrc/moe_kernels.cu:306-415 (one block per (expert, 32 columns),
// direct global loads, blocks launched for empty experts too).
#include <atomic>

#include "common.cuh"

namespace sy {

constexpr int GV_CONSUMER_WARPS = 8;
constexpr int GV_CONSUMERS = GV_CONSUMER_WARPS * 32;
constexpr int GV_THREADS = GV_CONSUMERS + 32;   // + the producer warp
constexpr int GV_ROWS = 8;                      // activation rows per pass
constexpr int GV_COLS = GV_CONSUMER_WARPS;      // output columns per stage
constexpr int GV_MAX_E = 256;
constexpr int GV_MAX_STAGES = 12;
constexpr int GV_SMEM_BUDGET = 227 * 1024 - 2560;  // dynamic shared memory (the rest is static)

// One warp, one output column of one stage, NR activation rows: float32 dot products over the
// warp's 16-byte slices, xor-butterfly reduction, epilogue, store. NR is a compile-time
// constant so that no instruction is spent on rows that are not there.
template <typename T, bool SWIGLU, bool SCALE, int NR>
__device__ __forceinline__ void gemv_column(const T* __restrict__ wrow, const T* __restrict__ urow,
                                            const T* __restrict__ xs, int K, int lane, uint64_t* empty_bar,
                                            const T* __restrict__ scale, T* __restrict__ C, int row0, int col,
                                            int Nout) {
  float acc[NR], accu[NR];
#pragma unroll
  for (int r = 0; r < NR; ++r) acc[r] = accu[r] = 0.f;
#pragma unroll 2
  for (int kk = lane * 8; kk < K; kk += 256) {
    float wf[8], uf[8];
    unpack8<T>(*reinterpret_cast<const uint4*>(wrow + kk), wf);
    if (SWIGLU) unpack8<T>(*reinterpret_cast<const uint4*>(urow + kk), uf);
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      float xf[8];
      unpack8<T>(*reinterpret_cast<const uint4*>(xs + (size_t)r * K + kk), xf);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        acc[r] = fmaf(xf[q], wf[q], acc[r]);
        if (SWIGLU) accu[r] = fmaf(xf[q], uf[q], accu[r]);
      }
    }
  }
  // the stage is read: hand it back before the reduction
  __syncwarp();
  if (lane == 0) mbar_arrive(empty_bar);
#pragma unroll
  for (int r = 0; r < NR; ++r) {
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], o);
      if (SWIGLU) accu[r] += __shfl_xor_sync(0xffffffffu, accu[r], o);
    }
  }
  if (lane < NR) {
    float v = 0.f, g = 0.f;
#pragma unroll
    for (int r = 0; r < NR; ++r)
      if (r == lane) {
        v = acc[r];
        g = accu[r];
      }
    const int row = row0 + lane;
    T o;
    if (SWIGLU) o = epilogue_swiglu<T>(v, g);
    else if (SCALE) o = epilogue_scale<T>(v, scale[row]);
    else o = Elem<T>::from_f(v);
    C[(size_t)row * Nout + col] = o;
  }
}

template <typename T, bool SWIGLU, bool SCALE>
__global__ void __launch_bounds__(GV_THREADS, 1)
gemv_stream_kernel(const T* __restrict__ A, const int* __restrict__ a_rows, const T* __restrict__ B,
                   const int* __restrict__ offsets, int E, int Nout, int K, const T* __restrict__ scale,
                   T* __restrict__ C, int nstages, int* status) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ int s_off[GV_MAX_E + 1];
  __shared__ int s_used[GV_MAX_E];
  __shared__ int s_nused;
  __shared__ __align__(8) uint64_t full_bar[GV_MAX_STAGES];
  __shared__ __align__(8) uint64_t empty_bar[GV_MAX_STAGES];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int STAGE_ROWS = SWIGLU ? 2 * GV_COLS : GV_COLS;
  const uint32_t row_bytes = (uint32_t)K * sizeof(T);
  const uint32_t stage_bytes = STAGE_ROWS * row_bytes;
  T* xs = reinterpret_cast<T*>(smem);                                   // [GV_ROWS][K]
  unsigned char* ring = smem + (((size_t)GV_ROWS * row_bytes + 127) & ~(size_t)127);

  for (int i = threadIdx.x; i <= E; i += GV_THREADS) s_off[i] = offsets[i];
  if (threadIdx.x == 0) {
    for (int s = 0; s < nstages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], GV_CONSUMER_WARPS);
    }
    fence_barrier_init();
  }
  __syncthreads();
  if (warp == 0) {  // experts that have rows, in order
    int n = 0;
    for (int base = 0; base < E; base += 32) {
      int e = base + lane;
      bool has = e < E && s_off[e + 1] > s_off[e];
      unsigned m = __ballot_sync(0xffffffffu, has);
      if (has) s_used[n + __popc(m & ((1u << lane) - 1u))] = e;
      n += __popc(m);
    }
    if (lane == 0) s_nused = n;
  }
  __syncthreads();

  const int groups = Nout / GV_COLS;                    // units per expert
  const long long total = (long long)s_nused * groups;
  const int u_begin = (int)(total * blockIdx.x / gridDim.x);
  const int u_end = (int)(total * (blockIdx.x + 1) / gridDim.x);
  const int Nfull = SWIGLU ? 2 * Nout : Nout;

  if (warp == GV_CONSUMER_WARPS) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      int it = 0;
      bool alive = true;
      for (int u = u_begin; u < u_end && alive;) {
        const int ue = u / groups, e = s_used[ue];
        const int seg_end = min(u_end, (ue + 1) * groups);
        const int passes = (s_off[e + 1] - s_off[e] + GV_ROWS - 1) / GV_ROWS;
        const T* Be = B + (size_t)e * Nfull * K;
        for (int p = 0; p < passes && alive; ++p)
          for (int uu = u; uu < seg_end; ++uu, ++it) {
            const int s = it % nstages, use = it / nstages;
            if (use > 0 && !mbar_wait(&empty_bar[s], (use - 1) & 1)) {
              *status = DS_TIMEOUT_EMPTY;
              alive = false;
              break;
            }
            const int col0 = (uu - ue * groups) * GV_COLS;
            unsigned char* dst = ring + (size_t)s * stage_bytes;
            mbar_arrive_expect_tx(&full_bar[s], stage_bytes);
            bulk_g2s(dst, Be + (size_t)col0 * K, GV_COLS * row_bytes, &full_bar[s]);
            if (SWIGLU) bulk_g2s(dst + GV_COLS * row_bytes, Be + (size_t)(Nout + col0) * K, GV_COLS * row_bytes, &full_bar[s]);
          }
        u = seg_end;
      }
      if (!alive) {
        // gave up: let the copies already issued land before the block can exit
        for (int j = it > nstages ? it - nstages : 0; j < it; ++j)
          mbar_wait(&full_bar[j % nstages], (j / nstages) & 1, 10000000ull);
      }
    }
    return;
  }

  // -------------------------------------------------------------------- consumers
  int it = 0;
  bool alive = true;
  // A warp that gave up on a wait keeps walking the loops (so that the named barriers below
  // still see all eight warps) but skips every wait, load and store.
  for (int u = u_begin; u < u_end;) {
    const int ue = u / groups, e = s_used[ue];
    const int seg_end = min(u_end, (ue + 1) * groups);
    const int row_begin = s_off[e], row_end = s_off[e + 1];
    for (int r0 = row_begin; r0 < row_end; r0 += GV_ROWS) {
      const int nr = min(GV_ROWS, row_end - r0);
      // this pass's activation rows into shared memory (after everyone left the previous pass)
      named_barrier_sync(1, GV_CONSUMERS);
      const int vec_per_row = K >> 3;
      for (int c = threadIdx.x; c < nr * vec_per_row; c += GV_CONSUMERS) {
        int r = c / vec_per_row, v = c - r * vec_per_row;
        int src = a_rows ? a_rows[r0 + r] : r0 + r;
        reinterpret_cast<uint4*>(xs)[(size_t)r * vec_per_row + v] =
            __ldg(reinterpret_cast<const uint4*>(A + (size_t)src * K) + v);
      }
      named_barrier_sync(1, GV_CONSUMERS);

      for (int uu = u; uu < seg_end; ++uu, ++it) {
        const int s = it % nstages, use = it / nstages;
        if (alive && !mbar_wait(&full_bar[s], use & 1)) {
          *status = DS_TIMEOUT_FULL;
          alive = false;
        }
        if (!alive) continue;
        const unsigned char* stage = ring + (size_t)s * stage_bytes;
        const T* wrow = reinterpret_cast<const T*>(stage + (size_t)warp * row_bytes);
        const T* urow = reinterpret_cast<const T*>(stage + (size_t)(GV_COLS + warp) * row_bytes);
        const int col = (uu - ue * groups) * GV_COLS + warp;
#define SY_GEMV_CASE(NR)                                                                                         \
  case NR:                                                                                                       \
    gemv_column<T, SWIGLU, SCALE, NR>(wrow, urow, xs, K, lane, &empty_bar[s], scale, C, r0, col, Nout);         \
    break;
        switch (nr) {
          SY_GEMV_CASE(1) SY_GEMV_CASE(2) SY_GEMV_CASE(3) SY_GEMV_CASE(4)
          SY_GEMV_CASE(5) SY_GEMV_CASE(6) SY_GEMV_CASE(7) SY_GEMV_CASE(8)
        }
#undef SY_GEMV_CASE
      }
    }
    u = seg_end;
  }
}

template <typename T, bool SWIGLU, bool SCALE>
static int launch_gemv(const void* A, const int32_t* a_rows, const void* B, const int32_t* offsets, int E, int Nout,
                       int K, const void* scale, void* C, cudaStream_t stream) {
  int sms = 0;
  int rc = device_sm_count(&sms);
  if (rc != SY_OK) return rc;
  int* status = device_status_word();
  if (!status) return SY_ERR_CUDA;
  const size_t row_bytes = (size_t)K * sizeof(T);
  const size_t x_bytes = ((size_t)GV_ROWS * row_bytes + 127) & ~(size_t)127;
  const size_t stage_bytes = (size_t)(SWIGLU ? 2 : 1) * GV_COLS * row_bytes;
  if (x_bytes + 2 * stage_bytes > (size_t)GV_SMEM_BUDGET)
    return fail(SY_ERR_ARGUMENT, "grouped_gemv: k_dim=%d does not leave room for two stages of shared memory", K);
  int nstages = (int)((GV_SMEM_BUDGET - x_bytes) / stage_bytes);
  if (nstages > GV_MAX_STAGES) nstages = GV_MAX_STAGES;
  const size_t smem = x_bytes + (size_t)nstages * stage_bytes;
  auto kern = gemv_stream_kernel<T, SWIGLU, SCALE>;
  static std::atomic<int> configured[MAX_DEVICES];
  int dev = 0;
  SY_CUDA(cudaGetDevice(&dev));
  if (!configured[dev].load(std::memory_order_acquire)) {
    SY_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GV_SMEM_BUDGET));
    configured[dev].store(1, std::memory_order_release);
  }
  kern<<<sms, GV_THREADS, smem, stream>>>(static_cast<const T*>(A), a_rows, static_cast<const T*>(B), offsets, E, Nout,
                                          K, static_cast<const T*>(scale), static_cast<T*>(C), nstages, status);
  return check_cuda(cudaGetLastError(), "grouped_gemv launch");
}

template <typename T>
static int dispatch_gemv(const void* A, const int32_t* a_rows, const void* B, const int32_t* offsets, int E, int Nout,
                         int K, int swiglu, const void* scale, void* C, cudaStream_t stream) {
  if (swiglu) return launch_gemv<T, true, false>(A, a_rows, B, offsets, E, Nout, K, nullptr, C, stream);
  if (scale) return launch_gemv<T, false, true>(A, a_rows, B, offsets, E, Nout, K, scale, C, stream);
  return launch_gemv<T, false, false>(A, a_rows, B, offsets, E, Nout, K, nullptr, C, stream);
}

}  // namespace sy

extern "C" int sy_grouped_gemv(const void* A, const int32_t* a_rows, const void* B, const int32_t* offsets,
                               int n_experts, int rows, int n_out, int k_dim, int swiglu, const void* scale, void* C,
                               int dtype, void* stream) {
  using namespace sy;
  SY_REQUIRE(rows >= 0 && n_experts >= 1 && n_experts <= GV_MAX_E, "grouped_gemv: 1..%d experts (got %d)", GV_MAX_E,
             n_experts);
  SY_REQUIRE(k_dim > 0 && k_dim % 8 == 0, "grouped_gemv: k_dim must be a multiple of 8 (got %d)", k_dim);
  SY_REQUIRE(n_out > 0 && n_out % GV_COLS == 0, "grouped_gemv: n_out must be a multiple of %d (got %d)", GV_COLS, n_out);
  SY_REQUIRE(!(swiglu && scale), "grouped_gemv: swiglu and scale are separate epilogues");
  SY_REQUIRE(dtype == SY_DTYPE_F16 || dtype == SY_DTYPE_BF16, "grouped_gemv: dtype must be f16 or bf16");
  if (rows == 0) return SY_OK;
  SY_REQUIRE(A && B && offsets && C, "grouped_gemv: null pointer");
  SY_REQUIRE(((uintptr_t)A % 16 == 0) && ((uintptr_t)B % 16 == 0), "grouped_gemv: A and B must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return dtype == SY_DTYPE_F16
             ? dispatch_gemv<__half>(A, a_rows, B, offsets, n_experts, n_out, k_dim, swiglu, scale, C, s)
             : dispatch_gemv<__nv_bfloat16>(A, a_rows, B, offsets, n_experts, n_out, k_dim, swiglu, scale, C, s);
}

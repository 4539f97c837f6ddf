// grouped_gemm: every expert's slice of the sorted batch on the tcgen05 tensor cores.
//
// Orientation. The weight tile is the MMA's M operand and the token rows are its N operand
// ("C^T = W . X^T"): an instruction multiplies 128 weight rows by up to 128 token rows over 16
// k. That keeps M = 128 full no matter how few rows an expert has, so the same kernel is a
// weight stream for a handful of rows and a compute-bound GEMM for thousands; N is rounded up
// to a multiple of 16 per tile.
//
// One tile = (expert, 128 token rows, a pair of 128-row weight tiles that share the token
// operand). With SwiGLU fused the pair is gate rows [c, c+128) and up rows [c, c+128) of the
// same output columns, so the epilogue has both halves in tensor memory; otherwise it is 256
// consecutive output columns. The grid is persistent (one block per SM); tiles are numbered on
// the device from `offsets` (expert-major, an expert's row tiles adjacent so that its weights
// are read from HBM once and then hit L2) and dealt round-robin, so nothing about the batch
// is read back to the host.
//
// A block is fourteen warps with fixed roles, connected by mbarriers:
//   warp 0      TMA producer: the two weight tiles of each 64-wide k block, 128-byte swizzle;
//   warps 2-9   gather producers: the tile's token rows, picked from the UNSORTED activations
//               through a_rows, loaded 16 bytes per thread (prefetched one k block ahead in
//               registers) and stored to shared memory in the same swizzled layout;
//   warp 1      MMA issuer: one thread, tcgen05.mma into one of two accumulator pairs in
//               tensor memory; tcgen05.commit releases the stage / publishes the accumulators;
//   warps 10-13 epilogue: tcgen05.ld of the accumulators (a thread owns one output column and
//               walks the token rows), SwiGLU or router-weight scaling with the 16-bit
//               rounding points, stores. It overlaps the next tile's main loop.
// Four 48 KB stages; tensor memory: 2 buffers x 2 accumulators x 128 columns = all 512.
//
// An output element is a sum over k in instruction order that does not depend on which other
// rows share the tile or on the tile's N, so a row's bits are the same on one GPU and inside
// an expert-parallel segment.
//
// Replaces switchyard/csrc/moe_kernels.cu:159-298 (64x64x32 WMMA tiles, one block per tile,
// tile list built by torch on the host).
#include <cuda.h>

#include <atomic>
#include <mutex>
#include <type_traits>

#include "common.cuh"

namespace sy {

constexpr int GM_BK = 64;                          // k per stage: 128-byte rows
constexpr int GM_BM = 128;                         // weight rows per MMA tile
constexpr int GM_BN = 128;                         // token rows per tile
constexpr int GM_STAGES = 4;
constexpr int GM_TILE_BYTES = GM_BM * GM_BK * 2;   // 16 KB
constexpr int GM_STAGE_BYTES = 3 * GM_TILE_BYTES;  // W0, W1, X
constexpr int GM_GATHER_WARPS = 8;
constexpr int GM_EPI_WARPS = 4;
constexpr int GM_THREADS = (2 + GM_GATHER_WARPS + GM_EPI_WARPS) * 32;
constexpr int GM_TMEM_COLS = 512;
constexpr int GM_MAX_E = 256;
constexpr int GM_SMEM = GM_STAGES * GM_STAGE_BYTES + 1024;  // + room to align to 1024
constexpr uint64_t GM_WAIT_NS = 1000000000ull;

struct Tile {
  int e, cb, row0, nvalid;
};

// Tile t of the device-side numbering; `cursor` walks the experts monotonically.
__device__ __forceinline__ Tile locate_tile(int t, int& cursor, const int* tile_start, const int* off) {
  while (tile_start[cursor + 1] <= t) ++cursor;
  const int e = cursor, local = t - tile_start[e];
  const int n = off[e + 1] - off[e], row_tiles = (n + GM_BN - 1) / GM_BN;
  Tile tile;
  tile.e = e;
  tile.cb = local / row_tiles;
  tile.row0 = off[e] + (local % row_tiles) * GM_BN;
  tile.nvalid = min(GM_BN, off[e + 1] - tile.row0);
  return tile;
}

template <typename T, bool SWIGLU, bool SCALE>
__global__ void __launch_bounds__(GM_THREADS, 1)
gemm_umma_kernel(const __grid_constant__ CUtensorMap w_map, const T* __restrict__ A,
                 const int* __restrict__ a_rows, const int* __restrict__ offsets, int E, int Nout, int K,
                 const T* __restrict__ scale, T* __restrict__ C, int* status) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[GM_STAGES];
  __shared__ __align__(8) uint64_t empty_bar[GM_STAGES];
  __shared__ __align__(8) uint64_t acc_full[2];
  __shared__ __align__(8) uint64_t acc_empty[2];
  __shared__ uint32_t s_tmem;
  __shared__ int s_off[GM_MAX_E + 1];
  __shared__ int s_tile_start[GM_MAX_E + 2];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  unsigned char* stages =
      reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);

  const int col_blocks = SWIGLU ? (Nout + GM_BM - 1) / GM_BM : (Nout + 2 * GM_BM - 1) / (2 * GM_BM);
  const int Nfull = SWIGLU ? 2 * Nout : Nout;
  const int k_blocks = (K + GM_BK - 1) / GM_BK;

  for (int i = threadIdx.x; i <= E; i += GM_THREADS) s_off[i] = offsets[i];
  if (threadIdx.x == 0) {
    for (int s = 0; s < GM_STAGES; ++s) {
      mbar_init(&full_bar[s], 1 + GM_GATHER_WARPS);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], GM_EPI_WARPS);
    }
    fence_barrier_init();
    prefetch_tensormap(&w_map);
  }
  __syncthreads();
  if (warp == 0) {  // exclusive prefix of tiles per expert
    int carry = 0;
    for (int base = 0; base < E; base += 32) {
      int e = base + lane;
      int n = e < E ? s_off[e + 1] - s_off[e] : 0;
      int tiles = ((n + GM_BN - 1) / GM_BN) * col_blocks, inc = tiles;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int y = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += y;
      }
      if (e < E) s_tile_start[e] = carry + inc - tiles;
      carry += __shfl_sync(0xffffffffu, inc, 31);
    }
    if (lane == 0) {
      s_tile_start[E] = carry;
      s_tile_start[E + 1] = 0x7fffffff;  // sentinel: the cursor never walks past E
    }
  }
  if (warp == 1) {
    tmem_alloc(&s_tmem, GM_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = s_tmem;
  const int total_tiles = s_tile_start[E];

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int it = 0, cursor = 0;
      bool alive = true;
      for (int t = blockIdx.x; t < total_tiles && alive; t += gridDim.x) {
        const Tile tile = locate_tile(t, cursor, s_tile_start, s_off);
        const int y0 = tile.e * Nfull + (SWIGLU ? tile.cb * GM_BM : tile.cb * 2 * GM_BM);
        const int y1 = SWIGLU ? tile.e * Nfull + Nout + tile.cb * GM_BM : y0 + GM_BM;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % GM_STAGES, use = it / GM_STAGES;
          if (use > 0 && !mbar_wait(&empty_bar[s], (use - 1) & 1, GM_WAIT_NS)) {
            *status = DS_TIMEOUT_EMPTY;
            alive = false;
            break;
          }
          unsigned char* st = stages + (size_t)s * GM_STAGE_BYTES;
          mbar_arrive_expect_tx(&full_bar[s], 2 * GM_TILE_BYTES);
          tma_load_2d(st, &w_map, kb * GM_BK, y0, &full_bar[s]);
          tma_load_2d(st + GM_TILE_BYTES, &w_map, kb * GM_BK, y1, &full_bar[s]);
        }
      }
      if (!alive)  // let the copies already issued land before the block can exit
        for (int j = it > GM_STAGES ? it - GM_STAGES : 0; j < it; ++j)
          mbar_wait(&full_bar[j % GM_STAGES], (j / GM_STAGES) & 1, 10000000ull);
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const int fmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
      int it = 0, cursor = 0, tile_no = 0;
      bool alive = true;
      for (int t = blockIdx.x; t < total_tiles && alive; t += gridDim.x, ++tile_no) {
        const Tile tile = locate_tile(t, cursor, s_tile_start, s_off);
        const int buf = tile_no & 1, use_t = tile_no >> 1;
        if (use_t > 0) {
          if (!mbar_wait(&acc_empty[buf], (use_t - 1) & 1, GM_WAIT_NS)) {
            *status = DS_TIMEOUT_TMEM;
            alive = false;
            break;
          }
          tc_fence_after_sync();
        }
        const int n_mma = max(16, (tile.nvalid + 15) & ~15);
        const uint32_t idesc = umma_idesc(fmt, GM_BM, n_mma);
        const uint32_t d0 = tmem + buf * 2 * GM_BN, d1 = d0 + GM_BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % GM_STAGES;
          if (!mbar_wait(&full_bar[s], (it / GM_STAGES) & 1, GM_WAIT_NS)) {
            *status = DS_TIMEOUT_FULL;
            alive = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t base = smem_u32(stages + (size_t)s * GM_STAGE_BYTES);
#pragma unroll
          for (int ks = 0; ks < GM_BK / 16; ++ks) {
            const uint64_t a0 = umma_desc_k_sw128(base + ks * 32);
            const uint64_t a1 = umma_desc_k_sw128(base + GM_TILE_BYTES + ks * 32);
            const uint64_t b = umma_desc_k_sw128(base + 2 * GM_TILE_BYTES + ks * 32);
            const uint32_t accumulate = (kb | ks) != 0;
            umma_f16(d0, a0, b, idesc, accumulate);
            umma_f16(d1, a1, b, idesc, accumulate);
          }
          umma_commit(&empty_bar[s]);  // the stage is free once these MMAs have read it
        }
        if (alive) umma_commit(&acc_full[buf]);
      }
    }
  } else if (warp < 2 + GM_GATHER_WARPS) {
    // ---------------------------------------------------------------- gather producers
    const int g = threadIdx.x - 64;
    const int c = g & 7, rsub = g >> 3;  // 16-byte chunk of the 128-byte row; row within a group of 32
    int it = 0, cursor = 0;
    bool alive = true;
    for (int t = blockIdx.x; t < total_tiles && alive; t += gridDim.x) {
      const Tile tile = locate_tile(t, cursor, s_tile_start, s_off);
      const T* src[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = rsub + 32 * i;
        src[i] = nullptr;
        if (r < tile.nvalid) {
          const int row = a_rows ? a_rows[tile.row0 + r] : tile.row0 + r;
          src[i] = A + (size_t)row * K + c * 8;
        }
      }
      uint4 cur[4], nxt[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        cur[i] = make_uint4(0, 0, 0, 0);
        if (src[i] && c * 8 < K) cur[i] = __ldg(reinterpret_cast<const uint4*>(src[i]));
      }
      for (int kb = 0; kb < k_blocks; ++kb, ++it) {
        const int k_next = (kb + 1) * GM_BK + c * 8;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          nxt[i] = make_uint4(0, 0, 0, 0);
          if (src[i] && kb + 1 < k_blocks && k_next < K)
            nxt[i] = __ldg(reinterpret_cast<const uint4*>(src[i] + (size_t)(kb + 1) * GM_BK));
        }
        const int s = it % GM_STAGES, use = it / GM_STAGES;
        if (use > 0 && !mbar_wait(&empty_bar[s], (use - 1) & 1, GM_WAIT_NS)) {
          *status = DS_TIMEOUT_EMPTY;
          alive = false;
          break;
        }
        unsigned char* x = stages + (size_t)s * GM_STAGE_BYTES + 2 * GM_TILE_BYTES;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int r = rsub + 32 * i;
          if (r < tile.nvalid) *reinterpret_cast<uint4*>(x + r * 128 + ((c ^ (r & 7)) << 4)) = cur[i];
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&full_bar[s]);
#pragma unroll
        for (int i = 0; i < 4; ++i) cur[i] = nxt[i];
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int q = warp & 3;  // the quarter of tensor memory's lanes this warp may read
    int cursor = 0, tile_no = 0;
    bool alive = true;
    for (int t = blockIdx.x; t < total_tiles && alive; t += gridDim.x, ++tile_no) {
      const Tile tile = locate_tile(t, cursor, s_tile_start, s_off);
      const int buf = tile_no & 1, use_t = tile_no >> 1;
      if (!mbar_wait(&acc_full[buf], use_t & 1, GM_WAIT_NS)) {
        *status = DS_TIMEOUT_MMA;
        alive = false;
        break;
      }
      tc_fence_after_sync();
      const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16) + buf * 2 * GM_BN;
      const int wrow = q * 32 + lane;
      const int col0 = SWIGLU ? tile.cb * GM_BM + wrow : tile.cb * 2 * GM_BM + wrow;
      const int col1 = col0 + GM_BM;  // second accumulator's column (not used with SwiGLU)
      for (int n0 = 0; n0 < tile.nvalid; n0 += 8) {
        uint32_t v0[8], v1[8];
        tmem_ld_x8(taddr + n0, v0);
        tmem_ld_x8(taddr + GM_BN + n0, v1);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int row = tile.row0 + n0 + j;
          if (n0 + j < tile.nvalid) {
            const float f0 = __uint_as_float(v0[j]), f1 = __uint_as_float(v1[j]);
            if (SWIGLU) {
              if (col0 < Nout) C[(size_t)row * Nout + col0] = epilogue_swiglu<T>(f0, f1);
            } else if (SCALE) {
              const T sc = scale[row];
              if (col0 < Nout) C[(size_t)row * Nout + col0] = epilogue_scale<T>(f0, sc);
              if (col1 < Nout) C[(size_t)row * Nout + col1] = epilogue_scale<T>(f1, sc);
            } else {
              if (col0 < Nout) C[(size_t)row * Nout + col0] = Elem<T>::from_f(f0);
              if (col1 < Nout) C[(size_t)row * Nout + col1] = Elem<T>::from_f(f1);
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
  }

  // every role ends here; tensor memory goes back before the block exits
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, GM_TMEM_COLS);
  }
}

// ---- host side ------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int encode_fn(EncodeTiledFn* out) {
  static std::atomic<EncodeTiledFn> cached{nullptr};
  EncodeTiledFn fn = cached.load(std::memory_order_acquire);
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    SY_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
    if (q != cudaDriverEntryPointSuccess || !p)
      return fail(SY_ERR_CUDA, "grouped_gemm: the driver does not provide cuTensorMapEncodeTiled");
    fn = reinterpret_cast<EncodeTiledFn>(p);
    cached.store(fn, std::memory_order_release);
  }
  *out = fn;
  return SY_OK;
}

// Tensor map over the stacked expert weights as a [rows, K] matrix; box = 128 rows x 64 k.
static int weight_map(CUtensorMap* map, const void* B, uint64_t rows, uint64_t K, int dtype) {
  EncodeTiledFn encode;
  int rc = encode_fn(&encode);
  if (rc != SY_OK) return rc;
  cuuint64_t dims[2] = {K, rows};
  cuuint64_t strides[1] = {K * 2};
  cuuint32_t box[2] = {GM_BK, GM_BM};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = encode(map, dtype == SY_DTYPE_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                      2, const_cast<void*>(B), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(SY_ERR_CUDA, "grouped_gemm: cuTensorMapEncodeTiled failed (%d)", (int)r);
  return SY_OK;
}

template <typename T, bool SWIGLU, bool SCALE>
static int launch_gemm(const CUtensorMap& map, const void* A, const int32_t* a_rows, const int32_t* offsets, int E,
                       int Nout, int K, const void* scale, void* C, cudaStream_t stream) {
  int sms = 0;
  int rc = device_sm_count(&sms);
  if (rc != SY_OK) return rc;
  int* status = device_status_word();
  if (!status) return SY_ERR_CUDA;
  auto kern = gemm_umma_kernel<T, SWIGLU, SCALE>;
  static std::atomic<int> configured[MAX_DEVICES];
  int dev = 0;
  SY_CUDA(cudaGetDevice(&dev));
  if (!configured[dev].load(std::memory_order_acquire)) {
    SY_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GM_SMEM));
    configured[dev].store(1, std::memory_order_release);
  }
  kern<<<sms, GM_THREADS, GM_SMEM, stream>>>(map, static_cast<const T*>(A), a_rows, offsets, E, Nout, K,
                                             static_cast<const T*>(scale), static_cast<T*>(C), status);
  return check_cuda(cudaGetLastError(), "grouped_gemm launch");
}

template <typename T>
static int dispatch_gemm(const CUtensorMap& map, const void* A, const int32_t* a_rows, const int32_t* offsets, int E,
                         int Nout, int K, int swiglu, const void* scale, void* C, cudaStream_t stream) {
  if (swiglu) return launch_gemm<T, true, false>(map, A, a_rows, offsets, E, Nout, K, nullptr, C, stream);
  if (scale) return launch_gemm<T, false, true>(map, A, a_rows, offsets, E, Nout, K, scale, C, stream);
  return launch_gemm<T, false, false>(map, A, a_rows, offsets, E, Nout, K, nullptr, C, stream);
}

}  // namespace sy

extern "C" int sy_grouped_gemm(const void* A, const int32_t* a_rows, const void* B, const int32_t* offsets,
                               int n_experts, int rows, int n_out, int k_dim, int swiglu, const void* scale, void* C,
                               int dtype, void* stream) {
  using namespace sy;
  SY_REQUIRE(rows >= 0 && n_experts >= 1 && n_experts <= GM_MAX_E, "grouped_gemm: 1..%d experts (got %d)", GM_MAX_E,
             n_experts);
  SY_REQUIRE(k_dim > 0 && k_dim % 8 == 0, "grouped_gemm: k_dim must be a multiple of 8 (got %d)", k_dim);
  SY_REQUIRE(n_out > 0 && n_out % 8 == 0, "grouped_gemm: n_out must be a multiple of 8 (got %d)", n_out);
  SY_REQUIRE(!(swiglu && scale), "grouped_gemm: swiglu and scale are separate epilogues");
  SY_REQUIRE(dtype == SY_DTYPE_F16 || dtype == SY_DTYPE_BF16, "grouped_gemm: dtype must be f16 or bf16");
  if (rows == 0) return SY_OK;
  SY_REQUIRE(A && B && offsets && C, "grouped_gemm: null pointer");
  SY_REQUIRE(((uintptr_t)A % 16 == 0) && ((uintptr_t)B % 16 == 0), "grouped_gemm: A and B must be 16-byte aligned");
  const uint64_t n_full = (uint64_t)(swiglu ? 2 : 1) * n_out;
  CUtensorMap map;
  int rc = weight_map(&map, B, (uint64_t)n_experts * n_full, (uint64_t)k_dim, dtype);
  if (rc != SY_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return dtype == SY_DTYPE_F16
             ? dispatch_gemm<__half>(map, A, a_rows, offsets, n_experts, n_out, k_dim, swiglu, scale, C, s)
             : dispatch_gemm<__nv_bfloat16>(map, A, a_rows, offsets, n_experts, n_out, k_dim, swiglu, scale, C, s);
}

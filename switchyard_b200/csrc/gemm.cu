// grouped_gemm and grouped_gemv: every expert's slice of the sorted batch on the tcgen05 tensor
// cores. One kernel in two shapes (see Shape below): "gemm" for compute-bound batches, "gemv"
// for decode, where the layer is a stream over expert weights.
//
// Orientation. The weight tile is the MMA's M operand and the token rows are its N operand
// ("C^T = W . X^T"): an instruction multiplies 128 weight rows by up to 128 token rows over 16
// k. That keeps M = 128 full no matter how few rows an expert has, so the same code is a
// weight stream for a handful of rows and a GEMM for thousands; N is rounded up to a multiple
// of 16 per tile. (A CUDA-core weight stream was built first and measured on a B200: float32
// FMA keeps up with HBM3e only below about four rows per expert, 1.2 TB/s at 64 tokens, so the
// decode path streams through the tensor cores too.)
//
// One tile = (expert, a block of token rows, a block of output columns). The grid is
// persistent (one block per SM); tiles are numbered on the device from `offsets` (expert-major,
// an expert's row tiles adjacent so that its weights are read from HBM once and then hit L2)
// and dealt round-robin, so nothing about the batch is read back to the host.
//
// A block is fourteen warps with fixed roles, connected by mbarriers:
//   warp 0      TMA producer: the weight tiles of each k block, 128-byte swizzle;
//   warps 2-9   gather producers: the tile's token rows, picked from the UNSORTED activations
//               through a_rows, 16-byte cp.async copies straight into the same swizzled layout,
//               several k blocks in flight per thread;
//   warp 1      MMA issuer: one thread, tcgen05.mma into one of two accumulator buffers in
//               tensor memory; tcgen05.commit releases the stage / publishes the accumulators;
//   warps 10-13 epilogue: tcgen05.ld of the accumulators (a thread owns one output column and
//               walks the token rows), SwiGLU or router-weight scaling with the 16-bit
//               rounding points, results staged in shared memory and written out as whole
//               128/256-byte row segments (16 bytes per thread; the destination may be a peer
//               GPU). It overlaps the next tile's main loop.
//
// An output element is a sum over k in instruction order that does not depend on which other
// rows share the tile or on the tile's N, so a row's bits are the same on one GPU and inside
// an expert-parallel segment (within one shape; the two shapes are separate modes).
//
// Replaces switchyard/csrc/moe_kernels.cu:159-298 (64x64x32 WMMA tiles, one block per tile,
// tile list built by torch on the host) and l.306-415 (CUDA-core GEMV, one block per expert and
// 32 columns, blocks launched for empty experts too).
#include <cuda.h>

#include <atomic>
#include <mutex>
#include <type_traits>

#include "common.cuh"

namespace sy {

constexpr int GM_ATOM_K = 64;                      // k per swizzle atom: 128-byte rows
constexpr int GM_BM = 128;                         // weight rows per accumulator (UMMA M)
constexpr int GM_GATHER_WARPS = 8;
constexpr int GM_EPI_WARPS = 4;
constexpr int GM_THREADS = (2 + GM_GATHER_WARPS + GM_EPI_WARPS) * 32;
constexpr int GM_MAX_E = 256;
constexpr int GM_RING_BYTES = 192 * 1024;          // shared-memory ring of stages
constexpr int GM_EPI_ROWS = 64;                    // token rows the epilogue stages per pass
constexpr int GM_EPI_BYTES = GM_EPI_ROWS * GM_BM * 2;  // staged output tile: 64 rows x 128 columns
constexpr int GM_SMEM = GM_RING_BYTES + GM_EPI_BYTES + 1024;  // + room to align the ring to 1024
constexpr uint64_t GM_WAIT_NS = 1000000000ull;

// Two shapes of the same kernel.
//   PAIR   (mode "gemm"): 128 token rows per tile, two 128-row weight tiles sharing them (two
//          accumulators), 48 KB stages x 4: the compute-bound shape.
//   !PAIR  (mode "gemv"): 64 token rows per tile, one 128-row weight tile (with SwiGLU: 64 gate
//          rows + 64 up rows of the same columns) over 128 k per stage (two swizzle atoms), so a
//          stage carries the same 32 KB of weights and the same eight MMAs as a PAIR stage, but
//          tiles are half as large and twice as many: less imbalance when every tile is one
//          pass over an expert's weights.
template <bool PAIR> struct Shape {
  static constexpr int BN = PAIR ? 128 : 64;               // token rows per tile (UMMA N max)
  static constexpr int BOX_ROWS = PAIR ? 128 : 64;         // weight rows per TMA box (two boxes per atom)
  static constexpr int KATOMS = PAIR ? 1 : 2;              // 64-wide k atoms per stage
  static constexpr int BK = KATOMS * GM_ATOM_K;            // k per stage
  static constexpr int W_ATOM_BYTES = 2 * BOX_ROWS * 128;  // weight bytes of one atom (both boxes)
  static constexpr int X_ATOM_BYTES = BN * 128;
  static constexpr int W_BYTES = KATOMS * W_ATOM_BYTES;    // weight bytes per stage (32 KB either way)
  static constexpr int X_BYTES = KATOMS * X_ATOM_BYTES;
  static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
  static constexpr int STAGES = GM_RING_BYTES / STAGE_BYTES;
  static constexpr int ACCS = PAIR ? 2 : 1;                // accumulators per tile
  static constexpr int BUF_COLS = ACCS * BN;               // tensor-memory columns per buffer
  static constexpr int TMEM_COLS = 2 * BUF_COLS;           // two buffers: 512 or 128
};

struct Tile {
  int e, cb, row0, nvalid;
};

// Optional per-role cycle accounting (compiled in only with -DSY_PROFILE; used when tuning).
#ifdef SY_PROFILE
__device__ long long g_prof[256][16];
#define SY_PROF_DECL(n) long long n = 0
#define SY_PROF_BEGIN(t) long long t = clock64()
#define SY_PROF_ADD(acc, t) acc += clock64() - t
#define SY_PROF_STORE(slot, v) g_prof[blockIdx.x][slot] = (v)
#else
#define SY_PROF_DECL(n)
#define SY_PROF_BEGIN(t)
#define SY_PROF_ADD(acc, t)
#define SY_PROF_STORE(slot, v)
#endif

// Rows come in ranges [begin, end). Normally an expert has one range: its slice of the sorted
// batch. In an expert-parallel mailbox an expert has `ranges_per_expert` of them, one per
// sender, and its tile rows are their concatenation: the expert's weights are streamed once for
// all senders. Tile t of the device-side numbering belongs to expert e (weights B[e]) and covers
// rows [r0, r0 + nvalid) of that concatenation; `cursor` walks the experts monotonically.
template <int BN>
__device__ __forceinline__ Tile locate_tile(int t, int& cursor, const int* tile_start, const int* expert_rows) {
  while (tile_start[cursor + 1] <= t) ++cursor;
  const int e = cursor, local = t - tile_start[e];
  const int n = expert_rows[e], row_tiles = (n + BN - 1) / BN;
  Tile tile;
  tile.e = e;
  tile.cb = local / row_tiles;
  tile.row0 = (local % row_tiles) * BN;
  tile.nvalid = min(BN, n - tile.row0);
  return tile;
}

// Row r of expert e's concatenated ranges: the range it falls in (g) and its row in A / C space.
__device__ __forceinline__ int map_row(int e, int r, int ranges_per_expert, const int* begin, const int* end, int& g) {
  g = e * ranges_per_expert;
  for (int len = end[g] - begin[g]; r >= len; len = end[g] - begin[g]) {
    r -= len;
    ++g;
  }
  return begin[g] + r;
}

template <typename T, bool SWIGLU, bool SCALE, bool PAIR>
__global__ void __launch_bounds__(GM_THREADS, 1)
gemm_umma_kernel(const __grid_constant__ CUtensorMap w_map, const T* __restrict__ A,
                 const int* __restrict__ a_rows, const int* __restrict__ begins, const int* __restrict__ ends, int E,
                 int group_div, int Nout, int K, const T* __restrict__ scale, T* __restrict__ C,
                 const unsigned long long* __restrict__ c_table, int* status) {
  using S = Shape<PAIR>;
  constexpr int BN = S::BN, STAGES = S::STAGES, STAGE_BYTES = S::STAGE_BYTES;
  // output columns per tile
  constexpr int COLS = SWIGLU ? (PAIR ? GM_BM : GM_BM / 2) : (PAIR ? 2 * GM_BM : GM_BM);
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t acc_full[2];
  __shared__ __align__(8) uint64_t acc_empty[2];
  __shared__ uint32_t s_tmem;
  __shared__ int s_begin[GM_MAX_E];       // row ranges
  __shared__ int s_end[GM_MAX_E];
  __shared__ int s_rows[GM_MAX_E];        // rows per expert (all its ranges)
  __shared__ int s_map_row[2][GM_BM];     // per accumulator buffer: the tile's rows in A / C space
  __shared__ int s_map_grp[2][GM_BM];     // ... and the range each row belongs to
  __shared__ int s_tile_start[GM_MAX_E + 2];
  __shared__ float s_xch[2][GM_BM / 2][9];  // up-projection values handed to the gate warps (!PAIR SwiGLU)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  unsigned char* stages =
      reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* out_tile = stages + GM_RING_BYTES;  // the epilogue's staged output rows

  const int col_blocks = (Nout + COLS - 1) / COLS;
  const int Nfull = SWIGLU ? 2 * Nout : Nout;
  const int k_blocks = (K + S::BK - 1) / S::BK;

  // Set-up that touches none of the kernel's inputs comes first, so that under programmatic
  // dependent launch it overlaps the tail of the previous kernel.
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
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
  if (warp == 1) {
    tmem_alloc(&s_tmem, S::TMEM_COLS);
    tmem_relinquish();
  }
  pdl_wait();  // row ranges, activations, scale: all written by earlier kernels
  for (int i = threadIdx.x; i < E; i += GM_THREADS) {
    const int b = begins[i], e = ends[i];
    s_begin[i] = b;
    s_end[i] = e > b ? e : b;
  }
  __syncthreads();
  const int EL = E / group_div;  // experts; E counts row ranges
  if (warp == 0) {  // rows per expert and the exclusive prefix of tiles per expert
    int carry = 0;
    for (int base = 0; base < EL; base += 32) {
      int e = base + lane;
      int n = 0;
      if (e < EL)
        for (int g = e * group_div; g < (e + 1) * group_div; ++g) n += s_end[g] - s_begin[g];
      if (e < EL) s_rows[e] = n;
      int tiles = ((n + BN - 1) / BN) * col_blocks, inc = tiles;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int y = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += y;
      }
      if (e < EL) s_tile_start[e] = carry + inc - tiles;
      carry += __shfl_sync(0xffffffffu, inc, 31);
    }
    if (lane == 0) {
      s_tile_start[EL] = carry;
      s_tile_start[EL + 1] = 0x7fffffff;  // sentinel: the cursor never walks past the last expert
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = s_tmem;
  const int total_tiles = s_tile_start[EL];

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int it = 0, cursor = 0;
      bool alive = true;
      SY_PROF_DECL(w_empty);
      SY_PROF_BEGIN(t_role);
      for (int t = blockIdx.x; t < total_tiles && alive; t += gridDim.x) {
        const Tile tile = locate_tile<BN>(t, cursor, s_tile_start, s_rows);
        const int y0 = tile.e * Nfull + tile.cb * COLS;
        const int y1 = SWIGLU ? y0 + Nout : y0 + S::BOX_ROWS;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES, use = it / STAGES;
          SY_PROF_BEGIN(t_w);
          if (use > 0 && !mbar_wait(&empty_bar[s], (use - 1) & 1, GM_WAIT_NS)) {
            *status = DS_TIMEOUT_EMPTY;
            alive = false;
            break;
          }
          SY_PROF_ADD(w_empty, t_w);
          unsigned char* st = stages + (size_t)s * STAGE_BYTES;
          mbar_arrive_expect_tx(&full_bar[s], S::W_BYTES);
#pragma unroll
          for (int a = 0; a < S::KATOMS; ++a) {
            const int kx = kb * S::BK + a * GM_ATOM_K;
            tma_load_2d(st + a * S::W_ATOM_BYTES, &w_map, kx, y0, &full_bar[s]);
            tma_load_2d(st + a * S::W_ATOM_BYTES + S::BOX_ROWS * 128, &w_map, kx, y1, &full_bar[s]);
          }
        }
      }
      SY_PROF_STORE(0, w_empty);
      SY_PROF_STORE(1, clock64() - t_role);
      if (!alive)  // let the copies already issued land before the block can exit
        for (int j = it > STAGES ? it - STAGES : 0; j < it; ++j)
          mbar_wait(&full_bar[j % STAGES], (j / STAGES) & 1, 10000000ull);
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const int fmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
      const uint32_t ring_lo = umma_desc_lo(smem_u32(stages));
      int it = 0, cursor = 0, tile_no = 0;
      bool alive = true;
      SY_PROF_DECL(w_full);
      SY_PROF_DECL(w_acc);
      SY_PROF_BEGIN(t_role);
      for (int t = blockIdx.x; t < total_tiles && alive; t += gridDim.x, ++tile_no) {
        const Tile tile = locate_tile<BN>(t, cursor, s_tile_start, s_rows);
        const int buf = tile_no & 1, use_t = tile_no >> 1;
        if (use_t > 0) {
          SY_PROF_BEGIN(t_w);
          if (!mbar_wait(&acc_empty[buf], (use_t - 1) & 1, GM_WAIT_NS)) {
            *status = DS_TIMEOUT_TMEM;
            alive = false;
            break;
          }
          SY_PROF_ADD(w_acc, t_w);
          tc_fence_after_sync();
        }
        const int n_mma = max(16, (tile.nvalid + 15) & ~15);
        const uint32_t idesc = umma_idesc(fmt, GM_BM, n_mma);
        const uint32_t d0 = tmem + buf * S::BUF_COLS, d1 = d0 + BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          SY_PROF_BEGIN(t_w);
          if (!mbar_wait(&full_bar[s], (it / STAGES) & 1, GM_WAIT_NS)) {
            *status = DS_TIMEOUT_FULL;
            alive = false;
            break;
          }
          SY_PROF_ADD(w_full, t_w);
          tc_fence_after_sync();
          const uint32_t lo = ring_lo + s * (STAGE_BYTES >> 4);  // descriptor low word of the stage's first tile
#pragma unroll
          for (int ks = 0; ks < S::BK / 16; ++ks) {
            const uint32_t accumulate = (kb | ks) != 0;
            const int atom = ks >> 2, within = (ks & 3) * 2;  // 32 bytes per 16 k inside the 128-byte atom
            const uint32_t a_lo = lo + atom * (S::W_ATOM_BYTES >> 4) + within;
            const uint32_t b_lo = lo + (S::W_BYTES >> 4) + atom * (S::X_ATOM_BYTES >> 4) + within;
            umma_f16_lohi(d0, a_lo, b_lo, UMMA_DESC_HI_K_SW128, idesc, accumulate);
            if (PAIR) umma_f16_lohi(d1, a_lo + (S::BOX_ROWS * 128 >> 4), b_lo, UMMA_DESC_HI_K_SW128, idesc, accumulate);
          }
          umma_commit(&empty_bar[s]);  // the stage is free once these MMAs have read it
        }
        if (alive) umma_commit(&acc_full[buf]);
      }
      SY_PROF_STORE(2, w_full);
      SY_PROF_STORE(3, w_acc);
      SY_PROF_STORE(4, clock64() - t_role);
      SY_PROF_STORE(5, (long long)it);
    }
  } else if (warp < 2 + GM_GATHER_WARPS) {
    // ---------------------------------------------------------------- gather producers
    // 16-byte asynchronous copies straight into the swizzled stage, DEPTH k blocks in flight
    // per thread (commit groups), so that the L2 round trip of a gathered row is overlapped
    // with the stages before it. A stage is published (proxy fence, then one arrive per warp)
    // once the group that filled it has landed; filling runs ahead across tile boundaries.
    constexpr int CHUNKS = S::BK / 8;                 // 16-byte chunks per token row per stage
    constexpr int ROWS_PER_PASS = GM_GATHER_WARPS * 32 / CHUNKS;
    constexpr int GI = BN / ROWS_PER_PASS;
    constexpr int DEPTH = STAGES - 1;
    const int g = threadIdx.x - 64;
    const int c = g % CHUNKS, rsub = g / CHUNKS;      // chunk of the row; row within a pass
    const int xoff = (c >> 3) * S::X_ATOM_BYTES;      // the atom the chunk belongs to
    const int cc = c & 7;
    int issued = 0, published = 0, cursor = 0;
    bool alive = true;
    SY_PROF_DECL(w_empty);
    SY_PROF_DECL(w_group);
    SY_PROF_DECL(w_rows);
    SY_PROF_BEGIN(t_role);
    for (int t = blockIdx.x; t < total_tiles && alive; t += gridDim.x) {
      const Tile tile = locate_tile<BN>(t, cursor, s_tile_start, s_rows);
      const T* src[GI];
      SY_PROF_BEGIN(t_r);
#pragma unroll
      for (int i = 0; i < GI; ++i) {
        const int r = rsub + ROWS_PER_PASS * i;
        src[i] = nullptr;
        if (r < tile.nvalid) {
          int g;
          const int at = map_row(tile.e, tile.row0 + r, group_div, s_begin, s_end, g);
          const int row = a_rows ? a_rows[at] : at;
          src[i] = A + (size_t)row * K + c * 8;
        }
      }
      SY_PROF_ADD(w_rows, t_r);
      for (int kb = 0; kb < k_blocks; ++kb) {
        const int s = issued % STAGES, use = issued / STAGES;
        SY_PROF_BEGIN(t_w);
        if (use > 0 && !mbar_wait(&empty_bar[s], (use - 1) & 1, GM_WAIT_NS)) {
          *status = DS_TIMEOUT_EMPTY;
          alive = false;
          break;
        }
        SY_PROF_ADD(w_empty, t_w);
        unsigned char* x = stages + (size_t)s * STAGE_BYTES + S::W_BYTES + xoff;
        const uint32_t bytes = kb * S::BK + c * 8 < K ? 16u : 0u;  // beyond K: zero fill
#pragma unroll
        for (int i = 0; i < GI; ++i) {
          const int r = rsub + ROWS_PER_PASS * i;
          if (src[i]) cp_async_16(x + r * 128 + ((cc ^ (r & 7)) << 4), bytes ? src[i] + (size_t)kb * S::BK : src[i], bytes);
        }
        cp_async_commit();
        ++issued;
        if (issued - published > DEPTH) {
          SY_PROF_BEGIN(t_g);
          cp_async_wait<DEPTH>();
          SY_PROF_ADD(w_group, t_g);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&full_bar[published % STAGES]);
          ++published;
        }
      }
    }
    if (threadIdx.x == 64) {
      SY_PROF_STORE(6, w_empty);
      SY_PROF_STORE(7, w_group);
      SY_PROF_STORE(8, w_rows);
      SY_PROF_STORE(9, clock64() - t_role);
    }
    cp_async_wait<0>();
    fence_proxy_async_smem();
    __syncwarp();
    for (; published < issued; ++published)
      if (lane == 0) mbar_arrive(&full_bar[published % STAGES]);
  } else {
    // ---------------------------------------------------------------- epilogue
    // A warp that gives up on a wait keeps walking the tiles (the exchange barrier below must
    // still see all four warps) but skips every wait, load and store.
    const int q = warp & 3;  // the quarter of tensor memory's lanes this warp may read
    int cursor = 0, tile_no = 0, chunk_no = 0;
    bool alive = true;
    SY_PROF_DECL(w_accf);
    SY_PROF_BEGIN(t_role);
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++tile_no) {
      const Tile tile = locate_tile<BN>(t, cursor, s_tile_start, s_rows);
      const int buf = tile_no & 1, use_t = tile_no >> 1;
      SY_PROF_BEGIN(t_w);
      if (alive && !mbar_wait(&acc_full[buf], use_t & 1, GM_WAIT_NS)) {
        *status = DS_TIMEOUT_MMA;
        alive = false;
      }
      SY_PROF_ADD(w_accf, t_w);
      tc_fence_after_sync();
      const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16) + buf * S::BUF_COLS;
      const int wrow = q * 32 + lane;
      const int et = threadIdx.x - (2 + GM_GATHER_WARPS) * 32;  // 0..127 among the epilogue threads
      // the tile's rows in A / C space (and the range of each), once per tile for all four warps
      int* map_row_s = s_map_row[buf];
      int* map_grp_s = s_map_grp[buf];
      if (et < tile.nvalid) {
        int g;
        map_row_s[et] = map_row(tile.e, tile.row0 + et, group_div, s_begin, s_end, g);
        map_grp_s[et] = g;
      }
      named_barrier_sync(3, GM_EPI_WARPS * 32);
      if (!c_table) {
        // Local destination: every thread stores its own column's values directly (2 bytes per
        // store, a warp covers 64 contiguous bytes of a row); L2 merges them, and the epilogue
        // stays short enough to hide behind the next tile's main loop.
        if (PAIR || !SWIGLU) {
          const int col0 = tile.cb * COLS + wrow;
          const int col1 = col0 + GM_BM;  // the second accumulator's column (PAIR without SwiGLU)
          for (int n0 = 0; n0 < tile.nvalid && alive; n0 += 8) {
            uint32_t v0[8], v1[8];
            tmem_ld_x8(taddr + n0, v0);
            if (PAIR) tmem_ld_x8(taddr + BN + n0, v1);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (n0 + j < tile.nvalid) {
                const int row = map_row_s[n0 + j];
                const float f0 = __uint_as_float(v0[j]), f1 = PAIR ? __uint_as_float(v1[j]) : 0.f;
                if (SWIGLU) {
                  if (col0 < Nout) C[(size_t)row * Nout + col0] = epilogue_swiglu<T>(f0, f1);
                } else if (SCALE) {
                  const T sc = scale[row];
                  if (col0 < Nout) C[(size_t)row * Nout + col0] = epilogue_scale<T>(f0, sc);
                  if (PAIR && col1 < Nout) C[(size_t)row * Nout + col1] = epilogue_scale<T>(f1, sc);
                } else {
                  if (col0 < Nout) C[(size_t)row * Nout + col0] = Elem<T>::from_f(f0);
                  if (PAIR && col1 < Nout) C[(size_t)row * Nout + col1] = Elem<T>::from_f(f1);
                }
              }
            }
          }
        } else {
          // one accumulator: lanes 0-63 hold the gate rows, lanes 64-127 the up rows of the same
          // 64 output columns. Warps 2,3 pass their values to warps 0,1 through shared memory.
          const int j64 = wrow & 63;
          const int col = tile.cb * COLS + j64;
          for (int n0 = 0; n0 < tile.nvalid; n0 += 8, ++chunk_no) {
            uint32_t v[8];
            if (alive) {
              tmem_ld_x8(taddr + n0, v);
              tmem_ld_wait();
            }
            float* slot = s_xch[chunk_no & 1][j64];
            if (q >= 2 && alive) {
#pragma unroll
              for (int j = 0; j < 8; ++j) slot[j] = __uint_as_float(v[j]);
            }
            named_barrier_sync(2, GM_EPI_WARPS * 32);
            if (q < 2 && alive) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                if (n0 + j < tile.nvalid && col < Nout)
                  C[(size_t)map_row_s[n0 + j] * Nout + col] = epilogue_swiglu<T>(__uint_as_float(v[j]), slot[j]);
              }
            }
          }
        }
      } else {
        // Destination given by c_table (usually a peer GPU): results go through a shared-memory
        // tile so that memory is written in 16-byte pieces, a whole 128- or 256-byte row segment
        // per group of threads, instead of one 2-byte store per thread (NVLink carries small
        // stores poorly): up to GM_EPI_ROWS token rows x OC output columns per pass.
        constexpr int OC = SWIGLU && !PAIR ? GM_BM / 2 : GM_BM;   // output columns per pass
        constexpr int ORB = OC * 2;                               // bytes per staged row
        constexpr int TPR = ORB / 16;                             // threads per row when copying out
        constexpr int STORE_ACCS = (PAIR && !SWIGLU) ? 2 : 1;
#pragma unroll 1
        for (int acc = 0; acc < STORE_ACCS; ++acc) {
#pragma unroll 1
          for (int nb = 0; nb < tile.nvalid; nb += GM_EPI_ROWS) {
            const int nrows = min(GM_EPI_ROWS, tile.nvalid - nb);
            // ---- phase 1: tensor memory -> registers -> epilogue arithmetic -> staged tile
            if (PAIR || !SWIGLU) {
              for (int n0 = nb; n0 < nb + nrows; n0 += 8) {
                uint32_t v0[8], v1[8];
                if (alive) {
                  tmem_ld_x8(taddr + acc * BN + n0, v0);
                  if (SWIGLU) tmem_ld_x8(taddr + BN + n0, v1);
                  tmem_ld_wait();
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  if (alive && n0 + j < tile.nvalid) {
                    const float f0 = __uint_as_float(v0[j]);
                    T o;
                    if (SWIGLU) o = epilogue_swiglu<T>(f0, __uint_as_float(v1[j]));
                    else if (SCALE) o = epilogue_scale<T>(f0, scale[map_row_s[n0 + j]]);
                    else o = Elem<T>::from_f(f0);
                    *reinterpret_cast<T*>(out_tile + (n0 + j - nb) * ORB + wrow * 2) = o;
                  }
                }
              }
            } else {
              // one accumulator: lanes 0-63 hold the gate rows, lanes 64-127 the up rows of the
              // same 64 output columns. Warps 2,3 pass their values to warps 0,1 through shared
              // memory (double-buffered by chunk, one barrier per chunk).
              const int j64 = wrow & 63;
              for (int n0 = nb; n0 < nb + nrows; n0 += 8, ++chunk_no) {
                uint32_t v[8];
                if (alive) {
                  tmem_ld_x8(taddr + n0, v);
                  tmem_ld_wait();
                }
                float* slot = s_xch[chunk_no & 1][j64];
                if (q >= 2 && alive) {
#pragma unroll
                  for (int j = 0; j < 8; ++j) slot[j] = __uint_as_float(v[j]);
                }
                named_barrier_sync(2, GM_EPI_WARPS * 32);
                if (q < 2 && alive) {
#pragma unroll
                  for (int j = 0; j < 8; ++j)
                    if (n0 + j < tile.nvalid)
                      *reinterpret_cast<T*>(out_tile + (n0 + j - nb) * ORB + j64 * 2) =
                          epilogue_swiglu<T>(__uint_as_float(v[j]), slot[j]);
                }
              }
            }
            named_barrier_sync(3, GM_EPI_WARPS * 32);
            // ---- phase 2: staged tile -> memory, 16 bytes per thread, whole row segments
            const int col = tile.cb * COLS + acc * GM_BM + (et % TPR) * 8;
            if (alive && col < Nout) {
              for (int r = et / TPR; r < nrows; r += GM_EPI_WARPS * 32 / TPR) {
                // c_table[g] is where row s_begin[g] of range g lands
                const int g = map_grp_s[nb + r];
                T* dst = reinterpret_cast<T*>(c_table[g]) + (size_t)(map_row_s[nb + r] - s_begin[g]) * Nout + col;
                *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(out_tile + r * ORB + (et % TPR) * 16);
              }
            }
            named_barrier_sync(3, GM_EPI_WARPS * 32);
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0 && alive) mbar_arrive(&acc_empty[buf]);
    }
    if (threadIdx.x == 320) {
      SY_PROF_STORE(10, w_accf);
      SY_PROF_STORE(11, clock64() - t_role);
    }
  }

  // every role ends here; tensor memory goes back before the block exits
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, S::TMEM_COLS);
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

// Tensor map over the stacked expert weights as a [rows, K] matrix; box = box_rows x 64 k.
static int weight_map(CUtensorMap* map, const void* B, uint64_t rows, uint64_t K, int dtype, int box_rows) {
  EncodeTiledFn encode;
  int rc = encode_fn(&encode);
  if (rc != SY_OK) return rc;
  cuuint64_t dims[2] = {K, rows};
  cuuint64_t strides[1] = {K * 2};
  cuuint32_t box[2] = {GM_ATOM_K, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = encode(map, dtype == SY_DTYPE_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                      2, const_cast<void*>(B), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(SY_ERR_CUDA, "grouped_gemm: cuTensorMapEncodeTiled failed (%d)", (int)r);
  return SY_OK;
}

struct GroupedArgs {
  const void* A;
  const int32_t* a_rows;
  const void* B;
  const int32_t* begins;   // [groups] first row of each group
  const int32_t* ends;     // [groups] one past its last row
  int groups;              // number of row ranges (experts x ranges per expert)
  int group_div;           // ranges per expert: ranges [e*group_div, (e+1)*group_div) are expert e's rows
  int n_out, k_dim;
  const void* scale;
  void* C;
  const unsigned long long* c_table;  // optional per-group output row pointers
  int dtype;
  cudaStream_t stream;
};

template <typename T, bool SWIGLU, bool SCALE, bool PAIR>
static int launch_gemm(const GroupedArgs& a) {
  int sms = 0;
  int rc = device_sm_count(&sms);
  if (rc != SY_OK) return rc;
  int* status = device_status_word();
  if (!status) return SY_ERR_CUDA;
  CUtensorMap map;
  rc = weight_map(&map, a.B, (uint64_t)(a.groups / a.group_div) * (SWIGLU ? 2 : 1) * a.n_out, (uint64_t)a.k_dim,
                  a.dtype, Shape<PAIR>::BOX_ROWS);
  if (rc != SY_OK) return rc;
  auto kern = gemm_umma_kernel<T, SWIGLU, SCALE, PAIR>;
  static std::atomic<int> configured[MAX_DEVICES];
  int dev = 0;
  SY_CUDA(cudaGetDevice(&dev));
  if (!configured[dev].load(std::memory_order_acquire)) {
    SY_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GM_SMEM));
    configured[dev].store(1, std::memory_order_release);
  }
  return launch_kernel(kern, sms, GM_THREADS, GM_SMEM, a.stream, "grouped tcgen05 launch", map,
                       static_cast<const T*>(a.A), a.a_rows, a.begins, a.ends, a.groups, a.group_div, a.n_out, a.k_dim,
                       static_cast<const T*>(a.scale), static_cast<T*>(a.C), a.c_table, status);
}

template <typename T, bool PAIR>
static int dispatch_gemm(const GroupedArgs& a, int swiglu) {
  if (swiglu) return launch_gemm<T, true, false, PAIR>(a);
  if (a.scale) return launch_gemm<T, false, true, PAIR>(a);
  return launch_gemm<T, false, false, PAIR>(a);
}

// Shared argument checks and dtype dispatch of the tensor-core entry points.
int grouped_umma(bool pair, const char* name, const GroupedArgs& a, int rows, int swiglu) {
  SY_REQUIRE(rows >= 0 && a.groups >= 1 && a.groups <= GM_MAX_E, "%s: 1..%d groups (got %d)", name, GM_MAX_E, a.groups);
  SY_REQUIRE(a.group_div >= 1 && a.groups % a.group_div == 0, "%s: %d groups do not divide by %d", name, a.groups,
             a.group_div);
  SY_REQUIRE(a.k_dim > 0 && a.k_dim % 8 == 0, "%s: k_dim must be a multiple of 8 (got %d)", name, a.k_dim);
  SY_REQUIRE(a.n_out > 0 && a.n_out % 8 == 0, "%s: n_out must be a multiple of 8 (got %d)", name, a.n_out);
  SY_REQUIRE(!(swiglu && a.scale), "%s: swiglu and scale are separate epilogues", name);
  SY_REQUIRE(a.dtype == SY_DTYPE_F16 || a.dtype == SY_DTYPE_BF16, "%s: dtype must be f16 or bf16", name);
  if (rows == 0) return SY_OK;
  SY_REQUIRE(a.A && a.B && a.begins && a.ends && (a.C || a.c_table), "%s: null pointer", name);
  SY_REQUIRE(((uintptr_t)a.A % 16 == 0) && ((uintptr_t)a.B % 16 == 0) && ((uintptr_t)a.C % 16 == 0),
             "%s: A, B and C must be 16-byte aligned", name);
  if (a.dtype == SY_DTYPE_F16) return pair ? dispatch_gemm<__half, true>(a, swiglu) : dispatch_gemm<__half, false>(a, swiglu);
  return pair ? dispatch_gemm<__nv_bfloat16, true>(a, swiglu) : dispatch_gemm<__nv_bfloat16, false>(a, swiglu);
}

}  // namespace sy

#ifdef SY_PROFILE
extern "C" int sy_prof_read(long long* out, int blocks) {
  return sy::check_cuda(cudaMemcpyFromSymbol(out, sy::g_prof, sizeof(long long) * 16 * blocks), "prof read");
}
#endif

extern "C" int sy_grouped_gemm(const void* A, const int32_t* a_rows, const void* B, const int32_t* offsets,
                               int n_experts, int rows, int n_out, int k_dim, int swiglu, const void* scale, void* C,
                               int dtype, void* stream) {
  sy::GroupedArgs a{A, a_rows, B, offsets, offsets ? offsets + 1 : nullptr, n_experts, 1, n_out, k_dim,
                    scale, C, nullptr, dtype, static_cast<cudaStream_t>(stream)};
  return sy::grouped_umma(true, "grouped_gemm", a, rows, swiglu);
}

extern "C" int sy_grouped_gemv(const void* A, const int32_t* a_rows, const void* B, const int32_t* offsets,
                               int n_experts, int rows, int n_out, int k_dim, int swiglu, const void* scale, void* C,
                               int dtype, void* stream) {
  sy::GroupedArgs a{A, a_rows, B, offsets, offsets ? offsets + 1 : nullptr, n_experts, 1, n_out, k_dim,
                    scale, C, nullptr, dtype, static_cast<cudaStream_t>(stream)};
  return sy::grouped_umma(false, "grouped_gemv", a, rows, swiglu);
}

extern "C" int sy_grouped_segments(const void* A, const void* B, const int32_t* begins, const int32_t* ends,
                                   int n_groups, int groups_per_expert, int rows_bound, int n_out, int k_dim, int swiglu,
                                   const void* scale, void* C, const uint64_t* c_table, int dtype, int compute_shape,
                                   void* stream) {
  sy::GroupedArgs a{A, nullptr, B, begins, ends, n_groups, groups_per_expert, n_out, k_dim, scale, C,
                    reinterpret_cast<const unsigned long long*>(c_table), dtype, static_cast<cudaStream_t>(stream)};
  return sy::grouped_umma(compute_shape != 0, "grouped_segments", a, rows_bound, swiglu);
}

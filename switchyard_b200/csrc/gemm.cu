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
#include <string.h>
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
  int phase, e, cb, row0, nvalid;
};

// One contraction over the row ranges: activations A (optionally gathered through a_rows),
// expert weights behind `map`, an epilogue, a destination. The fused expert FFN is two of them
// (gate/up with SwiGLU, then down with the router-weight scale) run by ONE launch.
struct Problem {
  CUtensorMap map;                       // [experts * n_full, K] weights, box 64 k x BOX_ROWS
  const void* A;
  const int* a_rows;
  const void* scale;
  void* C;
  const unsigned long long* c_table;     // optional per-range output row pointers
  int Nout, K, swiglu, pad_;
};

struct KernelArgs {
  Problem p[2];
  const int* begins;                     // [ranges]
  const int* ends;
  int ranges, group_div;                 // expert e owns ranges [e*group_div, (e+1)*group_div)
  int n_problems;                        // 1, or 2 = fused FFN: p[1] reads what p[0] wrote
  int* ready;                            // fused only: [experts] finished p[0] tiles, then [1] block counter
  int* status;
};

// Rows come in ranges [begin, end). Normally an expert has one range: its slice of the sorted
// batch. In an expert-parallel mailbox an expert has `group_div` of them, one per sender, and
// its tile rows are their concatenation: the expert's weights are streamed once for all
// senders. Tiles are numbered problem by problem, expert-major inside a problem; `cursor` walks
// the experts monotonically within a problem.
template <int BN>
__device__ __forceinline__ Tile locate_tile(int t, int tiles0, int& seen, int& cursor,
                                            const int (*tile_start)[GM_MAX_E + 2], const int* expert_rows) {
  const int phase = t >= tiles0 ? 1 : 0;
  if (phase != seen) {
    seen = phase;
    cursor = 0;
  }
  const int tl = t - (phase ? tiles0 : 0);
  const int* start = tile_start[phase];
  while (start[cursor + 1] <= tl) ++cursor;
  const int e = cursor, local = tl - start[e];
  const int n = expert_rows[e], row_tiles = (n + BN - 1) / BN;
  Tile tile;
  tile.phase = phase;
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

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// The epilogue of one tile, specialised on the epilogue kind so that its inner loops carry no
// run-time switches: accumulators -> SwiGLU / router-weight scale / plain rounding -> memory.
template <typename T, bool PAIR, bool SWIGLU, bool SCALE>
__device__ __forceinline__ void epilogue_tile(const Tile& tile, int buf, uint32_t tmem, int q, int lane, int et, bool alive,
                                              int& chunk_no, int Nout, int COLS, const T* __restrict__ scale,
                                              T* __restrict__ C, const unsigned long long* __restrict__ c_table,
                                              int group_div, const int* s_begin, const int* s_end, int* map_row_s,
                                              int* map_grp_s, float (*s_xch)[GM_BM / 2][9], unsigned char* out_tile) {
  using S = Shape<PAIR>;
  constexpr int BN = S::BN;
  const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16) + buf * S::BUF_COLS;
  const int wrow = q * 32 + lane;
  // With several ranges per expert the tile's rows in A / C space (and the range of each) are
  // looked up once per tile for all four warps; with one range they are consecutive.
  const bool mapped = group_div > 1;
  const int row_base = s_begin[tile.e * group_div] + tile.row0;
  if (mapped) {
    if (et < tile.nvalid) {
      int gr;
      map_row_s[et] = map_row(tile.e, tile.row0 + et, group_div, s_begin, s_end, gr);
      map_grp_s[et] = gr;
    }
    named_barrier_sync(3, GM_EPI_WARPS * 32);
  }
  constexpr bool exchange = !PAIR && SWIGLU;  // one accumulator: gate rows in lanes 0-63, up rows in 64-127
  if (!c_table) {
    // Local destination: every thread stores its own column's values directly (2 bytes per
    // store, a warp covers 64 contiguous bytes of a row); L2 merges them, and the epilogue
    // stays short enough to hide behind the next tile's main loop.
    if (!exchange) {
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
            const int row = mapped ? map_row_s[n0 + j] : row_base + n0 + j;
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
      // Warps 2,3 (up rows) pass their values to warps 0,1 (gate rows) through shared memory.
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
              C[(size_t)(mapped ? map_row_s[n0 + j] : row_base + n0 + j) * Nout + col] =
                  epilogue_swiglu<T>(__uint_as_float(v[j]), slot[j]);
          }
        }
      }
    }
  } else {
    // Destination given by c_table (usually a peer GPU): results go through a shared-memory
    // tile so that memory is written in 16-byte pieces, a whole 128- or 256-byte row segment
    // per group of threads, instead of one 2-byte store per thread (NVLink carries small
    // stores poorly): up to GM_EPI_ROWS token rows x OC output columns per pass.
    constexpr int OC = exchange ? GM_BM / 2 : GM_BM;  // output columns per pass
    constexpr int ORB = OC * 2;                       // bytes per staged row
    constexpr int TPR = ORB / 16;                     // threads per row when copying out
    constexpr int store_accs = (PAIR && !SWIGLU) ? 2 : 1;
#pragma unroll 1
    for (int acc = 0; acc < store_accs; ++acc) {
#pragma unroll 1
      for (int nb = 0; nb < tile.nvalid; nb += GM_EPI_ROWS) {
        const int nrows = min(GM_EPI_ROWS, tile.nvalid - nb);
        // ---- phase 1: tensor memory -> registers -> epilogue arithmetic -> staged tile
        if (!exchange) {
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
                else if (SCALE) o = epilogue_scale<T>(f0, scale[mapped ? map_row_s[n0 + j] : row_base + n0 + j]);
                else o = Elem<T>::from_f(f0);
                *reinterpret_cast<T*>(out_tile + (n0 + j - nb) * ORB + wrow * 2) = o;
              }
            }
          }
        } else {
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
            const int gr = mapped ? map_grp_s[nb + r] : tile.e;
            const int row = mapped ? map_row_s[nb + r] : row_base + nb + r;
            T* dst = reinterpret_cast<T*>(c_table[gr]) + (size_t)(row - s_begin[gr]) * Nout + col;
            *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(out_tile + r * ORB + (et % TPR) * 16);
          }
        }
        named_barrier_sync(3, GM_EPI_WARPS * 32);
      }
    }
  }
}

template <typename T, bool PAIR>
__global__ void __launch_bounds__(GM_THREADS, 1) gemm_umma_kernel(const __grid_constant__ KernelArgs args) {
  using S = Shape<PAIR>;
  constexpr int BN = S::BN, STAGES = S::STAGES, STAGE_BYTES = S::STAGE_BYTES;
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t acc_full[2];
  __shared__ __align__(8) uint64_t acc_empty[2];
  __shared__ uint32_t s_tmem;
  __shared__ int s_begin[GM_MAX_E];       // row ranges
  __shared__ int s_end[GM_MAX_E];
  __shared__ int s_rows[GM_MAX_E];        // rows per expert (all its ranges)
  __shared__ int s_tile_start[2][GM_MAX_E + 2];
  __shared__ int s_map_row[2][GM_BM];     // per accumulator buffer: the tile's rows in A / C space
  __shared__ int s_map_grp[2][GM_BM];     // ... and the range each row belongs to
  __shared__ float s_xch[2][GM_BM / 2][9];  // up-projection values handed to the gate warps (!PAIR SwiGLU)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  unsigned char* stages =
      reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* out_tile = stages + GM_RING_BYTES;  // the epilogue's staged output rows
  int* status = args.status;
  const int E = args.ranges, group_div = args.group_div, NP = args.n_problems;
  const int EL = E / group_div;  // experts; E counts row ranges

  // per-problem tile geometry
  auto cols_of = [&](int ph) {
    return args.p[ph].swiglu ? (PAIR ? GM_BM : GM_BM / 2) : (PAIR ? 2 * GM_BM : GM_BM);
  };
  auto col_blocks_of = [&](int ph) { return (args.p[ph].Nout + cols_of(ph) - 1) / cols_of(ph); };
  auto k_blocks_of = [&](int ph) { return (args.p[ph].K + S::BK - 1) / S::BK; };

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
    prefetch_tensormap(&args.p[0].map);
    if (NP > 1) prefetch_tensormap(&args.p[1].map);
  }
  if (warp == 1) {
    tmem_alloc(&s_tmem, S::TMEM_COLS);
    tmem_relinquish();
  }
  pdl_wait();  // row ranges, activations, scale: all written by earlier kernels
  for (int i = threadIdx.x; i < E; i += GM_THREADS) {
    const int b = args.begins[i], e = args.ends[i];
    s_begin[i] = b;
    s_end[i] = e > b ? e : b;
  }
  __syncthreads();
  if (warp == 0) {  // rows per expert and, per problem, the exclusive prefix of tiles per expert
    for (int ph = 0; ph < NP; ++ph) {
      const int col_blocks = col_blocks_of(ph);
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
        if (e < EL) s_tile_start[ph][e] = carry + inc - tiles;
        carry += __shfl_sync(0xffffffffu, inc, 31);
      }
      if (lane == 0) {
        s_tile_start[ph][EL] = carry;
        s_tile_start[ph][EL + 1] = 0x7fffffff;  // sentinel: the cursor never walks past the last expert
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = s_tmem;
  const int tiles0 = s_tile_start[0][EL];
  const int total_tiles = tiles0 + (NP > 1 ? s_tile_start[1][EL] : 0);

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int it = 0, cursor = 0, seen = 0;
      bool alive = true;
      // streaming shape: an expert's weights are read once, so they are marked evict-first in L2
      const uint64_t policy = l2_policy_evict_first();
      for (int t = blockIdx.x; t < total_tiles && alive; t += gridDim.x) {
        const Tile tile = locate_tile<BN>(t, tiles0, seen, cursor, s_tile_start, s_rows);
        const Problem& P = args.p[tile.phase];
        const int Nfull = P.swiglu ? 2 * P.Nout : P.Nout;
        const int y0 = tile.e * Nfull + tile.cb * cols_of(tile.phase);
        const int y1 = P.swiglu ? y0 + P.Nout : y0 + S::BOX_ROWS;
        const int k_blocks = k_blocks_of(tile.phase);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES, use = it / STAGES;
          if (use > 0 && !mbar_wait(&empty_bar[s], (use - 1) & 1, GM_WAIT_NS)) {
            *status = DS_TIMEOUT_EMPTY;
            alive = false;
            break;
          }
          unsigned char* st = stages + (size_t)s * STAGE_BYTES;
          mbar_arrive_expect_tx(&full_bar[s], S::W_BYTES);
#pragma unroll
          for (int a = 0; a < S::KATOMS; ++a) {
            const int kx = kb * S::BK + a * GM_ATOM_K;
            if (PAIR) {
              tma_load_2d(st + a * S::W_ATOM_BYTES, &P.map, kx, y0, &full_bar[s]);
              tma_load_2d(st + a * S::W_ATOM_BYTES + S::BOX_ROWS * 128, &P.map, kx, y1, &full_bar[s]);
            } else {
              tma_load_2d_hint(st + a * S::W_ATOM_BYTES, &P.map, kx, y0, &full_bar[s], policy);
              tma_load_2d_hint(st + a * S::W_ATOM_BYTES + S::BOX_ROWS * 128, &P.map, kx, y1, &full_bar[s], policy);
            }
          }
        }
      }
      if (!alive)  // let the copies already issued land before the block can exit
        for (int j = it > STAGES ? it - STAGES : 0; j < it; ++j)
          mbar_wait(&full_bar[j % STAGES], (j / STAGES) & 1, 10000000ull);
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const int fmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
      const uint32_t ring_lo = umma_desc_lo(smem_u32(stages));
      int it = 0, cursor = 0, seen = 0, tile_no = 0;
      bool alive = true;
      for (int t = blockIdx.x; t < total_tiles && alive; t += gridDim.x, ++tile_no) {
        const Tile tile = locate_tile<BN>(t, tiles0, seen, cursor, s_tile_start, s_rows);
        const int k_blocks = k_blocks_of(tile.phase);
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
        const uint32_t d0 = tmem + buf * S::BUF_COLS, d1 = d0 + BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(&full_bar[s], (it / STAGES) & 1, GM_WAIT_NS)) {
            *status = DS_TIMEOUT_FULL;
            alive = false;
            break;
          }
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
    int issued = 0, published = 0, cursor = 0, seen = 0;
    bool alive = true;
    for (int t = blockIdx.x; t < total_tiles && alive; t += gridDim.x) {
      const Tile tile = locate_tile<BN>(t, tiles0, seen, cursor, s_tile_start, s_rows);
      const Problem& P = args.p[tile.phase];
      const int K = P.K, k_blocks = k_blocks_of(tile.phase);
      if (tile.phase == 1) {
        // fused FFN: this tile reads what the expert's gate/up tiles wrote. Wait (bounded)
        // until all of them have been stored; they sit earlier in every block's tile list.
        const int need = ((s_rows[tile.e] + BN - 1) / BN) * col_blocks_of(0);
        int ok = lane == 0 ? (ld_acquire_gpu(args.ready + tile.e) >= need) : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) {
          // Not there yet. The gate/up tile it waits for may be this block's own, and that tile's
          // last stages are filled but not yet published: publish everything first, then wait.
          cp_async_wait<0>();
          fence_proxy_async_smem();
          __syncwarp();
          for (; published < issued; ++published)
            if (lane == 0) mbar_arrive(&full_bar[published % STAGES]);
          if (lane == 0) {
            const uint64_t start = global_timer_ns();
            while (ld_acquire_gpu(args.ready + tile.e) < need) {
              if (global_timer_ns() - start > GM_WAIT_NS) {
                *status = DS_TIMEOUT_FLAG;
                break;
              }
            }
          }
          __syncwarp();
        }
      }
      const T* A = static_cast<const T*>(P.A);
      const T* src[GI];
#pragma unroll
      for (int i = 0; i < GI; ++i) {
        const int r = rsub + ROWS_PER_PASS * i;
        src[i] = nullptr;
        if (r < tile.nvalid) {
          int gr;
          const int at = map_row(tile.e, tile.row0 + r, group_div, s_begin, s_end, gr);
          const int row = P.a_rows ? P.a_rows[at] : at;
          src[i] = A + (size_t)row * K + c * 8;
        }
      }
      for (int kb = 0; kb < k_blocks; ++kb) {
        const int s = issued % STAGES, use = issued / STAGES;
        if (use > 0 && !mbar_wait(&empty_bar[s], (use - 1) & 1, GM_WAIT_NS)) {
          *status = DS_TIMEOUT_EMPTY;
          alive = false;
          break;
        }
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
          cp_async_wait<DEPTH>();
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&full_bar[published % STAGES]);
          ++published;
        }
      }
    }
    cp_async_wait<0>();
    fence_proxy_async_smem();
    __syncwarp();
    for (; published < issued; ++published)
      if (lane == 0) mbar_arrive(&full_bar[published % STAGES]);
  } else {
    // ---------------------------------------------------------------- epilogue
    // A warp that gives up on a wait keeps walking the tiles (the barriers below must still
    // see all four warps) but skips every wait, load and store.
    const int q = warp & 3;  // the quarter of tensor memory's lanes this warp may read
    const int et = threadIdx.x - (2 + GM_GATHER_WARPS) * 32;  // 0..127 among the epilogue threads
    int cursor = 0, seen = 0, tile_no = 0, chunk_no = 0;
    bool alive = true;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++tile_no) {
      const Tile tile = locate_tile<BN>(t, tiles0, seen, cursor, s_tile_start, s_rows);
      const Problem& P = args.p[tile.phase];
      const int Nout = P.Nout, COLS = cols_of(tile.phase);
      const bool swiglu = P.swiglu != 0;
      const T* scale = static_cast<const T*>(P.scale);
      T* C = static_cast<T*>(P.C);
      const unsigned long long* c_table = P.c_table;
      const int buf = tile_no & 1, use_t = tile_no >> 1;
      if (alive && !mbar_wait(&acc_full[buf], use_t & 1, GM_WAIT_NS)) {
        *status = DS_TIMEOUT_MMA;
        alive = false;
      }
      tc_fence_after_sync();
      if (swiglu)
        epilogue_tile<T, PAIR, true, false>(tile, buf, tmem, q, lane, et, alive, chunk_no, Nout, COLS, scale, C, c_table,
                                            group_div, s_begin, s_end, s_map_row[buf], s_map_grp[buf], s_xch, out_tile);
      else if (scale)
        epilogue_tile<T, PAIR, false, true>(tile, buf, tmem, q, lane, et, alive, chunk_no, Nout, COLS, scale, C, c_table,
                                            group_div, s_begin, s_end, s_map_row[buf], s_map_grp[buf], s_xch, out_tile);
      else
        epilogue_tile<T, PAIR, false, false>(tile, buf, tmem, q, lane, et, alive, chunk_no, Nout, COLS, scale, C, c_table,
                                             group_div, s_begin, s_end, s_map_row[buf], s_map_grp[buf], s_xch, out_tile);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0 && alive) mbar_arrive(&acc_empty[buf]);
      if (NP > 1 && tile.phase == 0) {
        // fused FFN: publish this gate/up tile. All four warps' stores first (barrier), then
        // one thread makes them visible device-wide and counts the tile for its expert.
        named_barrier_sync(3, GM_EPI_WARPS * 32);
        if (et == 0) {
          __threadfence();
          atomicAdd(args.ready + tile.e, 1);
        }
      }
    }
  }

  // every role ends here; tensor memory goes back before the block exits
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, S::TMEM_COLS);
  }
  if (NP > 1 && threadIdx.x == 0) {
    // fused FFN: the last block out clears the per-expert counters for the next launch
    __threadfence();
    if (atomicAdd(args.ready + EL, 1) == (int)gridDim.x - 1) {
      for (int e = 0; e <= EL; ++e) args.ready[e] = 0;
      __threadfence();
    }
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
      return fail(SY_ERR_CUDA, "grouped kernel: the driver does not provide cuTensorMapEncodeTiled");
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
  if (r != CUDA_SUCCESS) return fail(SY_ERR_CUDA, "grouped kernel: cuTensorMapEncodeTiled failed (%d)", (int)r);
  return SY_OK;
}

// One contraction as the entry points describe it.
struct ProblemDesc {
  const void* A;
  const int32_t* a_rows;
  const void* B;
  int n_out, k_dim, swiglu;
  const void* scale;
  void* C;
  const unsigned long long* c_table;
};

struct GroupedArgs {
  ProblemDesc p[2];
  int n_problems;
  const int32_t* begins;   // [ranges] first row of each range
  const int32_t* ends;     // [ranges] one past its last row
  int ranges;              // number of row ranges (experts x ranges per expert)
  int group_div;           // ranges per expert: ranges [e*group_div, (e+1)*group_div) are expert e's rows
  int32_t* ready;          // fused FFN scratch: experts + 1 ints, zero before the first launch
  int dtype;
  cudaStream_t stream;
};

template <typename T, bool PAIR>
static int launch_gemm(const GroupedArgs& a) {
  int sms = 0;
  int rc = device_sm_count(&sms);
  if (rc != SY_OK) return rc;
  KernelArgs k;
  memset(&k, 0, sizeof(k));
  k.status = device_status_word();
  if (!k.status) return SY_ERR_CUDA;
  const int experts = a.ranges / a.group_div;
  for (int i = 0; i < a.n_problems; ++i) {
    const ProblemDesc& d = a.p[i];
    rc = weight_map(&k.p[i].map, d.B, (uint64_t)experts * (d.swiglu ? 2 : 1) * d.n_out, (uint64_t)d.k_dim, a.dtype,
                    Shape<PAIR>::BOX_ROWS);
    if (rc != SY_OK) return rc;
    k.p[i].A = d.A;
    k.p[i].a_rows = d.a_rows;
    k.p[i].scale = d.scale;
    k.p[i].C = d.C;
    k.p[i].c_table = d.c_table;
    k.p[i].Nout = d.n_out;
    k.p[i].K = d.k_dim;
    k.p[i].swiglu = d.swiglu;
  }
  k.begins = a.begins;
  k.ends = a.ends;
  k.ranges = a.ranges;
  k.group_div = a.group_div;
  k.n_problems = a.n_problems;
  k.ready = a.ready;
  auto kern = gemm_umma_kernel<T, PAIR>;
  static std::atomic<int> configured[MAX_DEVICES];
  int dev = 0;
  SY_CUDA(cudaGetDevice(&dev));
  if (!configured[dev].load(std::memory_order_acquire)) {
    SY_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GM_SMEM));
    configured[dev].store(1, std::memory_order_release);
  }
  return launch_kernel(kern, sms, GM_THREADS, GM_SMEM, a.stream, "grouped tcgen05 launch", k);
}

// Shared argument checks and dtype dispatch of the tensor-core entry points.
int grouped_umma(bool pair, const char* name, const GroupedArgs& a, int rows) {
  SY_REQUIRE(rows >= 0 && a.ranges >= 1 && a.ranges <= GM_MAX_E, "%s: 1..%d row ranges (got %d)", name, GM_MAX_E,
             a.ranges);
  SY_REQUIRE(a.group_div >= 1 && a.ranges % a.group_div == 0, "%s: %d ranges do not divide by %d", name, a.ranges,
             a.group_div);
  SY_REQUIRE(a.dtype == SY_DTYPE_F16 || a.dtype == SY_DTYPE_BF16, "%s: dtype must be f16 or bf16", name);
  for (int i = 0; i < a.n_problems; ++i) {
    const ProblemDesc& d = a.p[i];
    SY_REQUIRE(d.k_dim > 0 && d.k_dim % 8 == 0, "%s: k_dim must be a multiple of 8 (got %d)", name, d.k_dim);
    SY_REQUIRE(d.n_out > 0 && d.n_out % 8 == 0, "%s: n_out must be a multiple of 8 (got %d)", name, d.n_out);
    SY_REQUIRE(!(d.swiglu && d.scale), "%s: swiglu and scale are separate epilogues", name);
  }
  if (rows == 0) return SY_OK;
  SY_REQUIRE(a.begins && a.ends, "%s: null pointer", name);
  for (int i = 0; i < a.n_problems; ++i) {
    const ProblemDesc& d = a.p[i];
    SY_REQUIRE(d.A && d.B && (d.C || d.c_table), "%s: null pointer", name);
    SY_REQUIRE(((uintptr_t)d.A % 16 == 0) && ((uintptr_t)d.B % 16 == 0) && ((uintptr_t)d.C % 16 == 0),
               "%s: A, B and C must be 16-byte aligned", name);
  }
  SY_REQUIRE(a.n_problems == 1 || a.ready, "%s: the fused form needs its scratch", name);
  if (a.dtype == SY_DTYPE_F16) return pair ? launch_gemm<__half, true>(a) : launch_gemm<__half, false>(a);
  return pair ? launch_gemm<__nv_bfloat16, true>(a) : launch_gemm<__nv_bfloat16, false>(a);
}

static GroupedArgs single(const void* A, const int32_t* a_rows, const void* B, const int32_t* begins,
                          const int32_t* ends, int ranges, int group_div, int n_out, int k_dim, int swiglu,
                          const void* scale, void* C, const unsigned long long* c_table, int dtype, void* stream) {
  GroupedArgs a;
  memset(&a, 0, sizeof(a));
  a.p[0] = ProblemDesc{A, a_rows, B, n_out, k_dim, swiglu, scale, C, c_table};
  a.n_problems = 1;
  a.begins = begins;
  a.ends = ends;
  a.ranges = ranges;
  a.group_div = group_div;
  a.dtype = dtype;
  a.stream = static_cast<cudaStream_t>(stream);
  return a;
}

}  // namespace sy

extern "C" int sy_grouped_gemm(const void* A, const int32_t* a_rows, const void* B, const int32_t* offsets,
                               int n_experts, int rows, int n_out, int k_dim, int swiglu, const void* scale, void* C,
                               int dtype, void* stream) {
  return sy::grouped_umma(true, "grouped_gemm",
                          sy::single(A, a_rows, B, offsets, offsets ? offsets + 1 : nullptr, n_experts, 1, n_out, k_dim,
                                     swiglu, scale, C, nullptr, dtype, stream),
                          rows);
}

extern "C" int sy_grouped_gemv(const void* A, const int32_t* a_rows, const void* B, const int32_t* offsets,
                               int n_experts, int rows, int n_out, int k_dim, int swiglu, const void* scale, void* C,
                               int dtype, void* stream) {
  return sy::grouped_umma(false, "grouped_gemv",
                          sy::single(A, a_rows, B, offsets, offsets ? offsets + 1 : nullptr, n_experts, 1, n_out, k_dim,
                                     swiglu, scale, C, nullptr, dtype, stream),
                          rows);
}

extern "C" int sy_grouped_segments(const void* A, const void* B, const int32_t* begins, const int32_t* ends,
                                   int n_groups, int groups_per_expert, int rows_bound, int n_out, int k_dim, int swiglu,
                                   const void* scale, void* C, const uint64_t* c_table, int dtype, int compute_shape,
                                   void* stream) {
  return sy::grouped_umma(compute_shape != 0, "grouped_segments",
                          sy::single(A, nullptr, B, begins, ends, n_groups, groups_per_expert, n_out, k_dim, swiglu,
                                     scale, C, reinterpret_cast<const unsigned long long*>(c_table), dtype, stream),
                          rows_bound);
}

extern "C" size_t sy_expert_ffn_scratch_bytes(int n_experts) { return sizeof(int32_t) * (size_t)(n_experts + 1); }

extern "C" int sy_expert_ffn(const void* x, const int32_t* a_rows, const void* gate_up, const void* down,
                             const int32_t* begins, const int32_t* ends, int n_ranges, int ranges_per_expert,
                             int rows_bound, int hidden, int inter, const void* wsorted, void* act, void* y,
                             const uint64_t* y_table, int32_t* scratch, int dtype, int compute_shape, void* stream) {
  using namespace sy;
  SY_REQUIRE(wsorted, "expert_ffn: null router weights");
  GroupedArgs a;
  memset(&a, 0, sizeof(a));
  a.p[0] = ProblemDesc{x, a_rows, gate_up, inter, hidden, 1, nullptr, act, nullptr};
  a.p[1] = ProblemDesc{act, nullptr, down, hidden, inter, 0, wsorted, y,
                       reinterpret_cast<const unsigned long long*>(y_table)};
  a.n_problems = 2;
  a.begins = begins;
  a.ends = ends;
  a.ranges = n_ranges;
  a.group_div = ranges_per_expert;
  a.ready = scratch;
  a.dtype = dtype;
  a.stream = static_cast<cudaStream_t>(stream);
  return grouped_umma(compute_shape != 0, "expert_ffn", a, rows_bound);
}

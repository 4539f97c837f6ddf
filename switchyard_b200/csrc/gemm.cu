// grouped_gemm and grouped_gemv: every expert's slice of the sorted batch on the tcgen05 tensor
// cores. One persistent kernel in three shapes (see Shape below): "gemv" streams expert weights
// past a handful of token rows (decode), "gemm" is the compute-bound shape, alone or as CTA pairs.
//
// One tile = (expert, a block of token rows, a block of output columns). The grid is
// persistent (one block per SM); tiles are numbered on the device from `offsets` (expert-major,
// an expert's row tiles adjacent so that its weights are read from HBM once and then hit L2)
// and dealt round-robin, so nothing about the batch is read back to the host.
//
// A block is fourteen warps with fixed roles, connected by mbarriers:
//   warp 0      TMA producer: the weight boxes of each k block (128-byte swizzle) and, when a
//               tile's token rows are contiguous in memory (no a_rows, one range per expert),
//               the token box too;
//   warps 2-9   gather producers, for token rows that are NOT contiguous (picked from the
//               unsorted activations through a_rows, or spread over several ranges): 16-byte
//               cp.async copies straight into the same swizzled layout; idle otherwise;
//   warp 1      MMA issuer: one thread, tcgen05.mma into one of two accumulator buffers in
//               tensor memory; tcgen05.commit releases the stage / publishes the accumulators;
//   warps 10-13 epilogue: tcgen05.ld of the accumulators, SwiGLU or router-weight scaling with
//               the 16-bit rounding points, stores to C or to per-range destinations (a peer
//               GPU's mailbox). It overlaps the next tile's main loop.
//
// An output element is a sum over k in instruction order that does not depend on which other
// rows share the tile, so a row's bits are the same on one GPU and inside an expert-parallel
// segment (within one mode).
//
// What was measured on a B200 and dropped: a CUDA-core weight stream (float32 FMA keeps up with
// HBM3e only below about four rows per expert); TMA row gather (tile::gather4) for the token
// rows (about 47 ns per four-row instruction per SM: a quarter of what the compute shape needs);
// one cp.async gather for all rows with a thread-blocking wait per stage (the wait serialised
// the stages). Gathering 16-byte pieces through the load/store unit tops out near 960 TFLOP/s
// for the whole kernel, which is why compute-bound callers sort the rows first.
//
// Replaces switchyard/csrc/moe_kernels.cu:159-298 (64x64x32 WMMA tiles, one block per tile,
// tile list built by torch on the host) and l.306-415 (CUDA-core GEMV, one block per expert and
// 32 columns, blocks launched for empty experts too).
#include <cuda.h>

#include <atomic>
#include <mutex>
#include <stdlib.h>
#include <string.h>
#include <type_traits>

#include "common.cuh"
#include "ep_push.cuh"

namespace sy {


constexpr int GM_ATOM_K = 64;                      // k per swizzle atom: 128-byte rows
constexpr int GM_BM = 128;                         // weight rows per accumulator (UMMA M)
constexpr int GM_GATHER_WARPS = 8;
constexpr int GM_EPI_WARPS = 4;
constexpr int GM_THREADS = (2 + GM_GATHER_WARPS + GM_EPI_WARPS) * 32;
constexpr int GM_MAX_E = 256;
#ifndef SY_RING_KB
#define SY_RING_KB 192
#endif
constexpr int GM_RING_BYTES = SY_RING_KB * 1024;   // shared-memory ring of stages
constexpr int GM_MAX_BN = 256;                      // most token rows in a tile (any shape)
constexpr int GM_EPI_ROWS = 64;                    // token rows the epilogue stages per pass
constexpr int GM_EPI_BYTES = GM_EPI_ROWS * GM_BM * 2;  // staged output tile: 64 rows x 128 columns
constexpr int GM_SMEM = GM_RING_BYTES + GM_EPI_BYTES + 1024;  // + room to align the ring to 1024
constexpr int GM_MAX_RANKS = EP_MAX_RANKS;          // ranks of an expert-parallel group
constexpr int COMBINE_K = 8;                       // most choices per token the fused combine handles

// Three shapes of the same kernel.
//   SH_STREAM (mode "gemv"): the weight tile is the MMA's M operand (128 weight rows; with
//            SwiGLU 64 gate rows + 64 up rows of the same columns) and up to 64 token rows are
//            its N operand, rounded up to 16 per tile; 128 k per stage (two swizzle atoms). M
//            stays full however few rows an expert has: a weight stream for a handful of rows.
//   SH_PAIR  (mode "gemm"): the usual orientation. 128 token rows are M, 256 weight rows are N
//            (with SwiGLU 128 gate + 128 up rows of the same columns): one 128x256x16 MMA per
//            16 k, and an epilogue thread owns a token row, so it writes 16 bytes of a row at a
//            time and needs no exchange for SwiGLU. 48 KB stages x 4.
//   SH_DUO   (mode "gemm", many rows per expert): two CTAs on neighbouring SMs work as one
//            (tcgen05 cta_group::2). A tile is 256 token rows (128 gathered by each CTA) by 256
//            weight rows (128 loaded by each CTA); the pair's MMAs read both halves. Per MMA a
//            CTA fills 2/3 of the shared memory a PAIR tile needs. 128 k per stage: 64 KB stages x 3.
enum { SH_STREAM = 0, SH_PAIR = 1, SH_DUO = 2 };
template <int SH> struct Shape {
  static constexpr bool STREAM = SH == SH_STREAM, PAIR = SH == SH_PAIR, DUO = SH == SH_DUO;
  static constexpr int BN = STREAM ? 64 : DUO ? 256 : 128;  // token rows per tile
  static constexpr int XR = STREAM ? 64 : 128;              // token rows one CTA stages
  static constexpr int WR = PAIR ? 256 : 128;               // weight rows one CTA stages
  static constexpr int BOX_ROWS = WR / 2;                   // weight rows per TMA box (two boxes per atom)
  static constexpr int KATOMS = PAIR ? 1 : 2;               // 64-wide k atoms per stage
  static constexpr int BK = KATOMS * GM_ATOM_K;             // k per stage
  static constexpr int W_ATOM_BYTES = WR * 128;             // weight bytes of one atom (both boxes)
  static constexpr int X_ATOM_BYTES = XR * 128;
  static constexpr int W_BYTES = KATOMS * W_ATOM_BYTES;     // weight bytes per stage
  static constexpr int X_BYTES = KATOMS * X_ATOM_BYTES;
  static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;     // 48 KB, or 64 KB for DUO
  static constexpr int STAGES = GM_RING_BYTES / STAGE_BYTES;
  static constexpr int BUF_COLS = STREAM ? BN : 256;        // tensor-memory columns per accumulator buffer
  static constexpr int TMEM_COLS = 2 * BUF_COLS;            // two buffers: 128 or 512
  static constexpr int CTAS = DUO ? 2 : 1;                  // CTAs that share a tile
  static constexpr int GATHER_GROUP = GM_GATHER_WARPS / STAGES;  // gather warps per slot of the ring
};

struct Tile {
  int phase, e, cb, row0, nvalid;
};

// One contraction over the row ranges: activations A (optionally gathered through a_rows),
// expert weights behind `map`, an epilogue, a destination. The fused expert FFN is two of them
// (gate/up with SwiGLU, then down with the router-weight scale) run by ONE launch.
struct Problem {
  CUtensorMap map;                       // [experts * n_full, K] weights, box 64 k x BOX_ROWS
  CUtensorMap xmap;                      // [rows, K] activations, box 64 k x XR; used when x_tma
  const void* A;
  const int* a_rows;
  const void* scale;
  void* C;
  int use_table;                         // results go through the table of per-range row pointers
  int Nout, K, swiglu;
  int x_tma;                             // A's rows are the ranges' rows themselves (no a_rows, one range per
                                         // expert): a tile's rows are contiguous and come by TMA, not by gather
};

// Expert-parallel mode (arrive != nullptr). The rows sit in this rank's mailbox, one slot of `cap`
// rows per sender. The kernel itself waits (bounded) for every sender's arrival flag, reads the
// senders' metadata (meta[s] = per + 1 rebased offsets | first row in the sender's sort | rows),
// builds the row ranges (range e * R + s = sender s's rows of local expert e) and the table of
// where each range's results go (into the SENDER's result buffer, at the rows its own sort gave
// them), and when its last result tile has been stored it release-stores the layer's epoch into
// every sender's return flag. With push.counter set the kernel first does the layer's dispatch
// itself (csrc/ep_push.cuh: this rank's rows into the owners' mailboxes, their arrival flags) and
// advances the epoch when it ends; otherwise a dispatch launch has done both before it.
struct EpArgs {
  const int* arrive;
  const int* meta;
  int* epoch_counter;
  int R, per, cap, out_row_bytes;
  unsigned char* y[GM_MAX_RANKS];
  int* ret_flag[GM_MAX_RANKS];
  PushArgs push;
};

// Combine fused into the last problem's epilogue (streaming shape, local results): every result
// tile counts, per token and column block, the rows of that token it has stored; whoever stores
// a token's last row sums the token's rows of that column block in ascending row order (which is
// ascending expert order, the combine kernel's order) and writes the layer's output.
struct CombineArgs {
  void* out;                             // [n_tokens, Nout]; nullptr: no combine
  const int* token;                      // [rows] token of each sorted row
  const int* pos_of;                     // [n_tokens * k] sorted row of each choice
  int* arrivals;                         // [n_tokens * column blocks] zero before and after the launch
  int k, rows;
};

struct KernelArgs {
  Problem p[2];
  const int* begins;                     // [ranges]
  const int* ends;
  const unsigned long long* c_table;     // [ranges] optional per-range output row pointers
  int ranges, group_div;                 // expert e owns ranges [e*group_div, (e+1)*group_div)
  int weight_div;                        // the weights of "expert" e (a group of ranges) are those of expert
                                         // e / weight_div: > 1 when an expert's ranges are tiled separately
  int n_problems;                        // 1, or 2 = fused FFN: p[1] reads what p[0] wrote
  int* ready;                            // fused: [experts] finished p[0] tiles, then [1] blocks that have left
  int* status;
  unsigned long long wait_ns;            // limit of every wait in the kernel
  EpArgs ep;
  CombineArgs cmb;
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

// The epilogue of one STREAM tile, specialised on the epilogue kind so that its inner loops
// carry no run-time switches: accumulators -> SwiGLU / router-weight scale / plain rounding ->
// memory. A thread owns one weight row (= output column) and walks the token rows.
template <typename T, bool SWIGLU, bool SCALE>
__device__ __forceinline__ void epilogue_stream(const Tile& tile, int buf, uint32_t tmem, int q, int lane, int et, bool alive,
                                                int& chunk_no, int Nout, int colbase, const T* __restrict__ scale,
                                                T* __restrict__ C, const unsigned long long* __restrict__ c_table,
                                                int group_div, const int* s_begin, const int* s_end, int* map_row_s,
                                                int* map_grp_s, float (*s_xch)[GM_BM / 2][9], unsigned char* out_tile) {
  using S = Shape<SH_STREAM>;
  const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16) + buf * S::BUF_COLS;
  const int wrow = q * 32 + lane;
  // With several ranges per expert the tile's rows in A / C space (and the range of each) are
  // looked up once per tile for all four warps; with one range they are consecutive.
  const bool mapped = group_div > 1;
  const int row_base = s_begin[tile.e * group_div] + tile.row0;
  if (mapped) {
    for (int i = et; i < tile.nvalid; i += GM_EPI_WARPS * 32) {
      int gr;
      map_row_s[i] = map_row(tile.e, tile.row0 + i, group_div, s_begin, s_end, gr);
      map_grp_s[i] = gr;
    }
    named_barrier_sync(3, GM_EPI_WARPS * 32);
  }
  constexpr bool exchange = SWIGLU;  // gate rows in lanes 0-63, up rows in 64-127
  if (!c_table) {
    // Local destination: every thread stores its own column's values directly (2 bytes per
    // store, a warp covers 64 contiguous bytes of a row); L2 merges them, and the epilogue
    // stays short enough to hide behind the next tile's main loop.
    if (!exchange) {
      const int col0 = colbase + wrow;
      for (int n0 = 0; n0 < tile.nvalid && alive; n0 += 8) {
        uint32_t v0[8];
        tmem_ld_x8(taddr + n0, v0);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (n0 + j < tile.nvalid && col0 < Nout) {
            const int row = mapped ? map_row_s[n0 + j] : row_base + n0 + j;
            const float f0 = __uint_as_float(v0[j]);
            C[(size_t)row * Nout + col0] = SCALE ? epilogue_scale<T>(f0, scale[row]) : Elem<T>::from_f(f0);
          }
        }
      }
    } else {
      // Warps 2,3 (up rows) pass their values to warps 0,1 (gate rows) through shared memory.
      const int j64 = wrow & 63;
      const int col = colbase + j64;
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
#pragma unroll 1
    for (int nb = 0; nb < tile.nvalid; nb += GM_EPI_ROWS) {
      const int nrows = min(GM_EPI_ROWS, tile.nvalid - nb);
      // ---- phase 1: tensor memory -> registers -> epilogue arithmetic -> staged tile
      if (!exchange) {
        for (int n0 = nb; n0 < nb + nrows; n0 += 8) {
          uint32_t v0[8];
          if (alive) {
            tmem_ld_x8(taddr + n0, v0);
            tmem_ld_wait();
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (alive && n0 + j < tile.nvalid) {
              const float f0 = __uint_as_float(v0[j]);
              T o;
              if (SCALE) o = epilogue_scale<T>(f0, scale[mapped ? map_row_s[n0 + j] : row_base + n0 + j]);
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
      const int col = colbase + (et % TPR) * 8;
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

template <typename T> __device__ __forceinline__ uint32_t pack2(T a, T b) {
  return (uint32_t) reinterpret_cast<const uint16_t&>(a) | ((uint32_t) reinterpret_cast<const uint16_t&>(b) << 16);
}

// The epilogue of one PAIR / DUO tile. A thread owns one TOKEN row of the tile (its lane of
// tensor memory) and walks the output columns, sixteen at a time: SwiGLU pairs a gate column
// with its up column from the same row, so nothing is exchanged between threads, and results
// leave as 16-byte stores, two per step, to the row's place in C or behind c_table (a peer GPU).
template <typename T, int SH, bool SWIGLU, bool SCALE>
__device__ __forceinline__ void epilogue_rows(const Tile& tile, int buf, uint32_t tmem, int q, int lane, int cr, bool alive,
                                              int Nout, int colbase, const T* __restrict__ scale, T* __restrict__ C,
                                              const unsigned long long* __restrict__ c_table, int group_div,
                                              const int* s_begin, const int* s_end) {
  using S = Shape<SH>;
  const int trow = cr * S::XR + q * 32 + lane;  // this thread's row of the tile
  if (!alive || cr * S::XR + q * 32 >= tile.nvalid) return;  // the whole warp is past the tile's end
  const bool valid = trow < tile.nvalid;
  const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16) + buf * S::BUF_COLS;
  T* dst = nullptr;
  T sc = Elem<T>::from_f(0.f);
  if (valid) {
    int gr = tile.e * group_div, row;
    if (group_div > 1) row = map_row(tile.e, tile.row0 + trow, group_div, s_begin, s_end, gr);
    else row = s_begin[gr] + tile.row0 + trow;
    // c_table[g] is where row s_begin[g] of range g lands
    dst = (c_table ? reinterpret_cast<T*>(c_table[gr]) + (size_t)(row - s_begin[gr]) * Nout : C + (size_t)row * Nout) + colbase;
    if (SCALE) sc = scale[row];
  }
  // Accumulator columns: SwiGLU tiles hold [gate | up] groups of G columns (PAIR: one group of
  // 128 + 128; DUO: each CTA's weight rows are 64 + 64, so two groups); plain tiles hold the
  // 256 output columns in order. Sixteen output columns per step; the next step's accumulators
  // are already on their way from tensor memory while this step's are turned into stores.
  constexpr int G = S::DUO ? 64 : 128;
  constexpr int OUT_COLS = SWIGLU ? 128 : 256;
  const bool wide = (reinterpret_cast<uintptr_t>(dst) & 31) == 0;  // this row's segments are 32-byte aligned
  constexpr int STEPS = OUT_COLS / 16;
  uint32_t a[2][16], b[2][16];
  auto fetch = [&](int step, int slot) {
    const int oc = step * 16;
    if (SWIGLU) {
      const int gc = (oc / G) * 2 * G + (oc % G);
      tmem_ld_x16(taddr + gc, a[slot]);
      tmem_ld_x16(taddr + gc + G, b[slot]);
    } else {
      tmem_ld_x16(taddr + oc, a[slot]);
    }
  };
  fetch(0, 0);
  tmem_ld_wait();
#pragma unroll
  for (int step = 0; step < STEPS; ++step) {
    const int oc = step * 16, slot = step & 1;
    if (colbase + oc >= Nout) break;  // warp-uniform
    if (step + 1 < STEPS) fetch(step + 1, slot ^ 1);
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      T lo, hi;
      if (SWIGLU) {
        lo = epilogue_swiglu<T>(__uint_as_float(a[slot][2 * j]), __uint_as_float(b[slot][2 * j]));
        hi = epilogue_swiglu<T>(__uint_as_float(a[slot][2 * j + 1]), __uint_as_float(b[slot][2 * j + 1]));
      } else if (SCALE) {
        lo = epilogue_scale<T>(__uint_as_float(a[slot][2 * j]), sc);
        hi = epilogue_scale<T>(__uint_as_float(a[slot][2 * j + 1]), sc);
      } else {
        lo = Elem<T>::from_f(__uint_as_float(a[slot][2 * j]));
        hi = Elem<T>::from_f(__uint_as_float(a[slot][2 * j + 1]));
      }
      o[j] = pack2<T>(lo, hi);
    }
    if (valid) {
      if (wide && colbase + oc + 16 <= Nout) {
        st_global_32(dst + oc, o);  // a whole 32-byte sector per store
      } else {
        *reinterpret_cast<uint4*>(dst + oc) = make_uint4(o[0], o[1], o[2], o[3]);
        if (colbase + oc + 8 < Nout) *reinterpret_cast<uint4*>(dst + oc + 8) = make_uint4(o[4], o[5], o[6], o[7]);
      }
    }
    tmem_ld_wait();  // the next step's accumulators have arrived
  }
}

// Sorts eight ints ascending with a fixed network of compare-exchanges (registers only).
__device__ __forceinline__ void sort8(int (&v)[8]) {
#define SY_CSWAP(a, b)            \
  {                               \
    const int lo = min(v[a], v[b]); \
    v[b] = max(v[a], v[b]);       \
    v[a] = lo;                    \
  }
  SY_CSWAP(0, 1) SY_CSWAP(2, 3) SY_CSWAP(4, 5) SY_CSWAP(6, 7)
  SY_CSWAP(0, 2) SY_CSWAP(1, 3) SY_CSWAP(4, 6) SY_CSWAP(5, 7)
  SY_CSWAP(1, 2) SY_CSWAP(5, 6) SY_CSWAP(0, 4) SY_CSWAP(3, 7)
  SY_CSWAP(1, 5) SY_CSWAP(2, 6)
  SY_CSWAP(1, 4) SY_CSWAP(3, 6)
  SY_CSWAP(2, 4) SY_CSWAP(3, 5)
  SY_CSWAP(3, 4)
#undef SY_CSWAP
}

// Combine fused into the streaming shape's last epilogue. Called by the four epilogue warps
// after they have stored a result tile (nvalid rows x up to 128 columns of y). Every row's
// thread counts the row for its (token, column block); the thread that brings the count to the
// number of rows the token has finishes the token for this column block: the token's rows,
// read back through L2, summed in float32 in ascending row order (rows are sorted by expert, so
// this is the order of the combine kernel: expert id, ties by slot) and rounded once.
template <typename T>
__device__ __forceinline__ void epilogue_combine(const Tile& tile, int et, int row_base, int Nout, int colbase,
                                                 const CombineArgs& cb, const T* __restrict__ y, int col_blocks,
                                                 int* s_final, int* s_nfinal) {
  const int k = cb.k, rows = cb.rows;
  if (et == 0) *s_nfinal = 0;
  named_barrier_sync(3, GM_EPI_WARPS * 32);  // every warp's stores of this tile have been issued
  if (et < tile.nvalid) {
    const int t = cb.token[row_base + et];
    int have = 0;  // rows this token has (choices that the sort gave a row)
    for (int j = 0; j < k; ++j) {
      const int p = cb.pos_of[(size_t)t * k + j];
      have += p >= 0 && p < rows;
    }
    __threadfence();
    int* counter = cb.arrivals + (size_t)t * col_blocks + tile.cb;
    if (atomicAdd(counter, 1) + 1 == have) {
      *counter = 0;  // nobody else touches it in this launch; the next launch finds zero
      __threadfence();
      s_final[atomicAdd(s_nfinal, 1)] = t;
    }
  }
  named_barrier_sync(3, GM_EPI_WARPS * 32);
  const int nfinal = *s_nfinal;
  const int chunk = et & 15, lane8 = et >> 4;  // sixteen 16-byte chunks per 128 columns; eight tokens at a time
  const int col = colbase + chunk * 8;
  if (col >= Nout) return;
  for (int f = lane8; f < nfinal; f += GM_EPI_WARPS * 32 / 16) {
    const int t = s_final[f];
    int pos[COMBINE_K];
#pragma unroll
    for (int j = 0; j < COMBINE_K; ++j) {
      const int p = j < k ? cb.pos_of[(size_t)t * k + j] : -1;
      pos[j] = p >= 0 && p < rows ? p : 0x7fffffff;
    }
    sort8(pos);
    uint4 v[COMBINE_K];
#pragma unroll
    for (int j = 0; j < COMBINE_K; ++j)
      if (pos[j] != 0x7fffffff) v[j] = __ldcg(reinterpret_cast<const uint4*>(y + (size_t)pos[j] * Nout + col));
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < COMBINE_K; ++j)
      if (pos[j] != 0x7fffffff) {
        float fv[8];
        unpack8<T>(v[j], fv);
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[q] += fv[q];
      }
    __align__(16) T r[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) r[q] = Elem<T>::from_f(acc[q]);
    *reinterpret_cast<uint4*>(static_cast<T*>(cb.out) + (size_t)t * Nout + col) = *reinterpret_cast<const uint4*>(r);
  }
}

template <typename T, int SH>
__global__ void __launch_bounds__(GM_THREADS, 1) gemm_umma_kernel(const __grid_constant__ KernelArgs args) {
  using S = Shape<SH>;
  constexpr bool STREAM = S::STREAM, PAIR = S::PAIR, DUO = S::DUO;
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
  __shared__ int s_map_row[2][GM_MAX_BN];  // per accumulator buffer: the tile's rows in A / C space
  __shared__ int s_map_grp[2][GM_MAX_BN];  // ... and the range each row belongs to
  __shared__ float s_xch[2][GM_BM / 2][9];  // up-projection values handed to the gate warps (one-accumulator SwiGLU)
  __shared__ unsigned long long s_ctab[GM_MAX_E];  // per-range output row pointers (given, or built in expert-parallel mode)
  __shared__ int s_flag_ok;
  __shared__ int s_epoch;
  __shared__ int s_push_seg[GM_MAX_RANKS + 1];
  __shared__ int s_push_done[2];
  __shared__ int s_final[GM_MAX_BN];       // fused combine: tokens this tile completes
  __shared__ int s_nfinal;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  unsigned char* stages =
      reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* out_tile = stages + GM_RING_BYTES;  // the epilogue's staged output rows
  int* status = args.status;
  const uint64_t GM_WAIT_NS = args.wait_ns;
  const int E = args.ranges, group_div = args.group_div, NP = args.n_problems;
  const int EL = E / group_div;  // experts; E counts row ranges
  // DUO: the two CTAs of a cluster share every tile; `unit` numbers the clusters.
  const int cr = DUO ? (int)cluster_ctarank() : 0;
  const int unit = DUO ? (int)blockIdx.x >> 1 : (int)blockIdx.x;
  const int units = DUO ? (int)gridDim.x >> 1 : (int)gridDim.x;

  // per-problem tile geometry: output columns per tile, and the first weight row (= output
  // column) this CTA loads for a tile (DUO: each CTA loads half of the tile's weight rows)
  auto cols_of = [&](int ph) { return args.p[ph].swiglu ? (STREAM ? GM_BM / 2 : GM_BM) : (STREAM ? GM_BM : 2 * GM_BM); };
  auto col_blocks_of = [&](int ph) { return (args.p[ph].Nout + cols_of(ph) - 1) / cols_of(ph); };
  auto k_blocks_of = [&](int ph) { return (args.p[ph].K + S::BK - 1) / S::BK; };
  auto colbase_of = [&](const Tile& tile) { return tile.cb * cols_of(tile.phase); };
  auto wbase_of = [&](const Tile& tile) { return colbase_of(tile) + cr * (cols_of(tile.phase) >> 1); };

  // the gather warps work only if some problem's token rows do not come by TMA
  const bool gather_on = !(args.p[0].x_tma && (NP == 1 || args.p[1].x_tma));

  // Set-up that touches none of the kernel's inputs comes first, so that under programmatic
  // dependent launch it overlaps the tail of the previous kernel.
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      // the weights' expect_tx arrive plus one arrive per gather warp of the slot (both CTAs'
      // in DUO, where only the leader's full barriers are used)
      mbar_init(&full_bar[s], 1 + (gather_on ? S::CTAS * S::GATHER_GROUP : 0));
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], S::CTAS * GM_EPI_WARPS);  // DUO: the leader's, for both CTAs' epilogues
    }
    fence_barrier_init();
    for (int ph = 0; ph < NP; ++ph) {
      prefetch_tensormap(&args.p[ph].map);
      if (args.p[ph].x_tma) prefetch_tensormap(&args.p[ph].xmap);
    }
  }
  if (warp == 1) {
    if (DUO) {
      tmem_alloc_pair(&s_tmem, S::TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(&s_tmem, S::TMEM_COLS);
      tmem_relinquish();
    }
  }
  pdl_wait();  // row ranges, activations, scale: all written by earlier kernels
  if (args.ep.arrive) {
    // expert-parallel: wait for every sender's rows, then build the ranges and the result table
    const int R = args.ep.R, per = args.ep.per, cap = args.ep.cap;
    const bool pushes = args.ep.push.counter != nullptr;
    const int epoch = *args.ep.epoch_counter + (pushes ? 1 : 0);
    if (threadIdx.x == 0) {
      s_flag_ok = 1;
      s_epoch = epoch;
    }
    if (pushes) push_rows(args.ep.push, epoch, status, s_push_seg, s_push_done);  // the layer's dispatch, in this launch
    __syncthreads();
    if ((int)threadIdx.x < R && !wait_flag(args.ep.arrive + threadIdx.x, epoch, GM_WAIT_NS)) {
      *status = DS_TIMEOUT_FLAG;
      s_flag_ok = 0;
    }
    __syncthreads();
    const bool ok = s_flag_ok != 0;
    for (int g = threadIdx.x; g < E; g += GM_THREADS) {
      const int e = g / R, s = g - e * R;
      const volatile int* m = args.ep.meta + s * (per + 3);  // written by another GPU: no cached read
      const int lo = ok ? m[e] : 0, hi = ok ? min(m[e + 1], cap) : 0;
      s_begin[g] = s * cap + lo;
      s_end[g] = s * cap + (hi > lo ? hi : lo);
      s_ctab[g] = reinterpret_cast<unsigned long long>(args.ep.y[s]) +
                  (unsigned long long)((ok ? m[per + 1] : 0) + lo) * (unsigned long long)args.ep.out_row_bytes;
    }
    fence_proxy_async_all();  // the mailbox rows were written by plain (remote) stores; TMA may read them next
  } else {
    for (int i = threadIdx.x; i < E; i += GM_THREADS) {
      const int b = args.begins[i], e = args.ends[i];
      s_begin[i] = b;
      s_end[i] = e > b ? e : b;
      if (args.c_table) s_ctab[i] = args.c_table[i];
    }
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
  if (DUO) cluster_sync_all();  // the other CTA's barriers exist before anything arrives on them
  tc_fence_after_sync();
  const uint32_t tmem = s_tmem;
  const int tiles0 = s_tile_start[0][EL];
  const int total_tiles = tiles0 + (NP > 1 ? s_tile_start[1][EL] : 0);
  // token rows of a STREAM tile's MMA: a multiple of 16
  auto n_mma_of = [](int nvalid) { return max(16, (nvalid + 15) & ~15); };

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    // The whole warp walks the tiles; lane 0 waits for the slot and announces the stage's bytes,
    // then each box of the stage is issued by its own lane (issuing a TMA load keeps a thread
    // busy for about a hundred clocks; three to six boxes in a row would make this thread the
    // bottleneck of the ring).
    int it = 0, cursor = 0, seen = 0;
    bool alive = true;
    // streaming shape: an expert's weights are read once, so they are marked evict-first in L2
    const uint64_t policy = l2_policy_evict_first();
    for (int t = unit; t < total_tiles && alive; t += units) {
      const Tile tile = locate_tile<BN>(t, tiles0, seen, cursor, s_tile_start, s_rows);
      const Problem& P = args.p[tile.phase];
      const int Nfull = P.swiglu ? 2 * P.Nout : P.Nout;
      const int y0 = (tile.e / args.weight_div) * Nfull + wbase_of(tile);
      const int y1 = P.swiglu ? y0 + P.Nout : y0 + S::BOX_ROWS;
      const int k_blocks = k_blocks_of(tile.phase);
      // contiguous token rows: the tile's first row in A (rows past the tile's end belong to the
      // next expert or are zero-filled past A's end; their accumulator rows are never read)
      const int xrow = s_begin[tile.e] + tile.row0 + cr * S::XR;
      const uint32_t stage_bytes = S::W_BYTES + (P.x_tma ? S::X_BYTES : 0);
      // this lane's box within a stage: atom a = lane / 3; kind 0, 1 = the two weight boxes, 2 = token rows
      const int atom = lane / 3, kind = lane % 3;
      const bool has_box = atom < S::KATOMS && (kind < 2 || P.x_tma);
      const void* map = kind < 2 ? static_cast<const void*>(&P.map) : static_cast<const void*>(&P.xmap);
      const int by = kind == 0 ? y0 : kind == 1 ? y1 : xrow;
      const int boff = kind == 0   ? atom * S::W_ATOM_BYTES
                       : kind == 1 ? atom * S::W_ATOM_BYTES + S::BOX_ROWS * 128
                                   : S::W_BYTES + atom * S::X_ATOM_BYTES;
      // One stage: lane 0 waits for the slot and announces the bytes, then every box is issued by
      // its lane. `boxes`: 3 = the whole stage; 1 = claim the slot, announce the whole stage's
      // bytes, send only the weight boxes; 2 = only the token box of a stage claimed earlier.
      auto issue_stage = [&](int kb, int g, int boxes) -> bool {
        const int s = g % STAGES, use = g / STAGES;
        int ok = 1;
        if (lane == 0 && (boxes & 1)) {
          if (use > 0) ok = (int)mbar_wait(&empty_bar[s], (use - 1) & 1, GM_WAIT_NS);
          // DUO: both CTAs' bytes are counted on the leader's barrier
          if (ok && cr == 0) mbar_arrive_expect_tx(&full_bar[s], S::CTAS * stage_bytes);
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);  // also orders the other lanes' loads after the wait
        if (!ok) {
          if (lane == 0) *status = DS_TIMEOUT_EMPTY;
          return false;
        }
        if (has_box && (boxes & (kind < 2 ? 1 : 2))) {
          unsigned char* dst = stages + (size_t)s * STAGE_BYTES + boff;
          const int kx = kb * S::BK + atom * GM_ATOM_K;
          if (DUO) tma_load_2d_pair(dst, map, kx, by, cluster_map(&full_bar[s], 0));
          else if (STREAM && kind < 2) tma_load_2d_hint(dst, map, kx, by, &full_bar[s], policy);
          else tma_load_2d(dst, map, kx, by, &full_bar[s]);
        }
        return true;
      };
      int ahead = 0;  // stages of this tile whose weight boxes are already on their way
      if (tile.phase == 1 && P.x_tma) {
        // fused FFN: the token rows are what the expert's gate/up tiles wrote. Wait (bounded) until
        // all of them have been stored; they sit earlier in every block's tile list and their own
        // loads are already in flight, so nothing here holds them up.
        // When every gate/up tile of the launch runs in the first round (a handful of tokens: at
        // most one tile per block), HBM is far from busy and this tile's weights do not depend on
        // the wait: their boxes go out first, the token boxes follow after the wait. With more
        // tiles than blocks that was measured to hurt (the early weights take bandwidth from the
        // gate/up tiles the wait is for: 6 % slower at 64 tokens), so it is not done there.
        if (STREAM && tiles0 <= units) {
          ahead = min(STAGES, k_blocks);
          for (int j = 0; j < ahead && alive; ++j) alive = issue_stage(j, it + j, 1);
          if (!alive) break;
        }
        const int need = ((s_rows[tile.e] + BN - 1) / BN) * col_blocks_of(0) * S::CTAS;
        int ok = 1;
        if (lane == 0 && ld_acquire_gpu(args.ready + tile.e) < need) {
          const uint64_t start = global_timer_ns();
          while (ld_acquire_gpu(args.ready + tile.e) < need) {
            if (global_timer_ns() - start > GM_WAIT_NS) {
              *status = DS_TIMEOUT_FLAG;
              ok = 0;
              break;
            }
          }
        }
        if (!__shfl_sync(0xffffffffu, ok, 0)) {
          alive = false;
          break;
        }
        fence_proxy_async_all();  // they were written by plain stores; TMA reads them next
        for (int j = 0; j < ahead; ++j) issue_stage(j, it + j, 2);
        it += ahead;
      }
      for (int kb = ahead; kb < k_blocks && alive; ++kb, ++it) alive = issue_stage(kb, it, 3);
    }
    if (!alive && cr == 0 && lane == 0)  // let the copies already issued land before the block can exit
      for (int j = it > STAGES ? it - STAGES : 0; j < it; ++j) mbar_wait(&full_bar[j % STAGES], (j / STAGES) & 1, 10000000ull);
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    // One thread. STREAM: weights are the M operand, token rows the N operand. PAIR / DUO: token
    // rows are M and weight rows N (256 of them per instruction). DUO: the leader CTA's thread
    // issues for both CTAs; its commits reach both CTAs' barriers.
    if (lane == 0 && cr == 0) {
      const int fmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
      const uint32_t ring_lo = umma_desc_lo(smem_u32(stages));
      int it = 0, cursor = 0, seen = 0, tile_no = 0;
      bool alive = true;
      for (int t = unit; t < total_tiles && alive; t += units, ++tile_no) {
        const Tile tile = locate_tile<BN>(t, tiles0, seen, cursor, s_tile_start, s_rows);
        const int k_blocks = k_blocks_of(tile.phase);
        const int buf = tile_no & 1, use_t = tile_no >> 1;
        if (use_t > 0) {
          const bool ok = DUO ? mbar_wait_cluster(&acc_empty[buf], (use_t - 1) & 1, GM_WAIT_NS)
                              : mbar_wait(&acc_empty[buf], (use_t - 1) & 1, GM_WAIT_NS);
          if (!ok) {
            *status = DS_TIMEOUT_TMEM;
            alive = false;
            break;
          }
          tc_fence_after_sync();
        }
        const uint32_t idesc = umma_idesc(fmt, DUO ? 2 * GM_BM : GM_BM, STREAM ? n_mma_of(tile.nvalid) : 2 * GM_BM);
        const uint32_t d = tmem + buf * S::BUF_COLS;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const bool ok = DUO ? mbar_wait_cluster(&full_bar[s], (it / STAGES) & 1, GM_WAIT_NS)
                              : mbar_wait(&full_bar[s], (it / STAGES) & 1, GM_WAIT_NS);
          if (!ok) {
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
            const uint32_t w_lo = lo + atom * (S::W_ATOM_BYTES >> 4) + within;
            const uint32_t x_lo = lo + (S::W_BYTES >> 4) + atom * (S::X_ATOM_BYTES >> 4) + within;
            if (DUO) umma_f16_lohi_pair(d, x_lo, w_lo, UMMA_DESC_HI_K_SW128, idesc, accumulate);
            else if (PAIR) umma_f16_lohi(d, x_lo, w_lo, UMMA_DESC_HI_K_SW128, idesc, accumulate);
            else umma_f16_lohi(d, w_lo, x_lo, UMMA_DESC_HI_K_SW128, idesc, accumulate);
          }
          // the stage is free once these MMAs have read it
          if (DUO) umma_commit_pair(&empty_bar[s], 3);
          else umma_commit(&empty_bar[s]);
        }
        if (alive) {
          if (DUO) umma_commit_pair(&acc_full[buf], 3);
          else umma_commit(&acc_full[buf]);
        }
      }
    }
  } else if (warp < 2 + GM_GATHER_WARPS) {
    if (gather_on) {
    // ---------------------------------------------------------------- gather producers
    // The tile's token rows, 16-byte asynchronous copies straight into the swizzled stage.
    // Each slot of the ring has its own warps (GROUP of them, splitting the rows): they wait for
    // the slot, issue the stage's copies, wait for them to land, make them visible to the tensor
    // core (proxy fence) and arrive on the stage's barrier. Waiting for data therefore stalls
    // only that slot's warps; the other slots fill meanwhile, and a stage is handed to the MMA
    // issuer the moment it is complete. (A warp must see every use of its slot: an mbarrier
    // parity wait tells the previous phase from the current one, not from older ones.)
    // DUO: this CTA stages its half of the tile's rows and arrives on the leader's barrier.
    constexpr int CHUNKS = S::BK / 8;            // 16-byte chunks per token row per stage
    constexpr int RPI = 32 / CHUNKS;             // token rows one warp-wide copy instruction covers
    constexpr int ITERS = S::XR / RPI;           // instructions per full stage
    constexpr int OWN = S::XR / 32;              // row indices each lane keeps per tile
    static_assert(ITERS * RPI == S::XR && OWN * 32 == S::XR && 32 % (S::GATHER_GROUP * RPI) == 0, "gather geometry");
    constexpr int GROUP = S::GATHER_GROUP;       // warps per slot
    const int gw = warp - 2;                     // 0..7
    const int slot = gw % STAGES, part = gw / STAGES;  // part >= GROUP: a spare warp
    const int c = lane % CHUNKS, sub = lane / CHUNKS;  // chunk of the row; row within an instruction
    const int xatom = (c >> 3) * S::X_ATOM_BYTES, cc = c & 7;  // atom of the chunk; chunk within the 128-byte row
    int it = 0, cursor = 0, seen = 0;
    bool alive = true;
    for (int t = unit; t < total_tiles && alive; t += units) {
      const Tile tile = locate_tile<BN>(t, tiles0, seen, cursor, s_tile_start, s_rows);
      const Problem& P = args.p[tile.phase];
      const int K = P.K, k_blocks = k_blocks_of(tile.phase);
      // which of this tile's stages land in this warp's slot
      const int first_kb = (slot - it % STAGES + STAGES) % STAGES;
      const int it0 = it;
      it += k_blocks;
      if (first_kb >= k_blocks || part >= GROUP) continue;
      if (tile.phase == 1 && !P.x_tma) {
        // fused FFN: this tile reads what the expert's gate/up tiles wrote. Wait (bounded)
        // until all of them have been stored; they sit earlier in every block's tile list, and
        // everything this warp filled for them has already been handed over.
        const int need = ((s_rows[tile.e] + BN - 1) / BN) * col_blocks_of(0) * S::CTAS;
        int ok = 1;
        if (lane == 0 && ld_acquire_gpu(args.ready + tile.e) < need) {
          const uint64_t start = global_timer_ns();
          while (ld_acquire_gpu(args.ready + tile.e) < need) {
            if (global_timer_ns() - start > GM_WAIT_NS) {
              *status = DS_TIMEOUT_FLAG;
              ok = 0;
              break;
            }
          }
        }
        if (!__shfl_sync(0xffffffffu, ok, 0)) break;  // one bounded wait per warp, not one per tile
      }
      // Row indices: lane l keeps those of the CTA's rows l, l + 32, ...; DUO: the second CTA
      // stages the tile's rows from 128 on.
      const int mine = min(max(tile.nvalid - cr * S::XR, 0), S::XR);  // valid rows this CTA stages
      int own[OWN];
#pragma unroll
      for (int j = 0; j < OWN; ++j) {
        const int r = lane + 32 * j;
        own[j] = 0;
        if (r < mine) {
          int gr;
          const int at = map_row(tile.e, tile.row0 + cr * S::XR + r, group_div, s_begin, s_end, gr);
          own[j] = P.a_rows ? P.a_rows[at] : at;
        }
      }
      const T* A = static_cast<const T*>(P.A) + c * 8;
      const int iters = P.x_tma ? 0 : (mine + RPI - 1) / RPI;  // rows that come by TMA need no copies here
      for (int kb = first_kb; kb < k_blocks; kb += STAGES) {
        const int g = it0 + kb, s = g % STAGES, use = g / STAGES;
        if (use > 0) {
          int ok = lane == 0 ? (int)mbar_wait(&empty_bar[s], (use - 1) & 1, GM_WAIT_NS) : 1;
          ok = __shfl_sync(0xffffffffu, ok, 0);  // also orders the other lanes' copies after the wait
          if (!ok) {
            if (lane == 0) *status = DS_TIMEOUT_EMPTY;
            alive = false;
            break;
          }
        }
        unsigned char* x = stages + (size_t)s * STAGE_BYTES + S::W_BYTES;
        const bool in_k = kb * S::BK + c * 8 < K;  // beyond K: zero fill
        const size_t koff = in_k ? (size_t)kb * S::BK : 0;
        const uint32_t bytes = in_k ? 16u : 0u;
#pragma unroll
        for (int i0 = 0; i0 < ITERS; i0 += GROUP) {
          const int i = i0 + part;
          if (i < iters) {  // warp-uniform
            const int r = i * RPI + sub;
            // row r's index sits in lane r % 32, register r / 32 (= i * RPI / 32 for every lane)
            const int row = __shfl_sync(0xffffffffu, own[(i0 * RPI) >> 5], r & 31);
            if (r < mine) cp_async_16(x + xatom + r * 128 + ((cc ^ (r & 7)) << 4), A + (size_t)row * K + koff, bytes);
          }
        }
        cp_async_commit();
        cp_async_wait<0>();
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (DUO) mbar_arrive_cluster(cluster_map(&full_bar[s], 0));
          else mbar_arrive(&full_bar[s]);
        }
      }
    }
    }  // gather_on
  } else {
    // ---------------------------------------------------------------- epilogue
    // A warp that gives up on a wait keeps walking the tiles (the barriers below must still
    // see all four warps) but skips every wait, load and store.
    const int q = warp & 3;  // the quarter of tensor memory's lanes this warp may read
    const int et = threadIdx.x - (2 + GM_GATHER_WARPS) * 32;  // 0..127 among the epilogue threads
    int cursor = 0, seen = 0, tile_no = 0, chunk_no = 0;
    bool alive = true;
    for (int t = unit; t < total_tiles; t += units, ++tile_no) {
      const Tile tile = locate_tile<BN>(t, tiles0, seen, cursor, s_tile_start, s_rows);
      const Problem& P = args.p[tile.phase];
      const int Nout = P.Nout, colbase = colbase_of(tile);
      const bool swiglu = P.swiglu != 0;
      const T* scale = static_cast<const T*>(P.scale);
      T* C = static_cast<T*>(P.C);
      const unsigned long long* c_table = P.use_table ? s_ctab : nullptr;
      const int buf = tile_no & 1, use_t = tile_no >> 1;
      if (alive && !mbar_wait(&acc_full[buf], use_t & 1, GM_WAIT_NS)) {
        *status = DS_TIMEOUT_MMA;
        alive = false;
      }
      tc_fence_after_sync();
      if constexpr (STREAM) {
        if (swiglu)
          epilogue_stream<T, true, false>(tile, buf, tmem, q, lane, et, alive, chunk_no, Nout, colbase, scale, C, c_table,
                                          group_div, s_begin, s_end, s_map_row[buf], s_map_grp[buf], s_xch, out_tile);
        else if (scale)
          epilogue_stream<T, false, true>(tile, buf, tmem, q, lane, et, alive, chunk_no, Nout, colbase, scale, C, c_table,
                                          group_div, s_begin, s_end, s_map_row[buf], s_map_grp[buf], s_xch, out_tile);
        else
          epilogue_stream<T, false, false>(tile, buf, tmem, q, lane, et, alive, chunk_no, Nout, colbase, scale, C, c_table,
                                           group_div, s_begin, s_end, s_map_row[buf], s_map_grp[buf], s_xch, out_tile);
      } else {
        if (swiglu)
          epilogue_rows<T, SH, true, false>(tile, buf, tmem, q, lane, cr, alive, Nout, colbase, scale, C, c_table, group_div,
                                            s_begin, s_end);
        else if (scale)
          epilogue_rows<T, SH, false, true>(tile, buf, tmem, q, lane, cr, alive, Nout, colbase, scale, C, c_table, group_div,
                                            s_begin, s_end);
        else
          epilogue_rows<T, SH, false, false>(tile, buf, tmem, q, lane, cr, alive, Nout, colbase, scale, C, c_table, group_div,
                                             s_begin, s_end);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0 && alive) {
        if (DUO) mbar_arrive_cluster(cluster_map(&acc_empty[buf], 0));
        else mbar_arrive(&acc_empty[buf]);
      }
      if (NP > 1 && tile.phase == 0) {
        // fused FFN: publish this gate/up tile. All four warps' stores first (barrier), then
        // one thread makes them visible device-wide and counts the tile for its expert.
        fence_proxy_async_all();  // the rows just stored may be read back by TMA
        named_barrier_sync(3, GM_EPI_WARPS * 32);
        if (et == 0) {
          __threadfence();
          atomicAdd(args.ready + tile.e, 1);
        }
      }
      if constexpr (STREAM) {
        if (args.cmb.out && tile.phase == NP - 1)
          epilogue_combine<T>(tile, et, s_begin[tile.e * group_div] + tile.row0, Nout, colbase, args.cmb,
                              static_cast<const T*>(P.C), col_blocks_of(tile.phase), s_final, &s_nfinal);
      }
    }
  }

  // every role ends here; tensor memory goes back before the block exits
  tc_fence_before_sync();
  __syncthreads();
  if (DUO) cluster_sync_all();  // neither CTA leaves while the other may still signal or read it
  if (warp == 1) {
    tc_fence_after_sync();
    if (DUO) tmem_dealloc_pair(tmem, S::TMEM_COLS);
    else tmem_dealloc(tmem, S::TMEM_COLS);
  }
  if (NP > 1 && threadIdx.x == 0) {
    // fused FFN: the last block out clears the per-expert counters for the next launch. In
    // expert-parallel mode it also tells every sender that its results are in place: every
    // block's result stores (into the senders' memory) precede its count here, behind a
    // system-scope fence, and by now no block reads the mailboxes or their metadata any more.
    if (args.ep.arrive) __threadfence_system();
    else __threadfence();
    if (atomicAdd(args.ready + EL, 1) == (int)gridDim.x - 1) {
      for (int e = 0; e <= EL; ++e) args.ready[e] = 0;
      if (args.ep.arrive) {
        __threadfence_system();
        const int epoch = s_epoch;
        for (int r = 0; r < args.ep.R; ++r) st_relaxed_sys(args.ep.ret_flag[r], epoch);  // released by the fence above
        if (args.ep.push.counter) *args.ep.epoch_counter = epoch;  // the combine that follows reads it
        __threadfence();
      } else {
        __threadfence();
      }
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

// Tensor map over activations whose rows are the ranges' rows themselves, as a [rows, K]
// matrix; box = box_rows x 64 k.
static int activation_map(CUtensorMap* map, const void* A, uint64_t rows, uint64_t K, int dtype, int box_rows) {
  EncodeTiledFn encode;
  int rc = encode_fn(&encode);
  if (rc != SY_OK) return rc;
  cuuint64_t dims[2] = {K, rows};
  cuuint64_t strides[1] = {K * 2};
  cuuint32_t box[2] = {GM_ATOM_K, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = encode(map, dtype == SY_DTYPE_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                      2, const_cast<void*>(A), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(SY_ERR_CUDA, "grouped kernel: cuTensorMapEncodeTiled (activations) failed (%d)", (int)r);
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
  int use_table;           // results go through GroupedArgs::c_table (or the table built in expert-parallel mode)
};

struct GroupedArgs {
  ProblemDesc p[2];
  int n_problems;
  const int32_t* begins;   // [ranges] first row of each range
  const int32_t* ends;     // [ranges] one past its last row
  const unsigned long long* c_table;
  int ranges;              // number of row ranges (experts x ranges per expert)
  int group_div;           // ranges per expert: ranges [e*group_div, (e+1)*group_div) are expert e's rows
  int weight_div;          // 0 / 1: a group of ranges is an expert; n: n consecutive groups share an expert's weights
  int forced_shape;        // -1: chosen here; else SH_PAIR / SH_DUO as the caller asked
  int32_t* ready;          // fused FFN scratch: experts + 1 ints, zero before the first launch
  int rows;                // upper bound of the row indices in begins / ends
  int dtype;
  EpArgs ep;               // ep.arrive != nullptr: expert-parallel mode
  CombineArgs cmb;         // cmb.out != nullptr: combine fused into the last epilogue
  cudaStream_t stream;
};

// The grid is persistent and its blocks wait on one another (fused FFN: a down tile waits for
// gate/up tiles that other blocks own), so it must not be larger than what is resident at once.
// Asked once per device and kernel: blocks (or clusters of two) that fit, capped at one per SM
// (pair of SMs). The answer assumes the GPU's shared memory is not held by other resident
// kernels: a caller that runs another shared-memory-hungry kernel concurrently on the same GPU
// must not overlap it with the fused launches.
template <typename T, int SH>
static int resident_units(int sms, int* out) {
  static std::atomic<int> cached[MAX_DEVICES];
  int dev = 0;
  SY_CUDA(cudaGetDevice(&dev));
  int units = cached[dev].load(std::memory_order_acquire);
  if (!units) {
    auto kern = gemm_umma_kernel<T, SH>;
    SY_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GM_SMEM));
    if (SH == SH_DUO) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(sms & ~1);
      cfg.blockDim = dim3(GM_THREADS);
      cfg.dynamicSmemBytes = GM_SMEM;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 2;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      SY_CUDA(cudaOccupancyMaxActiveClusters(&units, kern, &cfg));
      if (units > sms / 2) units = sms / 2;
    } else {
      int per_sm = 0;
      SY_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, GM_THREADS, GM_SMEM));
      units = per_sm >= 1 ? sms : 0;
    }
    if (units < 1) return fail(SY_ERR_CUDA, "grouped kernel: no block of the tcgen05 kernel fits on this device");
    cached[dev].store(units, std::memory_order_release);
  }
  *out = units;
  return SY_OK;
}

template <typename T, int SH>
static int launch_gemm(const GroupedArgs& a) {
  int sms = 0;
  int rc = device_sm_count(&sms);
  if (rc != SY_OK) return rc;
  KernelArgs k;
  memset(&k, 0, sizeof(k));
  k.status = device_status_word();
  if (!k.status) return SY_ERR_CUDA;
  const int weight_div = a.weight_div > 1 ? a.weight_div : 1;
  const int experts = a.ranges / a.group_div / weight_div;
  k.weight_div = weight_div;
  for (int i = 0; i < a.n_problems; ++i) {
    const ProblemDesc& d = a.p[i];
    rc = weight_map(&k.p[i].map, d.B, (uint64_t)experts * (d.swiglu ? 2 : 1) * d.n_out, (uint64_t)d.k_dim, a.dtype,
                    Shape<SH>::BOX_ROWS);
    if (rc != SY_OK) return rc;
    k.p[i].x_tma = !d.a_rows && a.group_div == 1 && a.rows > 0;
    if (k.p[i].x_tma) {
      rc = activation_map(&k.p[i].xmap, d.A, (uint64_t)a.rows, (uint64_t)d.k_dim, a.dtype, Shape<SH>::XR);
      if (rc != SY_OK) return rc;
    }
    k.p[i].A = d.A;
    k.p[i].a_rows = d.a_rows;
    k.p[i].scale = d.scale;
    k.p[i].C = d.C;
    k.p[i].use_table = d.use_table;
    k.p[i].Nout = d.n_out;
    k.p[i].K = d.k_dim;
    k.p[i].swiglu = d.swiglu;
  }
  k.begins = a.begins;
  k.ends = a.ends;
  k.c_table = a.c_table;
  k.ranges = a.ranges;
  k.group_div = a.group_div;
  k.n_problems = a.n_problems;
  k.ready = a.ready;
  k.wait_ns = wait_limit_ns();
  k.ep = a.ep;
  k.cmb = a.cmb;
  int units = 0;
  rc = resident_units<T, SH>(sms, &units);
  if (rc != SY_OK) return rc;
  auto kern = gemm_umma_kernel<T, SH>;
  if (SH == SH_DUO)
    return launch_cluster_kernel(kern, 2, 2 * units, GM_THREADS, GM_SMEM, a.stream, "grouped tcgen05 launch", k);
  return launch_kernel(kern, units, GM_THREADS, GM_SMEM, a.stream, "grouped tcgen05 launch", k);
}

// Which compute tile a batch gets. Measured on a B200 at OLMoE sizes, whole layer, Zipf-skewed
// routing: the CTA-pair tile (256 token rows) wins by 3 % at 1024 rows per expert on average and
// loses 1-6 % at 512 and 128, where more of its rows are padding; uniform routing moves the
// crossover down, and the fused kernel alone gains up to 8 %. So: CTA pairs from 768 rows per
// expert on average, for plain sorted batches (one range per expert, contiguous rows);
// SY_GEMM_TILE=single|pair in the environment (read once) forces one. The two produce the same
// bits (the same MMAs in the same k order).
constexpr int GM_DUO_MIN_MEAN_ROWS = 768;
static std::atomic<int> g_forced_tile{-2};  // -2: not looked up yet; -1: automatic; else a shape
static int forced_tile() {
  int f = g_forced_tile.load(std::memory_order_relaxed);
  if (f == -2) {
    const char* v = getenv("SY_GEMM_TILE");
    f = v && v[0] == 's' ? SH_PAIR : v && v[0] == 'p' ? SH_DUO : -1;
    g_forced_tile.store(f, std::memory_order_relaxed);
  }
  return f;
}
static int compute_shape_for(const GroupedArgs& a, int rows) {
  if (a.forced_shape == SH_PAIR || a.forced_shape == SH_DUO) return a.forced_shape;
  bool plain = a.group_div == 1 && !a.ep.arrive;
  for (int i = 0; i < a.n_problems; ++i) plain = plain && !a.p[i].a_rows && !a.p[i].use_table;
  if (plain && forced_tile() >= 0) return forced_tile();
  return plain && rows >= a.ranges * GM_DUO_MIN_MEAN_ROWS ? SH_DUO : SH_PAIR;
}

// Shared argument checks and dtype dispatch of the tensor-core entry points.
int grouped_umma(bool pair, const char* name, const GroupedArgs& args, int rows) {
  GroupedArgs a = args;
  a.rows = rows;
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
  SY_REQUIRE(a.ep.arrive || (a.begins && a.ends), "%s: null pointer", name);
  for (int i = 0; i < a.n_problems; ++i) {
    const ProblemDesc& d = a.p[i];
    SY_REQUIRE(d.A && d.B && (d.C || d.use_table), "%s: null pointer", name);
    SY_REQUIRE(!d.use_table || a.c_table || a.ep.arrive, "%s: no table of result rows", name);
    SY_REQUIRE(((uintptr_t)d.A % 16 == 0) && ((uintptr_t)d.B % 16 == 0) && ((uintptr_t)d.C % 16 == 0),
               "%s: A, B and C must be 16-byte aligned", name);
  }
  SY_REQUIRE(a.n_problems == 1 || a.ready, "%s: the fused form needs its scratch", name);
  const int shape = pair ? compute_shape_for(a, rows) : SH_STREAM;
  SY_REQUIRE(!a.cmb.out || shape == SH_STREAM, "%s: the fused combine belongs to the streaming shape", name);
  if (a.dtype == SY_DTYPE_F16)
    return shape == SH_DUO    ? launch_gemm<__half, SH_DUO>(a)
           : shape == SH_PAIR ? launch_gemm<__half, SH_PAIR>(a)
                              : launch_gemm<__half, SH_STREAM>(a);
  return shape == SH_DUO    ? launch_gemm<__nv_bfloat16, SH_DUO>(a)
         : shape == SH_PAIR ? launch_gemm<__nv_bfloat16, SH_PAIR>(a)
                            : launch_gemm<__nv_bfloat16, SH_STREAM>(a);
}

static GroupedArgs single(const void* A, const int32_t* a_rows, const void* B, const int32_t* begins,
                          const int32_t* ends, int ranges, int group_div, int n_out, int k_dim, int swiglu,
                          const void* scale, void* C, const unsigned long long* c_table, int dtype, void* stream) {
  GroupedArgs a;
  memset(&a, 0, sizeof(a));
  a.p[0] = ProblemDesc{A, a_rows, B, n_out, k_dim, swiglu, scale, C, c_table != nullptr};
  a.n_problems = 1;
  a.forced_shape = -1;
  a.begins = begins;
  a.ends = ends;
  a.c_table = c_table;
  a.ranges = ranges;
  a.group_div = group_div;
  a.dtype = dtype;
  a.stream = static_cast<cudaStream_t>(stream);
  return a;
}

// Both projections of the expert FFN as one launch's two problems.
static GroupedArgs ffn_pair(const void* x, const int32_t* a_rows, const void* gate_up, const void* down, int hidden,
                            int inter, const void* wsorted, void* act, void* y, int y_through_table, int32_t* scratch,
                            int dtype, void* stream) {
  GroupedArgs a;
  memset(&a, 0, sizeof(a));
  a.p[0] = ProblemDesc{x, a_rows, gate_up, inter, hidden, 1, nullptr, act, 0};
  a.p[1] = ProblemDesc{act, nullptr, down, hidden, inter, 0, wsorted, y, y_through_table};
  a.n_problems = 2;
  a.forced_shape = -1;
  a.ready = scratch;
  a.dtype = dtype;
  a.stream = static_cast<cudaStream_t>(stream);
  return a;
}

}  // namespace sy

extern "C" int sy_force_compute_tile(int tile) {
  SY_REQUIRE(tile >= 0 && tile <= 2, "force_compute_tile: 0 = automatic, 1 = one CTA per tile, 2 = CTA pairs (got %d)", tile);
  sy::g_forced_tile.store(tile == 0 ? -1 : tile == 1 ? sy::SH_PAIR : sy::SH_DUO, std::memory_order_relaxed);
  return SY_OK;
}

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
  GroupedArgs a = ffn_pair(x, a_rows, gate_up, down, hidden, inter, wsorted, act, y, y_table != nullptr, scratch, dtype,
                           stream);
  a.begins = begins;
  a.ends = ends;
  a.c_table = reinterpret_cast<const unsigned long long*>(y_table);
  a.ranges = n_ranges;
  a.group_div = ranges_per_expert;
  return grouped_umma(compute_shape != 0, "expert_ffn", a, rows_bound);
}

extern "C" size_t sy_expert_ffn_combine_scratch_bytes(int n_experts, int n_tokens, int hidden) {
  return sizeof(int32_t) * ((size_t)(n_experts + 1) + (size_t)n_tokens * ((hidden + sy::GM_BM - 1) / sy::GM_BM));
}

extern "C" int sy_expert_ffn_combine(const void* x, const int32_t* token, const void* gate_up, const void* down,
                                     const int32_t* offsets, int n_experts, int rows, int hidden, int inter,
                                     const void* wsorted, void* act, void* y, const int32_t* pos_of, int top_k,
                                     int n_tokens, void* out, int32_t* scratch, int dtype, void* stream) {
  using namespace sy;
  SY_REQUIRE(wsorted && token && pos_of && out && offsets, "expert_ffn_combine: null pointer");
  SY_REQUIRE(top_k >= 1 && top_k <= COMBINE_K && n_tokens >= 0 && rows == n_tokens * top_k,
             "expert_ffn_combine: rows must be n_tokens * top_k with top_k <= %d (got %d, %d, %d)", COMBINE_K, rows,
             n_tokens, top_k);
  SY_REQUIRE((uintptr_t)out % 16 == 0, "expert_ffn_combine: out must be 16-byte aligned");
  GroupedArgs a = ffn_pair(x, token, gate_up, down, hidden, inter, wsorted, act, y, 0, scratch, dtype, stream);
  a.begins = offsets;
  a.ends = offsets + 1;
  a.ranges = n_experts;
  a.group_div = 1;
  a.cmb.out = out;
  a.cmb.token = token;
  a.cmb.pos_of = pos_of;
  a.cmb.arrivals = scratch ? scratch + n_experts + 1 : nullptr;
  a.cmb.k = top_k;
  a.cmb.rows = rows;
  return grouped_umma(false, "expert_ffn_combine", a, rows);
}

namespace sy {
int make_push_args(PushArgs* out, const char* name, const void* h, const int32_t* token, const void* wsorted,
                   const int32_t* offsets, int rows_bound, int experts_per_rank, int n_ranks, int self_rank,
                   int row_bytes, int capacity, void* const* x_dst, void* const* w_dst, int32_t* const* meta_dst,
                   int32_t* const* flag_dst, int32_t* counter, int64_t* stats);
}

extern "C" int sy_ep_expert_ffn(const void* x_mail, const void* w_mail, const int32_t* meta, const int32_t* arrive_flags,
                                int32_t* epoch_counter, int n_ranks, int experts_per_rank, int capacity,
                                const void* gate_up, const void* down, int hidden, int inter, void* act,
                                void* const* y_dst, int32_t* const* ret_flag_dst, int32_t* scratch, int dtype,
                                int compute_shape, const void* push_h, const int32_t* push_token,
                                const void* push_wsorted, const int32_t* push_offsets, int push_rows_bound,
                                int self_rank, void* const* x_dst, void* const* w_dst, int32_t* const* meta_dst,
                                int32_t* const* flag_dst, int32_t* push_counter, int64_t* stats, void* stream) {
  using namespace sy;
  SY_REQUIRE(n_ranks >= 1 && n_ranks <= GM_MAX_RANKS && experts_per_rank >= 1 && capacity >= 1,
             "ep_expert_ffn: 1..%d ranks (got %d)", GM_MAX_RANKS, n_ranks);
  SY_REQUIRE(compute_shape >= 0 && compute_shape <= 4, "ep_expert_ffn: compute_shape 0..4 (got %d)", compute_shape);
  SY_REQUIRE(x_mail && w_mail && meta && arrive_flags && epoch_counter && y_dst && ret_flag_dst,
             "ep_expert_ffn: null pointer");
  GroupedArgs a = ffn_pair(x_mail, nullptr, gate_up, down, hidden, inter, w_mail, act, nullptr, 1, scratch, dtype, stream);
  a.ranges = n_ranks * experts_per_rank;
  a.group_div = n_ranks;
  if (compute_shape >= 3) {
    // every sender's rows of an expert are tiled on their own: a range is then contiguous in the
    // mailbox, its token rows come as TMA boxes, and its tiles follow the expert's other ranges
    // (the weights are re-read from L2)
    a.group_div = 1;
    a.weight_div = n_ranks;
    a.forced_shape = compute_shape == 3 ? SH_PAIR : SH_DUO;
  } else if (compute_shape == 2) {
    a.forced_shape = SH_DUO;
  }
  a.ep.arrive = arrive_flags;
  a.ep.meta = meta;
  a.ep.epoch_counter = epoch_counter;
  a.ep.R = n_ranks;
  a.ep.per = experts_per_rank;
  a.ep.cap = capacity;
  a.ep.out_row_bytes = hidden * 2;
  for (int r = 0; r < n_ranks; ++r) {
    a.ep.y[r] = static_cast<unsigned char*>(y_dst[r]);
    a.ep.ret_flag[r] = ret_flag_dst[r];
    SY_REQUIRE(a.ep.y[r] && a.ep.ret_flag[r] && (uintptr_t)a.ep.y[r] % 16 == 0, "ep_expert_ffn: bad target for rank %d", r);
  }
  if (push_counter) {  // the dispatch runs in this launch's prologue
    int rc = make_push_args(&a.ep.push, "ep_expert_ffn", push_h, push_token, push_wsorted, push_offsets, push_rows_bound,
                            experts_per_rank, n_ranks, self_rank, hidden * 2, capacity, x_dst, w_dst, meta_dst, flag_dst,
                            push_counter, stats);
    if (rc != SY_OK) return rc;
  }
  return grouped_umma(compute_shape != 0, "ep_expert_ffn", a, n_ranks * capacity);
}

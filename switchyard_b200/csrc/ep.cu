// Expert-parallel transport for one process per GPU.
//
// Every rank owns a "window" of device memory that its peers map (CUDA IPC, or peer access in
// one process): a mailbox per sender (rows, router weights, per-expert offsets) and the buffer
// `y` that its own combine reads. One layer, per rank, all on the rank's stream, no host read:
//
//   dispatch    one launch: every sorted row goes to the rank that owns its expert, written
//               straight into that rank's mailbox over NVLink (its own rows too, locally);
//               rebased offsets, the segment's first row and its row count go with it; when the
//               last block is done, a release-store of the layer's epoch into every receiver's
//               arrival flag publishes the mailbox;
//   wait+build  one block waits (bounded) for all senders' arrival flags, then turns the
//               mailboxes' offsets into row groups (expert-major, one group per sender and local
//               expert) and into the table of where each group's results must land: in the
//               sender's `y`, at the rows the sender's own sort gave them;
//   experts     the grouped tcgen05 kernel twice over those groups (csrc/gemm.cu); the second
//               launch's epilogue stores each result row through the table, i.e. directly into
//               the sender's memory: the return trip is fused into the down projection;
//   signal      release-store of the epoch into every sender's return flag;
//   wait        before the combine, one block waits for every owner's return flag.
//
// The five transport steps take three launches: the dispatch's last block goes on to wait and
// build (sy_ep_dispatch_build), and the combine kernel signals and waits before it sums
// (sy_ep_combine). The separate entry points remain for callers that schedule the steps
// themselves.
//
// Flags only ever grow: the epoch is a per-rank layer counter kept in device memory (the
// dispatch's last block advances it, the later kernels of the layer read it), so nothing is
// reset between layers, the host passes no per-layer value, and a layer can be captured in a
// CUDA graph and replayed. All ranks run the same sequence of layers, so their counters agree.
// A mailbox is overwritten by layer n+1's dispatch only after its sender has passed layer n's
// return wait, which the receiver signals after it has finished reading the mailbox.
//
// Every wait is bounded; on expiry the kernel records DS_TIMEOUT_FLAG in the status word and
// lets the stream continue (the layer's output is then garbage and the host raises when it
// next reads the status). Kernels that wait for another rank's flag must run on different GPUs
// than the kernels that set it.
//
// Replaces the per-pair gather + three copies + event of switchyard/ep.py:193-223, the
// per-segment ffn + copy back + event of l.239-262, and the event waits of l.264-272.
#include <string.h>

#include "combine.cuh"

namespace sy {

constexpr int EP_MAX_RANKS = 16;
constexpr int EP_THREADS = 256;
constexpr uint64_t EP_WAIT_NS = 2000000000ull;

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Waits until *flag >= epoch; false after EP_WAIT_NS.
__device__ __forceinline__ bool wait_flag(const int* flag, int epoch) {
  if (ld_acquire_sys(flag) >= epoch) return true;
  const uint64_t start = global_timer_ns();
  for (uint32_t spin = 1;; ++spin) {
    if (ld_acquire_sys(flag) >= epoch) return true;
    if ((spin & 63u) == 0) {
      if (global_timer_ns() - start > EP_WAIT_NS) return false;
      __nanosleep(200);
    }
  }
}

struct ReturnTargets {
  unsigned char* y[EP_MAX_RANKS];   // sender s's result buffer (its window's y)
  int* flag[EP_MAX_RANKS];          // sender s's return flag for this rank
};

// What the dispatch's last block needs to go on with "wait + build" (arrive == nullptr: it does not).
struct BuildArgs {
  const int* arrive;                // this rank's arrival flags, one per sender
  const int* meta;                  // this rank's mailbox metadata, [R][per + 3]
  int* begins;
  int* ends;
  unsigned long long* c_table;
  int out_row_bytes;
};

// Row groups and result destinations from the senders' metadata; groups are expert-major:
// group g = e * R + s holds sender s's rows for local expert e. Run by one block once every
// sender's arrival flag has been seen (ok) or a wait has given up (!ok: empty groups).
__device__ __forceinline__ void build_groups(const int* meta, int per, int R, int cap, const ReturnTargets& rt,
                                             int out_row_bytes, bool ok, int* __restrict__ begins, int* __restrict__ ends,
                                             unsigned long long* __restrict__ c_table) {
  const int meta_ints = per + 3;
  for (int g = threadIdx.x; g < R * per; g += EP_THREADS) {
    const int e = g / R, s = g - e * R;
    const volatile int* m = meta + s * meta_ints;  // written by another GPU: no cached read
    const int lo = ok ? m[e] : 0, hi = ok ? min(m[e + 1], cap) : 0;
    begins[g] = s * cap + lo;
    ends[g] = s * cap + (hi > lo ? hi : lo);
    c_table[g] = reinterpret_cast<unsigned long long>(rt.y[s]) + (unsigned long long)(m[per + 1] + lo) * out_row_bytes;
  }
}

struct DispatchTargets {
  unsigned char* x[EP_MAX_RANKS];   // receiver d's mailbox rows for this sender
  unsigned char* w[EP_MAX_RANKS];   // ... router weights
  int* meta[EP_MAX_RANKS];          // ... [per+1 rebased offsets | first row | row count]
  int* flag[EP_MAX_RANKS];          // ... arrival flag of this sender
};

__global__ void __launch_bounds__(EP_THREADS)
ep_dispatch_kernel(const uint4* __restrict__ h, const int* __restrict__ token, const unsigned short* __restrict__ wsorted,
                   const int* __restrict__ offsets, int M, int per, int R, int vec_per_row, int cap,
                   DispatchTargets tg, int* done_counter, int* epoch_counter, int* status, BuildArgs build,
                   ReturnTargets rt) {
  __shared__ int s_seg[EP_MAX_RANKS + 1];
  __shared__ int s_last;
  __shared__ int s_ok;
  pdl_launch_dependents();
  pdl_wait();  // offsets, token, wsorted come from the sort before this kernel
  if (threadIdx.x <= R) s_seg[threadIdx.x] = offsets[threadIdx.x * per];
  __syncthreads();
  if (blockIdx.x == 0) {
    const int meta_ints = per + 3;
    for (int t = threadIdx.x; t < R * meta_ints; t += EP_THREADS) {
      const int d = t / meta_ints, j = t - d * meta_ints;
      int v;
      if (j <= per) v = offsets[d * per + j] - s_seg[d];
      else if (j == per + 1) v = s_seg[d];
      else v = min(s_seg[d + 1] - s_seg[d], cap);
      tg.meta[d][j] = v;
    }
  }
  for (int row = blockIdx.x; row < M; row += gridDim.x) {
    int d = 0;
    while (d + 1 < R && s_seg[d + 1] <= row) ++d;
    const int r = row - s_seg[d];
    if (r >= cap) {  // cannot happen when the caller respects max_tokens; never write past a mailbox
      if (threadIdx.x == 0) *status = DS_BAD_INDEX;
      continue;
    }
    const uint4* src = h + (size_t)token[row] * vec_per_row;
    uint4* dst = reinterpret_cast<uint4*>(tg.x[d]) + (size_t)r * vec_per_row;
    for (int i = threadIdx.x; i < vec_per_row; i += EP_THREADS) dst[i] = __ldg(src + i);
    if (threadIdx.x == 0) reinterpret_cast<unsigned short*>(tg.w[d])[r] = wsorted[row];
  }
  // last block out publishes the mailboxes
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    s_last = atomicAdd(done_counter, 1) == (int)gridDim.x - 1;
  }
  __syncthreads();
  if (s_last) {
    const int epoch = *epoch_counter + 1;  // only this block reads it; every other block is done
    __threadfence_system();
    if (threadIdx.x < R) st_release_sys(tg.flag[threadIdx.x], epoch);
    __syncthreads();
    if (threadIdx.x == 0) {
      *done_counter = 0;
      *epoch_counter = epoch;  // read by the layer's later kernels, which follow in stream order
      s_ok = 1;
    }
    if (build.arrive) {
      // wait + build in the same launch: this block is the last one with anything to do
      __syncthreads();
      if (threadIdx.x < R && !wait_flag(build.arrive + threadIdx.x, epoch)) {
        *status = DS_TIMEOUT_FLAG;
        s_ok = 0;
      }
      __syncthreads();
      build_groups(build.meta, per, R, cap, rt, build.out_row_bytes, s_ok != 0, build.begins, build.ends, build.c_table);
    }
  }
}

__global__ void __launch_bounds__(EP_THREADS)
ep_wait_build_kernel(const int* arrive_flags, const int* meta, int per, int R, int cap,
                     ReturnTargets rt, int out_row_bytes, const int* epoch_counter, int* __restrict__ begins,
                     int* __restrict__ ends, unsigned long long* __restrict__ c_table, int* status) {
  __shared__ int s_ok;
  pdl_launch_dependents();
  pdl_wait();  // the epoch was advanced by the dispatch before this kernel
  const int epoch = *epoch_counter;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < R && !wait_flag(arrive_flags + threadIdx.x, epoch)) {
    *status = DS_TIMEOUT_FLAG;
    s_ok = 0;
  }
  __syncthreads();
  build_groups(meta, per, R, cap, rt, out_row_bytes, s_ok != 0, begins, ends, c_table);
}

__global__ void ep_signal_kernel(ReturnTargets rt, int R, const int* epoch_counter) {
  pdl_launch_dependents();
  pdl_wait();  // every result row of the kernel before this one has been stored
  const int epoch = *epoch_counter;
  __threadfence_system();
  if (threadIdx.x < R) st_release_sys(rt.flag[threadIdx.x], epoch);
}

__global__ void ep_wait_kernel(const int* flags, int n, const int* epoch_counter, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  const int epoch = *epoch_counter;
  if (threadIdx.x < n && !wait_flag(flags + threadIdx.x, epoch)) *status = DS_TIMEOUT_FLAG;
}

// signal + wait + combine in one launch. Block 0 tells every sender that its results are in
// place (this kernel follows the expert kernel in stream order); then every block waits
// (bounded) until all owners have said the same to this rank, and sums its token's rows.
// A rank without tokens still launches one block: its peers wait for its signal.
template <typename T>
__global__ void __launch_bounds__(COMBINE_THREADS)
ep_combine_kernel(ReturnTargets rt, const int* ret_flags, int R, const int* epoch_counter, const T* __restrict__ y,
                  const int* __restrict__ pos_of, const int* __restrict__ idx, int n_tokens, int k, int H,
                  T* __restrict__ out, int* status) {
  __shared__ int s_row[COMBINE_MAX_K];
  pdl_launch_dependents();
  pdl_wait();  // every result row of the kernel before this one has been stored
  const int epoch = *epoch_counter;
  if (blockIdx.x == 0) {
    __threadfence_system();
    if (threadIdx.x < R) st_release_sys(rt.flag[threadIdx.x], epoch);
  }
  if (threadIdx.x < R && !wait_flag(ret_flags + threadIdx.x, epoch)) *status = DS_TIMEOUT_FLAG;
  __syncthreads();
  if ((int)blockIdx.x < n_tokens) combine_token<T, true>(y, pos_of, idx, k, H, out, blockIdx.x, s_row);
}

}  // namespace sy

namespace sy {
static int dispatch(const void* h, const int32_t* token, const void* wsorted, const int32_t* offsets, int m,
                    int experts_per_rank, int n_ranks, int row_bytes, int capacity, void* const* x_dst, void* const* w_dst,
                    int32_t* const* meta_dst, int32_t* const* flag_dst, int32_t* done_counter, int32_t* epoch_counter,
                    const BuildArgs& build, const ReturnTargets& rt, void* stream) {
  SY_REQUIRE(n_ranks >= 1 && n_ranks <= EP_MAX_RANKS, "ep_dispatch: 1..%d ranks (got %d)", EP_MAX_RANKS, n_ranks);
  SY_REQUIRE(m >= 0 && experts_per_rank >= 1 && capacity >= 1, "ep_dispatch: bad sizes");
  SY_REQUIRE(row_bytes > 0 && row_bytes % 16 == 0, "ep_dispatch: row size must be a multiple of 16 bytes");
  SY_REQUIRE(offsets && x_dst && w_dst && meta_dst && flag_dst && done_counter && epoch_counter,
             "ep_dispatch: null pointer");
  SY_REQUIRE(m == 0 || (h && token && wsorted), "ep_dispatch: null pointer");
  DispatchTargets tg;
  for (int d = 0; d < n_ranks; ++d) {
    tg.x[d] = static_cast<unsigned char*>(x_dst[d]);
    tg.w[d] = static_cast<unsigned char*>(w_dst[d]);
    tg.meta[d] = meta_dst[d];
    tg.flag[d] = flag_dst[d];
    SY_REQUIRE(tg.x[d] && tg.w[d] && tg.meta[d] && tg.flag[d] && (uintptr_t)tg.x[d] % 16 == 0,
               "ep_dispatch: bad target for rank %d", d);
  }
  int sms = 0;
  int rc = device_sm_count(&sms);
  if (rc != SY_OK) return rc;
  int* status = device_status_word();
  if (!status) return SY_ERR_CUDA;
  int blocks = m < 1 ? 1 : (m < sms * 4 ? m : sms * 4);
  return launch_kernel(ep_dispatch_kernel, blocks, EP_THREADS, 0, static_cast<cudaStream_t>(stream), "ep_dispatch launch",
                       static_cast<const uint4*>(h), token, static_cast<const unsigned short*>(wsorted), offsets, m,
                       experts_per_rank, n_ranks, row_bytes / 16, capacity, tg, done_counter, epoch_counter, status, build, rt);
}
}  // namespace sy

extern "C" int sy_ep_dispatch(const void* h, const int32_t* token, const void* wsorted, const int32_t* offsets, int m,
                              int experts_per_rank, int n_ranks, int row_bytes, int capacity, void* const* x_dst,
                              void* const* w_dst, int32_t* const* meta_dst, int32_t* const* flag_dst,
                              int32_t* done_counter, int32_t* epoch_counter, void* stream) {
  sy::BuildArgs none;
  memset(&none, 0, sizeof(none));
  sy::ReturnTargets rt;
  memset(&rt, 0, sizeof(rt));
  return sy::dispatch(h, token, wsorted, offsets, m, experts_per_rank, n_ranks, row_bytes, capacity, x_dst, w_dst, meta_dst,
                      flag_dst, done_counter, epoch_counter, none, rt, stream);
}

extern "C" int sy_ep_dispatch_build(const void* h, const int32_t* token, const void* wsorted, const int32_t* offsets, int m,
                                    int experts_per_rank, int n_ranks, int row_bytes, int capacity, void* const* x_dst,
                                    void* const* w_dst, int32_t* const* meta_dst, int32_t* const* flag_dst,
                                    int32_t* done_counter, int32_t* epoch_counter, const int32_t* arrive_flags,
                                    const int32_t* meta, void* const* y_dst, int out_row_bytes, int32_t* begins,
                                    int32_t* ends, uint64_t* c_table, void* stream) {
  using namespace sy;
  SY_REQUIRE(n_ranks >= 1 && n_ranks <= EP_MAX_RANKS, "ep_dispatch_build: 1..%d ranks (got %d)", EP_MAX_RANKS, n_ranks);
  SY_REQUIRE(arrive_flags && meta && y_dst && begins && ends && c_table, "ep_dispatch_build: null pointer");
  BuildArgs build{arrive_flags, meta, begins, ends, reinterpret_cast<unsigned long long*>(c_table), out_row_bytes};
  ReturnTargets rt;
  memset(&rt, 0, sizeof(rt));
  for (int s = 0; s < n_ranks; ++s) {
    rt.y[s] = static_cast<unsigned char*>(y_dst[s]);
    SY_REQUIRE(rt.y[s], "ep_dispatch_build: null result buffer for rank %d", s);
  }
  return dispatch(h, token, wsorted, offsets, m, experts_per_rank, n_ranks, row_bytes, capacity, x_dst, w_dst, meta_dst,
                  flag_dst, done_counter, epoch_counter, build, rt, stream);
}

extern "C" int sy_ep_wait_build(const int32_t* arrive_flags, const int32_t* meta, int experts_per_rank, int n_ranks,
                                int capacity, void* const* y_dst, int out_row_bytes, const int32_t* epoch_counter,
                                int32_t* begins, int32_t* ends, uint64_t* c_table, void* stream) {
  using namespace sy;
  SY_REQUIRE(n_ranks >= 1 && n_ranks <= EP_MAX_RANKS && experts_per_rank >= 1, "ep_wait_build: bad sizes");
  SY_REQUIRE(arrive_flags && meta && y_dst && begins && ends && c_table && epoch_counter, "ep_wait_build: null pointer");
  ReturnTargets rt;
  for (int s = 0; s < n_ranks; ++s) {
    rt.y[s] = static_cast<unsigned char*>(y_dst[s]);
    rt.flag[s] = nullptr;
    SY_REQUIRE(rt.y[s], "ep_wait_build: null result buffer for rank %d", s);
  }
  int* status = device_status_word();
  if (!status) return SY_ERR_CUDA;
  return launch_kernel(ep_wait_build_kernel, 1, EP_THREADS, 0, static_cast<cudaStream_t>(stream), "ep_wait_build launch",
                       arrive_flags, meta, experts_per_rank, n_ranks, capacity, rt, out_row_bytes, epoch_counter, begins,
                       ends, reinterpret_cast<unsigned long long*>(c_table), status);
}

extern "C" int sy_ep_signal(int32_t* const* flag_dst, int n_ranks, const int32_t* epoch_counter, void* stream) {
  using namespace sy;
  SY_REQUIRE(n_ranks >= 1 && n_ranks <= EP_MAX_RANKS && flag_dst && epoch_counter, "ep_signal: bad arguments");
  ReturnTargets rt;
  for (int s = 0; s < n_ranks; ++s) {
    rt.y[s] = nullptr;
    rt.flag[s] = flag_dst[s];
    SY_REQUIRE(rt.flag[s], "ep_signal: null flag for rank %d", s);
  }
  return launch_kernel(ep_signal_kernel, 1, 32, 0, static_cast<cudaStream_t>(stream), "ep_signal launch", rt, n_ranks,
                       epoch_counter);
}

extern "C" int sy_ep_wait(const int32_t* flags, int n, const int32_t* epoch_counter, void* stream) {
  using namespace sy;
  SY_REQUIRE(flags && epoch_counter && n >= 1 && n <= 32, "ep_wait: bad arguments");
  int* status = device_status_word();
  if (!status) return SY_ERR_CUDA;
  return launch_kernel(ep_wait_kernel, 1, 32, 0, static_cast<cudaStream_t>(stream), "ep_wait launch", flags, n,
                       epoch_counter, status);
}

extern "C" int sy_ep_combine(int32_t* const* flag_dst, const int32_t* ret_flags, int n_ranks, const int32_t* epoch_counter,
                             const void* y, const int32_t* pos_of, const int32_t* idx, int n_tokens, int top_k, int hidden,
                             void* out, int dtype, void* stream) {
  using namespace sy;
  SY_REQUIRE(n_ranks >= 1 && n_ranks <= EP_MAX_RANKS && flag_dst && ret_flags && epoch_counter, "ep_combine: bad arguments");
  SY_REQUIRE(n_tokens >= 0 && top_k >= 1 && top_k <= COMBINE_MAX_K, "ep_combine: top_k must be 1..8 (got %d)", top_k);
  SY_REQUIRE(hidden > 0 && hidden % 8 == 0, "ep_combine: hidden must be a multiple of 8 (got %d)", hidden);
  SY_REQUIRE(dtype == SY_DTYPE_F16 || dtype == SY_DTYPE_BF16, "ep_combine: dtype must be f16 or bf16");
  SY_REQUIRE(n_tokens == 0 || (y && pos_of && idx && out), "ep_combine: null pointer");
  SY_REQUIRE(((uintptr_t)y % 16 == 0) && ((uintptr_t)out % 16 == 0), "ep_combine: y and out must be 16-byte aligned");
  ReturnTargets rt;
  memset(&rt, 0, sizeof(rt));
  for (int s = 0; s < n_ranks; ++s) {
    rt.flag[s] = flag_dst[s];
    SY_REQUIRE(rt.flag[s], "ep_combine: null flag for rank %d", s);
  }
  int* status = device_status_word();
  if (!status) return SY_ERR_CUDA;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int blocks = n_tokens > 0 ? n_tokens : 1;  // a rank without tokens still signals
  if (dtype == SY_DTYPE_F16)
    return launch_kernel(ep_combine_kernel<__half>, blocks, COMBINE_THREADS, 0, s, "ep_combine launch", rt, ret_flags,
                         n_ranks, epoch_counter, static_cast<const __half*>(y), pos_of, idx, n_tokens, top_k, hidden,
                         static_cast<__half*>(out), status);
  return launch_kernel(ep_combine_kernel<__nv_bfloat16>, blocks, COMBINE_THREADS, 0, s, "ep_combine launch", rt, ret_flags,
                       n_ranks, epoch_counter, static_cast<const __nv_bfloat16*>(y), pos_of, idx, n_tokens, top_k, hidden,
                       static_cast<__nv_bfloat16*>(out), status);
}

// ---- CUDA IPC helpers: how the ranks' windows are mapped into one another (set-up time) ----
extern "C" int sy_ipc_export(void* ptr, unsigned char* handle64, uint64_t* offset_out) {
  using namespace sy;
  SY_REQUIRE(ptr && handle64 && offset_out, "ipc_export: null pointer");
  // the handle names the whole allocation that contains ptr; find its base
  typedef int (*RangeFn)(unsigned long long*, size_t*, unsigned long long);
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  SY_CUDA(cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &q));
  if (q != cudaDriverEntryPointSuccess || !fn) return fail(SY_ERR_CUDA, "ipc_export: no cuMemGetAddressRange");
  unsigned long long base = 0;
  size_t size = 0;
  int r = reinterpret_cast<RangeFn>(fn)(&base, &size, (unsigned long long)(uintptr_t)ptr);
  if (r != 0) return fail(SY_ERR_CUDA, "ipc_export: cuMemGetAddressRange failed (%d)", r);
  cudaIpcMemHandle_t h;
  SY_CUDA(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>((uintptr_t)base)));
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(handle64, &h, 64);
  *offset_out = (uint64_t)((uintptr_t)ptr - (uintptr_t)base);
  return SY_OK;
}

extern "C" int sy_ipc_open(const unsigned char* handle64, uint64_t offset, void** ptr_out) {
  using namespace sy;
  SY_REQUIRE(handle64 && ptr_out, "ipc_open: null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* base = nullptr;
  SY_CUDA(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
  *ptr_out = static_cast<unsigned char*>(base) + offset;
  return SY_OK;
}

extern "C" int sy_ipc_close(void* ptr, uint64_t offset) {
  using namespace sy;
  if (!ptr) return SY_OK;
  SY_CUDA(cudaIpcCloseMemHandle(static_cast<unsigned char*>(ptr) - offset));
  return SY_OK;
}

// Expert-parallel transport: how sorted rows reach the GPU that owns their expert and how the
// results come back, without the host taking part.
//
// Every rank owns a "window" of device memory that its peers can address (peer access inside one
// process, CUDA IPC between processes): a mailbox per sender (rows, router weights, per-expert
// offsets), flags, and the buffer `y` that its own combine reads. One layer, per rank, on the
// rank's stream:
//
//   dispatch    (sy_ep_dispatch) every sorted row goes to the rank that owns its expert, written
//               straight into that rank's mailbox over NVLink (the rank's own rows too, locally),
//               together with the rebased per-expert offsets, the segment's first row and its row
//               count. Blocks count the rows they have stored per destination; the block that
//               completes a destination release-stores the layer's epoch into that receiver's
//               arrival flag at once, so a receiver never waits for rows bound elsewhere;
//   experts     (sy_ep_expert_ffn, csrc/gemm.cu) the fused expert kernel waits for all senders'
//               arrival flags itself, builds its row ranges from the mailboxes' offsets in shared
//               memory, and its down-projection epilogue stores each result row into the SENDER's
//               `y` at the row the sender's own sort gave it: the return trip is part of the
//               epilogue. The block that stores the last result tile release-stores the epoch
//               into every sender's return flag;
//   combine     (sy_ep_combine) waits for every owner's return flag, then sums each token's rows.
//
// Flags only ever grow: the epoch is a per-rank layer counter kept in device memory (the
// dispatch's last block advances it, the later kernels of the layer read it), so nothing is
// reset between layers, the host passes no per-layer value, and a layer can be captured in a
// CUDA graph and replayed. All ranks run the same sequence of layers, so their counters agree.
// A mailbox is overwritten by layer n+1's dispatch only after its sender has passed layer n's
// return wait, which the receiver signals after it has finished reading the mailbox.
//
// Every wait is bounded (sy_set_wait_limit_ns); on expiry the kernel records DS_TIMEOUT_FLAG in
// the status word and lets the stream continue (the layer's output is then garbage and the host
// raises when it next reads the status). Kernels that wait for another rank's flag must run on
// different GPUs than the kernels that set it, unless the caller orders them itself so that
// every flag is already set when its waiter starts (ranks sharing one GPU: stream events).
//
// Replaces the per-pair gather + three copies + event of switchyard/ep.py:193-223, the
// per-segment ffn + copy back + event of l.239-262, and the event waits of l.264-272.
#include <string.h>

#include "combine.cuh"

namespace sy {

constexpr int EP_MAX_RANKS = 16;
constexpr int EP_THREADS = 256;

struct DispatchTargets {
  unsigned char* x[EP_MAX_RANKS];   // receiver d's mailbox rows for this sender
  unsigned char* w[EP_MAX_RANKS];   // ... router weights
  int* meta[EP_MAX_RANKS];          // ... [per+1 rebased offsets | first row | row count]
  int* flag[EP_MAX_RANKS];          // ... arrival flag of this sender
};

// counters: [R] units stored per destination (a row counts one, the metadata one), [1] blocks
// that have finished; all zero between launches. stats: [0] rows sent to other ranks, [1] rows
// kept, accumulated over the layers (read by the host when it wants them).
__global__ void __launch_bounds__(EP_THREADS)
ep_dispatch_kernel(const uint4* __restrict__ h, const int* __restrict__ token, const unsigned short* __restrict__ wsorted,
                   const int* __restrict__ offsets, int per, int R, int self, int vec_per_row, int cap, DispatchTargets tg,
                   int* counters, int* epoch_counter, long long* stats, int* status) {
  __shared__ int s_seg[EP_MAX_RANKS + 1];
  pdl_launch_dependents();
  pdl_wait();  // offsets, token, wsorted come from the sort before this kernel
  if ((int)threadIdx.x <= R) s_seg[threadIdx.x] = offsets[threadIdx.x * per];
  __syncthreads();
  const int epoch = *epoch_counter + 1;  // advanced by the last block out, after every block has read it
  const int rows = s_seg[R];

  // One more unit of destination d is in place: n rows (or the metadata). The caller's stores
  // come first (block barrier), then a system-scope fence, then the count; whoever completes
  // the destination publishes it.
  auto stored = [&](int d, int n) {
    __syncthreads();
    if (threadIdx.x == 0 && n > 0) {
      __threadfence_system();
      const int target = s_seg[d + 1] - s_seg[d] + 1;
      if (atomicAdd(counters + d, n) + n == target) st_release_sys(tg.flag[d], epoch);
    }
  };

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
    __syncthreads();
    if ((int)threadIdx.x < R) {  // one thread per destination: fence, count the metadata, maybe publish
      __threadfence_system();
      const int d = threadIdx.x, target = s_seg[d + 1] - s_seg[d] + 1;
      if (atomicAdd(counters + d, 1) + 1 == target) st_release_sys(tg.flag[d], epoch);
    }
    if (threadIdx.x == 0 && stats) {
      const int kept = s_seg[self + 1] - s_seg[self];
      stats[0] += rows - kept;
      stats[1] += kept;
    }
  }
  int cur = -1, n_cur = 0, d = 0;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    while (d + 1 < R && s_seg[d + 1] <= row) ++d;
    if (d != cur) {
      if (cur >= 0) stored(cur, n_cur);
      cur = d;
      n_cur = 0;
    }
    ++n_cur;
    const int r = row - s_seg[d];
    if (r >= cap) {  // cannot happen when the caller respects its capacity; never write past a mailbox
      if (threadIdx.x == 0) *status = DS_BAD_INDEX;
      continue;
    }
    const uint4* src = h + (size_t)token[row] * vec_per_row;
    uint4* dst = reinterpret_cast<uint4*>(tg.x[d]) + (size_t)r * vec_per_row;
    for (int i = threadIdx.x; i < vec_per_row; i += EP_THREADS) dst[i] = __ldg(src + i);
    if (threadIdx.x == 0) reinterpret_cast<unsigned short*>(tg.w[d])[r] = wsorted[row];
  }
  if (cur >= 0) stored(cur, n_cur);
  // the last block out advances the epoch and leaves the counters at zero for the next layer
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(counters + R, 1) == (int)gridDim.x - 1) {
      for (int i = 0; i <= R; ++i) counters[i] = 0;
      *epoch_counter = epoch;  // read by the layer's later kernels, which follow in stream order
      __threadfence();
    }
  }
}

__global__ void ep_wait_kernel(const int* flags, int n, const int* epoch_counter, int epoch_offset, int* status,
                               unsigned long long wait_ns) {
  pdl_launch_dependents();
  pdl_wait();
  const int epoch = *epoch_counter + epoch_offset;
  if ((int)threadIdx.x < n && !wait_flag(flags + threadIdx.x, epoch, wait_ns)) *status = DS_TIMEOUT_FLAG;
}

// wait + combine in one launch: every block waits (bounded) until all owners have stored this
// rank's results (their expert kernels signal), then sums its token's rows. y is read with L1
// bypassed: its rows were stored by other GPUs.
template <typename T>
__global__ void __launch_bounds__(COMBINE_THREADS)
ep_combine_kernel(const int* ret_flags, int R, const int* epoch_counter, const T* __restrict__ y,
                  const int* __restrict__ pos_of, const int* __restrict__ idx, int n_tokens, int k, int H,
                  T* __restrict__ out, int* status, unsigned long long wait_ns) {
  __shared__ int s_row[COMBINE_MAX_K];
  pdl_launch_dependents();
  pdl_wait();
  const int epoch = *epoch_counter;
  if ((int)threadIdx.x < R && !wait_flag(ret_flags + threadIdx.x, epoch, wait_ns)) *status = DS_TIMEOUT_FLAG;
  __syncthreads();
  if ((int)blockIdx.x < n_tokens) combine_token<T, true>(y, pos_of, idx, k, H, out, blockIdx.x, s_row, n_tokens * k);
}

}  // namespace sy

extern "C" size_t sy_ep_dispatch_scratch_bytes(int n_ranks) { return sizeof(int32_t) * (size_t)(n_ranks + 1); }

extern "C" int sy_ep_dispatch(const void* h, const int32_t* token, const void* wsorted, const int32_t* offsets,
                              int rows_bound, int experts_per_rank, int n_ranks, int self_rank, int row_bytes,
                              int capacity, void* const* x_dst, void* const* w_dst, int32_t* const* meta_dst,
                              int32_t* const* flag_dst, int32_t* counters, int32_t* epoch_counter, int64_t* stats,
                              void* stream) {
  using namespace sy;
  SY_REQUIRE(n_ranks >= 1 && n_ranks <= EP_MAX_RANKS, "ep_dispatch: 1..%d ranks (got %d)", EP_MAX_RANKS, n_ranks);
  SY_REQUIRE(self_rank >= 0 && self_rank < n_ranks, "ep_dispatch: rank %d of %d", self_rank, n_ranks);
  SY_REQUIRE(rows_bound >= 0 && experts_per_rank >= 1 && capacity >= 1, "ep_dispatch: bad sizes");
  SY_REQUIRE(row_bytes > 0 && row_bytes % 16 == 0, "ep_dispatch: row size must be a multiple of 16 bytes");
  SY_REQUIRE(offsets && x_dst && w_dst && meta_dst && flag_dst && counters && epoch_counter, "ep_dispatch: null pointer");
  SY_REQUIRE(rows_bound == 0 || (h && token && wsorted), "ep_dispatch: null pointer");
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
  // rows_bound (the caller's sorted rows, known on the host) only sizes the grid; the kernel
  // takes the real row count from offsets
  const int blocks = rows_bound < 1 ? 1 : (rows_bound < sms * 4 ? rows_bound : sms * 4);
  return launch_kernel(ep_dispatch_kernel, blocks, EP_THREADS, 0, static_cast<cudaStream_t>(stream), "ep_dispatch launch",
                       static_cast<const uint4*>(h), token, static_cast<const unsigned short*>(wsorted), offsets,
                       experts_per_rank, n_ranks, self_rank, row_bytes / 16, capacity, tg, counters, epoch_counter,
                       reinterpret_cast<long long*>(stats), status);
}

extern "C" int sy_ep_wait(const int32_t* flags, int n, const int32_t* epoch_counter, int epoch_offset, void* stream) {
  using namespace sy;
  SY_REQUIRE(flags && epoch_counter && n >= 1 && n <= 32, "ep_wait: bad arguments");
  int* status = device_status_word();
  if (!status) return SY_ERR_CUDA;
  return launch_kernel(ep_wait_kernel, 1, 32, 0, static_cast<cudaStream_t>(stream), "ep_wait launch", flags, n,
                       epoch_counter, epoch_offset, status, (unsigned long long)wait_limit_ns());
}

extern "C" int sy_ep_combine(const int32_t* ret_flags, int n_ranks, const int32_t* epoch_counter, const void* y,
                             const int32_t* pos_of, const int32_t* idx, int n_tokens, int top_k, int hidden, void* out,
                             int dtype, void* stream) {
  using namespace sy;
  SY_REQUIRE(n_ranks >= 1 && n_ranks <= EP_MAX_RANKS && ret_flags && epoch_counter, "ep_combine: bad arguments");
  SY_REQUIRE(n_tokens >= 0 && top_k >= 1 && top_k <= COMBINE_MAX_K, "ep_combine: top_k must be 1..8 (got %d)", top_k);
  SY_REQUIRE(hidden > 0 && hidden % 8 == 0, "ep_combine: hidden must be a multiple of 8 (got %d)", hidden);
  SY_REQUIRE(dtype == SY_DTYPE_F16 || dtype == SY_DTYPE_BF16, "ep_combine: dtype must be f16 or bf16");
  SY_REQUIRE(n_tokens == 0 || (y && pos_of && idx && out), "ep_combine: null pointer");
  SY_REQUIRE(((uintptr_t)y % 16 == 0) && ((uintptr_t)out % 16 == 0), "ep_combine: y and out must be 16-byte aligned");
  int* status = device_status_word();
  if (!status) return SY_ERR_CUDA;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned long long wait_ns = wait_limit_ns();
  const int blocks = n_tokens > 0 ? n_tokens : 1;  // a rank without tokens still waits: its mailbox slots are reused
  if (dtype == SY_DTYPE_F16)
    return launch_kernel(ep_combine_kernel<__half>, blocks, COMBINE_THREADS, 0, s, "ep_combine launch", ret_flags, n_ranks,
                         epoch_counter, static_cast<const __half*>(y), pos_of, idx, n_tokens, top_k, hidden,
                         static_cast<__half*>(out), status, wait_ns);
  return launch_kernel(ep_combine_kernel<__nv_bfloat16>, blocks, COMBINE_THREADS, 0, s, "ep_combine launch", ret_flags,
                       n_ranks, epoch_counter, static_cast<const __nv_bfloat16*>(y), pos_of, idx, n_tokens, top_k, hidden,
                       static_cast<__nv_bfloat16*>(out), status, wait_ns);
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

// Expert-parallel transport: how sorted rows reach the GPU that owns their expert and how the
// results come back, without the host taking part.
//
// Every rank owns a "window" of device memory that its peers can address (peer access inside one
// process, CUDA IPC between processes): a mailbox per sender (rows, router weights, per-expert
// offsets), flags, and the buffer `y` that its own combine reads. One layer, per rank, on the
// rank's stream:
//
//   dispatch    (csrc/ep_push.cuh) every sorted row goes to the rank that owns its expert, written
//               straight into that rank's mailbox over NVLink (the rank's own rows too, locally),
//               together with the rebased per-expert offsets, the segment's first row and its row
//               count; the block that stores last release-stores the layer's epoch into every
//               receiver's arrival flag. It runs in the prologue of the expert kernel (one launch
//               less on the critical path), or as a launch of its own (sy_ep_dispatch) for callers
//               that must order the steps themselves;
//   experts     (sy_ep_expert_ffn, csrc/gemm.cu) the fused expert kernel waits for all senders'
//               arrival flags itself, builds its row ranges from the mailboxes' offsets in shared
//               memory, and its down-projection epilogue stores each result row into the SENDER's
//               `y` at the row the sender's own sort gave it: the return trip is part of the
//               epilogue. The last block out release-stores the epoch into every sender's return
//               flag;
//   combine     (sy_ep_combine) waits for every owner's return flag, then sums each token's rows.
//
// Flags only ever grow: the epoch is a per-rank layer counter kept in device memory (advanced
// when the dispatch is complete, read by the layer's later kernels), so nothing is
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
#include <stdlib.h>
#include <string.h>

#include "combine.cuh"
#include "ep_push.cuh"

namespace sy {

constexpr int EP_THREADS = 256;

// The dispatch as a launch of its own (the expert kernel can also do it in its prologue, see
// sy_ep_expert_ffn): push, and the block that completes it advances the epoch that the layer's
// later kernels read.
__global__ void __launch_bounds__(EP_THREADS)
ep_dispatch_kernel(PushArgs p, int* epoch_counter, int* status) {
  __shared__ int s_seg[EP_MAX_RANKS + 1];
  __shared__ int s_done[2];
  pdl_launch_dependents();
  pdl_wait();  // offsets, token, wsorted come from the sort before this kernel
  const int epoch = *epoch_counter + 1;  // advanced below, once everything is stored
  if (push_rows(p, epoch, status, s_seg, s_done) && threadIdx.x == 0) {
    *epoch_counter = epoch;
    __threadfence();
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
                  T* __restrict__ out, const T* __restrict__ residual, int* status, unsigned long long wait_ns) {
  __shared__ int s_row[COMBINE_MAX_K];
  pdl_launch_dependents();
  pdl_wait();
  const int epoch = *epoch_counter;
  if ((int)threadIdx.x < R && !wait_flag(ret_flags + threadIdx.x, epoch, wait_ns)) *status = DS_TIMEOUT_FLAG;
  __syncthreads();
  if ((int)blockIdx.x < n_tokens) combine_token<T, true>(y, pos_of, idx, k, H, out, blockIdx.x, s_row, n_tokens * k, residual);
}

}  // namespace sy

namespace sy {
// Fills and checks the dispatch arguments shared by sy_ep_dispatch and sy_ep_expert_ffn.
int make_push_args(PushArgs* out, const char* name, const void* h, const int32_t* token, const void* wsorted,
                   const int32_t* offsets, int rows_bound, int experts_per_rank, int n_ranks, int self_rank,
                   int row_bytes, int capacity, void* const* x_dst, void* const* w_dst, int32_t* const* meta_dst,
                   int32_t* const* flag_dst, int32_t* counter, int64_t* stats) {
  SY_REQUIRE(n_ranks >= 1 && n_ranks <= EP_MAX_RANKS, "%s: 1..%d ranks (got %d)", name, EP_MAX_RANKS, n_ranks);
  SY_REQUIRE(self_rank >= 0 && self_rank < n_ranks, "%s: rank %d of %d", name, self_rank, n_ranks);
  SY_REQUIRE(rows_bound >= 0 && experts_per_rank >= 1 && capacity >= 1, "%s: bad sizes", name);
  SY_REQUIRE(row_bytes > 0 && row_bytes % 16 == 0, "%s: row size must be a multiple of 16 bytes", name);
  SY_REQUIRE(offsets && x_dst && w_dst && meta_dst && flag_dst && counter, "%s: null pointer", name);
  SY_REQUIRE(rows_bound == 0 || (h && token && wsorted), "%s: null pointer", name);
  PushArgs p;
  memset(&p, 0, sizeof(p));
  p.h = static_cast<const uint4*>(h);
  p.token = token;
  p.wsorted = static_cast<const unsigned short*>(wsorted);
  p.offsets = offsets;
  p.per = experts_per_rank;
  p.R = n_ranks;
  p.self = self_rank;
  p.vec_per_row = row_bytes / 16;
  p.cap = capacity;
  for (int d = 0; d < n_ranks; ++d) {
    p.x[d] = static_cast<unsigned char*>(x_dst[d]);
    p.w[d] = static_cast<unsigned char*>(w_dst[d]);
    p.meta[d] = meta_dst[d];
    p.flag[d] = flag_dst[d];
    SY_REQUIRE(p.x[d] && p.w[d] && p.meta[d] && p.flag[d] && (uintptr_t)p.x[d] % 16 == 0, "%s: bad target for rank %d",
               name, d);
  }
  p.counter = counter;
  // SY_PUSH_FENCE=sys in the environment (read once): every block fences at system scope before it
  // counts its rows, instead of at GPU scope with one system-scope fence by the completing block
  // (3 us slower per layer on a B200; kept as a conservative switch)
  static const int fence_sys = [] {
    const char* v = getenv("SY_PUSH_FENCE");
    return v && v[0] == 's' ? 1 : 0;
  }();
  p.block_fence_sys = fence_sys;
  p.stats = reinterpret_cast<long long*>(stats);
  *out = p;
  return SY_OK;
}
}  // namespace sy

extern "C" size_t sy_ep_dispatch_scratch_bytes(int n_ranks) { return sizeof(int32_t); }

extern "C" int sy_ep_dispatch(const void* h, const int32_t* token, const void* wsorted, const int32_t* offsets,
                              int rows_bound, int experts_per_rank, int n_ranks, int self_rank, int row_bytes,
                              int capacity, void* const* x_dst, void* const* w_dst, int32_t* const* meta_dst,
                              int32_t* const* flag_dst, int32_t* counters, int32_t* epoch_counter, int64_t* stats,
                              void* stream) {
  using namespace sy;
  SY_REQUIRE(epoch_counter, "ep_dispatch: null pointer");
  PushArgs p;
  int rc = make_push_args(&p, "ep_dispatch", h, token, wsorted, offsets, rows_bound, experts_per_rank, n_ranks, self_rank,
                          row_bytes, capacity, x_dst, w_dst, meta_dst, flag_dst, counters, stats);
  if (rc != SY_OK) return rc;
  int sms = 0;
  rc = device_sm_count(&sms);
  if (rc != SY_OK) return rc;
  int* status = device_status_word();
  if (!status) return SY_ERR_CUDA;
  // rows_bound (the caller's sorted rows, known on the host) only sizes the grid; the kernel
  // takes the real row count from offsets
  const int per_block = EP_THREADS / 32;  // a warp per row
  const int want = (rows_bound + per_block - 1) / per_block;
  const int blocks = want < 1 ? 1 : (want < sms * 4 ? want : sms * 4);
  return launch_kernel(ep_dispatch_kernel, blocks, EP_THREADS, 0, static_cast<cudaStream_t>(stream), "ep_dispatch launch",
                       p, epoch_counter, status);
}

extern "C" int sy_ep_wait(const int32_t* flags, int n, const int32_t* epoch_counter, int epoch_offset, void* stream) {
  using namespace sy;
  SY_REQUIRE(flags && epoch_counter && n >= 1 && n <= 32, "ep_wait: bad arguments");
  int* status = device_status_word();
  if (!status) return SY_ERR_CUDA;
  return launch_kernel(ep_wait_kernel, 1, 32, 0, static_cast<cudaStream_t>(stream), "ep_wait launch", flags, n,
                       epoch_counter, epoch_offset, status, (unsigned long long)wait_limit_ns());
}

namespace sy {
static int ep_combine_launch(const char* name, const int32_t* ret_flags, int n_ranks, const int32_t* epoch_counter,
                             const void* y, const int32_t* pos_of, const int32_t* idx, int n_tokens, int top_k,
                             int hidden, const void* residual, bool wants_residual, void* out, int dtype, void* stream) {
  SY_REQUIRE(n_ranks >= 1 && n_ranks <= EP_MAX_RANKS && ret_flags && epoch_counter, "%s: bad arguments", name);
  SY_REQUIRE(n_tokens >= 0 && top_k >= 1 && top_k <= COMBINE_MAX_K, "%s: top_k must be 1..8 (got %d)", name, top_k);
  SY_REQUIRE(hidden > 0 && hidden % 8 == 0, "%s: hidden must be a multiple of 8 (got %d)", name, hidden);
  SY_REQUIRE(dtype == SY_DTYPE_F16 || dtype == SY_DTYPE_BF16, "%s: dtype must be f16 or bf16", name);
  SY_REQUIRE(n_tokens == 0 || (y && pos_of && idx && out && (residual || !wants_residual)), "%s: null pointer", name);
  SY_REQUIRE(((uintptr_t)y % 16 == 0) && ((uintptr_t)out % 16 == 0) && ((uintptr_t)residual % 16 == 0),
             "%s: y, residual and out must be 16-byte aligned", name);
  int* status = device_status_word();
  if (!status) return SY_ERR_CUDA;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned long long wait_ns = wait_limit_ns();
  const int blocks = n_tokens > 0 ? n_tokens : 1;  // a rank without tokens still waits: its mailbox slots are reused
  if (dtype == SY_DTYPE_F16)
    return launch_kernel(ep_combine_kernel<__half>, blocks, COMBINE_THREADS, 0, s, "ep_combine launch", ret_flags, n_ranks,
                         epoch_counter, static_cast<const __half*>(y), pos_of, idx, n_tokens, top_k, hidden,
                         static_cast<__half*>(out), static_cast<const __half*>(residual), status, wait_ns);
  return launch_kernel(ep_combine_kernel<__nv_bfloat16>, blocks, COMBINE_THREADS, 0, s, "ep_combine launch", ret_flags,
                       n_ranks, epoch_counter, static_cast<const __nv_bfloat16*>(y), pos_of, idx, n_tokens, top_k, hidden,
                       static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(residual), status, wait_ns);
}
}  // namespace sy

extern "C" int sy_ep_combine(const int32_t* ret_flags, int n_ranks, const int32_t* epoch_counter, const void* y,
                             const int32_t* pos_of, const int32_t* idx, int n_tokens, int top_k, int hidden, void* out,
                             int dtype, void* stream) {
  return sy::ep_combine_launch("ep_combine", ret_flags, n_ranks, epoch_counter, y, pos_of, idx, n_tokens, top_k, hidden,
                               nullptr, false, out, dtype, stream);
}

extern "C" int sy_ep_combine_add(const int32_t* ret_flags, int n_ranks, const int32_t* epoch_counter, const void* y,
                                 const int32_t* pos_of, const int32_t* idx, int n_tokens, int top_k, int hidden,
                                 const void* residual, void* out, int dtype, void* stream) {
  return sy::ep_combine_launch("ep_combine_add", ret_flags, n_ranks, epoch_counter, y, pos_of, idx, n_tokens, top_k,
                               hidden, residual, true, out, dtype, stream);
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

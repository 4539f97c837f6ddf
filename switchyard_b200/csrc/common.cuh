// Shared pieces of the sm_100a MoE kernels: status codes, the thread-local error message,
// 16-bit type helpers, and thin wrappers over the PTX this library uses directly
// (mbarrier, bulk async copies, tcgen05 / tensor memory).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/switchyard_b200.h"

namespace sy {

// ---- host-side error plumbing -------------------------------------------------------------
void set_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);
int check_cuda(cudaError_t e, const char* what);
int device_sm_count(int* out);           // SMs of the current device (cached per device)
int current_device_slot(int* out);       // current device ordinal, < SY_MAX_DEVICES
int* device_status_word();               // device address of this device's kernel status word
uint64_t wait_limit_ns();                // how long kernels wait for a flag or barrier before giving up

#define SY_CUDA(expr)                                           \
  do {                                                          \
    int _sy_rc = ::sy::check_cuda((expr), #expr);               \
    if (_sy_rc != SY_OK) return _sy_rc;                         \
  } while (0)

#define SY_REQUIRE(cond, ...)                                   \
  do {                                                          \
    if (!(cond)) return ::sy::fail(SY_ERR_ARGUMENT, __VA_ARGS__); \
  } while (0)

constexpr int MAX_DEVICES = 64;

// ---- programmatic dependent launch ----------------------------------------------------------
// The layer is a chain of short kernels. Each is launched with the programmatic-serialization
// attribute, lets its successor start as soon as it is resident (pdl_launch_dependents), does
// whatever does not touch its inputs (barrier and tensor-memory set-up), and only then waits
// for its predecessors to finish (pdl_wait). Launch latency and prologues overlap the previous
// kernel's tail; results are unchanged. SY_NO_PDL=1 in the environment turns it off.
bool pdl_enabled();

template <typename... KArgs, typename... Args>
int launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, const char* what,
                  Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return check_cuda(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...), what);
}

// The same for a kernel that runs as clusters of `cluster` CTAs along x.
template <typename... KArgs, typename... Args>
int launch_cluster_kernel(void (*kernel)(KArgs...), int cluster, dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                          const char* what, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  return check_cuda(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...), what);
}

#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

// ---- 16-bit element helpers ---------------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<__half> {
  using pair = __half2;
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
  static __device__ __forceinline__ float2 pair_to_f2(uint32_t bits) {
    return __half22float2(*reinterpret_cast<const __half2*>(&bits));
  }
};
template <> struct Elem<__nv_bfloat16> {
  using pair = __nv_bfloat162;
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
  static __device__ __forceinline__ float2 pair_to_f2(uint32_t bits) {
    // a bfloat16 is the upper half of a float
    return make_float2(__uint_as_float(bits << 16), __uint_as_float(bits & 0xffff0000u));
  }
};

// round a float through the 16-bit type and back (the epilogues' rounding points)
template <typename T> __device__ __forceinline__ float round16(float v) {
  return Elem<T>::to_f(Elem<T>::from_f(v));
}

// 8 consecutive 16-bit elements (one 16-byte vector) to 8 floats
template <typename T> __device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  float2 a = Elem<T>::pair_to_f2(v.x), b = Elem<T>::pair_to_f2(v.y);
  float2 c = Elem<T>::pair_to_f2(v.z), d = Elem<T>::pair_to_f2(v.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}

// SwiGLU and row-scale epilogues with the rounding points of op-by-op 16-bit PyTorch
// (linear -> silu -> mul -> linear -> mul): each intermediate is rounded to the 16-bit type.
template <typename T> __device__ __forceinline__ T epilogue_swiglu(float acc_gate, float acc_up) {
  float g = round16<T>(acc_gate), u = round16<T>(acc_up);
  // ex2.approx and the approximate divide are exact to about 2^-21: far inside the 16-bit
  // rounding that follows, and several times cheaper than expf and an IEEE divide
  float s = round16<T>(__fdividef(g, 1.f + __expf(-g)));
  return Elem<T>::from_f(s * u);
}
template <typename T> __device__ __forceinline__ T epilogue_scale(float acc, T scale) {
  return Elem<T>::from_f(round16<T>(acc) * Elem<T>::to_f(scale));
}

// ---- device status word -------------------------------------------------------------------
// Kernels with bounded waits record where they gave up here instead of trapping.
enum DeviceStatus : int {
  DS_OK = 0,
  DS_TIMEOUT_FULL = 1,     // a consumer never saw its stage filled
  DS_TIMEOUT_EMPTY = 2,    // the producer never got a stage back
  DS_TIMEOUT_MMA = 3,      // the epilogue never saw the accumulator committed
  DS_TIMEOUT_TMEM = 4,     // the issuer never got an accumulator back
  DS_TIMEOUT_FLAG = 5,     // a peer's arrival flag never came
  DS_BAD_INDEX = 6,        // an index outside its array was skipped
};

// ---- PTX wrappers -------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_inval(uint64_t* bar) {
  asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// make generic-proxy writes to shared memory visible to the async proxy (TMA, tcgen05)
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after `limit_ns` and returns false. Every wait in this library goes
// through here, so that a protocol error ends in a status code, not in a hung GPU.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint64_t limit_ns = 2000000000ull) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t start = global_timer_ns();
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 255u) == 0 && global_timer_ns() - start > limit_ns) return false;
  }
}

// ---- flags between GPUs ---------------------------------------------------------------------
// A flag is an int in one GPU's memory that another GPU's kernel stores an ever-growing epoch
// into (after a system-scope fence); the owner's kernels wait until it has reached the epoch they expect.
// The writer fences at system scope once and then stores every peer's flag relaxed: fence +
// relaxed store is a release, and the stores leave back to back, where a st.release per flag
// would first wait until the store before it has been acknowledged by its GPU (a round trip
// over NVLink per flag).
__device__ __forceinline__ void st_relaxed_sys(int* p, int v) {
  asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Waits until *flag >= epoch; gives up (false) after limit_ns. Every poll is an acquire load:
// measured on a B200, polling with relaxed loads and fencing once after the flag is seen
// (fence.acq_rel.sys in every waiting thread) is slower than this.
__device__ __forceinline__ bool wait_flag(const int* flag, int epoch, uint64_t limit_ns) {
  if (ld_acquire_sys(flag) >= epoch) return true;
  const uint64_t start = global_timer_ns();
  for (uint32_t spin = 1;; ++spin) {
    if (ld_acquire_sys(flag) >= epoch) return true;
    if ((spin & 31u) == 0) {
      if (global_timer_ns() - start > limit_ns) return false;
      __nanosleep(100);
    }
  }
}

// 1-D bulk copy global -> shared, completion counted in bytes on an mbarrier.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst_smem)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// 2-D tiled TMA load global -> shared of this CTA only, completion on an mbarrier.
__device__ __forceinline__ void tma_load_2d(void* dst_smem, const void* tensor_map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_u32(dst_smem)),
      "l"(tensor_map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
// Orders this thread's earlier generic-proxy accesses (plain loads and stores, global memory
// included) with later async-proxy ones (TMA), in both directions.
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
// 16-byte asynchronous copy global -> shared (src_bytes < 16 zero-fills the rest), tracked by
// per-thread commit groups.
__device__ __forceinline__ void cp_async_16(void* dst_smem, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst_smem)), "l"(src), "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
// The same with an L2 eviction policy: weights that are read exactly once should not push
// re-used data (activations, offsets) out of L2.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void tma_load_2d_hint(void* dst_smem, const void* tensor_map, int x, int y, uint64_t* bar,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], "
      "[%4], %5;" ::"r"(smem_u32(dst_smem)),
      "l"(tensor_map), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const void* tensor_map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tensor_map) : "memory");
}
__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b32 r;\n\t"
      "elect.sync r|p, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// One 32-byte store (a whole sector) to a 32-byte aligned global address.
__device__ __forceinline__ void st_global_32(void* p, const uint32_t (&v)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]),
               "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}

// One 16-bit element read through L2 (written by another block of the same launch).
template <typename T> __device__ __forceinline__ T ldcg16(const T* p) {
  unsigned short v;
  asm volatile("ld.global.cg.u16 %0, [%1];" : "=h"(v) : "l"(p));
  return reinterpret_cast<T&>(v);
}

// Warp-level 16x8x16 matrix multiply-accumulate (16-bit inputs, float32 accumulators): the small
// router GEMM of the fused routing kernel. The expert FFN does not use it.
template <typename T>
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1);
template <>
__device__ __forceinline__ void mma_16816<__half>(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                  uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma_16816<__nv_bfloat16>(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---- tcgen05 / tensor memory --------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(columns)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc], 16-bit inputs, fp32 accumulate, one CTA.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same with the descriptors given as (low word, shared high word): the high word of a
// K-major 128-byte-swizzle descriptor is constant, and the low word is an address that the
// issuing thread advances with a 32-bit add, which keeps its instruction count per MMA small.
__device__ __forceinline__ void umma_f16_lohi(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 da, {%1, %3};\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}" ::"r"(tmem_d),
      "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Low / high words of umma_desc_k_sw128.
__device__ __forceinline__ uint32_t umma_desc_lo(uint32_t smem_addr) { return ((smem_addr & 0x3ffff) >> 4) | (1u << 16); }
constexpr uint32_t UMMA_DESC_HI_K_SW128 = (1024u >> 4) | (1u << 14) | (2u << 29);
// All MMAs issued so far by this thread arrive on the mbarrier when they complete.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// ---- CTA pairs (clusters of two; tcgen05 cta_group::2) --------------------------------------
// In a pair the even CTA ("leader") issues MMAs that read both CTAs' shared memory and write
// both CTAs' tensor memory: 256 weight rows (128 per CTA) by N token rows (N/2 staged by each
// CTA), so each CTA loads half of what it would need alone for the same arithmetic.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of the same shared-memory object in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t cluster_map(const void* local, uint32_t rank) {
  uint32_t a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(smem_u32(local)), "r"(rank));
  return a;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait on a barrier that CTAs of the whole cluster arrive on.
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, uint64_t limit_ns) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  uint64_t start = global_timer_ns();
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if ((spin & 255u) == 0 && global_timer_ns() - start > limit_ns) return false;
  }
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// 2-D tiled TMA load into THIS CTA's shared memory whose completion bytes are counted on a
// barrier that may live in the other CTA of the pair (`bar_cluster_addr` from cluster_map).
__device__ __forceinline__ void tma_load_2d_pair(void* dst_smem, const void* tensor_map, int x, int y,
                                                 uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], "
      "[%4];" ::"r"(smem_u32(dst_smem)),
      "l"(tensor_map), "r"(x), "r"(y), "r"(bar_cluster_addr)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* dst_smem, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(columns)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(columns) : "memory");
}
// umma_f16_lohi across the pair (M = 256: 128 rows from each CTA's shared memory).
__device__ __forceinline__ void umma_f16_lohi_pair(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t hi,
                                                   uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 da, {%1, %3};\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, p;\n\t}" ::"r"(tmem_d),
      "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// All pair MMAs issued so far by this thread arrive, when complete, on the barrier at the
// same shared-memory offset in every CTA of `cta_mask` (a signal only; it moves no data).
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"(cta_mask)
      : "memory");
}
// 32 lanes x 8 consecutive 32-bit columns of tensor memory into 8 registers per thread.
__device__ __forceinline__ void tmem_ld_x8(uint32_t addr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(addr)
               : "memory");
}
// The same for 16 columns.
__device__ __forceinline__ void tmem_ld_x16(uint32_t addr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(addr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor for a K-major operand tile whose rows are 128 bytes
// (64 16-bit elements) laid out with the 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffff) >> 4);       // start address, 16-byte units
  d |= (uint64_t)1 << 16;                             // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;                   // stride byte offset: 8 rows x 128 B
  d |= (uint64_t)1 << 46;                             // descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;                             // 128-byte swizzle
  return d;
}
// Instruction descriptor: fp32 accumulator, both operands K-major, a/b format 0 = f16, 1 = bf16.
__device__ __forceinline__ uint32_t umma_idesc(int fmt16, int M, int N) {
  return (1u << 4) | ((uint32_t)fmt16 << 7) | ((uint32_t)fmt16 << 10) | ((uint32_t)(N >> 3) << 17) |
         ((uint32_t)(M >> 4) << 24);
}

}  // namespace sy

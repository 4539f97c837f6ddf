// Expert-parallel transport primitives: the dispatch store (rows of this GPU's activations,
// picked by index, written straight into a buffer that may live on a peer GPU), a contiguous
// device-to-device copy, and peer-access set-up.
// Replace switchyard/csrc/moe_kernels.cu:447-489.
#include "common.cuh"

namespace sy {

constexpr int GATHER_THREADS = 256;

// One block per row group; 16-byte loads from local memory, 16-byte stores to (possibly
// remote) memory. Stores to a peer are fire-and-forget over NVLink; all loads of a thread are
// issued before its stores.
__global__ void __launch_bounds__(GATHER_THREADS)
gather_rows_kernel(const uint4* __restrict__ src, const int* __restrict__ index, int n, int vec_per_row,
                   uint4* __restrict__ dst) {
  for (int row = blockIdx.x; row < n; row += gridDim.x) {
    const uint4* s = src + (size_t)index[row] * vec_per_row;
    uint4* d = dst + (size_t)row * vec_per_row;
    for (int i = threadIdx.x; i < vec_per_row; i += GATHER_THREADS) d[i] = __ldg(s + i);
  }
}

}  // namespace sy

extern "C" int sy_gather_rows(const void* src, const int32_t* index, int n, int row_bytes, void* dst, void* stream) {
  using namespace sy;
  SY_REQUIRE(n >= 0 && row_bytes > 0 && row_bytes % 16 == 0, "gather_rows: row size must be a multiple of 16 bytes");
  if (n == 0) return SY_OK;
  SY_REQUIRE(src && index && dst, "gather_rows: null pointer");
  SY_REQUIRE(((uintptr_t)src % 16 == 0) && ((uintptr_t)dst % 16 == 0), "gather_rows: 16-byte alignment");
  int sms = 0;
  int rc = device_sm_count(&sms);
  if (rc != SY_OK) return rc;
  int blocks = n < sms * 8 ? n : sms * 8;
  gather_rows_kernel<<<blocks, GATHER_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), index, n, row_bytes / 16, static_cast<uint4*>(dst));
  return check_cuda(cudaGetLastError(), "gather_rows launch");
}

extern "C" int sy_copy_async(void* dst, const void* src, size_t bytes, void* stream) {
  using namespace sy;
  if (bytes == 0) return SY_OK;
  SY_REQUIRE(dst && src, "copy_async: null pointer");
  SY_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, static_cast<cudaStream_t>(stream)));
  return SY_OK;
}

extern "C" int sy_enable_peer_access(int device, int peer, int* enabled_out) {
  using namespace sy;
  SY_REQUIRE(enabled_out, "enable_peer_access: null output");
  *enabled_out = 0;
  if (device == peer) {
    *enabled_out = 1;
    return SY_OK;
  }
  int can = 0;
  SY_CUDA(cudaDeviceCanAccessPeer(&can, device, peer));
  if (!can) return SY_OK;
  int prev = 0;
  SY_CUDA(cudaGetDevice(&prev));
  SY_CUDA(cudaSetDevice(device));
  cudaError_t e = cudaDeviceEnablePeerAccess(peer, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();  // clear the sticky-free error
    e = cudaSuccess;
  }
  cudaError_t back = cudaSetDevice(prev);
  SY_CUDA(e);
  SY_CUDA(back);
  *enabled_out = 1;
  return SY_OK;
}

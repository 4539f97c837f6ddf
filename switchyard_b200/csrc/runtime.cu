// Host-side runtime of the library: thread-local error text, per-device caches (SM count,
// address of the kernel status word), version and status entry points.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

#include <atomic>
#include <mutex>

#include "common.cuh"

namespace sy {

static thread_local char t_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_error, sizeof(t_error), fmt, ap);
  va_end(ap);
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_error, sizeof(t_error), fmt, ap);
  va_end(ap);
  return code;
}

bool pdl_enabled() {
  static const bool on = [] {
    const char* v = getenv("SY_NO_PDL");
    return !(v && v[0] == '1');
  }();
  return on;
}

// How long a kernel of this library waits for a flag or barrier before it gives up and records
// a status code. One value for all devices; SY_WAIT_LIMIT_MS in the environment sets the
// initial value (read once), sy_set_wait_limit_ns replaces it at run time.
static std::atomic<uint64_t> g_wait_limit_ns{0};

uint64_t wait_limit_ns() {
  uint64_t v = g_wait_limit_ns.load(std::memory_order_relaxed);
  if (v == 0) {
    v = 2000000000ull;
    const char* e = getenv("SY_WAIT_LIMIT_MS");
    if (e && e[0]) {
      const long long ms = atoll(e);
      if (ms > 0) v = (uint64_t)ms * 1000000ull;
    }
    g_wait_limit_ns.store(v, std::memory_order_relaxed);
  }
  return v;
}

int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return SY_OK;
  snprintf(t_error, sizeof(t_error), "CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
  return SY_ERR_CUDA;
}

// One status word per device: every device that loads the module gets its own copy.
__device__ int g_status_word;

struct DeviceInfo {
  std::atomic<int> ready{0};
  int sm_count = 0;
  int* status_word = nullptr;
};
static DeviceInfo g_devices[MAX_DEVICES];
static std::mutex g_device_mutex;

static int device_info(DeviceInfo** out) {
  int dev = -1;
  SY_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= MAX_DEVICES) return fail(SY_ERR_ARGUMENT, "device ordinal %d out of range", dev);
  DeviceInfo& d = g_devices[dev];
  if (!d.ready.load(std::memory_order_acquire)) {
    std::lock_guard<std::mutex> lock(g_device_mutex);
    if (!d.ready.load(std::memory_order_relaxed)) {
      SY_CUDA(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
      void* p = nullptr;
      SY_CUDA(cudaGetSymbolAddress(&p, g_status_word));
      d.status_word = static_cast<int*>(p);
      // (the word starts at zero: a __device__ variable without an initialiser is zero-filled
      // when the module is loaded, so nothing has to be enqueued or synchronised here)
      d.ready.store(1, std::memory_order_release);
    }
  }
  *out = &d;
  return SY_OK;
}

int device_sm_count(int* out) {
  DeviceInfo* d;
  int rc = device_info(&d);
  if (rc != SY_OK) return rc;
  *out = d->sm_count;
  return SY_OK;
}

int current_device_slot(int* out) {
  SY_CUDA(cudaGetDevice(out));
  return SY_OK;
}

int* device_status_word() {
  DeviceInfo* d;
  return device_info(&d) == SY_OK ? d->status_word : nullptr;
}

}  // namespace sy

extern "C" const char* sy_last_error(void) { return sy::t_error; }

extern "C" const char* sy_version(void) { return "switchyard_b200 0.1 (sm_100a)"; }

extern "C" int sy_set_wait_limit_ns(uint64_t limit_ns) {
  SY_REQUIRE(limit_ns >= 1000ull && limit_ns <= 60000000000ull, "set_wait_limit_ns: 1 us .. 60 s (got %llu ns)",
             (unsigned long long)limit_ns);
  sy::g_wait_limit_ns.store(limit_ns, std::memory_order_relaxed);
  return SY_OK;
}

extern "C" uint64_t sy_wait_limit_ns(void) { return sy::wait_limit_ns(); }

static const char* status_text(int v) {
  switch (v) {
    case sy::DS_TIMEOUT_FULL: return "a stage of the expert kernel's ring was never filled";
    case sy::DS_TIMEOUT_EMPTY: return "a stage of the expert kernel's ring was never released";
    case sy::DS_TIMEOUT_MMA: return "an accumulator was never committed";
    case sy::DS_TIMEOUT_TMEM: return "an accumulator was never drained";
    case sy::DS_TIMEOUT_FLAG: return "a flag (a peer's arrival or return signal, or an expert's readiness) never came";
    case sy::DS_BAD_INDEX: return "an index outside its array was skipped";
    default: return "unknown status";
  }
}

extern "C" int sy_device_status(void* stream, int* status_out) {
  int* word = sy::device_status_word();
  if (!word) return SY_ERR_CUDA;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int v = 0;
  SY_CUDA(cudaMemcpyAsync(&v, word, sizeof(int), cudaMemcpyDeviceToHost, s));
  SY_CUDA(cudaStreamSynchronize(s));
  if (v != 0) {
    SY_CUDA(cudaMemsetAsync(word, 0, sizeof(int), s));
    SY_CUDA(cudaStreamSynchronize(s));
  }
  if (status_out) *status_out = v;
  if (v != 0) return sy::fail(SY_ERR_DEVICE, "device status %d: %s", v, status_text(v));
  return SY_OK;
}

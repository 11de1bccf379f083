#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace polar_b200 {

static thread_local char tls_error[512] = "";
static std::atomic<uint64_t> g_launches{0};

int fail(int status, const char* msg, cudaError_t err) {
  if (err != cudaSuccess) {
    std::snprintf(tls_error, sizeof(tls_error), "%s: %s (%s)", msg, cudaGetErrorString(err),
                  cudaGetErrorName(err));
  } else {
    std::snprintf(tls_error, sizeof(tls_error), "%s", msg);
  }
  return status;
}

void clear_error() { tls_error[0] = 0; }

void count_launch(uint64_t n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int sm_count() {
  // Cached per device ordinal; 148 on B200.
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

namespace {
constexpr int kMaxDevices = 64;
int* g_status_host = nullptr;   // kMaxDevices words
int* g_status_dev = nullptr;
std::atomic<unsigned long long> g_wait_limit_ns{0};
}  // namespace

int* device_status_word(int* rc) {
  static std::once_flag once;
  static cudaError_t err = cudaSuccess;
  std::call_once(once, [] {
    err = cudaHostAlloc(reinterpret_cast<void**>(&g_status_host), kMaxDevices * sizeof(int),
                        cudaHostAllocMapped | cudaHostAllocPortable);
    if (err == cudaSuccess) {
      std::memset(g_status_host, 0, kMaxDevices * sizeof(int));
      // portable + unified addressing: the same device pointer is valid on every GPU
      err = cudaHostGetDevicePointer(reinterpret_cast<void**>(&g_status_dev), g_status_host, 0);
    }
  });
  if (err != cudaSuccess) {
    *rc = fail(POLAR_B200_ERR_CUDA, "status word allocation", err);
    return nullptr;
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    cudaGetLastError();
    dev = 0;
  }
  *rc = POLAR_B200_OK;
  return g_status_dev + dev;
}

int device_status_read(int device) {
  if (!g_status_host) return 0;
  if (device >= 0) return device < kMaxDevices ? *(volatile int*)(g_status_host + device) : 0;
  for (int d = 0; d < kMaxDevices; ++d)
    if (int v = *(volatile int*)(g_status_host + d)) return v;
  return 0;
}

void device_status_clear_all() {
  if (!g_status_host) return;
  for (int d = 0; d < kMaxDevices; ++d) *(volatile int*)(g_status_host + d) = 0;
}

unsigned long long wait_limit_ns(unsigned long long fallback) {
  const unsigned long long v = g_wait_limit_ns.load(std::memory_order_relaxed);
  return v ? v : fallback;
}

}  // namespace polar_b200

extern "C" {
int polar_b200_device_status(void) { return polar_b200::device_status_read(-1); }
int polar_b200_device_status_of(int device) { return device < 0 ? 0 : polar_b200::device_status_read(device); }
void polar_b200_device_status_clear(void) { polar_b200::device_status_clear_all(); }
int polar_b200_check_device_status(void) {
  using namespace polar_b200;
  const int code = device_status_read(-1);
  if (code == 0) return POLAR_B200_OK;
  static thread_local char msg[96];
  std::snprintf(msg, sizeof msg, "a bounded device-side wait gave up (code %d)", code);
  clear_error();
  return fail(POLAR_B200_ERR_TIMEOUT, msg);
}
void polar_b200_set_wait_limit_ns(uint64_t ns) { polar_b200::g_wait_limit_ns.store(ns, std::memory_order_relaxed); }
uint64_t polar_b200_wait_limit_ns(void) { return polar_b200::g_wait_limit_ns.load(std::memory_order_relaxed); }
const char* polar_b200_last_error(void) { return polar_b200::tls_error; }
int polar_b200_version(void) { return 100; }
int polar_b200_built_for_sm(void) { return 100; }
uint64_t polar_b200_launch_count(void) {
  return polar_b200::g_launches.load(std::memory_order_relaxed);
}
}

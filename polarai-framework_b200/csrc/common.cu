#include <atomic>
#include <cstdio>
#include <cstring>

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

}  // namespace polar_b200

extern "C" {
const char* polar_b200_last_error(void) { return polar_b200::tls_error; }
int polar_b200_version(void) { return 100; }
int polar_b200_built_for_sm(void) { return 100; }
uint64_t polar_b200_launch_count(void) {
  return polar_b200::g_launches.load(std::memory_order_relaxed);
}
}

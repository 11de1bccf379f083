// The CUDA-runtime policy for device_scope.hpp: current-device bookkeeping that leaves the
// caller's thread as it found it, and pooled events per device.
#pragma once

#include "device_scope.hpp"

#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>
#include <vector>

namespace polarai::backend::generic {

struct CudaApi {
  using Event = cudaEvent_t;
  static constexpr int kMaxDevices = 64;

  // cuCtxGetCurrent / cuCtxSetCurrent, looked up through the runtime so that the plugin
  // does not link the driver library.  With them a thread that had NO context current
  // gets exactly that back (cudaSetDevice(previous) would create a context on a GPU the
  // host may never have meant to touch).
  struct Driver {
    CUresult (*getCurrent)(CUcontext*) = nullptr;
    CUresult (*setCurrent)(CUcontext) = nullptr;
  };
  static const Driver& driver() {
    static Driver d = [] {
      Driver r;
      void* p = nullptr;
      cudaDriverEntryPointQueryResult q;
      if (cudaGetDriverEntryPoint("cuCtxGetCurrent", &p, cudaEnableDefault, &q) == cudaSuccess &&
          q == cudaDriverEntryPointSuccess)
        r.getCurrent = reinterpret_cast<CUresult (*)(CUcontext*)>(p);
      p = nullptr;
      if (cudaGetDriverEntryPoint("cuCtxSetCurrent", &p, cudaEnableDefault, &q) == cudaSuccess &&
          q == cudaDriverEntryPointSuccess)
        r.setCurrent = reinterpret_cast<CUresult (*)(CUcontext)>(p);
      if (!r.getCurrent || !r.setCurrent) r = Driver{};
      cudaGetLastError();
      return r;
    }();
    return d;
  }

  static DeviceToken current() {
    DeviceToken t;
    const Driver& d = driver();
    if (d.getCurrent) {
      CUcontext ctx = nullptr;
      if (d.getCurrent(&ctx) == CUDA_SUCCESS) {
        t.context = ctx;
        t.haveContext = true;
      }
    }
    // With no context current the runtime reports the thread's default (0) without
    // creating anything.
    if (cudaGetDevice(&t.device) != cudaSuccess) {
      cudaGetLastError();
      t.device = 0;
    }
    return t;
  }
  static bool enter(int ordinal) {
    if (cudaSetDevice(ordinal) == cudaSuccess) return true;
    cudaGetLastError();
    return false;
  }
  static void restore(const DeviceToken& t) {
    if (t.haveContext && driver().setCurrent) {
      driver().setCurrent(static_cast<CUcontext>(t.context));   // nullptr: "no context", as found
    } else if (cudaSetDevice(t.device) != cudaSuccess) {
      cudaGetLastError();
    }
  }

  // ---- events, pooled per device (creating one costs microseconds and a launch needs one) ----
  struct Pool {
    std::mutex mutex;
    std::vector<cudaEvent_t> free;
  };
  static Pool& pool(int ordinal) {
    static Pool pools[kMaxDevices];
    return pools[(ordinal >= 0 && ordinal < kMaxDevices) ? ordinal : 0];
  }
  // The device must be current: an event belongs to the device it was created on.
  static Event takeEvent(int ordinal) {
    Pool& p = pool(ordinal);
    {
      std::lock_guard<std::mutex> g(p.mutex);
      if (!p.free.empty()) {
        cudaEvent_t e = p.free.back();
        p.free.pop_back();
        return e;
      }
    }
    cudaEvent_t e = nullptr;
    if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    return e;
  }
  static void giveEvent(int ordinal, Event e) {
    if (!e) return;
    Pool& p = pool(ordinal);
    std::lock_guard<std::mutex> g(p.mutex);
    p.free.push_back(e);
  }
  static void destroyEvents(int ordinal) {
    Pool& p = pool(ordinal);
    std::lock_guard<std::mutex> g(p.mutex);
    for (cudaEvent_t e : p.free) cudaEventDestroy(e);
    p.free.clear();
  }

  static bool record(Event e, cudaStream_t s) { return ok(cudaEventRecord(e, s)); }
  static bool streamWait(cudaStream_t s, Event e) { return ok(cudaStreamWaitEvent(s, e, 0)); }
  static bool eventSync(Event e) { return ok(cudaEventSynchronize(e)); }
  static bool copyPeer(void* dst, int dstOrdinal, const void* src, int srcOrdinal, size_t bytes, cudaStream_t s) {
    // Direct over NVLink when peer access is on (enabled once per pair, best effort);
    // otherwise the runtime stages the copy itself.
    enablePeer(dstOrdinal, srcOrdinal);
    return ok(cudaMemcpyPeerAsync(dst, dstOrdinal, src, srcOrdinal, bytes, s));
  }

private:
  static bool ok(cudaError_t e) {
    if (e == cudaSuccess) return true;
    cudaGetLastError();
    return false;
  }
  // Called with `device` current.
  static void enablePeer(int device, int peer) {
    static std::mutex m;
    static bool tried[kMaxDevices][kMaxDevices] = {};
    if (device == peer || device < 0 || peer < 0 || device >= kMaxDevices || peer >= kMaxDevices) return;
    std::lock_guard<std::mutex> g(m);
    if (tried[device][peer]) return;
    tried[device][peer] = true;
    int can = 0;
    if (cudaDeviceCanAccessPeer(&can, device, peer) == cudaSuccess && can) {
      cudaError_t e = cudaDeviceEnablePeerAccess(peer, 0);
      if (e != cudaSuccess) cudaGetLastError();   // already enabled, or refused: the copy still works
    } else {
      cudaGetLastError();
    }
  }
};

using ScopedDevice = ScopedDeviceT<CudaApi>;

}  // namespace polarai::backend::generic

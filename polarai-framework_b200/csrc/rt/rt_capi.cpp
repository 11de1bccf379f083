// Flat C view of the runtime plugin (include/polar_b200_rt.h).
#include "b200_runtime.hpp"
#include "pool_backend_allocator.hpp"

#include <polarai/backend/generic/runtime/LaunchCommand.h>
#include <polarai/backend/generic/runtime/TensorInfo.h>
#include <polarai/backend/generic/runtime/api.h>

#include <polar_b200.h>
#include <polar_b200_rt.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

using namespace polarai::backend::generic;
using polarai::core::internal::LockType;

struct polar_b200_rt {
  Context* ctx = nullptr;
  std::vector<std::shared_ptr<Device>> devices;
  std::shared_ptr<PoolBackendAllocator> allocator;
  std::vector<std::string> names;
  std::string error;
};

namespace {
// A batch of inputs is hundreds of megabytes; one thread copies about 10 GB/s, well below what
// the upload over PCIe that follows can take.  Large copies are cut over a few threads.
void big_memcpy(void* dst, const void* src, uint64_t bytes) {
  constexpr uint64_t kChunk = 4ull << 20;
  // POLAR_B200_COPY_THREADS overrides the number of copying threads (default: the cores, at most 16)
  static const unsigned limit = [] {
    const char* e = std::getenv("POLAR_B200_COPY_THREADS");
    unsigned v = e ? (unsigned)std::strtoul(e, nullptr, 10) : 0u;
    unsigned hw = std::thread::hardware_concurrency();
    return v ? v : std::min(hw ? hw : 1u, 16u);
  }();
  uint64_t parts = std::min<uint64_t>(bytes / kChunk, limit);
  if (parts <= 1) {
    std::memcpy(dst, src, bytes);
    return;
  }
  const uint64_t per = ((bytes / parts) + 63) & ~63ull;
  std::vector<std::thread> workers;
  for (uint64_t i = 1; i < parts; ++i) {
    const uint64_t lo = i * per, hi = std::min(bytes, lo + per);
    if (lo >= hi) break;
    workers.emplace_back([=] {
      std::memcpy(static_cast<char*>(dst) + lo, static_cast<const char*>(src) + lo, hi - lo);
    });
  }
  std::memcpy(dst, src, std::min(bytes, per));
  for (auto& w : workers) w.join();
}

B200Device* dev(polar_b200_rt* rt, int i) {
  if (!rt || i < 0 || i >= (int)rt->devices.size()) return nullptr;
  return static_cast<B200Device*>(rt->devices[i].get());
}
int fail(polar_b200_rt* rt, int status, const std::string& msg) {
  if (rt) rt->error = msg;
  return status;
}
// After a synchronisation point: did a bounded device-side wait give up on that GPU?
int device_wait_status(polar_b200_rt* rt, B200Device* d) {
  if (int code = polar_b200_device_status_of(d->ordinal()))
    return fail(rt, POLAR_B200_ERR_TIMEOUT, d->getDeviceName() + ": a bounded device-side wait gave up (code " +
                                                std::to_string(code) + ")");
  return POLAR_B200_OK;
}
int allocator_status(polar_b200_rt* rt) {
  int s = rt->allocator->lastStatus();
  if (s) {
    rt->error = rt->allocator->lastError();
    rt->allocator->clearError();
  }
  return s;
}
}  // namespace

extern "C" {

polar_b200_rt* polar_b200_rt_open(void) {
  auto* rt = new polar_b200_rt();
  rt->ctx = initContext();
  rt->devices = rt->ctx->getDevices();
  rt->allocator = std::make_shared<PoolBackendAllocator>();
  for (auto& d : rt->devices) {
    rt->allocator->registerDevice(*d);
    rt->names.push_back(d->getDeviceName());
  }
  return rt;
}

void polar_b200_rt_close(polar_b200_rt* rt) {
  if (!rt) return;
  for (auto& d : rt->devices) static_cast<B200Device*>(d.get())->synchronize();
  rt->allocator.reset();
  rt->devices.clear();
  closeContext(rt->ctx);
  delete rt;
}

int polar_b200_rt_device_count(polar_b200_rt* rt) { return rt ? (int)rt->devices.size() : 0; }

const char* polar_b200_rt_device_name(polar_b200_rt* rt, int device) {
  return dev(rt, device) ? rt->names[device].c_str() : "";
}

int polar_b200_rt_allocate(polar_b200_rt* rt, int device, uint64_t va, uint64_t bytes) {
  B200Device* d = dev(rt, device);
  if (!d) return fail(rt, POLAR_B200_ERR_INVALID, "no such device");
  rt->allocator->allocate(MemoryRecord{va, bytes}, *d);
  return allocator_status(rt);
}

int polar_b200_rt_deallocate(polar_b200_rt* rt, uint64_t va, uint64_t bytes) {
  if (!rt) return POLAR_B200_ERR_INVALID;
  rt->allocator->deallocate(MemoryRecord{va, bytes});
  return allocator_status(rt);
}

int polar_b200_rt_write(polar_b200_rt* rt, uint64_t va, uint64_t bytes, const void* src) {
  if (!rt || (!src && bytes)) return fail(rt, POLAR_B200_ERR_INVALID, "null source");
  MemoryRecord rec{va, bytes};
  void* host = rt->allocator->beginOverwrite(rec);
  if (int s = allocator_status(rt)) return s;
  if (!host) return fail(rt, POLAR_B200_ERR_CUDA, "no host memory for the record");
  big_memcpy(host, src, bytes);
  rt->allocator->endOverwrite(rec);   // the upload to the devices that hold the record starts here
  return allocator_status(rt);
}

int polar_b200_rt_host_begin_write(polar_b200_rt* rt, uint64_t va, uint64_t bytes, void** host) {
  if (!rt || !host) return fail(rt, POLAR_B200_ERR_INVALID, "null handle or result pointer");
  *host = rt->allocator->beginOverwrite(MemoryRecord{va, bytes});
  if (int s = allocator_status(rt)) return s;
  return *host ? POLAR_B200_OK : fail(rt, POLAR_B200_ERR_CUDA, "no host memory for the record");
}

int polar_b200_rt_host_end_write(polar_b200_rt* rt, uint64_t va, uint64_t bytes) {
  if (!rt) return POLAR_B200_ERR_INVALID;
  rt->allocator->endOverwrite(MemoryRecord{va, bytes});
  return allocator_status(rt);
}

int polar_b200_rt_read(polar_b200_rt* rt, uint64_t va, uint64_t bytes, void* dst) {
  if (!rt || (!dst && bytes)) return fail(rt, POLAR_B200_ERR_INVALID, "null destination");
  MemoryRecord rec{va, bytes};
  rt->allocator->lock(rec, LockType::READ);
  if (int s = allocator_status(rt)) return s;
  void* host = rt->allocator->get(rec);
  if (!host) {
    rt->allocator->release(rec);
    return fail(rt, POLAR_B200_ERR_CUDA, "no host memory for the record");
  }
  big_memcpy(dst, host, bytes);
  rt->allocator->release(rec);
  for (auto& d : rt->devices) {
    auto* bd = static_cast<B200Device*>(d.get());
    if (int s = bd->takeStatus()) return fail(rt, s, bd->lastError());
    if (bd->ready())
      if (int s = device_wait_status(rt, bd)) return s;
  }
  return POLAR_B200_OK;
}

int polar_b200_rt_launch(polar_b200_rt* rt, int device, struct LaunchCommand* cmd) {
  B200Device* d = dev(rt, device);
  if (!d || !cmd) return fail(rt, POLAR_B200_ERR_INVALID, "no such device or null command");
  // Locks as the operations' gen() methods take them: the result (last tensor argument; the
  // last two for the one builtin with two results) READ_WRITE, every other tensor READ.
  std::vector<uint64_t> tensors;
  for (uint64_t i = 0; i < cmd->argsCount; ++i)
    if (cmd->args[i].type == ArgDesc::TENSOR) tensors.push_back(i);
  const size_t n_results = std::min<size_t>(tensors.size(), (size_t)polar_b200_result_count(cmd->nativeKernelName));
  auto is_result = [&](uint64_t i) {
    for (size_t r = 0; r < n_results; ++r)
      if (tensors[tensors.size() - 1 - r] == i) return true;
    return false;
  };
  auto record_of = [](TensorInfo* t) {
    MemoryRecord r{t->virtAddr, 4};
    for (uint64_t k = 0; k < t->dims; ++k) r.allocationSize *= t->shape[k];
    return r;
  };
  std::vector<MemoryRecord> locked;
  auto unlock_all = [&] { for (auto& r : locked) rt->allocator->release(r, *d); };
  auto is_locked = [&](const MemoryRecord& r) {
    for (auto& l : locked) if (l == r) return true;
    return false;
  };
  for (uint64_t i : tensors) {
    if (!is_result(i)) continue;
    MemoryRecord r = record_of(static_cast<TensorInfo*>(cmd->args[i].arg));
    if (is_locked(r)) continue;
    rt->allocator->lock(r, *d, LockType::READ_WRITE);
    if (int s = allocator_status(rt)) { unlock_all(); return s; }
    locked.push_back(r);
  }
  for (uint64_t i : tensors) {
    if (is_result(i)) continue;
    MemoryRecord r = record_of(static_cast<TensorInfo*>(cmd->args[i].arg));
    if (is_locked(r)) continue;   // an in-place update reads what it writes
    rt->allocator->lock(r, *d, LockType::READ);
    if (int s = allocator_status(rt)) { unlock_all(); return s; }
    locked.push_back(r);
  }
  Event* evt = d->launch(*rt->allocator, *cmd, nullptr);
  int status = static_cast<B200Event*>(evt)->status();
  if (status) {
    rt->error = d->lastError();
    d->takeStatus();   // reported here
  }
  // Stream order protects the buffers; the locks can go as soon as the work is queued.
  unlock_all();
  delete evt;
  return status;
}

int polar_b200_rt_adopt(polar_b200_rt* rt, int device, uint64_t va, uint64_t bytes, void* device_ptr) {
  B200Device* d = dev(rt, device);
  if (!d) return fail(rt, POLAR_B200_ERR_INVALID, "no such device");
  rt->allocator->adoptExternal(MemoryRecord{va, bytes}, *d, device_ptr);
  return allocator_status(rt);
}

int polar_b200_rt_allreduce_fadd(polar_b200_rt* rt, int device, void* const* buffers, void* multicast, uint32_t rank,
                                 uint32_t world, uint32_t channel, uint64_t first, uint64_t count, const polar_b200_rt_update* updates,
                                 uint32_t n_updates, float scale_w, float scale_g) {
  B200Device* d = dev(rt, device);
  if (!d || (n_updates && !updates) || n_updates > POLAR_B200_MAX_UPDATE_SEGMENTS)
    return fail(rt, POLAR_B200_ERR_INVALID, "no such device, or a bad update list");
  // The kernel rewrites every weight record in place: taken READ_WRITE like any builtin's
  // output, so that host copies and other devices' copies become stale.
  std::vector<MemoryRecord> locked;
  polar_b200_update_segment seg[POLAR_B200_MAX_UPDATE_SEGMENTS];
  auto unlock_all = [&] { for (auto& r : locked) rt->allocator->release(r, *d); };
  for (uint32_t i = 0; i < n_updates; ++i) {
    const polar_b200_rt_update& u = updates[i];
    if ((u.weight_offset + u.count) * sizeof(float) > u.weight_bytes) {
      unlock_all();
      return fail(rt, POLAR_B200_ERR_INVALID, "update runs past its weight record");
    }
    MemoryRecord r{u.weight_va, u.weight_bytes};
    bool have = false;
    for (auto& l : locked) have = have || l == r;
    if (!have) {
      rt->allocator->lock(r, *d, LockType::READ_WRITE);
      if (int s = allocator_status(rt)) { unlock_all(); return s; }
      locked.push_back(r);
    }
    seg[i].weights = static_cast<float*>(d->getAllocator()->getPtr(r)) + u.weight_offset;
    seg[i].offset = u.grad_offset;
    seg[i].count = u.count;
  }
  int status = polar_b200_allreduce_fadd_multicast(buffers, multicast, rank, world, channel, first, count, seg, n_updates,
                                                   scale_w, scale_g, d->stream());
  if (status) rt->error = polar_b200_last_error();
  else for (auto& r : locked) d->pool().markWritten(r);
  unlock_all();
  return status;
}

int polar_b200_rt_barrier(polar_b200_rt* rt, int device) {
  B200Device* d = dev(rt, device);
  if (!d) return fail(rt, POLAR_B200_ERR_INVALID, "no such device");
  d->synchronize();
  if (int s = d->takeStatus()) return fail(rt, s, d->lastError());
  return device_wait_status(rt, d);
}

void* polar_b200_rt_device_ptr(polar_b200_rt* rt, int device, uint64_t va, uint64_t bytes) {
  B200Device* d = dev(rt, device);
  return d ? d->getAllocator()->getPtr(MemoryRecord{va, bytes}) : nullptr;
}

void* polar_b200_rt_stream(polar_b200_rt* rt, int device) {
  B200Device* d = dev(rt, device);
  return d ? (void*)d->stream() : nullptr;
}

uint64_t polar_b200_rt_bytes_in_use(polar_b200_rt* rt, int device) {
  B200Device* d = dev(rt, device);
  return d ? static_cast<B200Allocator*>(d->getAllocator().get())->bytesInUse() : 0;
}

int polar_b200_rt_set_memory_limit(polar_b200_rt* rt, int device, uint64_t bytes) {
  B200Device* d = dev(rt, device);
  if (!d) return fail(rt, POLAR_B200_ERR_INVALID, "no such device");
  static_cast<B200Allocator*>(d->getAllocator().get())->setLimit(bytes);
  return POLAR_B200_OK;
}

const char* polar_b200_rt_last_error(polar_b200_rt* rt) { return rt ? rt->error.c_str() : ""; }

}  // extern "C"

#include "pool_backend_allocator.hpp"

#include "b200_runtime.hpp"

#include <cuda_runtime.h>
#include <polar_b200.h>

#include <cstdio>
#include <cstdlib>

namespace polarai::backend::generic {

using core::internal::LockType;

namespace {
// The CUDA devices an allocator of this plugin meets are the plugin's own (the build has no
// RTTI; the provider tag is the reference's way to tell device kinds apart).
B200Device* asB200(Device& d) {
  return d.getProvider() == DeviceProvider::CUDA ? static_cast<B200Device*>(&d) : nullptr;
}
}  // namespace

void PoolBackendAllocator::freeHost(HostBlock& b) {
  // an upload may still be reading either buffer
  b.reading.settle();
  b.spareReading.settle();
  for (void* p : {b.ptr, b.spare}) {
    if (!p) continue;
    if (b.pinned) {
      cudaFreeHost(p);
    } else {
      std::free(p);
    }
  }
  b.ptr = b.spare = nullptr;
}

void* PoolBackendAllocator::allocHost(size_t bytes, bool* pinned) {
  void* p = nullptr;
  // Pinned, so that host<->device copies run at full PCIe/C2C rate and can be
  // asynchronous.
  if (*pinned && cudaMallocHost(&p, bytes) == cudaSuccess) return p;
  // No CUDA driver (a host-only process) or no pinnable memory left: pageable
  // memory holds the same data, copies are just slower.
  cudaGetLastError();
  *pinned = false;
  return std::malloc(bytes);
}

PoolBackendAllocator::~PoolBackendAllocator() {
  for (auto& kv : mHost) freeHost(kv.second);
}

void PoolBackendAllocator::registerDevice(Device& device) {
  std::unique_lock<std::recursive_mutex> guard(mMutex);
  for (auto& l : mLayers)
    if (l.device == &device) return;
  if (!device.hasAllocator()) return;
  auto layer = device.getAllocator();
  // When a device layer is short of memory it asks us to save the block first
  // (the reference's offload hook, LayerAllocator.cpp:238-249).
  layer->registerMemoryOffloadCallback([this](MemoryRecord rec, AllocatorLayerBase& from) {
    std::unique_lock<std::recursive_mutex> g(mMutex);
    auto it = mEntries.find(rec.virtualAddress);
    if (it == mEntries.end()) return;
    if (from.getTag(rec) == it->second.tag) {   // the evicted copy is the newest one
      ensureHost(rec);
      auto& hb = mHost[rec.virtualAddress];
      if (hb.tag != it->second.tag) {
        for (auto& l : mLayers)
          if (l.layer.get() == &from) l.device->copyToHost(rec, hb.ptr);
        hb.tag = it->second.tag;
      }
    }
  });
  mLayers.push_back(DeviceLayer{&device, layer});
}

PoolBackendAllocator::DeviceLayer* PoolBackendAllocator::layerOf(Device& device) {
  for (auto& l : mLayers)
    if (l.device == &device) return &l;
  for (auto& l : mLayers)
    if (*l.device == device) return &l;
  return nullptr;
}

bool PoolBackendAllocator::toRecord(const TensorInternal& t, MemoryRecord& out) {
  if (!mToRecord) {
    fail(POLAR_B200_ERR_UNSUPPORTED, "TensorInternal overload used without a tensor conversion installed");
    return false;
  }
  out = mToRecord(t);
  return true;
}

void PoolBackendAllocator::ensureHost(const MemoryRecord& record) {
  if (mHost.count(record.virtualAddress)) return;
  size_t bytes = record.allocationSize ? record.allocationSize : 4;
  bool pinned = true;
  void* p = allocHost(bytes, &pinned);
  if (!p) {
    fail(POLAR_B200_ERR_CUDA, "host allocation failed");
    return;
  }
  HostBlock& hb = mHost[record.virtualAddress];
  hb.ptr = p;
  hb.size = bytes;
  hb.tag = 0;
  hb.pinned = pinned;
}

void PoolBackendAllocator::updateHost(const MemoryRecord& record) {
  auto& e = mEntries[record.virtualAddress];
  ensureHost(record);
  auto hit = mHost.find(record.virtualAddress);
  if (hit == mHost.end() || hit->second.tag == e.tag) return;
  hit->second.reading.settle();   // nothing may still be reading the buffer that is about to be refilled
  for (auto& l : mLayers) {
    if (l.layer->isAllocated(record) && l.layer->getTag(record) == e.tag) {
      l.device->copyToHost(record, hit->second.ptr);   // synchronises that device's stream
      hit->second.tag = e.tag;
      return;
    }
  }
  // Nobody holds the newest version: a fresh record. The RAM copy is as good as any.
  hit->second.tag = e.tag;
}

// ---- allocate

void PoolBackendAllocator::allocate(const MemoryRecord& record, Device& device) {
  std::unique_lock<std::recursive_mutex> guard(mMutex);
  DeviceLayer* l = layerOf(device);
  if (!l) return fail(POLAR_B200_ERR_INVALID, "allocate: device is not registered");
  if (l->layer->isAllocated(record)) return;   // double allocation is a no-op
  l->layer->allocate(record);
  if (!l->layer->isAllocated(record)) return fail(POLAR_B200_ERR_CUDA, "device allocation failed");
  auto ins = mEntries.emplace(record.virtualAddress, Entry{});
  // A record already known elsewhere keeps its version; the new device copy is stale.
  l->layer->setTag(record, ins.second ? ins.first->second.tag : 0);
}

void PoolBackendAllocator::adoptExternal(const MemoryRecord& record, Device& device, void* devicePtr) {
  std::unique_lock<std::recursive_mutex> guard(mMutex);
  DeviceLayer* l = layerOf(device);
  B200Device* cuda = asB200(device);
  if (!l || !cuda) return fail(POLAR_B200_ERR_INVALID, "adopt: not a registered CUDA device of this plugin");
  if (mEntries.count(record.virtualAddress) || !cuda->pool().adoptExternal(record, devicePtr))
    return fail(POLAR_B200_ERR_INVALID, "adopt: the record exists already, or the pointer is null");
  auto ins = mEntries.emplace(record.virtualAddress, Entry{});
  l->layer->setTag(record, ins.first->second.tag);   // this device holds the newest (only) version
}

void PoolBackendAllocator::allocate(const MemoryRecord& record) {
  std::unique_lock<std::recursive_mutex> guard(mMutex);
  if (mHost.count(record.virtualAddress)) return;
  for (auto& l : mLayers)
    if (l.layer->isAllocated(record)) return;
  ensureHost(record);
  auto ins = mEntries.emplace(record.virtualAddress, Entry{});
  auto hit = mHost.find(record.virtualAddress);
  if (hit != mHost.end()) hit->second.tag = ins.first->second.tag;
}

void PoolBackendAllocator::allocate(const TensorInternal& tensor, Device& device) {
  MemoryRecord r;
  if (toRecord(tensor, r)) allocate(r, device);
}
void PoolBackendAllocator::allocate(const TensorInternal& tensor) {
  MemoryRecord r;
  if (toRecord(tensor, r)) allocate(r);
}

void PoolBackendAllocator::deallocate(const MemoryRecord& record) {
  std::unique_lock<std::recursive_mutex> guard(mMutex);
  auto it = mEntries.find(record.virtualAddress);
  if (it != mEntries.end() && !it->second.locks.empty())
    return fail(POLAR_B200_ERR_INVALID, "deallocate: record is locked");
  for (auto& l : mLayers)
    if (l.layer->isAllocated(record)) l.layer->deallocate(record);
  auto hit = mHost.find(record.virtualAddress);
  if (hit != mHost.end()) {
    freeHost(hit->second);
    mHost.erase(hit);
  }
  if (it != mEntries.end()) mEntries.erase(it);
}
void PoolBackendAllocator::deallocate(const TensorInternal& tensor) {
  MemoryRecord r;
  if (toRecord(tensor, r)) deallocate(r);
}

// ---- lock / release

void PoolBackendAllocator::lock(const MemoryRecord& record, Device& device, LockType type) {
  std::unique_lock<std::recursive_mutex> guard(mMutex);
  DeviceLayer* l = layerOf(device);
  if (!l) return fail(POLAR_B200_ERR_INVALID, "lock: device is not registered");
  Entry& e = mEntries[record.virtualAddress];
  if (type == LockType::READ_WRITE && !e.locks.empty())
    return fail(POLAR_B200_ERR_INVALID, "READ_WRITE lock requested for a record that is already locked");
  for (auto& lk : e.locks)
    if (lk.type == LockType::READ_WRITE)
      return fail(POLAR_B200_ERR_INVALID, "lock requested for a record under a READ_WRITE lock");
  if (!l->layer->isAllocated(record)) {
    l->layer->allocate(record);
    if (!l->layer->isAllocated(record)) return fail(POLAR_B200_ERR_CUDA, "device allocation failed");
    l->layer->setTag(record, 0);
  }
  if (l->layer->getTag(record) != e.tag) {
    // This device's copy is stale: fetch the newest one.
    auto hit = mHost.find(record.virtualAddress);
    bool host_has = hit != mHost.end() && hit->second.tag == e.tag;
    DeviceLayer* src = nullptr;
    if (!host_has)
      for (auto& o : mLayers)
        if (&o != l && o.layer->isAllocated(record) && o.layer->getTag(record) == e.tag) src = &o;
    B200Device* cuda = asB200(device);
    if (host_has) {
      // The new version may already be on its way (endOverwrite uploads ahead of use).
      if (!(cuda && cuda->pool().adoptStaged(record, e.tag))) {
        device.copyToDevice(record, hit->second.ptr);
        // From pinned memory that copy is asynchronous: the host block must not be written
        // or freed before it has run.
        if (cuda && hit->second.pinned) hit->second.reading.mark(cuda->ordinal(), cuda->stream());
      }
    } else if (src && mPeerCopy && mPeerCopy(device, *src->device, record)) {
      // copied by the installed hook
    } else if (src && cuda && asB200(*src->device)) {
      // CUDA device to CUDA device: a peer copy on the destination's stream, ordered after
      // the producer on the source's stream; no RAM staging, no host wait
      cuda->copyFromPeer(record, *asB200(*src->device));
    } else if (src) {
      // devices of another provider only promise copyToHost/copyToDevice
      updateHost(record);
      auto h2 = mHost.find(record.virtualAddress);
      if (h2 != mHost.end()) device.copyToDevice(record, h2->second.ptr);
    }
    // else: nobody has written the record yet; its contents are undefined by contract
  }
  if (type == LockType::READ_WRITE) e.tag++;
  l->layer->setTag(record, e.tag);
  e.locks.push_back(Lock{type, &device});
  l->layer->lock(record);
}

void PoolBackendAllocator::lock(const MemoryRecord& record, LockType type) {
  std::unique_lock<std::recursive_mutex> guard(mMutex);
  Entry& e = mEntries[record.virtualAddress];
  if (type == LockType::READ_WRITE && !e.locks.empty())
    return fail(POLAR_B200_ERR_INVALID, "READ_WRITE lock requested for a record that is already locked");
  for (auto& lk : e.locks)
    if (lk.type == LockType::READ_WRITE)
      return fail(POLAR_B200_ERR_INVALID, "lock requested for a record under a READ_WRITE lock");
  updateHost(record);
  if (type == LockType::READ_WRITE) {
    e.tag++;
    auto hit = mHost.find(record.virtualAddress);
    if (hit != mHost.end()) {
      hit->second.tag = e.tag;
      // The caller is about to write this buffer: an upload queued earlier must have read it.
      hit->second.reading.settle();
    }
  }
  e.locks.push_back(Lock{type, nullptr});
}

void* PoolBackendAllocator::beginOverwrite(const MemoryRecord& record) {
  std::unique_lock<std::recursive_mutex> guard(mMutex);
  Entry& e = mEntries[record.virtualAddress];
  if (!e.locks.empty()) {
    fail(POLAR_B200_ERR_INVALID, "overwrite requested for a record that is locked");
    return nullptr;
  }
  ensureHost(record);
  auto hit = mHost.find(record.virtualAddress);
  if (hit == mHost.end()) return nullptr;
  HostBlock& hb = hit->second;
  if (hb.reading.pending()) {
    // An upload is still reading the current buffer: take the other one (the old contents
    // are not needed), waiting only if that one is being read as well.
    if (!hb.spare) {
      bool pinned = hb.pinned;
      hb.spare = pinned ? allocHost(hb.size, &pinned) : nullptr;
      if (hb.spare && !pinned) {   // mixed kinds would confuse freeHost: do without a spare
        std::free(hb.spare);
        hb.spare = nullptr;
      }
    }
    if (hb.spare) {
      std::swap(hb.ptr, hb.spare);
      std::swap(hb.reading, hb.spareReading);
    }
    hb.reading.settle();
  }
  e.tag++;
  hb.tag = e.tag;
  e.locks.push_back(Lock{LockType::READ_WRITE, nullptr});
  return hb.ptr;
}

void PoolBackendAllocator::endOverwrite(const MemoryRecord& record) {
  std::unique_lock<std::recursive_mutex> guard(mMutex);
  release(record);
  auto it = mEntries.find(record.virtualAddress);
  auto hit = mHost.find(record.virtualAddress);
  if (it == mEntries.end() || hit == mHost.end() || !hit->second.pinned) return;
  for (auto& l : mLayers) {
    B200Device* cuda = asB200(*l.device);
    if (!cuda || !l.layer->isAllocated(record)) continue;
    if (cuda->pool().stage(record, hit->second.ptr, it->second.tag, nullptr))
      hit->second.reading.mark(cuda->ordinal(), cuda->uploadStream());
  }
}

void PoolBackendAllocator::lock(const TensorInternal& tensor, Device& device, LockType type) {
  MemoryRecord r;
  if (toRecord(tensor, r)) lock(r, device, type);
}
void PoolBackendAllocator::lock(const TensorInternal& tensor, LockType type) {
  MemoryRecord r;
  if (toRecord(tensor, r)) lock(r, type);
}

void PoolBackendAllocator::release(const MemoryRecord& record, Device& device) {
  std::unique_lock<std::recursive_mutex> guard(mMutex);
  auto it = mEntries.find(record.virtualAddress);
  if (it == mEntries.end()) return;
  auto& locks = it->second.locks;
  for (size_t i = 0; i < locks.size(); ++i) {
    if (locks[i].device && (locks[i].device == &device || *locks[i].device == device)) {
      locks.erase(locks.begin() + i);
      if (DeviceLayer* l = layerOf(device)) l->layer->release(record);
      return;
    }
  }
}

void PoolBackendAllocator::release(const MemoryRecord& record) {
  std::unique_lock<std::recursive_mutex> guard(mMutex);
  auto it = mEntries.find(record.virtualAddress);
  if (it == mEntries.end()) return;
  auto& locks = it->second.locks;
  for (size_t i = 0; i < locks.size(); ++i) {
    if (!locks[i].device) {
      locks.erase(locks.begin() + i);
      return;
    }
  }
}
void PoolBackendAllocator::release(const TensorInternal& tensor) {
  MemoryRecord r;
  if (toRecord(tensor, r)) release(r);
}

// ---- get

void* PoolBackendAllocator::get(const MemoryRecord& record) {
  std::unique_lock<std::recursive_mutex> guard(mMutex);
  auto hit = mHost.find(record.virtualAddress);
  return hit == mHost.end() ? nullptr : hit->second.ptr;
}
void* PoolBackendAllocator::get(const TensorInternal& tensor) {
  MemoryRecord r;
  return toRecord(tensor, r) ? get(r) : nullptr;
}
void* PoolBackendAllocator::getImpl(const MemoryRecord& record, Device& device) {
  std::unique_lock<std::recursive_mutex> guard(mMutex);
  DeviceLayer* l = layerOf(device);
  return l ? l->layer->getPtr(record) : nullptr;
}
void* PoolBackendAllocator::getImpl(const TensorInternal& tensor, Device& device) {
  MemoryRecord r;
  return toRecord(tensor, r) ? getImpl(r, device) : nullptr;
}

}  // namespace polarai::backend::generic

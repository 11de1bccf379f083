#include "pool_backend_allocator.hpp"

#include <cuda_runtime.h>
#include <polar_b200.h>

#include <cstdio>
#include <cstdlib>

namespace polarai::backend::generic {

using core::internal::LockType;

void PoolBackendAllocator::freeHost(HostBlock& b) {
  if (b.pinned) {
    cudaFreeHost(b.ptr);
  } else {
    std::free(b.ptr);
  }
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
  void* p = nullptr;
  size_t bytes = record.allocationSize ? record.allocationSize : 4;
  // Pinned, so that host<->device copies run at full PCIe/C2C rate and can be
  // asynchronous.
  bool pinned = true;
  if (cudaMallocHost(&p, bytes) != cudaSuccess) {
    // No CUDA driver (a host-only process) or no pinnable memory left: pageable
    // memory holds the same data, copies are just slower.
    cudaGetLastError();
    pinned = false;
    p = std::malloc(bytes);
    if (!p) {
      fail(POLAR_B200_ERR_CUDA, "host allocation failed");
      return;
    }
  }
  mHost[record.virtualAddress] = HostBlock{p, bytes, 0, pinned};
}

void PoolBackendAllocator::updateHost(const MemoryRecord& record) {
  auto& e = mEntries[record.virtualAddress];
  ensureHost(record);
  auto hit = mHost.find(record.virtualAddress);
  if (hit == mHost.end() || hit->second.tag == e.tag) return;
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
    if (host_has) {
      device.copyToDevice(record, hit->second.ptr);
    } else if (src && src->device->getProvider() == DeviceProvider::CUDA &&
               device.getProvider() == DeviceProvider::CUDA) {
      // CUDA device to CUDA device: a peer copy, no RAM staging
      cudaMemcpy(l->layer->getPtr(record), src->layer->getPtr(record), record.allocationSize,
                 cudaMemcpyDefault);
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
    if (hit != mHost.end()) hit->second.tag = e.tag;
  }
  e.locks.push_back(Lock{type, nullptr});
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

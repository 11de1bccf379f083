// BackendAllocator for hosts that drive B200 devices: pinned host memory as the
// RAM layer, one stream-ordered pool layer per registered device (the device's
// own AllocatorLayerBase), tag-based coherence between them.
//
// It plays the role of the reference's LayerAllocator
// (src/backend/generic/lib/allocators/LayerAllocator.cpp) behind the same
// BackendAllocator interface (include/polarai/backend/generic/BackendAllocator.hpp),
// with these differences: tensors stay device-resident between graphs (nothing is
// staged through RAM unless the newest copy really lives elsewhere), devices are
// looked up by pointer instead of by name string, and a stale device copy is
// refreshed straight from the device that holds the newest one.
#pragma once

#include <polarai/backend/generic/BackendAllocator.hpp>

#include <functional>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace polarai::backend::generic {

class PoolBackendAllocator final : public BackendAllocator {
public:
  PoolBackendAllocator() = default;
  ~PoolBackendAllocator() override;

  // How a TensorInternal becomes a MemoryRecord.  TensorInternal's accessors live
  // in the framework's core library; whoever links that library installs the
  // conversion.  Without it the TensorInternal overloads report an error.
  using TensorToRecord = std::function<MemoryRecord(const TensorInternal&)>;
  void setTensorConversion(TensorToRecord fn) { mToRecord = std::move(fn); }

  void registerDevice(Device& device) override;

  void allocate(const TensorInternal& tensor, Device& device) override;
  void allocate(const MemoryRecord& record, Device& device) override;
  void allocate(const MemoryRecord& record) override;
  void allocate(const TensorInternal& tensor) override;
  void deallocate(const TensorInternal& tensor) override;
  void deallocate(const MemoryRecord& record);

  void lock(const TensorInternal& tensor, Device& device, LockType type) override;
  void lock(const MemoryRecord& record, Device& device, LockType type) override;
  void lock(const MemoryRecord& record, LockType type) override;
  void lock(const TensorInternal& tensor, LockType type) override;

  void release(const MemoryRecord& record, Device& device) override;
  void release(const MemoryRecord& record) override;
  void release(const TensorInternal& tensor) override;

  void* get(const MemoryRecord& record) override;
  void* get(const TensorInternal& tensor) override;

  // Error state (the reference terminates the process instead).
  int lastStatus() const { return mStatus; }
  const char* lastError() const { return mError; }
  void clearError() { mStatus = 0; mError = ""; }

protected:
  void* getImpl(const TensorInternal& tensor, Device& device) override;
  void* getImpl(const MemoryRecord& record, Device& device) override;

private:
  struct HostBlock { void* ptr; size_t size; size_t tag; bool pinned; };
  static void freeHost(HostBlock& b);
  struct Lock { LockType type; Device* device; };  // device == nullptr: host
  struct Entry {
    size_t tag = 1;                       // newest version of the record
    std::vector<Lock> locks;
  };
  struct DeviceLayer { Device* device; std::shared_ptr<AllocatorLayerBase> layer; };

  DeviceLayer* layerOf(Device& device);
  bool toRecord(const TensorInternal& t, MemoryRecord& out);
  void ensureHost(const MemoryRecord& record);
  void updateHost(const MemoryRecord& record);   // pull the newest copy into RAM
  void fail(int status, const char* msg) { mStatus = status; mError = msg; }

  std::vector<DeviceLayer> mLayers;
  std::unordered_map<size_t, HostBlock> mHost;
  std::unordered_map<size_t, Entry> mEntries;
  TensorToRecord mToRecord;
  std::recursive_mutex mMutex;
  int mStatus = 0;
  const char* mError = "";
};

}  // namespace polarai::backend::generic

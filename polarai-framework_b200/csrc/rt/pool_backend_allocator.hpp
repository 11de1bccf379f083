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

#include "cuda_api.hpp"

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

  // ---- beyond the reference interface ----
  // Whole-record overwrite from the host (what a loader does): like a host READ_WRITE
  // lock, except that the old contents are NOT preserved, which lets the record keep TWO
  // pinned buffers and hand out the one no upload is still reading - the host fills
  // version v+1 while version v is still crossing PCIe.  endOverwrite() releases the lock
  // and starts uploading the new version to every CUDA device that holds the record, on
  // that device's upload stream and into a fresh block, so that the copy overlaps kernels
  // still reading the old version; the next device lock adopts the fresh block.
  void* beginOverwrite(const MemoryRecord& record);
  void endOverwrite(const MemoryRecord& record);
  // Device-to-device refresh used when both devices are CUDA devices of this plugin;
  // replaceable so that host-only tests can observe the choice.  Returns false when it
  // did not do the copy (the allocator then stages through host memory).
  // Makes caller-owned device memory the record's copy on `device` (see
  // B200Allocator::adoptExternal); the record starts as "newest on that device".
  void adoptExternal(const MemoryRecord& record, Device& device, void* devicePtr);
  using PeerCopyFn = std::function<bool(Device& dst, Device& src, const MemoryRecord&)>;
  void setPeerCopy(PeerCopyFn fn) { mPeerCopy = std::move(fn); }

  // Error state (the reference terminates the process instead).
  int lastStatus() const { return mStatus; }
  const char* lastError() const { return mError; }
  void clearError() { mStatus = 0; mError = ""; }

protected:
  void* getImpl(const TensorInternal& tensor, Device& device) override;
  void* getImpl(const MemoryRecord& record, Device& device) override;

private:
  // Host copy of a record.  `ptr` is the current buffer; `spare` a second one that
  // beginOverwrite() alternates with (allocated on first need).  `reading` / `spareReading`
  // track asynchronous uploads that may still be reading the respective buffer: the host
  // must not write or free a buffer before they have run.
  struct HostBlock {
    void* ptr = nullptr;
    size_t size = 0;
    size_t tag = 0;
    bool pinned = false;
    void* spare = nullptr;
    PendingRead<CudaApi> reading, spareReading;
  };
  static void freeHost(HostBlock& b);
  static void* allocHost(size_t bytes, bool* pinned);
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
  PeerCopyFn mPeerCopy;
  std::recursive_mutex mMutex;
  int mStatus = 0;
  const char* mError = "";
};

}  // namespace polarai::backend::generic

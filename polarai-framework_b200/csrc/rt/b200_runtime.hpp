// PolarAI device-runtime plugin for NVIDIA B200.
//
// Implements the reference's runtime boundary - the abstract classes Context,
// Device, Event (include/polarai/backend/generic/runtime/{Context,Device,Event}.hpp)
// and AllocatorLayerBase (include/polarai/backend/generic/AllocatorLayerBase.hpp) -
// on the CUDA runtime API, with precompiled sm_100a kernels reached through the
// C ABI of libpolar_b200.so.  It replaces src/backend/generic/runtime/cuda/
// (CudaContext, CudaDevice, CudaAllocator, CudaEvent), which JIT-links PTX and
// synchronises after every launch.
//
// Differences a caller can observe:
//  - device names are unique ("NVIDIA B200 #3"): the reference keys its
//    allocator maps by name (LayerAllocator.cpp:30,226-234) and eight identical
//    names would collide;
//  - getPtr() returns the device pointer itself (as the USM SYCL allocator does),
//    not the address of a handle;
//  - launch() is stream-ordered and does not synchronise; the returned Event
//    completes when the kernel has;
//  - memory comes from a per-device cudaMallocAsync pool that keeps freed blocks;
//  - the calling thread's current CUDA device is never changed: every method makes
//    its GPU current for its own duration only (device_scope.hpp), and a GPU is not
//    touched at all (no context, stream or pool on it) until it is first used, so a
//    host that enumerates eight devices and computes on one pays for one.
#pragma once

#include <polarai/backend/generic/AllocatorLayerBase.hpp>
#include <polarai/backend/generic/MemoryRecord.hpp>
#include <polarai/backend/generic/runtime/Context.hpp>
#include <polarai/backend/generic/runtime/Device.hpp>
#include <polarai/backend/generic/runtime/Event.hpp>

#include <cuda_runtime.h>

#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

namespace polarai::backend::generic {

class B200Device;

// Per-device memory layer on a stream-ordered pool.
class B200Allocator final : public AllocatorLayerBase {
public:
  explicit B200Allocator(B200Device& owner);
  ~B200Allocator() override;

  void registerMemoryOffloadCallback(MemoryOffloadCallbackT cb) override { mOffload = std::move(cb); }
  void allocate(MemoryRecord record) override;
  void deallocate(MemoryRecord record) override;
  void lock(MemoryRecord record) override;
  void release(MemoryRecord record) override;
  void* getPtr(MemoryRecord record) override;
  bool isAllocated(const MemoryRecord& record) const override;
  size_t getTag(MemoryRecord record) override;
  void setTag(MemoryRecord record, size_t tag) override;

  // ---- not part of the reference interface ----
  size_t bytesInUse() const { return mBytes; }
  void setLimit(size_t bytes) { mLimit = bytes; }   // 0 = no limit
  int lastError() const { return mLastError; }
  // Frees everything; the layer stays valid but empty (see ~B200Device).
  void shutdown();

  // "The record's block was just written by work queued on the device's main stream."
  // A later copyToHost of the record waits for exactly that work instead of for
  // everything queued on the stream.
  void markWritten(const MemoryRecord& record);
  // The event of the last markWritten (nullptr: never marked).
  cudaEvent_t writtenEvent(const MemoryRecord& record);

  // Upload ahead of use: version `tag` of the record is copied from pinned host memory
  // into a FRESH block on the device's upload stream, while kernels on the main stream
  // may still be reading the current block.  adoptStaged() swaps the fresh block in
  // (the main stream waits for the upload; the old block is freed in stream order).
  // `uploaded` receives an event (owned by the callee) that completes with the copy.
  bool stage(const MemoryRecord& record, const void* pinnedSrc, size_t tag, cudaEvent_t* uploaded);
  bool adoptStaged(const MemoryRecord& record, size_t tag);

  // Registers device memory the CALLER owns as the record's block (never freed, evicted or
  // replaced by this layer): how a gradient that must live in NVLink peer memory becomes a
  // record that launches can name.  False when the record already exists.
  bool adoptExternal(const MemoryRecord& record, void* devicePtr);

private:
  struct Block { void* ptr; size_t size; size_t tag; int locks; cudaEvent_t written; bool external = false; };
  struct Staged { void* ptr; size_t size; size_t tag; cudaEvent_t done; };
  bool evictFor(size_t bytes);
  bool ensurePool();
  void dropStaged(size_t va);

  B200Device& mOwner;
  cudaMemPool_t mPool = nullptr;
  bool mPoolTried = false;
  bool mDead = false;
  MemoryOffloadCallbackT mOffload;
  std::unordered_map<size_t, Block> mBlocks;          // by virtual address
  std::unordered_map<size_t, Staged> mStaged;         // uploaded ahead, not yet adopted
  std::unordered_set<size_t> mReleased;               // allocated, unlocked: may be evicted
  size_t mBytes = 0;
  size_t mLimit = 0;
  int mLastError = 0;
  mutable std::mutex mMutex;
};

class B200Event final : public Event {
public:
  B200Event(B200Device* device, cudaEvent_t evt, int status);
  ~B200Event() override;
  void wait() override;
  void addCallback(std::function<void()> cb) override { mCallbacks.push_back(std::move(cb)); }
  auto getDevice() -> Device* override;
  // polar_b200_status of the launch that produced this event.
  int status() const { return mStatus; }
  cudaEvent_t native() const { return mEvent; }

private:
  B200Device* mDevice;
  cudaEvent_t mEvent;
  int mStatus;
  std::vector<std::function<void()>> mCallbacks;
};

class B200Device final : public Device {
public:
  explicit B200Device(int ordinal);
  ~B200Device() override;

  auto getProvider() const -> DeviceProvider override { return DeviceProvider::CUDA; }
  auto getKind() const -> DeviceKind override { return DeviceKind::GPU; }
  auto getDeviceName() const -> std::string override { return mName; }
  auto isPartitionSupported(PartitionDomain) -> bool override { return false; }
  auto hasAllocator() -> bool override { return true; }
  auto partition(PartitionDomain) -> std::vector<std::shared_ptr<Device>> override { return {}; }
  auto getAllocator() -> std::shared_ptr<AllocatorLayerBase> override { return mAllocator; }
  bool operator==(const Device& other) const override { return mName == other.getDeviceName(); }

  void copyToHost(MemoryRecord record, void* dest) const override;
  void copyToDevice(MemoryRecord record, void* src) const override;
  auto launch(BackendAllocator&, LaunchCommand&, Event*) -> Event* override;
  void consumeEvent(Event* evt) override;
  // Kernels are precompiled for sm_100a; there is nothing to select.
  void selectBinary(std::vector<std::shared_ptr<ProgramDesc>>&) override {}

  // ---- not part of the reference interface ----
  int ordinal() const { return mOrdinal; }
  // The three streams of the device, created on first use: `stream` carries kernels and
  // ordinary copies; uploads ahead of use and targeted read-backs have their own so
  // that they overlap the kernels.
  cudaStream_t stream() const { ensureReady(); return mStream; }
  cudaStream_t uploadStream() const { ensureReady(); return mUpload; }
  cudaStream_t downloadStream() const { ensureReady(); return mDownload; }
  bool ready() const { return mReady; }
  B200Allocator& pool() { return *mAllocator; }
  int lastStatus() const { return mLastStatus; }
  // Returns the last error status and clears it, so that one failure is reported once.
  int takeStatus() { int s = mLastStatus; mLastStatus = 0; return s; }
  const std::string& lastError() const { return mLastError; }
  void synchronize() const;
  // Newest copy of the record lives on `src`: fetch it device to device, ordered after
  // the producer on src's stream and before later work on this device's stream.
  void copyFromPeer(MemoryRecord record, B200Device& src);

private:
  void ensureReady() const;

  int mOrdinal;
  mutable bool mReady = false;
  mutable std::mutex mInitMutex;
  mutable cudaStream_t mStream = nullptr;
  mutable cudaStream_t mUpload = nullptr;
  mutable cudaStream_t mDownload = nullptr;
  void* mWorkspace = nullptr;        // scratch for split-k matmuls, grown on demand
  uint64_t mWorkspaceBytes = 0;
  std::string mName;
  std::shared_ptr<B200Allocator> mAllocator;
  mutable int mLastStatus = 0;
  mutable std::string mLastError;
};

class B200Context final : public Context {
public:
  B200Context();
  ~B200Context() override = default;
  std::vector<std::shared_ptr<Device>>& getDevices() override { return mDevices; }

private:
  std::vector<std::shared_ptr<Device>> mDevices;
};

}  // namespace polarai::backend::generic

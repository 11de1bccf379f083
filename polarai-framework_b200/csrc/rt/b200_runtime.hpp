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
//  - memory comes from a per-device cudaMallocAsync pool that keeps freed blocks.
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
  B200Allocator(int ordinal, cudaStream_t stream);
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

  // Not part of the reference interface.
  size_t bytesInUse() const { return mBytes; }
  void setLimit(size_t bytes) { mLimit = bytes; }   // 0 = no limit
  int lastError() const { return mLastError; }

private:
  struct Block { void* ptr; size_t size; size_t tag; int locks; };
  bool evictFor(size_t bytes);

  int mOrdinal;
  cudaStream_t mStream;
  cudaMemPool_t mPool = nullptr;
  MemoryOffloadCallbackT mOffload;
  std::unordered_map<size_t, Block> mBlocks;          // by virtual address
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

  // Not part of the reference interface.
  int ordinal() const { return mOrdinal; }
  cudaStream_t stream() const { return mStream; }
  int lastStatus() const { return mLastStatus; }
  // Returns the last error status and clears it, so that one failure is reported once.
  int takeStatus() { int s = mLastStatus; mLastStatus = 0; return s; }
  const std::string& lastError() const { return mLastError; }
  void synchronize() const;
  cudaEvent_t takeEvent();
  void giveEvent(cudaEvent_t e);

private:
  int mOrdinal;
  cudaStream_t mStream = nullptr;
  void* mWorkspace = nullptr;        // scratch for split-k matmuls, grown on demand
  uint64_t mWorkspaceBytes = 0;
  std::string mName;
  std::shared_ptr<B200Allocator> mAllocator;
  mutable int mLastStatus = 0;
  mutable std::string mLastError;
  std::vector<cudaEvent_t> mEventPool;
  std::mutex mEventMutex;
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

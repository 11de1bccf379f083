#include "b200_runtime.hpp"

#include <polarai/backend/generic/BackendAllocator.hpp>
#include <polarai/backend/generic/runtime/LaunchCommand.h>
#include <polarai/backend/generic/runtime/TensorInfo.h>
#include <polarai/backend/generic/runtime/api.h>

#include <polar_b200.h>

#include <cstdio>
#include <cstdlib>

namespace polarai::backend::generic {

namespace {
// Environment switch for diagnostics, read once.
bool verbose() {
  static int v = -1;
  if (v < 0) v = std::getenv("POLAR_B200_VERBOSE") ? 1 : 0;
  return v == 1;
}
void note(const char* what, cudaError_t e) {
  if (e != cudaSuccess)
    std::fprintf(stderr, "[polar_rt_cuda] %s: %s\n", what, cudaGetErrorString(e));
}
}  // namespace

// ---------------------------------------------------------------- allocator

B200Allocator::B200Allocator(int ordinal, cudaStream_t stream) : mOrdinal(ordinal), mStream(stream) {
  cudaMemPoolProps props = {};
  props.allocType = cudaMemAllocationTypePinned;
  props.handleTypes = cudaMemHandleTypeNone;
  props.location.type = cudaMemLocationTypeDevice;
  props.location.id = ordinal;
  cudaError_t e = cudaMemPoolCreate(&mPool, &props);
  note("cudaMemPoolCreate", e);
  if (e == cudaSuccess) {
    // Keep freed blocks in the pool: graphs are evaluated again and again with
    // the same tensor sizes.
    unsigned long long keep = ~0ull;
    note("cudaMemPoolSetAttribute", cudaMemPoolSetAttribute(mPool, cudaMemPoolAttrReleaseThreshold, &keep));
  } else {
    mPool = nullptr;
  }
}

B200Allocator::~B200Allocator() {
  cudaSetDevice(mOrdinal);
  cudaStreamSynchronize(mStream);
  for (auto& kv : mBlocks) cudaFreeAsync(kv.second.ptr, mStream);
  cudaStreamSynchronize(mStream);
  if (mPool) cudaMemPoolDestroy(mPool);
}

bool B200Allocator::evictFor(size_t bytes) {
  // Frees released (unlocked) blocks until `bytes` fit under the limit, telling
  // the owner first so it can save the contents (the reference's offload hook:
  // CudaAllocator.hpp:35-48).
  while (mLimit && mBytes + bytes > mLimit && !mReleased.empty()) {
    size_t va = *mReleased.begin();
    auto it = mBlocks.find(va);
    mReleased.erase(mReleased.begin());
    if (it == mBlocks.end() || it->second.locks > 0) continue;
    MemoryRecord victim{va, it->second.size};
    if (mOffload) {
      mMutex.unlock();
      mOffload(victim, *this);
      mMutex.lock();
      it = mBlocks.find(va);
      if (it == mBlocks.end()) continue;
    }
    cudaFreeAsync(it->second.ptr, mStream);
    mBytes -= it->second.size;
    mBlocks.erase(it);
  }
  return !(mLimit && mBytes + bytes > mLimit);
}

void B200Allocator::allocate(MemoryRecord record) {
  std::unique_lock<std::mutex> guard(mMutex);
  if (mBlocks.count(record.virtualAddress)) return;  // double allocation is a no-op
  cudaSetDevice(mOrdinal);
  size_t bytes = record.allocationSize ? record.allocationSize : 4;
  if (!evictFor(bytes)) {
    mLastError = POLAR_B200_ERR_CUDA;
    std::fprintf(stderr, "[polar_rt_cuda] device %d: %zu bytes do not fit under the %zu byte limit\n",
                 mOrdinal, bytes, mLimit);
    return;
  }
  void* ptr = nullptr;
  cudaError_t e = mPool ? cudaMallocFromPoolAsync(&ptr, bytes, mPool, mStream)
                        : cudaMallocAsync(&ptr, bytes, mStream);
  if (e != cudaSuccess) {
    note("cudaMallocAsync", e);
    mLastError = POLAR_B200_ERR_CUDA;
    cudaGetLastError();
    return;
  }
  mBlocks[record.virtualAddress] = Block{ptr, bytes, 1, 0};
  mBytes += bytes;
}

void B200Allocator::deallocate(MemoryRecord record) {
  std::unique_lock<std::mutex> guard(mMutex);
  auto it = mBlocks.find(record.virtualAddress);
  if (it == mBlocks.end()) return;
  if (it->second.locks > 0) {
    std::fprintf(stderr, "[polar_rt_cuda] deallocate of a locked record %zu ignored\n", record.virtualAddress);
    mLastError = POLAR_B200_ERR_INVALID;
    return;
  }
  cudaSetDevice(mOrdinal);
  cudaFreeAsync(it->second.ptr, mStream);
  mBytes -= it->second.size;
  mReleased.erase(record.virtualAddress);
  mBlocks.erase(it);
}

void B200Allocator::lock(MemoryRecord record) {
  std::unique_lock<std::mutex> guard(mMutex);
  auto it = mBlocks.find(record.virtualAddress);
  if (it == mBlocks.end()) return;
  it->second.locks++;
  mReleased.erase(record.virtualAddress);
}

void B200Allocator::release(MemoryRecord record) {
  std::unique_lock<std::mutex> guard(mMutex);
  auto it = mBlocks.find(record.virtualAddress);
  if (it == mBlocks.end()) return;
  if (it->second.locks > 0) it->second.locks--;
  if (it->second.locks == 0) mReleased.insert(record.virtualAddress);
}

void* B200Allocator::getPtr(MemoryRecord record) {
  std::unique_lock<std::mutex> guard(mMutex);
  auto it = mBlocks.find(record.virtualAddress);
  return it == mBlocks.end() ? nullptr : it->second.ptr;
}

bool B200Allocator::isAllocated(const MemoryRecord& record) const {
  std::unique_lock<std::mutex> guard(mMutex);
  return mBlocks.count(record.virtualAddress) > 0;
}

size_t B200Allocator::getTag(MemoryRecord record) {
  std::unique_lock<std::mutex> guard(mMutex);
  auto it = mBlocks.find(record.virtualAddress);
  return it == mBlocks.end() ? 0 : it->second.tag;
}

void B200Allocator::setTag(MemoryRecord record, size_t tag) {
  std::unique_lock<std::mutex> guard(mMutex);
  auto it = mBlocks.find(record.virtualAddress);
  if (it != mBlocks.end()) it->second.tag = tag;
}

// -------------------------------------------------------------------- event

B200Event::B200Event(B200Device* device, cudaEvent_t evt, int status)
    : mDevice(device), mEvent(evt), mStatus(status) {}

B200Event::~B200Event() {
  if (mEvent) mDevice->giveEvent(mEvent);
}

void B200Event::wait() {
  if (mEvent) {
    cudaSetDevice(mDevice->ordinal());
    cudaError_t e = cudaEventSynchronize(mEvent);
    if (e != cudaSuccess) {
      note("cudaEventSynchronize", e);
      mStatus = POLAR_B200_ERR_CUDA;
    }
  }
  // Callbacks run on the waiting thread, after completion, once
  // (as src/backend/generic/runtime/cuda/CudaEvent.cpp:21-29 does).
  auto cbs = std::move(mCallbacks);
  mCallbacks.clear();
  for (auto& cb : cbs) cb();
}

auto B200Event::getDevice() -> Device* { return mDevice; }

// ------------------------------------------------------------------- device

B200Device::B200Device(int ordinal) : mOrdinal(ordinal) {
  cudaSetDevice(ordinal);
  cudaDeviceProp prop;
  std::string base = "CUDA device";
  if (cudaGetDeviceProperties(&prop, ordinal) == cudaSuccess) base = prop.name;
  mName = base + " #" + std::to_string(ordinal);
  note("cudaStreamCreate", cudaStreamCreateWithFlags(&mStream, cudaStreamNonBlocking));
  mAllocator = std::make_shared<B200Allocator>(ordinal, mStream);
}

B200Device::~B200Device() {
  cudaSetDevice(mOrdinal);
  if (mStream) cudaStreamSynchronize(mStream);
  if (mWorkspace) cudaFree(mWorkspace);
  mAllocator.reset();
  for (cudaEvent_t e : mEventPool) cudaEventDestroy(e);
  if (mStream) cudaStreamDestroy(mStream);
}

cudaEvent_t B200Device::takeEvent() {
  {
    std::unique_lock<std::mutex> guard(mEventMutex);
    if (!mEventPool.empty()) {
      cudaEvent_t e = mEventPool.back();
      mEventPool.pop_back();
      return e;
    }
  }
  cudaEvent_t e = nullptr;
  note("cudaEventCreate", cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  return e;
}

void B200Device::giveEvent(cudaEvent_t e) {
  std::unique_lock<std::mutex> guard(mEventMutex);
  mEventPool.push_back(e);
}

void B200Device::synchronize() const {
  cudaSetDevice(mOrdinal);
  cudaError_t e = cudaStreamSynchronize(mStream);
  if (e != cudaSuccess) {
    note("cudaStreamSynchronize", e);
    mLastStatus = POLAR_B200_ERR_CUDA;
    mLastError = cudaGetErrorString(e);
  }
}

void B200Device::copyToHost(MemoryRecord record, void* dest) const {
  void* src = mAllocator->getPtr(record);
  if (!src || !dest) {
    mLastStatus = POLAR_B200_ERR_INVALID;
    mLastError = "copyToHost: record is not allocated on this device";
    return;
  }
  cudaSetDevice(mOrdinal);
  cudaError_t e = cudaMemcpyAsync(dest, src, record.allocationSize, cudaMemcpyDeviceToHost, mStream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(mStream);
  if (e != cudaSuccess) {
    note("copyToHost", e);
    mLastStatus = POLAR_B200_ERR_CUDA;
    mLastError = cudaGetErrorString(e);
  }
}

void B200Device::copyToDevice(MemoryRecord record, void* src) const {
  void* dst = mAllocator->getPtr(record);
  if (!dst || !src) {
    mLastStatus = POLAR_B200_ERR_INVALID;
    mLastError = "copyToDevice: record is not allocated on this device";
    return;
  }
  cudaSetDevice(mOrdinal);
  // Stream-ordered: kernels launched afterwards on this device's stream see the
  // data.  From pageable memory the call returns once the source is staged;
  // from pinned memory it is asynchronous and the caller must not overwrite
  // `src` before the device's next synchronisation point.
  cudaError_t e = cudaMemcpyAsync(dst, src, record.allocationSize, cudaMemcpyHostToDevice, mStream);
  if (e != cudaSuccess) {
    note("copyToDevice", e);
    mLastStatus = POLAR_B200_ERR_CUDA;
    mLastError = cudaGetErrorString(e);
  }
}

auto B200Device::launch(BackendAllocator& allocator, LaunchCommand& cmd, Event* blocking) -> Event* {
  cudaSetDevice(mOrdinal);
  int status = POLAR_B200_OK;
  if (blocking) {
    // Work of this device is stream-ordered already; an event of another device
    // becomes a stream dependency instead of a host wait.
    auto* be = static_cast<B200Event*>(blocking);
    if (be->getDevice() != this && be->native())
      note("cudaStreamWaitEvent", cudaStreamWaitEvent(mStream, be->native(), 0));
  }
  constexpr uint64_t kMaxArgs = 8;
  polar_b200_arg args[kMaxArgs];
  const char* name = cmd.nativeKernelName ? cmd.nativeKernelName : "";
  if (cmd.argsCount > kMaxArgs || (cmd.argsCount && !cmd.args)) {
    status = POLAR_B200_ERR_UNSUPPORTED;
    mLastError = "launch: bad argument list";
  }
  for (uint64_t i = 0; status == POLAR_B200_OK && i < cmd.argsCount; ++i) {
    const ArgDesc& a = cmd.args[i];
    if (a.type == ArgDesc::TENSOR) {
      auto* t = static_cast<TensorInfo*>(a.arg);
      if (!t || t->dataType != 2 /* DataType::FLOAT */) {
        status = POLAR_B200_ERR_UNSUPPORTED;
        mLastError = "launch: only float tensors are supported";
        break;
      }
      MemoryRecord rec;
      rec.virtualAddress = t->virtAddr;
      rec.allocationSize = 4;
      for (uint64_t d = 0; d < t->dims; ++d) rec.allocationSize *= t->shape[d];
      args[i].is_tensor = 1;
      args[i].tensor.data = allocator.get<float>(rec, *this);
      args[i].tensor.dims = t->dims;
      args[i].tensor.shape = t->shape;
      args[i].scalar = 0.f;
      args[i].integer = 0;
      if (!args[i].tensor.data && rec.allocationSize) {
        status = POLAR_B200_ERR_INVALID;
        mLastError = "launch: tensor is not allocated on this device";
      }
    } else {
      args[i].is_tensor = 0;
      args[i].tensor = polar_b200_tensor{nullptr, 0, nullptr};
      args[i].scalar = 0.f;
      args[i].integer = 0;
      if (a.arg && a.size == 8) {
        args[i].integer = *static_cast<int64_t*>(a.arg);     // attributes such as a pooling window
      } else if (a.arg) {
        args[i].scalar = *static_cast<float*>(a.arg);
      }
    }
  }
  if (status == POLAR_B200_OK) {
    // Scratch for split-k matmuls is kept for the life of the device and only ever grows:
    // taking it from the stream-ordered pool per launch costs a physical allocation each
    // time the pool has been trimmed at a synchronisation point.
    const uint64_t need = polar_b200_launch_workspace_bytes(name, args, cmd.argsCount);
    if (need > mWorkspaceBytes) {
      if (mWorkspace) cudaFreeAsync(mWorkspace, mStream);
      mWorkspace = nullptr;
      mWorkspaceBytes = 0;
      void* p = nullptr;
      if (cudaMallocAsync(&p, need, mStream) == cudaSuccess) {
        mWorkspace = p;
        mWorkspaceBytes = need;
      } else {
        cudaGetLastError();   // the library then falls back to its own per-launch allocation
      }
    }
    status = polar_b200_launch_by_name(name, args, cmd.argsCount, need <= mWorkspaceBytes ? mWorkspace : nullptr,
                                       need <= mWorkspaceBytes ? mWorkspaceBytes : 0, mStream);
    if (status != POLAR_B200_OK) mLastError = polar_b200_last_error();
  }
  if (status != POLAR_B200_OK) {
    // The reference has no error channel here (its runtimes terminate); this one
    // reports and hands back an event that carries the status.
    std::fprintf(stderr, "[polar_rt_cuda] launch of '%s' (%s) failed: %s\n", name,
                 cmd.kernelName ? cmd.kernelName : "", mLastError.c_str());
    mLastStatus = status;
  } else if (verbose()) {
    std::fprintf(stderr, "[polar_rt_cuda] %s: launched %s\n", mName.c_str(), name);
  }
  cudaEvent_t evt = takeEvent();
  if (evt) note("cudaEventRecord", cudaEventRecord(evt, mStream));
  return new B200Event(this, evt, status);
}

void B200Device::consumeEvent(Event* evt) {
  if (!evt) return;
  evt->wait();
  delete evt;
}

// ------------------------------------------------------------------ context

B200Context::B200Context() {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    n = 0;
  }
  for (int i = 0; i < n; ++i) {
    int major = 0;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, i);
    if (major != 10) {
      std::fprintf(stderr, "[polar_rt_cuda] device %d is not sm_100: skipped (kernels are built for sm_100a only)\n", i);
      continue;
    }
    mDevices.push_back(std::make_shared<B200Device>(i));
  }
}

}  // namespace polarai::backend::generic

// The two symbols RuntimeDriver looks up with dlsym
// (src/backend/generic/runtime/driver/RuntimeDriver.cpp:39-46).
extern "C" {
polarai::backend::generic::Context* initContext() { return new polarai::backend::generic::B200Context(); }
void closeContext(polarai::backend::generic::Context* ctx) { delete ctx; }
}

#include "b200_runtime.hpp"

#include "cuda_api.hpp"

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
  if (e != cudaSuccess) {
    std::fprintf(stderr, "[polar_rt_cuda] %s: %s\n", what, cudaGetErrorString(e));
    cudaGetLastError();
  }
}
}  // namespace

// ---------------------------------------------------------------- allocator

B200Allocator::B200Allocator(B200Device& owner) : mOwner(owner) {}

bool B200Allocator::ensurePool() {
  // Called with the device current and mMutex held.
  if (mPoolTried) return mPool != nullptr;
  mPoolTried = true;
  cudaMemPoolProps props = {};
  props.allocType = cudaMemAllocationTypePinned;
  props.handleTypes = cudaMemHandleTypeNone;
  props.location.type = cudaMemLocationTypeDevice;
  props.location.id = mOwner.ordinal();
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
  return mPool != nullptr;
}

B200Allocator::~B200Allocator() { shutdown(); }

void B200Allocator::shutdown() {
  // Called by the owning device before its streams go away; whoever still holds this layer
  // afterwards (an allocator that outlives the context) finds it empty and inert.
  std::unique_lock<std::mutex> guard(mMutex);
  if (mDead) return;
  mDead = true;
  if (!mOwner.ready()) return;   // the GPU was never used: nothing was created on it
  ScopedDevice on(mOwner.ordinal());
  cudaStream_t s = mOwner.stream();
  cudaStreamSynchronize(mOwner.uploadStream());
  cudaStreamSynchronize(s);
  for (auto& kv : mStaged) {
    cudaFreeAsync(kv.second.ptr, s);
    CudaApi::giveEvent(mOwner.ordinal(), kv.second.done);
  }
  for (auto& kv : mBlocks) {
    if (!kv.second.external) cudaFreeAsync(kv.second.ptr, s);
    CudaApi::giveEvent(mOwner.ordinal(), kv.second.written);
  }
  cudaStreamSynchronize(s);
  mBlocks.clear();
  mStaged.clear();
  mReleased.clear();
  mBytes = 0;
  if (mPool) cudaMemPoolDestroy(mPool);
  mPool = nullptr;
}

bool B200Allocator::evictFor(size_t bytes) {
  // Frees released (unlocked) blocks until `bytes` fit under the limit, telling
  // the owner first so it can save the contents (the reference's offload hook:
  // CudaAllocator.hpp:35-48).  Called with the device current and mMutex held.
  while (mLimit && mBytes + bytes > mLimit && !mReleased.empty()) {
    size_t va = *mReleased.begin();
    auto it = mBlocks.find(va);
    mReleased.erase(mReleased.begin());
    if (it == mBlocks.end() || it->second.locks > 0 || it->second.external) continue;
    MemoryRecord victim{va, it->second.size};
    if (mOffload) {
      mMutex.unlock();
      mOffload(victim, *this);
      mMutex.lock();
      it = mBlocks.find(va);
      if (it == mBlocks.end()) continue;
    }
    dropStaged(va);
    cudaFreeAsync(it->second.ptr, mOwner.stream());
    CudaApi::giveEvent(mOwner.ordinal(), it->second.written);
    mBytes -= it->second.size;
    mBlocks.erase(it);
  }
  return !(mLimit && mBytes + bytes > mLimit);
}

void B200Allocator::allocate(MemoryRecord record) {
  std::unique_lock<std::mutex> guard(mMutex);
  if (mBlocks.count(record.virtualAddress)) return;  // double allocation is a no-op
  if (mDead) {
    mLastError = POLAR_B200_ERR_INVALID;
    return;
  }
  ScopedDevice on(mOwner.ordinal());
  cudaStream_t s = mOwner.stream();
  size_t bytes = record.allocationSize ? record.allocationSize : 4;
  if (!evictFor(bytes)) {
    mLastError = POLAR_B200_ERR_CUDA;
    std::fprintf(stderr, "[polar_rt_cuda] device %d: %zu bytes do not fit under the %zu byte limit\n",
                 mOwner.ordinal(), bytes, mLimit);
    return;
  }
  void* ptr = nullptr;
  cudaError_t e = ensurePool() ? cudaMallocFromPoolAsync(&ptr, bytes, mPool, s) : cudaMallocAsync(&ptr, bytes, s);
  if (e != cudaSuccess) {
    note("cudaMallocAsync", e);
    mLastError = POLAR_B200_ERR_CUDA;
    return;
  }
  mBlocks[record.virtualAddress] = Block{ptr, bytes, 1, 0, nullptr};
  mBytes += bytes;
}

void B200Allocator::dropStaged(size_t va) {
  auto st = mStaged.find(va);
  if (st == mStaged.end()) return;
  cudaFreeAsync(st->second.ptr, mOwner.uploadStream());
  CudaApi::giveEvent(mOwner.ordinal(), st->second.done);
  mBytes -= st->second.size;
  mStaged.erase(st);
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
  ScopedDevice on(mOwner.ordinal());
  dropStaged(record.virtualAddress);
  if (!it->second.external) {
    cudaFreeAsync(it->second.ptr, mOwner.stream());
    mBytes -= it->second.size;
  }
  CudaApi::giveEvent(mOwner.ordinal(), it->second.written);
  mReleased.erase(record.virtualAddress);
  mBlocks.erase(it);
}

bool B200Allocator::adoptExternal(const MemoryRecord& record, void* devicePtr) {
  std::unique_lock<std::mutex> guard(mMutex);
  if (mDead || !devicePtr || mBlocks.count(record.virtualAddress)) return false;
  Block b{devicePtr, record.allocationSize, 1, 0, nullptr};
  b.external = true;
  mBlocks[record.virtualAddress] = b;
  return true;
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

void B200Allocator::markWritten(const MemoryRecord& record) {
  std::unique_lock<std::mutex> guard(mMutex);
  auto it = mBlocks.find(record.virtualAddress);
  if (it == mBlocks.end()) return;
  ScopedDevice on(mOwner.ordinal());
  if (!it->second.written) it->second.written = CudaApi::takeEvent(mOwner.ordinal());
  // Re-recording an event is allowed: whoever waits on it afterwards waits for this point.
  if (it->second.written) note("cudaEventRecord(written)", cudaEventRecord(it->second.written, mOwner.stream()));
}

cudaEvent_t B200Allocator::writtenEvent(const MemoryRecord& record) {
  std::unique_lock<std::mutex> guard(mMutex);
  auto it = mBlocks.find(record.virtualAddress);
  return it == mBlocks.end() ? nullptr : it->second.written;
}

bool B200Allocator::stage(const MemoryRecord& record, const void* pinnedSrc, size_t tag, cudaEvent_t* uploaded) {
  std::unique_lock<std::mutex> guard(mMutex);
  if (uploaded) *uploaded = nullptr;
  auto it = mBlocks.find(record.virtualAddress);
  if (mDead || it == mBlocks.end() || it->second.locks > 0 || it->second.external || !pinnedSrc) return false;
  ScopedDevice on(mOwner.ordinal());
  const size_t va = record.virtualAddress, bytes = it->second.size;
  dropStaged(va);
  // The block being replaced must not be the eviction victim.
  const bool was_released = mReleased.erase(va) > 0;
  const bool fits = evictFor(bytes);
  if (mBlocks.find(va) == mBlocks.end()) return false;   // gone while the offload hook ran
  if (was_released) mReleased.insert(va);
  if (!fits) return false;
  cudaStream_t up = mOwner.uploadStream();
  void* ptr = nullptr;
  cudaError_t e = ensurePool() ? cudaMallocFromPoolAsync(&ptr, bytes, mPool, up) : cudaMallocAsync(&ptr, bytes, up);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return false;   // not an error: the ordinary upload at lock time still happens
  }
  const size_t copy = record.allocationSize < bytes ? record.allocationSize : bytes;
  e = cudaMemcpyAsync(ptr, pinnedSrc, copy, cudaMemcpyHostToDevice, up);
  cudaEvent_t done = e == cudaSuccess ? CudaApi::takeEvent(mOwner.ordinal()) : nullptr;
  if (done) e = cudaEventRecord(done, up);
  if (e != cudaSuccess || !done) {
    cudaGetLastError();
    cudaFreeAsync(ptr, up);
    CudaApi::giveEvent(mOwner.ordinal(), done);
    return false;
  }
  mStaged[va] = Staged{ptr, bytes, tag, done};
  mBytes += bytes;
  if (uploaded) *uploaded = done;
  return true;
}

bool B200Allocator::adoptStaged(const MemoryRecord& record, size_t tag) {
  std::unique_lock<std::mutex> guard(mMutex);
  auto st = mStaged.find(record.virtualAddress);
  auto it = mBlocks.find(record.virtualAddress);
  if (st == mStaged.end() || it == mBlocks.end() || st->second.tag != tag) return false;
  ScopedDevice on(mOwner.ordinal());
  cudaStream_t s = mOwner.stream();
  note("cudaStreamWaitEvent(upload)", cudaStreamWaitEvent(s, st->second.done, 0));
  // Kernels already queued on the main stream may still read the old block; freeing it on
  // that stream orders the free after them.
  cudaFreeAsync(it->second.ptr, s);
  mBytes -= it->second.size;
  it->second.ptr = st->second.ptr;
  it->second.size = st->second.size;
  CudaApi::giveEvent(mOwner.ordinal(), st->second.done);
  mStaged.erase(st);
  if (!it->second.written) it->second.written = CudaApi::takeEvent(mOwner.ordinal());
  if (it->second.written) cudaEventRecord(it->second.written, s);
  return true;
}

// -------------------------------------------------------------------- event

B200Event::B200Event(B200Device* device, cudaEvent_t evt, int status)
    : mDevice(device), mEvent(evt), mStatus(status) {}

B200Event::~B200Event() {
  if (mEvent) CudaApi::giveEvent(mDevice->ordinal(), mEvent);
}

void B200Event::wait() {
  if (mEvent) {
    ScopedDevice on(mDevice->ordinal());
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
  // Only the name is read here; nothing is created on the GPU until it is used.
  cudaDeviceProp prop;
  std::string base = "CUDA device";
  if (cudaGetDeviceProperties(&prop, ordinal) == cudaSuccess) {
    base = prop.name;
  } else {
    cudaGetLastError();
  }
  mName = base + " #" + std::to_string(ordinal);
  mAllocator = std::make_shared<B200Allocator>(*this);
}

void B200Device::ensureReady() const {
  if (mReady) return;
  std::lock_guard<std::mutex> g(mInitMutex);
  if (mReady) return;
  ScopedDevice on(mOrdinal);
  note("cudaStreamCreate", cudaStreamCreateWithFlags(&mStream, cudaStreamNonBlocking));
  note("cudaStreamCreate(upload)", cudaStreamCreateWithFlags(&mUpload, cudaStreamNonBlocking));
  note("cudaStreamCreate(download)", cudaStreamCreateWithFlags(&mDownload, cudaStreamNonBlocking));
  mReady = true;
}

B200Device::~B200Device() {
  if (!mReady) {
    mAllocator->shutdown();
    mAllocator.reset();
    return;
  }
  ScopedDevice on(mOrdinal);
  cudaStreamSynchronize(mUpload);
  cudaStreamSynchronize(mDownload);
  cudaStreamSynchronize(mStream);
  if (mWorkspace) cudaFree(mWorkspace);
  mAllocator->shutdown();
  mAllocator.reset();
  CudaApi::destroyEvents(mOrdinal);
  cudaStreamDestroy(mUpload);
  cudaStreamDestroy(mDownload);
  cudaStreamDestroy(mStream);
}

void B200Device::synchronize() const {
  if (!mReady) return;
  ScopedDevice on(mOrdinal);
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
  ScopedDevice on(mOrdinal);
  cudaError_t e;
  if (cudaEvent_t written = mAllocator->writtenEvent(record)) {
    // The record's last writer is known: wait for it alone, on the download stream, so
    // that work queued behind it (the next step of a pipelined host) keeps running.
    e = cudaStreamWaitEvent(downloadStream(), written, 0);
    if (e == cudaSuccess)
      e = cudaMemcpyAsync(dest, src, record.allocationSize, cudaMemcpyDeviceToHost, mDownload);
    if (e == cudaSuccess) e = cudaStreamSynchronize(mDownload);
  } else {
    e = cudaMemcpyAsync(dest, src, record.allocationSize, cudaMemcpyDeviceToHost, stream());
    if (e == cudaSuccess) e = cudaStreamSynchronize(mStream);
  }
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
  ScopedDevice on(mOrdinal);
  // Stream-ordered: kernels launched afterwards on this device's stream see the
  // data.  From pageable memory the call returns once the source is staged;
  // from pinned memory it is asynchronous and the owner of `src` must not overwrite
  // it before the copy has run (PoolBackendAllocator tracks that per host block).
  cudaError_t e = cudaMemcpyAsync(dst, src, record.allocationSize, cudaMemcpyHostToDevice, stream());
  if (e != cudaSuccess) {
    note("copyToDevice", e);
    mLastStatus = POLAR_B200_ERR_CUDA;
    mLastError = cudaGetErrorString(e);
    return;
  }
  mAllocator->markWritten(record);
}

void B200Device::copyFromPeer(MemoryRecord record, B200Device& src) {
  void* dst = mAllocator->getPtr(record);
  void* from = src.mAllocator->getPtr(record);
  if (!dst || !from) {
    mLastStatus = POLAR_B200_ERR_INVALID;
    mLastError = "copyFromPeer: record is not allocated on both devices";
    return;
  }
  if (!orderedPeerCopy<CudaApi>(dst, mOrdinal, stream(), from, src.mOrdinal, src.stream(), record.allocationSize)) {
    mLastStatus = POLAR_B200_ERR_CUDA;
    mLastError = "copyFromPeer: a CUDA call failed";
    return;
  }
  mAllocator->markWritten(record);
}

auto B200Device::launch(BackendAllocator& allocator, LaunchCommand& cmd, Event* blocking) -> Event* {
  ScopedDevice on(mOrdinal);
  cudaStream_t s = stream();
  int status = POLAR_B200_OK;
  if (blocking) {
    // Work of this device is stream-ordered already; an event of another device
    // becomes a stream dependency instead of a host wait.
    auto* be = static_cast<B200Event*>(blocking);
    if (be->getDevice() != this && be->native())
      note("cudaStreamWaitEvent", cudaStreamWaitEvent(s, be->native(), 0));
  }
  constexpr uint64_t kMaxArgs = 8;
  polar_b200_arg args[kMaxArgs];
  const char* name = cmd.nativeKernelName ? cmd.nativeKernelName : "";
  if (cmd.argsCount > kMaxArgs || (cmd.argsCount && !cmd.args)) {
    status = POLAR_B200_ERR_UNSUPPORTED;
    mLastError = "launch: bad argument list";
  }
  // the builtin writes its LAST tensor argument (its last two, for the one builtin with two results)
  MemoryRecord results[2] = {{0, 0}, {0, 0}};
  int n_seen = 0;
  const int n_results = polar_b200_result_count(name) > 1 ? 2 : 1;
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
      results[0] = results[1];
      results[1] = rec;
      ++n_seen;
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
      if (mWorkspace) cudaFreeAsync(mWorkspace, s);
      mWorkspace = nullptr;
      mWorkspaceBytes = 0;
      void* p = nullptr;
      if (cudaMallocAsync(&p, need, s) == cudaSuccess) {
        mWorkspace = p;
        mWorkspaceBytes = need;
      } else {
        cudaGetLastError();   // the library then falls back to its own per-launch allocation
      }
    }
    status = polar_b200_launch_by_name(name, args, cmd.argsCount, need <= mWorkspaceBytes ? mWorkspace : nullptr,
                                       need <= mWorkspaceBytes ? mWorkspaceBytes : 0, s);
    if (status != POLAR_B200_OK) mLastError = polar_b200_last_error();
  }
  if (status != POLAR_B200_OK) {
    // The reference has no error channel here (its runtimes terminate); this one
    // reports and hands back an event that carries the status.
    std::fprintf(stderr, "[polar_rt_cuda] launch of '%s' (%s) failed: %s\n", name,
                 cmd.kernelName ? cmd.kernelName : "", mLastError.c_str());
    mLastStatus = status;
  } else {
    for (int r = 0; r < n_results && r < n_seen; ++r) mAllocator->markWritten(results[1 - r]);
    if (verbose()) std::fprintf(stderr, "[polar_rt_cuda] %s: launched %s\n", mName.c_str(), name);
  }
  cudaEvent_t evt = CudaApi::takeEvent(mOrdinal);
  if (evt) note("cudaEventRecord", cudaEventRecord(evt, s));
  return new B200Event(this, evt, status);
}

void B200Device::consumeEvent(Event* evt) {
  if (!evt) return;
  evt->wait();
  delete evt;
}

// ------------------------------------------------------------------ context

B200Context::B200Context() {
  // Enumeration only: no device is made current and nothing is created on any GPU.
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    n = 0;
  }
  for (int i = 0; i < n; ++i) {
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, i) != cudaSuccess) cudaGetLastError();
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

// Test infrastructure: a second implementation of the reference's Device boundary
// that executes builtins on the host with the CPU oracle (oracle/builtins_oracle.c).
// It plays the role of the reference's MockDevice
// (tests/unit/backend/generic/lib/allocators/LayerAllocator.cpp:23-50 of the reference)
// but really computes, so that one graph - including the graphs getGradient builds -
// can be evaluated through the same Executor on this device and on the B200 device
// and the results compared.
#pragma once

#include <polarai/backend/generic/AllocatorLayerBase.hpp>
#include <polarai/backend/generic/BackendAllocator.hpp>
#include <polarai/backend/generic/runtime/Device.hpp>
#include <polarai/backend/generic/runtime/Event.hpp>
#include <polarai/backend/generic/runtime/LaunchCommand.h>
#include <polarai/backend/generic/runtime/TensorInfo.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <unordered_map>

extern "C" {
void oracle_set_threads(int n);
void oracle_ffill(float pattern, float* out, uint64_t n);
void oracle_fcopy(const float* in, float* out, uint64_t n);
void oracle_fadd(const float* a, float sa, const float* b, float sb, float* out, uint64_t n);
void oracle_fmul(const float* a, const float* b, float* out, uint64_t n);
void oracle_fdivide(const float* a, const float* b, float* out, uint64_t n);
void oracle_fsigmoid(const float* in, float* out, uint64_t n, int clamp);
void oracle_flogloss(const float* p, const float* y, float* out, uint64_t n);
void oracle_fmulconcat(const float* g, const float* l, float* out, uint64_t n);
void oracle_frelu(const float* in, float* out, uint64_t n);
void oracle_fsoftmax(const float* in, float* out, uint64_t n);
void oracle_fpool(const float* in, uint64_t h, uint64_t w, uint64_t wh, uint64_t ww, uint64_t sh, uint64_t sw, float* out);
void oracle_fconv2d(const float* in, uint64_t h, uint64_t w, const float* ker, uint64_t kh, uint64_t kw, float* out);
void oracle_ftranspose(const float* in, uint64_t rows, uint64_t cols, float* out);
void oracle_fmatmul(int tl, int tr, uint64_t m, uint64_t n, uint64_t k, const float* l, const float* r, float* out);
}

namespace polarai::backend::generic {

class OracleLayer final : public AllocatorLayerBase {
public:
  ~OracleLayer() override {
    for (auto& kv : mMem) std::free(kv.second);
  }
  void registerMemoryOffloadCallback(MemoryOffloadCallbackT) override {}
  void allocate(MemoryRecord r) override {
    if (!mMem.count(r.virtualAddress)) {
      mMem[r.virtualAddress] = std::calloc(1, r.allocationSize ? r.allocationSize : 4);
      mTags[r.virtualAddress] = 1;
    }
  }
  void deallocate(MemoryRecord r) override {
    auto it = mMem.find(r.virtualAddress);
    if (it != mMem.end()) {
      std::free(it->second);
      mMem.erase(it);
    }
  }
  void lock(MemoryRecord) override {}
  void release(MemoryRecord) override {}
  void* getPtr(MemoryRecord r) override {
    auto it = mMem.find(r.virtualAddress);
    return it == mMem.end() ? nullptr : it->second;
  }
  bool isAllocated(const MemoryRecord& r) const override { return mMem.count(r.virtualAddress) > 0; }
  size_t getTag(MemoryRecord r) override { return mTags[r.virtualAddress]; }
  void setTag(MemoryRecord r, size_t tag) override { mTags[r.virtualAddress] = tag; }

private:
  std::unordered_map<size_t, void*> mMem;
  std::unordered_map<size_t, size_t> mTags;
};

class OracleEvent final : public Event {
public:
  explicit OracleEvent(Device* d) : mDevice(d) {}
  void wait() override {
    for (auto& cb : mCallbacks) cb();
    mCallbacks.clear();
  }
  void addCallback(std::function<void()> cb) override { mCallbacks.push_back(std::move(cb)); }
  auto getDevice() -> Device* override { return mDevice; }

private:
  Device* mDevice;
  std::vector<std::function<void()>> mCallbacks;
};

class OracleDevice final : public Device {
public:
  explicit OracleDevice(std::string name = "oracle-cpu") : mName(std::move(name)), mLayer(std::make_shared<OracleLayer>()) {
    oracle_set_threads(8);
  }
  auto getProvider() const -> DeviceProvider override { return DeviceProvider::HOST; }
  auto getKind() const -> DeviceKind override { return DeviceKind::CPU; }
  std::string getDeviceName() const override { return mName; }
  bool hasAllocator() override { return true; }
  std::vector<std::shared_ptr<Device>> partition(PartitionDomain) override { return {}; }
  std::shared_ptr<AllocatorLayerBase> getAllocator() override { return mLayer; }
  bool operator==(const Device& d) const override { return d.getDeviceName() == getDeviceName(); }
  void copyToHost(MemoryRecord r, void* dest) const override {
    if (void* p = mLayer->getPtr(r)) std::memcpy(dest, p, r.allocationSize);
  }
  void copyToDevice(MemoryRecord r, void* src) const override {
    if (void* p = mLayer->getPtr(r)) std::memcpy(p, src, r.allocationSize);
  }
  void consumeEvent(Event* e) override {
    if (e) {
      e->wait();
      delete e;
    }
  }
  void selectBinary(std::vector<std::shared_ptr<ProgramDesc>>&) override {}
  int launches = 0;
  int failures = 0;

  Event* launch(BackendAllocator& alloc, LaunchCommand& cmd, Event*) override {
    ++launches;
    const std::string name = cmd.nativeKernelName;
    float* t[8] = {nullptr};
    uint64_t n[8] = {0};
    TensorInfo* ti[8] = {nullptr};
    float f[8] = {0};
    int64_t iv[8] = {0};
    for (uint64_t i = 0; i < cmd.argsCount && i < 8; ++i) {
      if (cmd.args[i].type == ArgDesc::TENSOR) {
        ti[i] = static_cast<TensorInfo*>(cmd.args[i].arg);
        MemoryRecord r{ti[i]->virtAddr, 4};
        n[i] = 1;
        for (uint64_t d = 0; d < ti[i]->dims; ++d) n[i] *= ti[i]->shape[d];
        r.allocationSize *= n[i];
        t[i] = alloc.get<float>(r, *this);
      } else if (cmd.args[i].size == 8) {
        iv[i] = *static_cast<int64_t*>(cmd.args[i].arg);
      } else {
        f[i] = *static_cast<float*>(cmd.args[i].arg);
      }
    }
    if (name == "ffill") oracle_ffill(f[0], t[1], n[1]);
    else if (name == "fcopy") oracle_fcopy(t[0], t[1], n[1]);
    else if (name == "fadd") oracle_fadd(t[0], f[1], t[2], f[3], t[4], n[4]);
    else if (name == "fmul") oracle_fmul(t[0], t[1], t[2], n[2]);
    else if (name == "fdivide") oracle_fdivide(t[0], t[1], t[2], n[2]);
    else if (name == "fsigmoid") oracle_fsigmoid(t[0], t[1], n[1], 1);
    else if (name == "flogloss") oracle_flogloss(t[0], t[1], t[2], n[2]);
    else if (name == "fmulconcat") oracle_fmulconcat(t[0], t[1], t[2], n[2]);
    else if (name == "frelu") oracle_frelu(t[0], t[1], n[1]);
    else if (name == "fsoftmax") oracle_fsoftmax(t[0], t[1], n[1]);
    else if (name == "fpool")
      oracle_fpool(t[0], ti[0]->shape[0], ti[0]->shape[1], iv[1], iv[2], iv[3], iv[4], t[5]);
    else if (name == "fconv2d")
      oracle_fconv2d(t[0], ti[0]->shape[0], ti[0]->shape[1], t[1], ti[1]->shape[0], ti[1]->shape[1], t[2]);
    else if (name == "ftranspose") oracle_ftranspose(t[0], ti[0]->shape[0], ti[0]->shape[1], t[1]);
    else if (name.rfind("fmatmul_", 0) == 0 && name.size() == 11) {
      int tl = name[8] == 't', tr = name[10] == 't';
      uint64_t m = tl ? ti[0]->shape[1] : ti[0]->shape[0], k = tl ? ti[0]->shape[0] : ti[0]->shape[1];
      uint64_t nn = tr ? ti[1]->shape[0] : ti[1]->shape[1];
      oracle_fmatmul(tl, tr, m, nn, k, t[0], t[1], t[2]);
    } else {
      ++failures;
      std::fprintf(stderr, "[oracle device] unknown kernel %s\n", name.c_str());
    }
    return new OracleEvent(this);
  }

private:
  std::string mName;
  std::shared_ptr<OracleLayer> mLayer;
};

}  // namespace polarai::backend::generic

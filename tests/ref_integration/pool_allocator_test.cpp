// Host-side unit tests of PoolBackendAllocator (csrc/rt/pool_backend_allocator.*), in the
// manner of the reference's allocator tests with a mock device
// (tests/unit/backend/generic/lib/allocators/LayerAllocator.cpp of the reference): two
// host-memory devices stand in for GPUs, so the coherence logic runs without CUDA.
#include "oracle_device.hpp"

#include <rt/pool_backend_allocator.hpp>

#include <gtest/gtest.h>

#include <cstring>
#include <vector>

using namespace polarai::backend::generic;
using polarai::core::internal::LockType;

class PoolAllocatorTest : public ::testing::Test {
protected:
  OracleDevice devA{"fake-gpu-0"}, devB{"fake-gpu-1"};
  PoolBackendAllocator alloc;
  void SetUp() override {
    alloc.registerDevice(devA);
    alloc.registerDevice(devB);
  }
  // the typed accessor lives in the base class; the derived class's own get() overloads hide it
  static float* ptr(BackendAllocator& a, const MemoryRecord& r, Device& d) { return a.get<float>(r, d); }
};

#define EXPECT_TRUE_(cond) EXPECT_FLOAT_EQ((cond) ? 1.0f : 0.0f, 1.0f)

TEST_F(PoolAllocatorTest, HostWriteReachesTheDeviceOnLock) {
  MemoryRecord r{1, 16 * sizeof(float)};
  alloc.allocate(r, devA);
  alloc.lock(r, LockType::READ_WRITE);                 // host write, as ath_load does
  auto* h = static_cast<float*>(alloc.get(r));
  for (int i = 0; i < 16; ++i) h[i] = float(i);
  alloc.release(r);
  alloc.lock(r, devA, LockType::READ);                 // the device copy is stale: refreshed from RAM
  for (int i = 0; i < 16; ++i) EXPECT_FLOAT_EQ(ptr(alloc, r, devA)[i], float(i));
  alloc.release(r, devA);
  EXPECT_TRUE_(alloc.lastStatus() == 0);
}

TEST_F(PoolAllocatorTest, DeviceWriteComesBackToTheHostAndCrossesDevices) {
  MemoryRecord r{100, 8 * sizeof(float)};
  alloc.allocate(r, devA);
  alloc.lock(r, devA, LockType::READ_WRITE);
  for (int i = 0; i < 8; ++i) ptr(alloc, r, devA)[i] = 2.0f * i;   // "kernel" output on device A
  alloc.release(r, devA);
  alloc.lock(r, devB, LockType::READ);                 // B has never seen the record: pulled from A
  for (int i = 0; i < 8; ++i) EXPECT_FLOAT_EQ(ptr(alloc, r, devB)[i], 2.0f * i);
  alloc.release(r, devB);
  alloc.lock(r, LockType::READ);                       // OutputNodeAccessor's path
  auto* h = static_cast<float*>(alloc.get(r));
  for (int i = 0; i < 8; ++i) EXPECT_FLOAT_EQ(h[i], 2.0f * i);
  alloc.release(r);
  // B overwrites; A must see B's version next time
  alloc.lock(r, devB, LockType::READ_WRITE);
  for (int i = 0; i < 8; ++i) ptr(alloc, r, devB)[i] = -1.0f;
  alloc.release(r, devB);
  alloc.lock(r, devA, LockType::READ);
  for (int i = 0; i < 8; ++i) EXPECT_FLOAT_EQ(ptr(alloc, r, devA)[i], -1.0f);
  alloc.release(r, devA);
  EXPECT_TRUE_(alloc.lastStatus() == 0);
}

TEST_F(PoolAllocatorTest, ConflictingLocksAreStatusesNotAborts) {
  MemoryRecord r{7, 4 * sizeof(float)};
  alloc.allocate(r, devA);
  alloc.lock(r, devA, LockType::READ);
  alloc.lock(r, devA, LockType::READ_WRITE);           // the reference dies here (FatalError)
  EXPECT_TRUE_(alloc.lastStatus() != 0);
  alloc.clearError();
  alloc.deallocate(r);                                 // still locked
  EXPECT_TRUE_(alloc.lastStatus() != 0);
  alloc.clearError();
  alloc.release(r, devA);
  alloc.lock(r, devA, LockType::READ_WRITE);           // fine now
  EXPECT_TRUE_(alloc.lastStatus() == 0);
  alloc.lock(r, devB, LockType::READ);                 // under a READ_WRITE lock elsewhere
  EXPECT_TRUE_(alloc.lastStatus() != 0);
  alloc.clearError();
  alloc.release(r, devA);
  alloc.deallocate(r);
  EXPECT_TRUE_(alloc.lastStatus() == 0);
  EXPECT_TRUE_(!devA.getAllocator()->isAllocated(r));
}

TEST_F(PoolAllocatorTest, DoubleAllocationIsANoOpAndUnknownDevicesAreRefused) {
  MemoryRecord r{9, 64};
  alloc.allocate(r, devA);
  void* p = ptr(alloc, r, devA);
  alloc.allocate(r, devA);
  EXPECT_TRUE_(ptr(alloc, r, devA) == p);
  OracleDevice stranger{"not-registered"};
  alloc.allocate(r, stranger);
  EXPECT_TRUE_(alloc.lastStatus() != 0);
}

TEST_F(PoolAllocatorTest, DeviceToDeviceRefreshGoesThroughThePeerCopyNotThroughRam) {
  // The CUDA plugin copies device to device on the destination's stream, ordered after the
  // producer; the allocator's part is to choose that path with the right pair of devices.
  MemoryRecord r{300, 8 * sizeof(float)};
  int calls = 0;
  std::string route;
  alloc.setPeerCopy([&](Device& dst, Device& src, const MemoryRecord& rec) {
    ++calls;
    route = src.getDeviceName() + "->" + dst.getDeviceName();
    std::memcpy(dst.getAllocator()->getPtr(rec), src.getAllocator()->getPtr(rec), rec.allocationSize);
    return true;
  });
  alloc.allocate(r, devA);
  alloc.lock(r, devA, LockType::READ_WRITE);
  for (int i = 0; i < 8; ++i) ptr(alloc, r, devA)[i] = 3.0f + i;
  alloc.release(r, devA);
  alloc.lock(r, devB, LockType::READ);
  EXPECT_TRUE_(calls == 1 && route == "fake-gpu-0->fake-gpu-1");
  for (int i = 0; i < 8; ++i) EXPECT_FLOAT_EQ(ptr(alloc, r, devB)[i], 3.0f + i);
  alloc.release(r, devB);
  EXPECT_TRUE_(alloc.get(r) == nullptr);               // no host copy was ever made
  // a hook that declines leaves the staging path through host memory in charge
  alloc.setPeerCopy([&](Device&, Device&, const MemoryRecord&) { ++calls; return false; });
  alloc.lock(r, devB, LockType::READ_WRITE);
  for (int i = 0; i < 8; ++i) ptr(alloc, r, devB)[i] = -2.0f * i;
  alloc.release(r, devB);
  alloc.lock(r, devA, LockType::READ);
  EXPECT_TRUE_(calls == 2);
  for (int i = 0; i < 8; ++i) EXPECT_FLOAT_EQ(ptr(alloc, r, devA)[i], -2.0f * i);
  alloc.release(r, devA);
  EXPECT_TRUE_(alloc.lastStatus() == 0);
}

TEST_F(PoolAllocatorTest, OverwriteReplacesTheRecordAndRespectsLocks) {
  MemoryRecord r{400, 4 * sizeof(float)};
  alloc.allocate(r, devA);
  for (int version = 1; version <= 3; ++version) {
    auto* h = static_cast<float*>(alloc.beginOverwrite(r));
    EXPECT_TRUE_(h != nullptr);
    for (int i = 0; i < 4; ++i) h[i] = 10.0f * version + i;
    alloc.endOverwrite(r);
    alloc.lock(r, devA, LockType::READ);                 // the device sees each new version
    for (int i = 0; i < 4; ++i) EXPECT_FLOAT_EQ(ptr(alloc, r, devA)[i], 10.0f * version + i);
    alloc.release(r, devA);
  }
  alloc.lock(r, devA, LockType::READ);
  EXPECT_TRUE_(alloc.beginOverwrite(r) == nullptr);      // locked on a device: refused, not aborted
  EXPECT_TRUE_(alloc.lastStatus() != 0);
  alloc.clearError();
  alloc.release(r, devA);
  EXPECT_TRUE_(alloc.beginOverwrite(r) != nullptr);
  alloc.endOverwrite(r);
  EXPECT_TRUE_(alloc.lastStatus() == 0);
}

// Scoped CUDA-device selection and cross-stream ordering for the runtime plugin, written
// against a small `Api` policy so that the logic runs on the host with a recording fake
// (tests/native/device_scope_test.cpp) and on the CUDA runtime in the plugin.
//
// Why it exists: a plugin that implements Device for eight GPUs must make "its" GPU
// current before almost every CUDA call.  The reference's driver calls initContext() and
// every Device method on the host's own thread (RuntimeDriver.cpp:39-50 of the reference)
// and expects nothing else about that thread to change; a plugin that leaves the last GPU
// it touched current makes the host's next kernel launch run on the wrong GPU with
// another GPU's pointers.  Every entry of the plugin therefore opens a ScopedDevice and
// the calling thread leaves with the device (and driver context) it came with.
#pragma once

#include <cstddef>
#include <cstdint>
#include <utility>
#include <vector>

namespace polarai::backend::generic {

// What a thread had current when a scope was opened.
struct DeviceToken {
  int device = 0;          // runtime's current device
  void* context = nullptr; // driver context that was current (nullptr: none yet)
  bool haveContext = false;  // `context` is meaningful (the driver entry points were found)
};

// Api must provide:
//   static DeviceToken current();            what the calling thread has now
//   static bool enter(int ordinal);          make `ordinal` current (creates its context if needed)
//   static void restore(const DeviceToken&); put a token's state back
template <class Api>
class ScopedDeviceT {
public:
  explicit ScopedDeviceT(int ordinal) : mToken(Api::current()) {
    // Already there: a context is current and it belongs to the wanted device.
    const bool there = mToken.device == ordinal && (!mToken.haveContext || mToken.context != nullptr);
    if (!there) {
      mOk = Api::enter(ordinal);
      mSwitched = true;
    }
  }
  ~ScopedDeviceT() {
    if (mSwitched) Api::restore(mToken);
  }
  ScopedDeviceT(const ScopedDeviceT&) = delete;
  ScopedDeviceT& operator=(const ScopedDeviceT&) = delete;
  bool ok() const { return mOk; }
  bool switched() const { return mSwitched; }

private:
  DeviceToken mToken;
  bool mOk = true;
  bool mSwitched = false;
};

// ---- ordering of work between the streams of two devices ---------------------------------
//
// Api must also provide (Stream, Event are opaque handles):
//   static Event takeEvent(int ordinal);  static void giveEvent(int ordinal, Event);
//   static bool record(Event, Stream);    static bool streamWait(Stream, Event);
//   static bool copyPeer(void* dst, int dstOrdinal, const void* src, int srcOrdinal, size_t, Stream);
//   static bool eventSync(Event);

// Copies `bytes` from a buffer of device `srcOrdinal` to one of device `dstOrdinal` so that
//  (1) the copy starts after everything queued so far on the SOURCE device's stream (the
//      kernel that produced the data may still be running),
//  (2) it runs on the DESTINATION device's stream, so that consumers queued there afterwards
//      see the data,
//  (3) work queued later on the source stream (which may overwrite the buffer) starts only
//      after the copy has read it.
// Nothing waits on the host.
template <class Api, class Stream>
bool orderedPeerCopy(void* dst, int dstOrdinal, Stream dstStream, const void* src, int srcOrdinal,
                     Stream srcStream, size_t bytes) {
  bool ok = true;
  typename Api::Event produced, consumed;
  {
    ScopedDeviceT<Api> onSrc(srcOrdinal);
    produced = Api::takeEvent(srcOrdinal);
    ok = ok && produced && Api::record(produced, srcStream);
  }
  {
    ScopedDeviceT<Api> onDst(dstOrdinal);
    ok = ok && Api::streamWait(dstStream, produced);
    ok = ok && Api::copyPeer(dst, dstOrdinal, src, srcOrdinal, bytes, dstStream);
    consumed = Api::takeEvent(dstOrdinal);
    ok = ok && consumed && Api::record(consumed, dstStream);
  }
  {
    ScopedDeviceT<Api> onSrc(srcOrdinal);
    ok = ok && Api::streamWait(srcStream, consumed);
  }
  // A stream wait refers to the state of the event at the time of the call, so both
  // events can go back to their pools at once.
  if (produced) Api::giveEvent(srcOrdinal, produced);
  if (consumed) Api::giveEvent(dstOrdinal, consumed);
  return ok;
}

// A host buffer that asynchronous host-to-device copies may still be reading.  The owner
// marks it after queuing each copy and settles it before the buffer is written or freed.
template <class Api>
class PendingRead {
public:
  PendingRead() = default;
  PendingRead(const PendingRead&) = delete;
  PendingRead& operator=(const PendingRead&) = delete;
  PendingRead(PendingRead&& o) noexcept : mMarks(std::move(o.mMarks)) { o.mMarks.clear(); }
  PendingRead& operator=(PendingRead&& o) noexcept {
    if (this != &o) {
      settle();
      mMarks = std::move(o.mMarks);
      o.mMarks.clear();
    }
    return *this;
  }
  ~PendingRead() { settle(); }

  // A copy out of the buffer was just queued on `stream` of device `ordinal`.
  template <class Stream>
  void mark(int ordinal, Stream stream) {
    ScopedDeviceT<Api> on(ordinal);
    // one mark per stream is enough: a later copy on the same stream finishes after an earlier one
    const std::uintptr_t key = (std::uintptr_t)stream;
    for (size_t i = 0; i < mMarks.size(); ++i) {
      if (mMarks[i].ordinal == ordinal && mMarks[i].stream == key) {
        Api::giveEvent(ordinal, mMarks[i].event);
        mMarks.erase(mMarks.begin() + i);
        break;
      }
    }
    typename Api::Event e = Api::takeEvent(ordinal);
    if (!e) return;
    if (Api::record(e, stream)) {
      mMarks.push_back(Mark{e, ordinal, key});
    } else {
      Api::giveEvent(ordinal, e);
    }
  }
  // Blocks the host until every marked copy has read the buffer.  No-op when nothing is pending.
  void settle() {
    for (auto& m : mMarks) {
      Api::eventSync(m.event);
      Api::giveEvent(m.ordinal, m.event);
    }
    mMarks.clear();
  }
  bool pending() const { return !mMarks.empty(); }

private:
  struct Mark {
    typename Api::Event event;
    int ordinal;
    std::uintptr_t stream;
  };
  std::vector<Mark> mMarks;
};

}  // namespace polarai::backend::generic

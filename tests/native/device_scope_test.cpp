// Host-side test of csrc/rt/device_scope.hpp with a recording stand-in for the CUDA calls:
// the calling thread's device and context come back as they were, the peer copy is ordered
// on both streams, and a host buffer under an asynchronous upload is not handed out early.
#include <rt/device_scope.hpp>

#include <cstdio>
#include <string>
#include <vector>

using namespace polarai::backend::generic;

namespace {

std::vector<std::string> g_log;
int g_failures = 0;

void expect(bool cond, const char* what) {
  if (!cond) {
    ++g_failures;
    std::printf("FAILED: %s\n", what);
  }
}

// A thread with a current device and context, eight fake GPUs, numbered events.
struct FakeApi {
  using Event = int;   // 0 = none
  static int device;
  static void* context;
  static int nextEvent;
  static int contextsCreated;
  static void* contextOf(int ordinal) { return reinterpret_cast<void*>(static_cast<long>(0x1000 + ordinal)); }

  static DeviceToken current() {
    DeviceToken t;
    t.device = device;
    t.context = context;
    t.haveContext = true;
    return t;
  }
  static bool enter(int ordinal) {
    g_log.push_back("enter " + std::to_string(ordinal));
    device = ordinal;
    context = contextOf(ordinal);
    ++contextsCreated;
    return true;
  }
  static void restore(const DeviceToken& t) {
    g_log.push_back("restore " + std::to_string(t.device) + (t.context ? "" : " (no context)"));
    device = t.device;
    context = t.context;
  }
  static Event takeEvent(int ordinal) {
    expect(device == ordinal, "an event is taken with its device current");
    return ++nextEvent;
  }
  static void giveEvent(int, Event) {}
  static bool record(Event e, int stream) {
    g_log.push_back("record e" + std::to_string(e) + " on s" + std::to_string(stream) + " dev " + std::to_string(device));
    return true;
  }
  static bool streamWait(int stream, Event e) {
    g_log.push_back("s" + std::to_string(stream) + " waits e" + std::to_string(e) + " dev " + std::to_string(device));
    return true;
  }
  static bool copyPeer(void*, int dstOrdinal, const void*, int srcOrdinal, size_t, int stream) {
    g_log.push_back("copy " + std::to_string(srcOrdinal) + "->" + std::to_string(dstOrdinal) + " on s" +
                    std::to_string(stream) + " dev " + std::to_string(device));
    return true;
  }
  static bool eventSync(Event e) {
    g_log.push_back("host waits e" + std::to_string(e));
    return true;
  }
};
int FakeApi::device = 0;
void* FakeApi::context = nullptr;
int FakeApi::nextEvent = 0;
int FakeApi::contextsCreated = 0;

using Scoped = ScopedDeviceT<FakeApi>;

void reset(int device, void* context) {
  g_log.clear();
  FakeApi::device = device;
  FakeApi::context = context;
  FakeApi::nextEvent = 0;
  FakeApi::contextsCreated = 0;
}

}  // namespace

int main() {
  // 1. a host working on GPU 0 enumerates and uses GPU 7: it leaves on GPU 0, same context
  reset(0, FakeApi::contextOf(0));
  {
    Scoped on(7);
    expect(FakeApi::device == 7, "inside the scope the wanted device is current");
    {
      Scoped again(7);   // nested use of the same device does not switch
      expect(!again.switched(), "a scope on the current device does nothing");
    }
    expect(FakeApi::device == 7, "the inner scope left the outer one's device");
  }
  expect(FakeApi::device == 0 && FakeApi::context == FakeApi::contextOf(0), "device and context are restored");
  expect(g_log.size() == 2 && g_log[0] == "enter 7" && g_log[1] == "restore 0", "one switch, one restore");

  // 2. a thread that never touched CUDA (no context) asks for GPU 0: device 0 is "current"
  //    only by default, so the scope must enter it - and must put "no context" back
  reset(0, nullptr);
  {
    Scoped on(0);
    expect(on.switched(), "a default device without a context is not 'already there'");
    expect(FakeApi::context == FakeApi::contextOf(0), "the context exists inside the scope");
  }
  expect(FakeApi::context == nullptr, "the thread is left without a context, as it was found");

  // 3. already on the device with a context: no call at all
  reset(3, FakeApi::contextOf(3));
  {
    Scoped on(3);
  }
  expect(g_log.empty(), "no switch when the device is current");

  // 4. ordered peer copy 1 -> 2 while the host thread sits on GPU 0
  reset(0, FakeApi::contextOf(0));
  int src_stream = 11, dst_stream = 22;
  char a[8], b[8];
  expect(orderedPeerCopy<FakeApi>(b, 2, dst_stream, a, 1, src_stream, sizeof a), "peer copy succeeds");
  std::vector<std::string> calls;
  for (auto& l : g_log)
    if (l.rfind("enter", 0) && l.rfind("restore", 0)) calls.push_back(l);
  const char* want[] = {"record e1 on s11 dev 1",    // after the producer on the source stream
                        "s22 waits e1 dev 2",        // the destination stream waits for it
                        "copy 1->2 on s22 dev 2",    // the copy runs on the destination stream
                        "record e2 on s22 dev 2",    // ...
                        "s11 waits e2 dev 1"};       // and later work on the source waits for the copy
  expect(calls.size() == 5, "five ordering calls");
  for (size_t i = 0; i < calls.size() && i < 5; ++i) expect(calls[i] == want[i], want[i]);
  expect(FakeApi::device == 0 && FakeApi::context == FakeApi::contextOf(0), "the host thread is back on GPU 0");
  for (auto& l : g_log) expect(l.find("host waits") == std::string::npos, "nothing waits on the host");

  // 5. a pinned buffer under upload: settle() waits for every stream that reads it, once
  reset(0, FakeApi::contextOf(0));
  {
    PendingRead<FakeApi> reading;
    expect(!reading.pending(), "fresh buffer: nothing pending");
    reading.settle();
    expect(g_log.empty(), "settle without a mark does nothing");
    reading.mark(1, 11);
    reading.mark(1, 11);   // a second copy on the same stream replaces the first mark
    reading.mark(2, 22);
    expect(reading.pending(), "marked");
    g_log.clear();
    reading.settle();
    int waits = 0;
    for (auto& l : g_log) waits += l.find("host waits") != std::string::npos;
    expect(waits == 2, "one host wait per stream that read the buffer");
    expect(!reading.pending(), "settled");
    g_log.clear();
    reading.settle();
    expect(g_log.empty(), "settling twice waits once");
    PendingRead<FakeApi> moved;
    reading.mark(1, 11);
    moved = std::move(reading);
    expect(moved.pending() && !reading.pending(), "a mark moves with its buffer");
  }
  expect(FakeApi::device == 0, "marks leave the host thread's device alone");

  std::printf("device_scope: %d failures\n", g_failures);
  return g_failures;
}

// A direct (non-JIT) implementation of polarai::backend::generic::Executor.
//
// The reference's Executor (include/polarai/backend/generic/Executor.hpp:36-61,
// src/backend/generic/lib/ExecutorImpl.cpp) lowers a graph through MLIR and an LLVM
// JIT into host code that calls the ath_* support routines.  This file provides the
// same class - same header, same member functions - without a compiler: the
// framework's own GraphCompiler::compile (src/core/graph/internal/GraphCompiler.cpp:21-110)
// is driven with a Generator whose functors RECORD the builtin program (per node:
// alloc, lock, invoke-loader or builtin launch, release; per cluster: barrier), and
// evaluate() replays the record through the reference's unchanged support routines
// (ath_device_select, ath_allocate, ath_lock, ath_load, ath_launch, ath_release,
// ath_barrier - src/backend/generic/runtime/support/routines.cpp:37-112), which in
// turn drive whatever devices the RuntimeDriver found - here the B200 plugin.
//
// Builtins are launched by native kernel name with LaunchCommand/ArgDesc/TensorInfo
// arguments in the order the MLIR lowering would have produced
// (utils/dialects/include/PolarGraph/PolarGraphOps.td; CodeGen.cpp:283-462).
#include <polarai/backend/generic/Executor.hpp>
#include <polarai/backend/generic/runtime/Event.hpp>
#include <polarai/backend/generic/runtime/GraphHandle.hpp>
#include <polarai/backend/generic/runtime/LaunchCommand.h>
#include <polarai/backend/generic/runtime/TensorInfo.h>
#include <polarai/core/Generator.hpp>
#include <polarai/core/context/internal/ContextInternal.hpp>
#include <polarai/core/graph/internal/GraphCompiler.hpp>
#include <polarai/core/loader/internal/AbstractLoaderInternal.hpp>
#include <polarai/core/node/internal/AbstractNodeInternal.hpp>
#include <polarai/core/node/internal/InputNodeInternal.hpp>
#include <polarai/backend/generic/runtime/BackendAccessor.hpp>
#include <polarai/loaders/internal/ConstantLoaderInternal.hpp>
#include <polarai/loaders/internal/DummyLoaderInternal.hpp>

#include <lib/allocators/LayerAllocator.hpp>
#include <runtime/driver/RuntimeDriver.hpp>
#include <runtime/host/HostDevice.hpp>
#include <runtime/support/api.hpp>

#include "data_parallel_plan.hpp"

#include <algorithm>
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <string>
#include <thread>
#include <unordered_map>
#include <variant>
#include <vector>

using namespace polarai::core;
using namespace polarai::core::internal;

namespace polarai::backend::generic {

namespace {

// A tensor as the runtime sees it: what goes into a TensorInfo.
struct TensorDesc {
  uint64_t virtAddr = 0;
  int dataType = 0;
  std::vector<uint64_t> shape;
};

struct Value : GenValueImplBase {
  bool isTensor = false;
  TensorDesc tensor;
  float scalar = 0.f;
  bool isInteger = false;   // an 8-byte integer attribute (pooling window, stride)
  int64_t integer = 0;
};

GenValue makeTensorValue(const TensorInternal& t) {
  auto v = std::make_shared<Value>();
  v->isTensor = true;
  v->tensor.virtAddr = t.getVirtualAddress();
  v->tensor.dataType = static_cast<int>(t.getDataType());
  for (size_t d : t.getShape().getShape()) v->tensor.shape.push_back(d);
  return GenValue{v};
}

struct Command {
  enum Kind { ALLOC, LOCK, RELEASE, LOAD, LAUNCH } kind;
  TensorDesc tensor;                  // ALLOC, LOCK, RELEASE, LOAD
  LockType lockType = LockType::READ; // LOCK
  std::string nativeName;             // LAUNCH
  std::vector<Value> args;            // LAUNCH, in LaunchCommand order
};

struct NodeRecord : GenNodeImplBase {
  std::string name;
  size_t nodeId = 0;
  size_t clusterId = 0;
  std::vector<GenValue> operands;
  GenValue result;
  std::vector<Command> commands;
  auto getOperand(size_t i) -> GenValue override { return operands.at(i); }
  auto getResult() -> GenValue override { return result; }
  auto getBatchIndex() -> GenValue override { return GenValue{}; }
};

struct Step {
  enum Kind { NODE, BARRIER } kind;
  std::shared_ptr<NodeRecord> node;
  uint64_t clusterId = 0;
};

struct GraphRecord : GenGraphImplBase {
  std::string name;
  std::vector<Step> steps;
};

// Where recorded commands go: a node body, a graph body, or nowhere (top level).
struct InsertionPoint : GenInsPointImplBase {
  NodeRecord* node = nullptr;
  GraphRecord* graph = nullptr;
};

// Installs recording functors for every builtin of the catalogue
// (include/polarai/core/internal/GenBuiltins.hpp:25-52).
class Recorder {
public:
  explicit Recorder(Generator& gen) { install(gen); }
  std::shared_ptr<GraphRecord> graph;
  std::vector<std::string> unsupported;

private:
  InsertionPoint mPoint;

  void emit(Command c) {
    if (mPoint.node) mPoint.node->commands.push_back(std::move(c));
  }
  static const Value& val(const GenValue& v) { return v.value<Value>(); }

  void launch(const char* name, std::initializer_list<GenValue> args) {
    Command c;
    c.kind = Command::LAUNCH;
    c.nativeName = name;
    for (const auto& a : args) c.args.push_back(val(a));
    emit(std::move(c));
  }
  void refuse(const char* what) { unsupported.emplace_back(what); }

  void install(Generator& g) {
    g.registerConstantFunctor([](Generator::SupportedConstantT c) {
      auto v = std::make_shared<Value>();
      v->scalar = std::visit([](auto x) { return static_cast<float>(x); }, c);
      return GenValue{v};
    });
    g.registerNodeFunctor([this](std::string_view name, size_t nodeId, size_t clusterId,
                                 const std::vector<TensorInternal*>& operands, TensorInternal& out) {
      auto n = std::make_shared<NodeRecord>();
      n->name = std::string(name);
      n->nodeId = nodeId;
      n->clusterId = clusterId;
      for (auto* t : operands) n->operands.push_back(makeTensorValue(*t));
      n->result = makeTensorValue(out);
      return GenNode{n};
    });
    g.registerGraphFunctor([this](std::string_view name, size_t) {
      graph = std::make_shared<GraphRecord>();
      graph->name = std::string(name);
      return GenGraph{graph};
    });
    g.registerSetInsertionPointFunctor(std::function<void(GenInsertionPoint)>(
        [this](GenInsertionPoint p) { mPoint = p.point<InsertionPoint>(); }));
    g.registerSetInsertionPointFunctor(std::function<void(GenNode)>([this](GenNode n) {
      mPoint.node = &n.node<NodeRecord>();
      mPoint.graph = nullptr;
    }));
    g.registerSetInsertionPointFunctor(std::function<void(GenGraph)>([this](GenGraph gr) {
      mPoint.node = nullptr;
      mPoint.graph = &gr.graph<GraphRecord>();
    }));
    g.registerGetInsertionPointFunctor([this]() {
      return GenInsertionPoint{std::make_shared<InsertionPoint>(mPoint)};
    });

    builtin_functor_t<builtin::Alloc> alloc = [this](GenValue t) {
      Command c;
      c.kind = Command::ALLOC;
      c.tensor = val(t).tensor;
      emit(std::move(c));
      return GenValue{};
    };
    g.registerFunctor<builtin::Alloc>(alloc);
    builtin_functor_t<builtin::Lock> lock = [this](GenValue t, LockType type) {
      Command c;
      c.kind = Command::LOCK;
      c.tensor = val(t).tensor;
      c.lockType = type;
      emit(std::move(c));
      return GenValue{};
    };
    g.registerFunctor<builtin::Lock>(lock);
    builtin_functor_t<builtin::Release> release = [this](GenValue t) {
      Command c;
      c.kind = Command::RELEASE;
      c.tensor = val(t).tensor;
      emit(std::move(c));
      return GenValue{};
    };
    g.registerFunctor<builtin::Release>(release);
    builtin_functor_t<builtin::InvokeLoader> load = [this](GenValue t) {
      Command c;
      c.kind = Command::LOAD;
      c.tensor = val(t).tensor;
      emit(std::move(c));
      return GenValue{};
    };
    g.registerFunctor<builtin::InvokeLoader>(load);
    builtin_functor_t<builtin::Barrier> barrier = [this](uint64_t clusterId) {
      if (mPoint.graph) mPoint.graph->steps.push_back(Step{Step::BARRIER, nullptr, clusterId});
    };
    g.registerFunctor<builtin::Barrier>(barrier);
    builtin_functor_t<builtin::NodeEval> eval = [this](GenGraph gr, GenNode n, const std::vector<GenValue>&) {
      auto& rec = gr.graph<GraphRecord>();
      auto node = std::shared_ptr<NodeRecord>(&n.node<NodeRecord>(), [keep = n](NodeRecord*) {});
      rec.steps.push_back(Step{Step::NODE, node, node->clusterId});
      return n.getResult();
    };
    g.registerFunctor<builtin::NodeEval>(eval);
    builtin_functor_t<builtin::Return> ret = [](std::optional<GenValue>) {};
    g.registerFunctor<builtin::Return>(ret);

    // Operation builtins -> native kernel names and LaunchCommand argument orders.
    builtin_functor_t<builtin::Add> add = [this](GenValue a, GenValue sa, GenValue b, GenValue sb, GenValue out) {
      launch("fadd", {a, sa, b, sb, out});
    };
    g.registerFunctor<builtin::Add>(add);
    builtin_functor_t<builtin::Copy> copy = [this](GenValue in, GenValue out) { launch("fcopy", {in, out}); };
    g.registerFunctor<builtin::Copy>(copy);
    builtin_functor_t<builtin::Divide> div = [this](GenValue n, GenValue d, GenValue out) {
      launch("fdivide", {n, d, out});
    };
    g.registerFunctor<builtin::Divide>(div);
    builtin_functor_t<builtin::LogLoss> ll = [this](GenValue p, GenValue y, GenValue out) {
      launch("flogloss", {p, y, out});
    };
    g.registerFunctor<builtin::LogLoss>(ll);
    builtin_functor_t<builtin::MatMul> mm = [this](GenValue l, GenValue r, GenValue out, bool tl, bool tr) {
      const char* names[2][2] = {{"fmatmul_f_f", "fmatmul_f_t"}, {"fmatmul_t_f", "fmatmul_t_t"}};
      launch(names[tl ? 1 : 0][tr ? 1 : 0], {l, r, out});
    };
    g.registerFunctor<builtin::MatMul>(mm);
    builtin_functor_t<builtin::Mul> mul = [this](GenValue a, GenValue b, GenValue out) { launch("fmul", {a, b, out}); };
    g.registerFunctor<builtin::Mul>(mul);
    builtin_functor_t<builtin::MulConcat> mc = [this](GenValue grad, GenValue local, GenValue out) {
      launch("fmulconcat", {grad, local, out});
    };
    g.registerFunctor<builtin::MulConcat>(mc);
    builtin_functor_t<builtin::Fill> fill = [this](GenValue pattern, GenValue out) { launch("ffill", {pattern, out}); };
    g.registerFunctor<builtin::Fill>(fill);
    builtin_functor_t<builtin::Sigmoid> sig = [this](GenValue in, GenValue out) { launch("fsigmoid", {in, out}); };
    g.registerFunctor<builtin::Sigmoid>(sig);

    builtin_functor_t<builtin::Conv2D> conv = [this](GenValue in, GenValue ker, GenValue out) {
      launch("fconv2d", {in, ker, out});
    };
    g.registerFunctor<builtin::Conv2D>(conv);
    // The window and the stride are attributes of the operation; they travel as four
    // 8-byte integer DATA arguments between the input and the output tensor.
    builtin_functor_t<builtin::Pool2D> pool = [this](GenValue in, GenValue out, const std::vector<int64_t>& window,
                                                     const std::vector<int64_t>& stride) {
      if (window.size() != 2 || stride.size() != 2) return refuse("Pool2D with a window that is not 2-D");
      auto attr = [](int64_t v) {
        auto a = std::make_shared<Value>();
        a->isInteger = true;
        a->integer = v;
        return GenValue{a};
      };
      launch("fpool", {in, attr(window[0]), attr(window[1]), attr(stride[0]), attr(stride[1]), out});
    };
    g.registerFunctor<builtin::Pool2D>(pool);
    builtin_functor_t<builtin::ReLU> relu = [this](GenValue in, GenValue out) { launch("frelu", {in, out}); };
    g.registerFunctor<builtin::ReLU>(relu);
    builtin_functor_t<builtin::Softmax> sm = [this](GenValue in, GenValue out) { launch("fsoftmax", {in, out}); };
    g.registerFunctor<builtin::Softmax>(sm);
    // Builtins no operation of the reference emits.  Transpose has a tensor in and a tensor
    // out like any other.  Slice's functor takes (index, tensor) and returns nothing
    // (GenBuiltins.hpp:147-149), so a generator cannot hand the sub-tensor to a consumer: no
    // launch can be recorded for it.  The device builtin "fslice" exists for callers by name.
    builtin_functor_t<builtin::Slice> sl = [this](GenValue, GenValue) { refuse("Slice (no result value to launch into)"); };
    g.registerFunctor<builtin::Slice>(sl);
    builtin_functor_t<builtin::Transpose> tp = [this](GenValue in, GenValue out) { launch("ftranspose", {in, out}); };
    g.registerFunctor<builtin::Transpose>(tp);
  }
};

TensorInfo infoOf(TensorDesc& d) {
  TensorInfo t;
  t.virtAddr = d.virtAddr;
  t.dataType = d.dataType;
  t.dims = d.shape.size();
  t.shape = d.shape.data();
  return t;
}

}  // namespace

// ---- constants filled on the device -------------------------------------------------------
// The reference fills a constant tensor element by element on the host and copies it over
// (ConstantLoaderInternal.cpp:24-31); gradient graphs create such ones/zeros tensors for every
// differentiated node (GraphInternal.cpp:242-251,282-292).  Here an input node fed by a
// ConstantLoader is placed on the compute device and its LOAD becomes one `ffill` launch -
// the builtin the reference registers (CodeGen.cpp:454-462) but never emits.
//
// This build has no RTTI (like the reference's), so a loader's dynamic type is read off its
// vtable pointer and compared with that of a ConstantLoaderInternal made here; the class has
// one vtable, emitted with its key function in the frontend library.
namespace {
struct ConstantPeek : polarai::loaders::internal::ConstantLoaderInternal {
  static float value(const polarai::loaders::internal::ConstantLoaderInternal& c) {
    return c.*(&ConstantPeek::mFloatValue);
  }
};
inline const void* vtableOf(const void* object) { return *static_cast<const void* const*>(object); }
}  // namespace

// ---- batch-sharded execution over several devices -------------------------------------------
// The reference's Executor accepts several devices but runs every node on the first one
// (ExecutorImpl.cpp:71-75; ath_device_select, routines.cpp:73-79).  When the caller declares
// which inputs are batch-sharded (polar_b200_executor_shard_inputs), this Executor replays the
// recorded program on EVERY selected device - one host thread and one allocator per device -
// with the rows of the sharded tensors divided among them, and sums the results of
// contractions over the batch across the devices (data_parallel_plan.hpp has the rules).
namespace {

namespace dp = polar_b200::dp;

// One device's copy of the world: its own allocator (tags and locks are per replica: the
// "same" record holds different rows on different devices) and the device itself.
struct Replica {
  std::shared_ptr<Device> device;
  std::shared_ptr<BackendAllocator> allocator;
};

// Reusable barrier for the replica threads.
class ThreadBarrier {
public:
  explicit ThreadBarrier(unsigned n) : mCount(n) {}
  void wait() {
    std::unique_lock<std::mutex> lk(mMutex);
    const unsigned gen = mGeneration;
    if (++mArrived == mCount) {
      mArrived = 0;
      ++mGeneration;
      mCv.notify_all();
    } else {
      mCv.wait(lk, [&] { return gen != mGeneration; });
    }
  }

private:
  std::mutex mMutex;
  std::condition_variable mCv;
  unsigned mCount, mArrived = 0, mGeneration = 0;
};

MemoryRecord recordOf(const TensorInternal& t) {
  return MemoryRecord{t.getVirtualAddress(), t.getSize() * polarai::core::sizeOfDataType(t.getDataType())};
}

// What Executor::getAllocator() hands out once a graph has run batch-sharded: host reads of a
// tensor are answered from the replicas - a replicated tensor from the first device, a
// sharded one gathered row block by row block into a buffer of the global size.  Everything
// the replicas do not know goes to the single-device allocator it wraps.
class ReplicaViewAllocator final : public BackendAllocator {
public:
  ReplicaViewAllocator(std::shared_ptr<BackendAllocator> single, std::vector<Replica>* replicas,
                       std::unordered_map<uint64_t, dp::Part>* parts)
      : mSingle(std::move(single)), mReplicas(replicas), mParts(parts) {}

  void registerDevice(Device& d) override { mSingle->registerDevice(d); }
  void allocate(const TensorInternal& t, Device& d) override { mSingle->allocate(t, d); }
  void allocate(const MemoryRecord& r, Device& d) override { mSingle->allocate(r, d); }
  void allocate(const MemoryRecord& r) override { mSingle->allocate(r); }
  void allocate(const TensorInternal& t) override { base().allocate(t); }
  void deallocate(const TensorInternal& t) override { base().deallocate(t); }
  void lock(const TensorInternal& t, Device& d, LockType type) override { mSingle->lock(t, d, type); }
  void lock(const MemoryRecord& r, Device& d, LockType type) override { mSingle->lock(r, d, type); }
  void release(const MemoryRecord& r, Device& d) override { mSingle->release(r, d); }

  void lock(const TensorInternal& t, LockType type) override { lock(recordOf(t), type); }
  void release(const TensorInternal& t) override { release(recordOf(t)); }
  void* get(const TensorInternal& t) override { return get(recordOf(t)); }

  void lock(const MemoryRecord& global, LockType type) override {
    const dp::Part part = partOf(global);
    if (part == dp::Part::UNKNOWN) return mSingle->lock(global, type);
    // OutputNodeAccessor asks for READ_WRITE even to read (OutputNodeAccessor.hpp:24); the view
    // serves reads: a write made through it would reach one device at most, so inputs are
    // changed through their loaders instead.
    (void)type;
    const size_t n = mReplicas->size();
    if (part == dp::Part::REPLICATED) {
      (*mReplicas)[0].allocator->lock(global, LockType::READ);
      return;
    }
    // sharded: gather the row blocks
    MemoryRecord local{global.virtualAddress, global.allocationSize / n};
    auto& buf = mGathered[global.virtualAddress];
    buf.resize(global.allocationSize);
    for (size_t r = 0; r < n; ++r) {
      auto& a = *(*mReplicas)[r].allocator;
      a.lock(local, LockType::READ);
      if (void* p = a.get(local)) std::memcpy(buf.data() + r * local.allocationSize, p, local.allocationSize);
      a.release(local);
    }
  }
  void release(const MemoryRecord& global) override {
    const dp::Part part = partOf(global);
    if (part == dp::Part::UNKNOWN) return mSingle->release(global);
    if (part == dp::Part::REPLICATED) (*mReplicas)[0].allocator->release(global);
  }
  void* get(const MemoryRecord& global) override {
    const dp::Part part = partOf(global);
    if (part == dp::Part::UNKNOWN) return mSingle->get(global);
    if (part == dp::Part::REPLICATED) return (*mReplicas)[0].allocator->get(global);
    auto it = mGathered.find(global.virtualAddress);
    return it == mGathered.end() ? nullptr : it->second.data();
  }

protected:
  void* getImpl(const TensorInternal&, Device&) override { return nullptr; }
  void* getImpl(const MemoryRecord&, Device&) override { return nullptr; }

private:
  // the tensor-keyed overloads live in the base interface (the derived class's own overloads hide them)
  TensorAllocator& base() { return *mSingle; }
  dp::Part partOf(const MemoryRecord& r) const {
    if (mReplicas->empty()) return dp::Part::UNKNOWN;
    auto it = mParts->find(r.virtualAddress);
    return it == mParts->end() ? dp::Part::UNKNOWN : it->second;
  }
  std::shared_ptr<BackendAllocator> mSingle;
  std::vector<Replica>* mReplicas;
  std::unordered_map<uint64_t, dp::Part>* mParts;
  std::unordered_map<uint64_t, std::vector<unsigned char>> mGathered;
};

}  // namespace

class ExecutorImpl {
public:
  using FilterFunctionT = Executor::FilterFunctionT;

  ExecutorImpl(bool debug, FilterFunctionT filter) : mDebug(debug), mFilter(std::move(filter)) {
    mAllocator = std::make_shared<LayerAllocator>();
    mRuntimeDriver = std::make_shared<RuntimeDriver>(debug);
    std::copy_if(mRuntimeDriver->getDeviceList().begin(), mRuntimeDriver->getDeviceList().end(),
                 std::back_inserter(mDevices), mFilter);
    for (auto& dev : mDevices) {
      if (debug) std::clog << "Registering " << dev->getDeviceName() << '\n';
      mAllocator->registerDevice(*dev);
    }
    mHost = std::make_shared<HostDevice>();
    registerSelf(true);
  }
  ~ExecutorImpl() { registerSelf(false); }
  void registerSelf(bool add);

  void addGraph(Graph& graph) {
    Generator generator;
    Recorder recorder(generator);
    GraphCompiler::compile(graph, generator);
    for (auto& u : recorder.unsupported)
      std::fprintf(stderr, "[polar_b200_executor] graph '%s' uses builtin %s, which this runtime does not implement\n",
                   graph.getName().getString(), u.c_str());
    mGraphs[graph.getName().getString()] = recorder.graph;
    if (mDebug && recorder.graph)
      std::clog << "Recorded graph " << recorder.graph->name << ": " << recorder.graph->steps.size() << " steps\n";
    if (recorder.graph && std::getenv("POLAR_B200_DUMP_PROGRAM")) dump(*recorder.graph);
  }

  // The recorded program as text, one line per runtime call, in the order evaluate() issues
  // them (POLAR_B200_DUMP_PROGRAM=1): what the reference's lowering to its runtime dialect
  // would contain for the same graph (utils/dialects/test/conversion/graph_to_runtime.mlir).
  static void dump(const GraphRecord& g) {
    std::printf("program %s\n", g.name.c_str());
    for (const auto& step : g.steps) {
      if (step.kind == Step::BARRIER) {
        std::printf("  barrier cluster=%llu\n", (unsigned long long)step.clusterId);
        continue;
      }
      const NodeRecord& n = *step.node;
      std::printf("  node %s id=%zu cluster=%zu\n", n.name.c_str(), n.nodeId, n.clusterId);
      for (const auto& c : n.commands) {
        switch (c.kind) {
          case Command::ALLOC: std::printf("    alloc va=%llu\n", (unsigned long long)c.tensor.virtAddr); break;
          case Command::LOCK:
            std::printf("    lock %s va=%llu\n", c.lockType == LockType::READ ? "read" : "read_write",
                        (unsigned long long)c.tensor.virtAddr);
            break;
          case Command::RELEASE: std::printf("    release va=%llu\n", (unsigned long long)c.tensor.virtAddr); break;
          case Command::LOAD: std::printf("    load va=%llu\n", (unsigned long long)c.tensor.virtAddr); break;
          case Command::LAUNCH: {
            std::printf("    launch %s", c.nativeName.c_str());
            for (const auto& v : c.args) {
              if (v.isTensor) std::printf(" T%llu", (unsigned long long)v.tensor.virtAddr);
              else if (v.isInteger) std::printf(" i%lld", (long long)v.integer);
              else std::printf(" f%g", v.scalar);
            }
            std::printf("\n");
            break;
          }
        }
      }
    }
    std::fflush(stdout);
  }

  void evaluate(Graph& graph) {
    auto it = mGraphs.find(graph.getName().getString());
    if (it == mGraphs.end() || !it->second) {
      std::fprintf(stderr, "[polar_b200_executor] evaluate: graph '%s' was not added\n", graph.getName().getString());
      return;
    }
    if (mDevices.empty()) {
      std::fprintf(stderr, "[polar_b200_executor] evaluate: no device\n");
      return;
    }
    GraphHandle handle;
    handle.allocator = mAllocator;
    handle.devices.push_back(mDevices.front());
    handle.devices.push_back(mHost);
    std::unordered_map<uint64_t, float> constants;   // input node -> fill value
    std::set<uint64_t> keeps;                        // input nodes whose loader writes nothing
    prepare(graph, handle, constants, keeps);
    if (mDevices.size() > 1 && !mShardInputs.empty()) {
      if (evaluateDataParallel(*it->second, handle, constants, keeps)) return;
      // not shardable: said on stderr; the graph runs on the first device like in the reference
    }
    std::vector<Event*> pending;
    for (auto& step : it->second->steps) {
      if (step.kind == Step::BARRIER) {
        if (!pending.empty()) ath_barrier(static_cast<uint32_t>(pending.size()), pending.data());
        for (Event* e : pending) delete e;
        pending.clear();
        continue;
      }
      NodeRecord& node = *step.node;
      Device* device = ath_device_select(&handle, node.nodeId);
      for (auto& c : node.commands) {
        TensorInfo ti = infoOf(c.tensor);
        switch (c.kind) {
          case Command::ALLOC: ath_allocate(&handle, *device, &ti); break;
          case Command::LOCK: ath_lock(&handle, *device, &ti, c.lockType); break;
          // Work on a device is stream-ordered, so the lock can go as soon as the
          // launch is queued; no event is attached.
          case Command::RELEASE: ath_release(&handle, *device, &ti, nullptr); break;
          case Command::LOAD: {
            auto cst = constants.find(node.nodeId);
            if (cst == constants.end()) {
              ath_load(&handle, node.nodeId, &ti);
              break;
            }
            ArgDesc fillArgs[2] = {{sizeof(float), &cst->second, ArgDesc::DATA}, {0, &ti, ArgDesc::TENSOR}};
            std::string kernelName = node.name + "_ffill";
            LaunchCommand cmd{kernelName.c_str(), 2, fillArgs, "ffill"};
            Event* evt = ath_launch(&handle, device, nullptr, cmd);
            if (evt) pending.push_back(evt);
            break;
          }
          case Command::LAUNCH: {
            std::vector<TensorInfo> infos(c.args.size());
            std::vector<ArgDesc> args(c.args.size());
            for (size_t i = 0; i < c.args.size(); ++i) {
              Value& v = c.args[i];
              if (v.isTensor) {
                infos[i] = infoOf(v.tensor);
                args[i] = ArgDesc{0, &infos[i], ArgDesc::TENSOR};
              } else if (v.isInteger) {
                args[i] = ArgDesc{sizeof(int64_t), &v.integer, ArgDesc::DATA};
              } else {
                args[i] = ArgDesc{sizeof(float), &v.scalar, ArgDesc::DATA};
              }
            }
            std::string kernelName = node.name + "_" + c.nativeName;
            LaunchCommand cmd{kernelName.c_str(), args.size(), args.data(), c.nativeName.c_str()};
            Event* evt = ath_launch(&handle, device, nullptr, cmd);
            if (evt) pending.push_back(evt);
            break;
          }
        }
      }
    }
    if (!pending.empty()) ath_barrier(static_cast<uint32_t>(pending.size()), pending.data());
    for (Event* e : pending) delete e;
  }

  // Loaders, host nodes and constants of a graph, as evaluate() needs them.  Input nodes run
  // on the host: their loaders fill host memory (ExecutorImpl.cpp:77-93) - except constants,
  // which are filled where they are used.
  void prepare(Graph& graph, GraphHandle& handle, std::unordered_map<uint64_t, float>& constants,
               std::set<uint64_t>& keeps) {
    auto& traversal = graph.traverse();
    auto ctx = graph.getContext().internal();
    polarai::loaders::internal::ConstantLoaderInternal constantProbe(ctx, 0, 0.0f);
    polarai::loaders::internal::DummyLoaderInternal dummyProbe(ctx, 0);
    for (const auto& cluster : traversal.getClusters()) {
      for (const auto& node : cluster.content) {
        auto& n = ctx->getRef<AbstractNodeInternal>(node.nodeIndex);
        if (n.getType() != NodeType::INPUT) continue;
        auto& inp = ctx->getRef<InputNodeInternal>(node.nodeIndex);
        auto& loader = ctx->getRef<AbstractLoaderInternal>(inp.getLoader());
        handle.mLoaders[node.nodeIndex] = &loader;
        if (vtableOf(&loader) == vtableOf(&dummyProbe)) keeps.insert(node.nodeIndex);
        if (mDeviceConstants && vtableOf(&loader) == vtableOf(&constantProbe)) {
          constants[node.nodeIndex] =
              ConstantPeek::value(static_cast<const polarai::loaders::internal::ConstantLoaderInternal&>(loader));
          continue;   // stays on the compute device: ath_device_select sends only host nodes to the host
        }
        handle.isHostNode.insert(node.nodeIndex);
      }
    }
  }

  bool evaluateDataParallel(GraphRecord& graph, GraphHandle& single, std::unordered_map<uint64_t, float>& constants,
                            std::set<uint64_t>& keeps);

  BackendAllocator& getAllocator() { return mView ? static_cast<BackendAllocator&>(*mView) : *mAllocator; }
  std::shared_ptr<BackendAllocator> getAllocatorPtr() {
    return mView ? std::static_pointer_cast<BackendAllocator>(mView) : mAllocator;
  }
  void setAllocator(std::shared_ptr<BackendAllocator>& allocator) {
    mAllocator = std::move(allocator);
    for (auto& dev : mDevices) mAllocator->registerDevice(*dev);
  }
  std::vector<std::shared_ptr<Device>>& getDevices() { return mDevices; }
  void shardInputs(const size_t* ids, size_t count) {
    mShardInputs.clear();
    for (size_t i = 0; i < count; ++i) mShardInputs.insert(ids[i]);
  }

private:
  bool mDebug;
  // POLAR_B200_HOST_CONSTANTS=1 keeps the reference's host-side constant fill
  bool mDeviceConstants = std::getenv("POLAR_B200_HOST_CONSTANTS") == nullptr;
  FilterFunctionT mFilter;
  // The driver owns the plugin library: it must outlive the devices' users.
  std::shared_ptr<RuntimeDriver> mRuntimeDriver;
  std::vector<std::shared_ptr<Device>> mDevices;
  std::shared_ptr<Device> mHost;
  std::shared_ptr<BackendAllocator> mAllocator;
  std::map<std::string, std::shared_ptr<GraphRecord>> mGraphs;
  // batch-sharded execution (empty until the caller declares sharded inputs)
  std::set<uint64_t> mShardInputs;                       // input node ids
  std::vector<Replica> mReplicas;                        // one per selected device, kept across graphs
  std::unordered_map<uint64_t, dp::Part> mParts;         // split of every tensor seen so far
  uint64_t mBatch = 0;
  std::shared_ptr<ReplicaViewAllocator> mView;
};

// Replays the recorded program on every selected device with the batch rows divided among
// them.  Returns false (after saying why) when the program cannot be split by rows.
bool ExecutorImpl::evaluateDataParallel(GraphRecord& graph, GraphHandle& single,
                                        std::unordered_map<uint64_t, float>& constants, std::set<uint64_t>& keeps) {
  const unsigned n = static_cast<unsigned>(mDevices.size());
  // 1. the program as the planner sees it
  struct Site { size_t step, cmd; };
  std::vector<dp::Op> ops;
  std::vector<Site> sites;
  auto argOf = [](const TensorDesc& t) {
    dp::Arg a;
    a.isTensor = true;
    a.va = t.virtAddr;
    a.shape = t.shape;
    return a;
  };
  for (size_t si = 0; si < graph.steps.size(); ++si) {
    if (graph.steps[si].kind != Step::NODE) continue;
    NodeRecord& node = *graph.steps[si].node;
    for (size_t ci = 0; ci < node.commands.size(); ++ci) {
      Command& c = node.commands[ci];
      dp::Op op;
      if (c.kind == Command::LOAD) {
        op.name = "load";
        op.args.push_back(argOf(c.tensor));
        op.declaredSharded = mShardInputs.count(node.nodeId) > 0;
        op.constant = constants.count(node.nodeId) > 0;
        op.keeps = keeps.count(node.nodeId) > 0;
      } else if (c.kind == Command::LAUNCH) {
        op.name = c.nativeName;
        for (auto& v : c.args) op.args.push_back(v.isTensor ? argOf(v.tensor) : dp::Arg{});
      } else {
        continue;
      }
      ops.push_back(std::move(op));
      sites.push_back(Site{si, ci});
    }
  }
  dp::Plan plan = dp::makePlan(ops, n, mParts, mBatch);
  if (!plan.ok) {
    std::fprintf(stderr, "[polar_b200_executor] graph '%s' cannot be split by rows over %u devices (%s): running on "
                         "the first device\n", graph.name.c_str(), n, plan.why.c_str());
    return false;
  }
  mBatch = plan.batch;
  // which node's result needs a sum over the devices once the node has released it
  std::unordered_map<size_t, TensorDesc> sumAfterStep;
  for (size_t i = 0; i < ops.size(); ++i)
    if (plan.sumAfter[i]) sumAfterStep[sites[i].step] = graph.steps[sites[i].step].node->commands[sites[i].cmd].args.back().tensor;

  // 2. one replica per device, kept across graphs (forward, gradient and update graphs share tensors)
  if (mReplicas.empty()) {
    for (auto& d : mDevices) {
      Replica r;
      r.device = d;
      r.allocator = std::make_shared<LayerAllocator>();
      r.allocator->registerDevice(*d);
      mReplicas.push_back(std::move(r));
    }
    mView = std::make_shared<ReplicaViewAllocator>(mAllocator, &mReplicas, &mParts);
  }

  // 3. host inputs are loaded ONCE, at their global size, and handed out by rows
  std::unordered_map<uint64_t, std::vector<float>> loaded;   // node id -> global data
  for (auto& step : graph.steps) {
    if (step.kind != Step::NODE) continue;
    NodeRecord& node = *step.node;
    if (constants.count(node.nodeId) || keeps.count(node.nodeId)) continue;
    for (auto& c : node.commands) {
      if (c.kind != Command::LOAD) continue;
      uint64_t count = 1;
      for (uint64_t d : c.tensor.shape) count *= d;
      auto& buf = loaded[node.nodeId];
      buf.assign(count, 0.0f);
      BackendAccessor<float> acc(buf.data(), c.tensor.shape.size(), c.tensor.shape.data());
      single.mLoaders[node.nodeId]->load(acc);
    }
  }

  // 4. replay, one host thread per device
  ThreadBarrier barrier(n);
  std::vector<std::vector<float>> partial(n);   // exchange slots
  std::vector<float> total;
  auto localDesc = [&](const TensorDesc& t) {
    TensorDesc l = t;
    auto it = plan.part.find(t.virtAddr);
    l.shape = dp::localShape(t.shape, it == plan.part.end() ? dp::Part::REPLICATED : it->second, n);
    return l;
  };
  auto bytesOf = [](const TensorDesc& t) {
    uint64_t b = 4;
    for (uint64_t d : t.shape) b *= d;
    return b;
  };
  auto work = [&](unsigned r) {
    Replica& rep = mReplicas[r];
    GraphHandle handle;
    handle.allocator = rep.allocator;
    handle.devices.push_back(rep.device);
    handle.devices.push_back(mHost);
    handle.mLoaders = single.mLoaders;
    handle.isHostNode = single.isHostNode;
    std::vector<Event*> pending;
    auto drain = [&] {
      if (!pending.empty()) ath_barrier(static_cast<uint32_t>(pending.size()), pending.data());
      for (Event* e : pending) delete e;
      pending.clear();
    };
    for (size_t si = 0; si < graph.steps.size(); ++si) {
      Step& step = graph.steps[si];
      if (step.kind == Step::BARRIER) {
        drain();
        continue;
      }
      NodeRecord& node = *step.node;
      Device* device = ath_device_select(&handle, node.nodeId);
      for (auto& c : node.commands) {
        TensorDesc local = localDesc(c.tensor);
        TensorInfo ti = infoOf(local);
        switch (c.kind) {
          case Command::ALLOC: ath_allocate(&handle, *device, &ti); break;
          case Command::LOCK: ath_lock(&handle, *device, &ti, c.lockType); break;
          case Command::RELEASE: ath_release(&handle, *device, &ti, nullptr); break;
          case Command::LOAD: {
            auto cst = constants.find(node.nodeId);
            if (cst != constants.end()) {
              ArgDesc fillArgs[2] = {{sizeof(float), &cst->second, ArgDesc::DATA}, {0, &ti, ArgDesc::TENSOR}};
              std::string kernelName = node.name + "_ffill";
              LaunchCommand cmd{kernelName.c_str(), 2, fillArgs, "ffill"};
              if (Event* evt = ath_launch(&handle, device, nullptr, cmd)) pending.push_back(evt);
              break;
            }
            auto src = loaded.find(node.nodeId);
            if (src == loaded.end()) break;   // a loader that writes nothing: the tensor keeps what it holds
            MemoryRecord rec{local.virtAddr, bytesOf(local)};
            if (void* dst = rep.allocator->get(rec)) {
              const bool sharded = plan.part[local.virtAddr] == dp::Part::SHARDED;
              const char* from = reinterpret_cast<const char*>(src->second.data()) + (sharded ? r * rec.allocationSize : 0);
              std::memcpy(dst, from, rec.allocationSize);
            }
            break;
          }
          case Command::LAUNCH: {
            std::vector<TensorDesc> locals(c.args.size());
            std::vector<TensorInfo> infos(c.args.size());
            std::vector<ArgDesc> args(c.args.size());
            for (size_t i = 0; i < c.args.size(); ++i) {
              Value& v = c.args[i];
              if (v.isTensor) {
                locals[i] = localDesc(v.tensor);
                infos[i] = infoOf(locals[i]);
                args[i] = ArgDesc{0, &infos[i], ArgDesc::TENSOR};
              } else if (v.isInteger) {
                args[i] = ArgDesc{sizeof(int64_t), &v.integer, ArgDesc::DATA};
              } else {
                args[i] = ArgDesc{sizeof(float), &v.scalar, ArgDesc::DATA};
              }
            }
            std::string kernelName = node.name + "_" + c.nativeName;
            LaunchCommand cmd{kernelName.c_str(), args.size(), args.data(), c.nativeName.c_str()};
            if (Event* evt = ath_launch(&handle, device, nullptr, cmd)) pending.push_back(evt);
            break;
          }
        }
      }
      auto sum = sumAfterStep.find(si);
      if (sum == sumAfterStep.end()) continue;
      // This node contracted over the batch: every device holds a partial sum of the whole
      // result.  Sum over the devices, in device order (the same bits on every device), through
      // host memory - the one exchange of a data-parallel step.  Generic over the Device
      // interface; the peer-memory kernel of the kernel library is the fast form for hosts that
      // run one process per GPU.
      drain();
      TensorDesc local = localDesc(sum->second);
      MemoryRecord rec{local.virtAddr, bytesOf(local)};
      const size_t count = rec.allocationSize / sizeof(float);
      rep.allocator->lock(rec, LockType::READ);
      partial[r].assign(static_cast<const float*>(rep.allocator->get(rec)),
                        static_cast<const float*>(rep.allocator->get(rec)) + count);
      rep.allocator->release(rec);
      barrier.wait();
      if (r == 0) {
        total = partial[0];
        for (unsigned d = 1; d < n; ++d)
          for (size_t i = 0; i < count; ++i) total[i] += partial[d][i];
      }
      barrier.wait();
      rep.allocator->lock(rec, LockType::READ_WRITE);
      std::memcpy(rep.allocator->get(rec), total.data(), rec.allocationSize);
      rep.allocator->release(rec);
      barrier.wait();   // `total` may be reused by the next sum
    }
    drain();
  };
  std::vector<std::thread> threads;
  for (unsigned r = 1; r < n; ++r) threads.emplace_back(work, r);
  work(0);
  for (auto& t : threads) t.join();
  return true;
}

namespace {
// Executor objects by the address of their device list (what Executor::getDevices() returns a
// reference to): the reference's Executor class has no room for new members.
std::mutex g_registryMutex;
std::map<const void*, ExecutorImpl*> g_registry;
}  // namespace

// ---- the public class declared by the reference header ----------------------

Executor::Executor(bool enableDebugOutput, FilterFunctionT filter)
    : mImpl(polarai::utils::makeShared<ExecutorImpl>(enableDebugOutput, std::move(filter))) {}
void Executor::addGraph(Graph& graph) { mImpl->addGraph(graph); }
void Executor::evaluate(Graph& graph) { mImpl->evaluate(graph); }
BackendAllocator& Executor::getAllocator() { return mImpl->getAllocator(); }
std::shared_ptr<BackendAllocator> Executor::getAllocatorPtr() { return mImpl->getAllocatorPtr(); }
void Executor::setAllocator(std::shared_ptr<BackendAllocator>& allocator) { mImpl->setAllocator(allocator); }
std::vector<std::shared_ptr<Device>>& Executor::getDevices() { return mImpl->getDevices(); }

void ExecutorImpl::registerSelf(bool add) {
  std::lock_guard<std::mutex> g(g_registryMutex);
  if (add) g_registry[&mDevices] = this;
  else g_registry.erase(&mDevices);
}

}  // namespace polarai::backend::generic

// Declared in include/polar_b200_executor.h.
void polar_b200_executor_shard_inputs(polarai::backend::generic::Executor& executor, const size_t* inputNodeIds,
                                      size_t count) {
  using namespace polarai::backend::generic;
  std::lock_guard<std::mutex> g(g_registryMutex);
  auto it = g_registry.find(&executor.getDevices());
  if (it != g_registry.end()) it->second->shardInputs(inputNodeIds, count);
}

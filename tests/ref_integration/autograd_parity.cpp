// Parity of whole graphs, autograd included, between the B200 device and the CPU
// oracle device, both driven through the same Executor with the unchanged
// Context/Graph/Node/Loader API:
//   logistic regression  L = LogLoss(Sigmoid(X . W), Y)   (BASELINE configuration 2)
//   forward graph, the gradient graph and the weight-update graph that
//   Graph::getGradient builds (src/core/graph/internal/GraphInternal.cpp:329-474),
//   evaluated in that order.
// The reference's autograd is taken as it is (its MatMul derivative multiplies by
// gradient[0] only, its learning rate is the built-in -0.01): the point is that both
// devices execute the identical builtin program and agree.
//
// Usage: autograd_parity [batch]        exit code 0 = parity holds (or no GPU: oracle only)
#include "oracle_device.hpp"

#include <polarai/backend/generic/Executor.hpp>
#include <polarai/core/context/Context.hpp>
#include <polarai/core/graph/Graph.hpp>
#include <polarai/core/node/InputNode.hpp>
#include <polarai/core/node/Node.hpp>
#include <polarai/core/node/OutputNode.hpp>
#include <polarai/core/node/internal/InputNodeInternal.hpp>
#include <polarai/loaders/MemcpyLoader.hpp>
#include <polarai/operation/LogLossOperation.hpp>
#include <polarai/operation/MatMulOperation.hpp>
#include <polarai/operation/SigmoidOperation.hpp>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>

using namespace polarai;
using namespace polarai::core;
using namespace polarai::operation;
using namespace polarai::backend::generic;

struct Result {
  std::vector<float> loss, weights;
  bool ok = false;
};

// Builds the graphs in a fresh Context and evaluates them on the executor's first device.
static Result runOn(Executor& executor, size_t batch, size_t nIn, std::vector<float> X, std::vector<float> W,
                    std::vector<float> Y) {
  Result res;
  // A roomy arena: the default one cannot grow (see HeterogeneousVector's copy on growth).
  core::Context context(utils::Allocator<utils::byte>(), 4000, 64);
  auto graph = context.create<Graph>("logreg");
  auto lx = context.create<loaders::MemcpyLoader>(X.data(), X.size() * sizeof(float));
  auto lw = context.create<loaders::MemcpyLoader>(W.data(), W.size() * sizeof(float));
  auto ly = context.create<loaders::MemcpyLoader>(Y.data(), Y.size() * sizeof(float));
  auto x = graph.create<InputNode>(TensorShape{batch, nIn}, DataType::FLOAT, true, lx.getPublicIndex(), "X");
  auto w = graph.create<InputNode>(TensorShape{nIn, 1}, DataType::FLOAT, false, lw.getPublicIndex(), "W");
  auto y = graph.create<InputNode>(TensorShape{batch, 1}, DataType::FLOAT, true, ly.getPublicIndex(), "Y");
  auto mm = graph.create<Node>(context.create<MatMulOperation>(false, false), "matmul");
  graph.connect(x, mm, MatMulOperation::LEFT);
  graph.connect(w, mm, MatMulOperation::RIGHT);
  auto sg = graph.create<Node>(context.create<SigmoidOperation>(), "sigmoid");
  graph.connect(mm, sg, SigmoidOperation::Unmarked);
  auto ll = graph.create<Node>(context.create<LogLossOperation>(), "logloss");
  graph.connect(sg, ll, LogLossOperation::PREDICTED);
  graph.connect(y, ll, LogLossOperation::GROUND_TRUTH);
  auto out = graph.create<OutputNode>("out");
  graph.connect(ll, out, Operation::Unmarked);

  auto [gradGraph, updGraph] = graph.getGradient(ll);

  executor.addGraph(graph);
  executor.addGraph(gradGraph);
  executor.addGraph(updGraph);
  executor.evaluate(graph);
  {
    auto acc = context.internal()->getRef<OutputNode>(out).getAccess<float>(executor.getAllocator());
    for (size_t i = 0; i < batch; ++i) res.loss.push_back(acc(i));
  }
  executor.evaluate(gradGraph);
  executor.evaluate(updGraph);
  {
    auto& wNode = context.internal()->getRef<core::internal::InputNodeInternal>(w);
    auto& tensor = *wNode.getTensorPtr();
    core::internal::TensorAllocator& alloc = executor.getAllocator();   // the base view: host access by tensor
    alloc.lock(tensor, core::internal::LockType::READ);
    auto* p = static_cast<float*>(alloc.get(tensor));
    for (size_t i = 0; i < nIn; ++i) res.weights.push_back(p[i]);
    alloc.release(tensor);
  }
  res.ok = true;
  return res;
}

int main(int argc, char** argv) {
  size_t batch = argc > 1 ? std::strtoul(argv[1], nullptr, 10) : 1;
  const size_t nIn = 784;
  std::mt19937 rng(0);
  std::normal_distribution<float> nx(0.f, 1.f), nw(0.f, 0.01f);
  std::vector<float> X(batch * nIn), W(nIn), Y(batch);
  for (auto& v : X) v = nx(rng);
  for (auto& v : W) v = nw(rng);
  for (auto& v : Y) v = (rng() & 1) ? 1.f : 0.f;

  // CPU: an executor with no driver devices, given the oracle device.
  Executor cpuExec(false, [](std::shared_ptr<Device>&) { return false; });
  auto oracle = std::make_shared<OracleDevice>();
  cpuExec.getDevices().push_back(oracle);
  cpuExec.getAllocator().registerDevice(*oracle);
  Result cpu = runOn(cpuExec, batch, nIn, X, W, Y);
  std::printf("oracle device: %d launches, loss[0]=%.7g, W[0] %.7g -> %.7g\n", oracle->launches, cpu.loss[0], W[0],
              cpu.weights[0]);
  if (oracle->failures) return 3;
  double moved = 0;
  for (size_t i = 0; i < nIn; ++i) moved += std::fabs(cpu.weights[i] - W[i]);
  if (!(moved > 0)) {
    std::printf("FAIL: the update graph did not change the weights\n");
    return 4;
  }

  if (batch == 1) {
    // With one row the reference's derivative chain is the textbook gradient:
    // dL/dW = ((p - y) / (p - p*p)) * ((1 - p) * p) * x, and W <- W - 0.01 * dL/dW.
    double z = 0;
    for (size_t i = 0; i < nIn; ++i) z += (double)X[i] * W[i];
    double p = 1.0 / (1.0 + std::exp(-z));
    double worst = 0, scale = 0;
    for (size_t i = 0; i < nIn; ++i) {
      double want = W[i] - 0.01 * (p - Y[0]) * X[i];
      worst = std::fmax(worst, std::fabs(cpu.weights[i] - want));
      scale = std::fmax(scale, std::fabs(want));
    }
    std::printf("batch 1: updated weights vs the analytic SGD step, max err / max|W| %.3g\n", worst / scale);
    if (worst / scale > 1e-4) return 5;
  }

  Executor gpuExec(false);
  if (gpuExec.getDevices().empty()) {
    std::printf("no B200 device: oracle-only run\n");
    return 0;
  }
  Result gpu = runOn(gpuExec, batch, nIn, X, W, Y);
  double lossErr = 0, wErr = 0, wScale = 0;
  for (size_t i = 0; i < batch; ++i)
    lossErr = std::fmax(lossErr, std::fabs(gpu.loss[i] - cpu.loss[i]) / std::fabs(cpu.loss[i]));
  for (size_t i = 0; i < nIn; ++i) {
    wErr = std::fmax(wErr, std::fabs(gpu.weights[i] - cpu.weights[i]));
    wScale = std::fmax(wScale, std::fabs(cpu.weights[i]));
  }
  std::printf("B200 device %s: loss max rel err %.3g, updated W max err / max|W| %.3g\n",
              gpuExec.getDevices().front()->getDeviceName().c_str(), lossErr, wErr / wScale);
  // fp32 GEMM / loss tolerance of the benchmark configuration
  bool ok = lossErr <= 1e-4 && wErr / wScale <= 1e-4;
  std::printf(ok ? "PARITY OK\n" : "PARITY FAILED\n");
  return ok ? 0 : 1;
}

// The Executor's batch-sharded evaluation on several devices, checked on the CPU: fake devices
// that compute with the oracle stand in for GPUs (oracle_device.hpp), the graph is built with
// the unchanged Context/Graph/Node/Loader API.
//
//   S  = Sigmoid(X . W)            X [B,I] and Y [B,H] are declared batch-sharded, W [I,H] is not
//   D  = Combine(1, S, -1, Y)
//   dW = X^T . D                   a contraction over the batch: summed over the devices
//   Wn = Combine(1, W, -0.1, dW)   the update every device applies to its replica
//
// One device, two devices and four devices must agree: S row for row (bit-exact - rows do not
// mix), dW and Wn up to the order of the batch sum; every device must have received the whole
// program.  With a GPU present the same comparison runs on the B200 devices.
//
// Usage: data_parallel_executor        exit code 0 = all comparisons hold
#include "oracle_device.hpp"

#include <polar_b200_executor.h>

#include <polarai/backend/generic/Executor.hpp>
#include <polarai/core/context/Context.hpp>
#include <polarai/core/graph/Graph.hpp>
#include <polarai/core/node/InputNode.hpp>
#include <polarai/core/node/Node.hpp>
#include <polarai/core/node/OutputNode.hpp>
#include <polarai/loaders/MemcpyLoader.hpp>
#include <polarai/operation/CombineOperation.hpp>
#include <polarai/operation/MatMulOperation.hpp>
#include <polarai/operation/SigmoidOperation.hpp>

#include <cmath>
#include <cstdio>
#include <random>
#include <vector>

using namespace polarai;
using namespace polarai::core;
using namespace polarai::operation;
using namespace polarai::backend::generic;

struct Result {
  std::vector<float> S, dW, Wn;
};

static Result runOn(Executor& executor, bool shard, size_t B, size_t I, size_t H, std::vector<float> X,
                    std::vector<float> W, std::vector<float> Y) {
  core::Context context(utils::Allocator<utils::byte>(), 4000, 64);
  auto graph = context.create<Graph>("dp_step");
  auto lx = context.create<loaders::MemcpyLoader>(X.data(), X.size() * sizeof(float));
  auto lw = context.create<loaders::MemcpyLoader>(W.data(), W.size() * sizeof(float));
  auto ly = context.create<loaders::MemcpyLoader>(Y.data(), Y.size() * sizeof(float));
  auto x = graph.create<InputNode>(TensorShape{B, I}, DataType::FLOAT, true, lx.getPublicIndex(), "X");
  auto w = graph.create<InputNode>(TensorShape{I, H}, DataType::FLOAT, false, lw.getPublicIndex(), "W");
  auto y = graph.create<InputNode>(TensorShape{B, H}, DataType::FLOAT, true, ly.getPublicIndex(), "Y");
  auto mm = graph.create<Node>(context.create<MatMulOperation>(false, false), "XW");
  graph.connect(x, mm, MatMulOperation::LEFT);
  graph.connect(w, mm, MatMulOperation::RIGHT);
  auto sg = graph.create<Node>(context.create<SigmoidOperation>(), "S");
  graph.connect(mm, sg, SigmoidOperation::Unmarked);
  auto df = graph.create<Node>(context.create<CombineOperation>(1.0f, -1.0f), "D");
  graph.connect(sg, df, CombineOperation::ALPHA);
  graph.connect(y, df, CombineOperation::BETA);
  auto gw = graph.create<Node>(context.create<MatMulOperation>(true, false), "dW");
  graph.connect(x, gw, MatMulOperation::LEFT);
  graph.connect(df, gw, MatMulOperation::RIGHT);
  auto up = graph.create<Node>(context.create<CombineOperation>(1.0f, -0.1f), "Wn");
  graph.connect(w, up, CombineOperation::ALPHA);
  graph.connect(gw, up, CombineOperation::BETA);
  auto outS = graph.create<OutputNode>("outS");
  graph.connect(sg, outS, Operation::Unmarked);
  auto outG = graph.create<OutputNode>("outG");
  graph.connect(gw, outG, Operation::Unmarked);
  auto outW = graph.create<OutputNode>("outW");
  graph.connect(up, outW, Operation::Unmarked);

  if (shard) {
    size_t ids[2] = {static_cast<size_t>(x), static_cast<size_t>(y)};
    polar_b200_executor_shard_inputs(executor, ids, 2);
  }
  executor.addGraph(graph);
  executor.evaluate(graph);
  Result res;
  auto read = [&](utils::Index node, size_t count, std::vector<float>& into) {
    auto acc = context.internal()->getRef<OutputNode>(node).getAccess<float>(executor.getAllocator());
    for (size_t i = 0; i < count; ++i) into.push_back(acc(i));
  };
  read(outS, B * H, res.S);
  read(outG, I * H, res.dW);
  read(outW, I * H, res.Wn);
  return res;
}

static int compare(const char* what, const Result& one, const Result& many) {
  int bad = 0;
  for (size_t i = 0; i < one.S.size(); ++i) bad += one.S[i] != many.S[i];
  double gErr = 0, gMax = 0, wErr = 0;
  for (size_t i = 0; i < one.dW.size(); ++i) {
    gErr = std::fmax(gErr, std::fabs(one.dW[i] - many.dW[i]));
    gMax = std::fmax(gMax, std::fabs(one.dW[i]));
    wErr = std::fmax(wErr, std::fabs(one.Wn[i] - many.Wn[i]));
  }
  std::printf("%s: S differs in %d of %zu entries; dW max err / max|dW| %.3g; Wn max err %.3g\n", what, bad, one.S.size(),
              gErr / gMax, wErr);
  return (bad == 0 && gErr / gMax <= 1e-5 && wErr <= 1e-5 * gMax) ? 0 : 1;
}

int main() {
  const size_t B = 96, I = 40, H = 24;
  std::mt19937 rng(3);
  std::normal_distribution<float> nd(0.f, 1.f);
  std::vector<float> X(B * I), W(I * H), Y(B * H);
  for (auto& v : X) v = nd(rng);
  for (auto& v : W) v = 0.1f * nd(rng);
  for (auto& v : Y) v = (rng() & 1) ? 1.f : 0.f;
  int failures = 0;

  auto withFakes = [&](unsigned n, bool shard, std::vector<std::shared_ptr<OracleDevice>>& devs) {
    Executor exec(false, [](std::shared_ptr<Device>&) { return false; });   // no driver devices
    for (unsigned d = 0; d < n; ++d) {
      devs.push_back(std::make_shared<OracleDevice>("fake-gpu-" + std::to_string(d)));
      exec.getDevices().push_back(devs.back());
      exec.getAllocator().registerDevice(*devs.back());
    }
    return runOn(exec, shard, B, I, H, X, W, Y);
  };
  std::vector<std::shared_ptr<OracleDevice>> d1, d2, d4, dn;
  Result one = withFakes(1, false, d1);
  Result two = withFakes(2, true, d2);
  Result four = withFakes(4, true, d4);
  failures += compare("2 fake devices vs 1", one, two);
  failures += compare("4 fake devices vs 1", one, four);
  std::printf("launches per device: 1 device %d | 2 devices %d %d | 4 devices %d %d %d %d\n", d1[0]->launches,
              d2[0]->launches, d2[1]->launches, d4[0]->launches, d4[1]->launches, d4[2]->launches, d4[3]->launches);
  for (auto& d : d2) failures += d->launches != d1[0]->launches || d->failures;
  for (auto& d : d4) failures += d->launches != d1[0]->launches || d->failures;
  // several devices but nothing declared: the reference's behaviour, everything on the first
  Result undeclared = withFakes(2, false, dn);
  failures += compare("2 fake devices, no declaration, vs 1", one, undeclared);
  failures += dn[1]->launches != 0;
  std::printf("undeclared: second device got %d launches\n", dn[1]->launches);

  Executor gpuExec(false);
  if (gpuExec.getDevices().size() >= 2) {
    // the same on the real devices: all selected B200s against the oracle's one-device result
    const size_t n = gpuExec.getDevices().size();
    const size_t Bg = 96 * n;   // any batch the devices divide
    std::vector<float> Xg(Bg * I), Yg(Bg * H);
    for (auto& v : Xg) v = nd(rng);
    for (auto& v : Yg) v = (rng() & 1) ? 1.f : 0.f;
    Executor cpu(false, [](std::shared_ptr<Device>&) { return false; });
    auto od = std::make_shared<OracleDevice>();
    cpu.getDevices().push_back(od);
    cpu.getAllocator().registerDevice(*od);
    Result ref = runOn(cpu, false, Bg, I, H, Xg, W, Yg);
    Result gpu = runOn(gpuExec, true, Bg, I, H, Xg, W, Yg);
    int bad = 0;
    double sErr = 0, gErr = 0, gMax = 0;
    for (size_t i = 0; i < ref.S.size(); ++i) sErr = std::fmax(sErr, std::fabs(ref.S[i] - gpu.S[i]) / std::fabs(ref.S[i]));
    for (size_t i = 0; i < ref.dW.size(); ++i) {
      gErr = std::fmax(gErr, std::fabs(ref.dW[i] - gpu.dW[i]));
      gMax = std::fmax(gMax, std::fabs(ref.dW[i]));
    }
    std::printf("%zu B200 devices vs the oracle on one device: S max rel err %.3g, dW max err / max|dW| %.3g\n", n, sErr,
                gErr / gMax);
    bad = !(sErr <= 1e-5 && gErr / gMax <= 1e-4);
    failures += bad;
  } else {
    std::printf("fewer than two B200 devices: fake devices only\n");
  }
  std::printf(failures ? "DATA PARALLEL FAILED\n" : "DATA PARALLEL OK\n");
  return failures;
}

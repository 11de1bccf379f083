// Host-side test of csrc/executor/data_parallel_plan.hpp: the split of an MLP-shaped program
// over devices follows from the declared batch inputs alone.
#include <executor/data_parallel_plan.hpp>

#include <cstdio>

using namespace polar_b200::dp;

static int g_failures = 0;
static void expect(bool c, const char* what) {
  if (!c) {
    ++g_failures;
    std::printf("FAILED: %s\n", what);
  }
}
static Arg T(uint64_t va, std::vector<uint64_t> shape) {
  Arg a;
  a.isTensor = true;
  a.va = va;
  a.shape = std::move(shape);
  return a;
}
static Arg S() { return Arg{}; }
static Op load(Arg t, bool sharded, bool constant = false, bool keeps = false) {
  Op o;
  o.name = "load";
  o.args = {t};
  o.declaredSharded = sharded;
  o.constant = constant;
  o.keeps = keeps;
  return o;
}
static Op op(const char* name, std::vector<Arg> args) {
  Op o;
  o.name = name;
  o.args = std::move(args);
  return o;
}

int main() {
  const uint64_t B = 64, I = 16, H = 12, O = 4;
  enum : uint64_t { X = 1, Y, W1, W2, ONES, Z1, HH, Z2, P, L, D, DW2, DH, OMH, SH, DZ1, DW1, LR };
  std::vector<Op> mlp = {
      load(T(X, {B, I}), true), load(T(Y, {B, O}), true), load(T(W1, {I, H}), false), load(T(W2, {H, O}), false),
      load(T(ONES, {B, H}), false, true),                               // a constant: follows its consumers
      op("fmatmul_f_f", {T(X, {B, I}), T(W1, {I, H}), T(Z1, {B, H})}),
      op("fsigmoid", {T(Z1, {B, H}), T(HH, {B, H})}),
      op("fmatmul_f_f", {T(HH, {B, H}), T(W2, {H, O}), T(Z2, {B, O})}),
      op("fsigmoid", {T(Z2, {B, O}), T(P, {B, O})}),
      op("flogloss", {T(P, {B, O}), T(Y, {B, O}), T(L, {B, O})}),
      op("fadd", {T(P, {B, O}), S(), T(Y, {B, O}), S(), T(D, {B, O})}),
      op("fmatmul_t_f", {T(HH, {B, H}), T(D, {B, O}), T(DW2, {H, O})}),      // contraction over the batch
      op("fmatmul_f_t", {T(D, {B, O}), T(W2, {H, O}), T(DH, {B, H})}),
      op("fadd", {T(ONES, {B, H}), S(), T(HH, {B, H}), S(), T(OMH, {B, H})}),
      op("fmul", {T(OMH, {B, H}), T(HH, {B, H}), T(SH, {B, H})}),
      op("fmul", {T(DH, {B, H}), T(SH, {B, H}), T(DZ1, {B, H})}),
      op("fmatmul_t_f", {T(X, {B, I}), T(DZ1, {B, H}), T(DW1, {I, H})}),
      op("fadd", {T(W2, {H, O}), S(), T(DW2, {H, O}), S(), T(W2, {H, O})}),
      op("fadd", {T(W1, {I, H}), S(), T(DW1, {I, H}), S(), T(W1, {I, H})}),
  };
  std::unordered_map<uint64_t, Part> known;
  Plan plan = makePlan(mlp, 2, known, 0);
  expect(plan.ok, "the MLP step is shardable");
  expect(plan.batch == B, "batch extent found from the declared inputs");
  for (uint64_t t : {X, Y, ONES, Z1, HH, Z2, P, L, D, DH, OMH, SH, DZ1})
    expect(plan.part[t] == Part::SHARDED, "batch-shaped tensors are split by rows");
  for (uint64_t t : {W1, W2, DW1, DW2}) expect(plan.part[t] == Part::REPLICATED, "weights and their gradients are replicated");
  int sums = 0;
  for (size_t i = 0; i < mlp.size(); ++i) {
    if (plan.sumAfter[i]) {
      ++sums;
      expect(mlp[i].name == "fmatmul_t_f", "only contractions over the batch need a sum over devices");
    }
  }
  expect(sums == 2, "two sums: dW2 and dW1");
  expect(localShape({B, I}, Part::SHARDED, 2) == std::vector<uint64_t>({B / 2, I}), "local shape halves the rows");
  expect(localShape({I, H}, Part::REPLICATED, 2) == std::vector<uint64_t>({I, H}), "replicated shape unchanged");

  // a later program of the same executor (a gradient graph) reads tensors the first one produced:
  // their split is remembered, and loaders that write nothing keep it
  std::vector<Op> later = {load(T(HH, {B, H}), false, false, true), load(T(W2, {H, O}), false, false, true),
                           op("fmatmul_f_f", {T(HH, {B, H}), T(W2, {H, O}), T(100, {B, O})})};
  Plan p2 = makePlan(later, 2, known, plan.batch);
  expect(p2.ok && p2.part[100] == Part::SHARDED, "splits carry over to later programs");

  // what cannot be a row split is refused, not mis-executed
  std::unordered_map<uint64_t, Part> k3;
  std::vector<Op> bad = {load(T(1, {B, I}), true), load(T(2, {B, I}), false),
                         op("fmul", {T(1, {B, I}), T(2, {B, I}), T(3, {B, I})})};
  expect(!makePlan(bad, 2, k3, 0).ok, "a replicated operand beside a sharded one is refused");
  k3.clear();
  std::vector<Op> soft = {load(T(1, {B, I}), true), op("fsoftmax", {T(1, {B, I}), T(2, {B, I})})};
  expect(!makePlan(soft, 2, k3, 0).ok, "a whole-tensor builtin on a split tensor is refused");
  k3.clear();
  std::vector<Op> odd = {load(T(1, {7, I}), true)};
  expect(!makePlan(odd, 2, k3, 0).ok, "a batch that does not divide is refused");
  k3.clear();
  std::vector<Op> tt = {load(T(1, {B, I}), true), load(T(2, {H, B}), false),
                        op("fmatmul_t_t", {T(1, {B, I}), T(2, {H, B}), T(3, {I, H})})};
  expect(!makePlan(tt, 2, k3, 0).ok, "a contraction whose right operand is not row-split is refused");
  // all-replicated programs stay valid (every device computes the same thing)
  k3.clear();
  std::vector<Op> rep = {load(T(1, {8, 8}), false), op("fsigmoid", {T(1, {8, 8}), T(2, {8, 8})})};
  Plan p5 = makePlan(rep, 2, k3, 0);
  expect(p5.ok && p5.part[2] == Part::REPLICATED, "nothing declared: everything replicated");

  std::printf("data_parallel_plan: %d failures\n", g_failures);
  return g_failures;
}

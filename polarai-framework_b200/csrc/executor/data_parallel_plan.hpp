// Batch-sharding plan for a recorded builtin program: which tensors are split by rows over
// the devices, which are replicated, and after which launches a sum over devices is due.
//
// The reference leaves this role empty: its Executor can be given several devices
// (include/polarai/backend/generic/Executor.hpp:36-61) but ath_device_select always answers
// devices.front() (src/backend/generic/runtime/support/routines.cpp:73-79, "TODO real device
// selection logic") and GraphPartitionPlanner is a placeholder
// (src/backend/generic/lib/GraphPartitionPlanner.cpp:18-41).  The plan made here is data
// parallelism: every device replays the same program on its share of the batch rows;
// everything follows from WHICH INPUTS the caller declares batch-sharded.
//
// Plain C++ over plain structs, so that the rules are testable on the host
// (tests/native/data_parallel_plan_test.cpp).
#pragma once

#include <cstdint>
#include <string>
#include <unordered_map>
#include <vector>

namespace polar_b200::dp {

enum class Part { UNKNOWN, REPLICATED, SHARDED };

struct Arg {
  bool isTensor = false;
  uint64_t va = 0;                 // virtual address of the tensor
  std::vector<uint64_t> shape;     // GLOBAL shape
};

struct Op {
  std::string name;                // native kernel name; "load" = an input node's loader
  std::vector<Arg> args;           // LaunchCommand order; the last tensor is the result
  bool declaredSharded = false;    // load: the caller declared this input batch-sharded
  bool constant = false;           // load: filled with one value (its split follows its consumers)
  bool keeps = false;              // load: the loader writes nothing (the tensor keeps what it holds)
};

struct Plan {
  bool ok = true;
  std::string why;                                  // when !ok: what cannot be sharded
  uint64_t batch = 0;                               // global extent of the sharded dimension
  std::unordered_map<uint64_t, Part> part;          // by virtual address
  std::vector<bool> sumAfter;                       // per op: its result is a per-device partial sum
};

inline bool isElementwise(const std::string& n) {
  static const char* names[] = {"fcopy", "fadd", "fmul", "fdivide", "fsigmoid", "flogloss", "frelu",
                                "fsigmoid_grad", "fsigmoid_logloss_grad"};
  for (const char* e : names)
    if (n == e) return true;
  return false;
}

// `known` carries the split of tensors that earlier programs of the same executor produced
// (a gradient graph reads the forward graph's activations); it is updated with this program's.
inline Plan makePlan(const std::vector<Op>& ops, unsigned devices, std::unordered_map<uint64_t, Part>& known,
                     uint64_t knownBatch) {
  Plan plan;
  plan.part = known;
  plan.batch = knownBatch;
  plan.sumAfter.assign(ops.size(), false);
  auto fail = [&](const std::string& why) {
    plan.ok = false;
    if (plan.why.empty()) plan.why = why;
  };
  auto partOf = [&](const Arg& a) {
    auto it = plan.part.find(a.va);
    return it == plan.part.end() ? Part::UNKNOWN : it->second;
  };
  auto shard = [&](const Arg& a, const std::string& what) {
    if (a.shape.empty()) return fail(what + ": a scalar cannot be split by rows");
    if (plan.batch == 0) plan.batch = a.shape[0];
    if (a.shape[0] != plan.batch) return fail(what + ": first extent differs from the batch");
    if (plan.batch % devices) return fail("the batch does not divide over the devices");
    plan.part[a.va] = Part::SHARDED;
  };
  // Two passes: the second one settles constants whose consumers come later in the program
  // than another consumer that left them undecided.
  for (int pass = 0; pass < 2 && plan.ok; ++pass) {
    for (size_t i = 0; i < ops.size() && plan.ok; ++i) {
      const Op& op = ops[i];
      std::vector<const Arg*> t;
      for (const Arg& a : op.args)
        if (a.isTensor) t.push_back(&a);
      if (t.empty()) continue;
      const Arg& out = *t.back();
      if (op.name == "load") {
        if (op.declaredSharded) shard(out, "declared input");
        else if (op.constant || op.keeps) { /* follows its consumers, or keeps what earlier programs decided */ }
        else if (partOf(out) == Part::UNKNOWN) plan.part[out.va] = Part::REPLICATED;
        continue;
      }
      if (op.name == "ffill") continue;   // like a constant load
      bool anySharded = false;
      for (size_t j = 0; j + 1 < t.size(); ++j) anySharded |= partOf(*t[j]) == Part::SHARDED;
      if (isElementwise(op.name)) {
        if (anySharded) {
          for (size_t j = 0; j + 1 < t.size(); ++j) {
            if (partOf(*t[j]) == Part::REPLICATED) return fail(op.name + ": a replicated operand beside a sharded one"), plan;
            shard(*t[j], op.name);         // settles undecided constants
          }
          shard(out, op.name);
        } else if (pass == 1 || partOf(*t[0]) == Part::REPLICATED) {
          for (size_t j = 0; j + 1 < t.size(); ++j)
            if (partOf(*t[j]) == Part::UNKNOWN) plan.part[t[j]->va] = Part::REPLICATED;
          plan.part[out.va] = Part::REPLICATED;
        }
        continue;
      }
      if (op.name == "fmulconcat" && t.size() == 3) {
        if (partOf(*t[0]) == Part::SHARDED) return fail("fmulconcat: the gradient scalar is sharded"), plan;
        plan.part[t[0]->va] = Part::REPLICATED;
        if (partOf(*t[1]) == Part::SHARDED) shard(out, op.name);
        else if (pass == 1 || partOf(*t[1]) == Part::REPLICATED) {
          plan.part[t[1]->va] = Part::REPLICATED;
          plan.part[out.va] = Part::REPLICATED;
        }
        continue;
      }
      if (op.name.rfind("fmatmul_", 0) == 0 && op.name.size() >= 11 && t.size() >= 3) {
        const bool tl = op.name[8] == 't', tr = op.name[10] == 't';
        const Part l = partOf(*t[0]), r = partOf(*t[1]);
        if (l != Part::SHARDED && r != Part::SHARDED) {
          if (pass == 1 || (l == Part::REPLICATED && r == Part::REPLICATED)) {
            plan.part[t[0]->va] = plan.part[t[1]->va] = Part::REPLICATED;
            for (size_t j = 2; j < t.size(); ++j) plan.part[t[j]->va] = Part::REPLICATED;
          }
        } else if (!tl && l == Part::SHARDED && r != Part::SHARDED) {
          // rows of the left operand are batch rows: the result is split the same way
          plan.part[t[1]->va] = Part::REPLICATED;
          for (size_t j = 2; j < t.size(); ++j) shard(*t[j], op.name);
        } else if (tl && !tr && l == Part::SHARDED && r != Part::REPLICATED) {
          // left stored [batch, m], right stored [batch, n]: the sum runs over the batch, so each
          // device holds a partial sum of the whole result
          shard(*t[1], op.name);
          if (op.name.size() > 11) return fail(op.name + ": a fused form over a batch contraction"), plan;
          plan.part[out.va] = Part::REPLICATED;
          plan.sumAfter[i] = true;
        } else {
          return fail(op.name + ": this combination of sharded operands is not a row split"), plan;
        }
        continue;
      }
      // whole-tensor builtins (fsoftmax, fpool, fconv2d, ftranspose, fslice, fsum ...): replicated only
      if (anySharded) return fail(op.name + ": not defined on a row split"), plan;
      if (pass == 1) {
        for (const Arg* a : t) plan.part[a->va] = Part::REPLICATED;
      }
    }
  }
  if (plan.ok) {
    for (auto& kv : plan.part)
      if (kv.second == Part::UNKNOWN) kv.second = Part::REPLICATED;
    known = plan.part;
  }
  return plan;
}

// Shape of a tensor on one device.
inline std::vector<uint64_t> localShape(const std::vector<uint64_t>& global, Part part, unsigned devices) {
  std::vector<uint64_t> s = global;
  if (part == Part::SHARDED && !s.empty()) s[0] /= devices;
  return s;
}

}  // namespace polar_b200::dp

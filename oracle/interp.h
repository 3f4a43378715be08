// TEST INFRASTRUCTURE, NOT PRODUCT CODE: CPU restatement of the reference interpreter and of
// its view-fused CPU evaluator. See interp.cc / realize.cc for the reference citations.
#pragma once
#include <vector>

#include "../kurumi_b200/csrc/core/graph.h"

namespace ko {

// One evaluated node. `wide` = the bytes hold f64 values although `dtype` names a narrower
// float (the "f64 interpreter run").
struct Val {
  ku::Shape shape;
  ku::DType dtype = ku::DType::F32;
  bool wide = false;
  std::vector<uint8_t> bytes;
};

uint64_t threefry2x32(uint64_t key, uint64_t counter);
float uniform_f32(uint64_t bits);

// Strict left fold of Sum / ReduceMax over `axis` of a row-major f32 buffer (interp/reduce.rs:67-84).
void reduce_f32(ku::OpKind k, const float* data, const ku::Shape& shape, size_t axis, float* out);
Val eval_op(const ku::Node& n, const std::vector<const Val*>& in, bool wide_mode);
ku::Tensor to_tensor(const Val& v);
std::vector<ku::Tensor> interpret_many(const ku::Graph& g, const std::vector<ku::NodeId>& ids, const ku::Feeds& feeds, bool wide_mode);

// kurumi_core/src/realize/eval.rs:22-27: the f32 view-fused evaluator, falling back to the
// interpreter when the graph leaves the fused path. `kernels` (optional) receives the number of
// passes over data, or -1 when the interpreter ran (realize/eval.rs:49-56).
ku::Tensor force(const ku::Graph& g, ku::NodeId id, const ku::Feeds& feeds, long* kernels);
// kurumi_core/src/realize/plan.rs:21-27: whether `root` can be compiled into a replayable plan (f32, fused ops, Inputs allowed).
bool plan_supported(const ku::Graph& g, ku::NodeId root);

}  // namespace ko

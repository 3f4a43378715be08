// Scheduler: walks a graph once and compiles it into a Program (buffer slots + kernel launches).
// The walk is the device analogue of kurumi_core/src/realize/sched.rs:32-104 and of the Metal
// backend's kurumi_metal/src/backend/eval_walk.rs:73-138: movement rewrites leaf views,
// elementwise ops grow one fused expression, and a reduction / softmax / contraction / attention
// / root is a kernel boundary. Differences that matter on a GPU: a contraction is left pending so
// the pointwise chain that consumes it becomes its epilogue; multi-consumer expressions are
// re-inlined into each consumer kernel instead of being written to memory; an op with no kernel
// is an error, never a CPU fallback.
#pragma once
#include <unordered_map>

#include "fuse.h"

namespace ku::cu {

struct PendingGemm {
  GemmDesc desc;
  int a_slot = -1, b_slot = -1;
  Shape out_shape;
  int result_slot = -1;  // set once the plain (un-fused) contraction has been emitted
  int uses = 0;          // dry run: kernels that read the accumulator
  bool fusable = true;   // dry run: every such kernel is a pointwise pass over the untouched result
};

class Scheduler {
 public:
  // `load` compiles a generated kernel (null = dry run: decide fusion only, emit nothing).
  // `plan` (from a dry run) says per pending contraction whether its consumer may become its epilogue.
  Scheduler(const KernelLoader* load, const Graph& g, int sm_count, const std::vector<bool>* plan);
  Program compile(const std::vector<NodeId>& roots);
  std::vector<bool> fuse_plan() const;

 private:
  bool dry() const { return load_ == nullptr; }
  int new_slot(Slot::Kind k, DType dt, const Shape& shape, NodeId node = 0);
  Fused buffer_value(int slot, DType dt, const Shape& shape) const;
  Fused value_of(NodeId id);
  Fused eval_node(NodeId id);
  Fused movement(const Node& n, Fused f);
  Fused elementwise(const Node& n, const std::vector<Fused>& in);
  Fused combine(OpKind op, DType dt, const std::vector<const Fused*>& in);
  Fused materialize(const Fused& f, int out_slot = -1);
  Fused resolve_acc(const Fused& f);
  int force_gemm(int id);
  Fused reduce(OpKind k, const Fused& f, size_t axis);
  Fused softmax(OpKind k, const Fused& f, size_t axis, float eps);
  Fused dot(const Node& n, const Fused& a, const Fused& b);
  Fused dot_general(DType dt, const Shape& out_shape, const Fused& a, const Fused& b, const std::vector<size_t>& lc,
                    const std::vector<size_t>& rc, const std::vector<size_t>& lb, const std::vector<size_t>& rb);
  Fused sdpa(const Node& n, const Fused& q, const Fused& k, const Fused& v);
  Fused attention(DType dt, const Shape& shape, bool causal, float scale, const Fused& q, const Fused& k, const Fused& v);
  // The decomposition Graph::sdpa records below its 1 GiB score-buffer threshold (kurumi_core/src/graph/ops/nn/attention.rs:97-113),
  // found again so that the same user call runs the same fused kernel at every size.
  struct SdpaMatch { NodeId q, k, v; bool causal; float scale; std::vector<NodeId> interior; };
  bool match_sdpa(NodeId id, SdpaMatch* m) const;
  Fused quant_matmul(const Node& n, const std::vector<Fused>& in);
  Fused indexing(const Node& n, const std::vector<Fused>& in);
  Fused dense(const Fused& f);   // the value in a contiguous buffer of its own layout (written out if it is not one already)
  Fused view_step(OpKind k, Fused f, const Shape& shape);
  Fused imm_value(const Shape& shape, DType dt, uint64_t bits) const;
  void emit_gemm(int id, const Fused* epi, int out_slot);
  void push_launch(const Emitted& e, const Fused& f, int out_slot, double flops = 0);
  void note_acc_use(const Fused& f, bool fusable_here);
  double leaf_bytes(const Fused& f) const;
  size_t op_nodes(const Fused& f) const;

  const KernelLoader* load_;
  const Graph& g_;
  int sm_;
  const std::vector<bool>* plan_;
  Program prog_;
  std::unordered_map<NodeId, Fused> memo_;
  std::unordered_map<NodeId, size_t> consumers_;
  std::vector<PendingGemm> gemms_;
  std::unordered_map<NodeId, SdpaMatch> sdpa_matches_;   // final dot_general of a recognised decomposition
  std::unordered_map<NodeId, bool> skipped_;             // interior nodes of those: never evaluated
};

// Compile `roots` of `g`: a dry run decides epilogue fusion, the second run emits kernels.
Program compile_program(Runtime& rt, const Graph& g, const std::vector<NodeId>& roots);
// Same walk without a device: every generated kernel is compiled to an sm_100a cubin by NVRTC and
// discarded. Returns the kernel family of each launch the program would issue.
std::vector<std::string> compile_check(const Graph& g, const std::vector<NodeId>& roots, int sm_count);

}  // namespace ku::cu

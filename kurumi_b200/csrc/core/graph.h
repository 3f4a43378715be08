// Graph IR: the closed primitive set, the append-only node arena, record-time dtype/shape
// inference, the op builders (surface ops decomposed to primitives) and the `amp` pass.
//
// Mirrors, for the primitives a device backend evaluates:
//   kurumi_core/src/graph/op.rs:12-127      Op / Node / NodeId
//   kurumi_core/src/graph.rs:29-112         arena, leaf builders, process-unique graph id
//   kurumi_core/src/graph/infer.rs:10-134   dtype and shape rules
//   kurumi_core/src/graph/check.rs:8-59     record-time guards (strict same-shape/same-dtype)
//   kurumi_core/src/graph/ops/**            builders / decompositions
//   kurumi_core/src/graph/pass/amp.rs:16-40 mixed-precision rewrite
//   kurumi_core/src/graph/inspect.rs:10-39  reachable (topological order)
#pragma once
#include <array>
#include <cstdint>
#include <memory>
#include <new>
#include <string>
#include <unordered_map>
#include <vector>

#include "dtype.h"

namespace ku {

using Shape = std::vector<size_t>;
using NodeId = uint32_t;

inline size_t numel(const Shape& s) { size_t n = 1; for (size_t d : s) n *= d; return n; }
std::string shape_str(const Shape& s);
std::vector<size_t> row_major_strides(const Shape& s);

// Host storage of tensors is obtained through two hooks, so that a device backend can hand out page-locked memory
// (a copy between such memory and the device runs at the full rate of the link and overlaps with kernels). The
// defaults are malloc and free. Elements are left uninitialised by resize(); assign(n, 0) still clears.
struct HostMem {
  static void* (*alloc)(size_t bytes);
  static void (*release)(void* p, size_t bytes);
  static void (*copy)(void* dst, const void* src, size_t bytes);   // large host-to-host copies (default: memcpy)
};
template <typename T>
struct HostAlloc {
  using value_type = T;
  HostAlloc() = default;
  template <typename U> HostAlloc(const HostAlloc<U>&) {}
  T* allocate(size_t n) {
    void* p = HostMem::alloc(n * sizeof(T));
    if (!p) throw std::bad_alloc();
    return static_cast<T*>(p);
  }
  void deallocate(T* p, size_t n) { HostMem::release(p, n * sizeof(T)); }
  template <typename U> void construct(U* p) noexcept { ::new (static_cast<void*>(p)) U; }
  template <typename U, typename... A> void construct(U* p, A&&... a) { ::new (static_cast<void*>(p)) U(std::forward<A>(a)...); }
  template <typename U> bool operator==(const HostAlloc<U>&) const { return true; }
  template <typename U> bool operator!=(const HostAlloc<U>&) const { return false; }
};
using Bytes = std::vector<uint8_t, HostAlloc<uint8_t>>;

// Host tensor (the reference's TensorVal): row-major, little-endian element bytes.
struct Tensor {
  Shape shape;
  DType dtype = DType::F32;
  Bytes bytes;
  size_t len() const { return bytes.size() / dtype_width(dtype); }
  template <typename T> const T* data() const { return reinterpret_cast<const T*>(bytes.data()); }
  template <typename T> T* data() { return reinterpret_cast<T*>(bytes.data()); }
  static Tensor make(DType dt, Shape shape) {
    Tensor t; t.dtype = dt; t.bytes.assign(std::max<size_t>(numel(shape), 0) * dtype_width(dt), 0); t.shape = std::move(shape); return t;
  }
  // storage left uninitialised: for results that are overwritten in full
  static Tensor make_uninit(DType dt, Shape shape) {
    Tensor t; t.dtype = dt; t.bytes.resize(numel(shape) * dtype_width(dt)); t.shape = std::move(shape); return t;
  }
  static Tensor from_f32(const float* p, size_t n, Shape shape) {
    Tensor t; t.dtype = DType::F32; t.shape = std::move(shape); t.bytes.resize(n * 4);
    if (n) std::memcpy(t.bytes.data(), p, n * 4);
    return t;
  }
};
using TensorPtr = std::shared_ptr<const Tensor>;

enum class OpKind : uint8_t {
  Const, Input, Iota, RandUniform, Cast, Bitcast, Detach,
  Add, Mul, Max, Neg, IDiv, And, Or, Xor, Shl, Shr, CmpLt, CmpEq, Where,
  Recip, Sqrt, Exp2, Log2, Sin, Floor,
  Sum, Prod, ReduceMax, Softmax, RmsNorm, Sdpa,
  Reshape, Permute, Expand, Slice, Flip, Pad, DotGeneral,
  QuantMatmul, ArgReduce,
  Gather, GatherAlong, Scatter, ScatterAlong, Argsort,
};
const char* op_name(OpKind k);
inline bool is_movement(OpKind k) { return k >= OpKind::Reshape && k <= OpKind::Pad; }
inline bool is_elementwise(OpKind k) { return (k >= OpKind::Cast && k <= OpKind::Floor); }

struct Op {
  OpKind kind = OpKind::Const;
  TensorPtr data;                              // Const
  Shape shape;                                 // Const/Input/Iota/RandUniform/Reshape/Expand target
  DType to = DType::F32;                       // Input/Iota dtype, Cast/Bitcast target
  size_t axis = 0;                             // Iota/Sum/Prod/ReduceMax/Softmax/RmsNorm
  float eps = 0.f;                             // RmsNorm
  bool causal = false;                         // Sdpa
  std::vector<size_t> perm;                    // Permute perm / Flip axes
  std::vector<std::array<size_t, 3>> ranges;   // Slice (start, end, step) / Pad (lo, hi, 0)
  std::vector<size_t> lc, rc, lb, rb;          // DotGeneral contract / batch axes
  uint8_t bits = 0;                            // QuantMatmul: 2, 4 or 8 bits per weight
  size_t group_size = 0;                       // QuantMatmul: weights per (scale, min) group along K
  bool symmetric = true;                       // QuantMatmul: no mins operand
  bool arg_min = false;                        // ArgReduce: index of the minimum instead of the maximum
  uint8_t combine = 0;                         // Scatter / ScatterAlong: 0 set, 1 add, 2 max, 3 min (kurumi_core/src/graph/op.rs:104-109)
  bool descending = false;                     // Argsort
};

struct Node {
  Op op;
  DType dtype;
  std::vector<NodeId> src;
  Shape shape;
};

class Graph {
 public:
  Graph();
  uint64_t id() const { return id_; }
  size_t size() const { return nodes_.size(); }
  const Node& node(NodeId i) const;   // throws on a bad id
  DType dtype(NodeId i) const { return node(i).dtype; }
  const Shape& shape(NodeId i) const { return node(i).shape; }

  // leaves
  NodeId constant(Tensor t);
  NodeId constant_f32(std::vector<float> v, Shape shape);
  NodeId input(Shape shape, DType dt);
  NodeId iota(Shape shape, size_t axis, DType dt);
  NodeId rand_uniform(Shape shape, uint64_t seed);
  NodeId rand_uniform_keyed(Shape shape, NodeId seed);
  NodeId cast(NodeId a, DType to);
  NodeId bitcast(NodeId a, DType to);
  NodeId detach(NodeId a);
  // primitives
  NodeId add(NodeId a, NodeId b);
  NodeId mul(NodeId a, NodeId b);
  NodeId max(NodeId a, NodeId b);
  NodeId neg(NodeId a);
  NodeId recip(NodeId a);
  NodeId sqrt(NodeId a);
  NodeId exp2(NodeId a);
  NodeId log2(NodeId a);
  NodeId sin(NodeId a);
  NodeId floor(NodeId a);
  NodeId idiv(NodeId a, NodeId b);
  NodeId shl(NodeId a, NodeId b);
  NodeId shr(NodeId a, NodeId b);
  NodeId bit_and(NodeId a, NodeId b);
  NodeId bit_or(NodeId a, NodeId b);
  NodeId bit_xor(NodeId a, NodeId b);
  NodeId cmp_lt(NodeId a, NodeId b);
  NodeId cmp_eq(NodeId a, NodeId b);
  NodeId select(NodeId cond, NodeId a, NodeId b);
  NodeId sum(NodeId a, size_t axis);
  NodeId prod(NodeId a, size_t axis);
  NodeId reduce_max(NodeId a, size_t axis);
  NodeId softmax(NodeId a, size_t axis);
  NodeId argmax(NodeId a, size_t axis);   // I64 index of the first maximum along the axis
  NodeId argmin(NodeId a, size_t axis);
  NodeId rmsnorm(NodeId a, size_t axis, float eps);
  // indexing along one axis (kurumi_core/src/graph/ops/core/indexing.rs:21-123): out-of-range indices are clamped by the
  // gathers and dropped by the scatters; updates fold into the operand in index order
  NodeId gather(NodeId operand, NodeId indices, size_t axis);          // out = operand[..axis] ++ indices.shape ++ operand[axis+1..]
  NodeId gather_along(NodeId operand, NodeId indices, size_t axis);    // out = indices.shape, one index per position
  NodeId scatter(NodeId operand, NodeId indices, NodeId updates, size_t axis, uint8_t combine);
  NodeId scatter_along(NodeId operand, NodeId indices, NodeId updates, size_t axis, uint8_t combine);
  NodeId argsort(NodeId a, size_t axis, bool descending);              // I64 permutation per line, stable
  NodeId sort(NodeId a, size_t axis, bool descending);                 // gather_along(a, argsort(a))
  NodeId reshape(NodeId a, Shape shape);
  NodeId permute(NodeId a, std::vector<size_t> perm);
  NodeId expand(NodeId a, Shape shape);
  NodeId slice_step(NodeId a, std::vector<std::array<size_t, 3>> ranges);
  NodeId flip(NodeId a, std::vector<size_t> axes);
  NodeId pad(NodeId a, std::vector<std::array<size_t, 2>> pads);
  NodeId dot_general(NodeId a, NodeId b, std::vector<size_t> lc, std::vector<size_t> rc, std::vector<size_t> lb,
                     std::vector<size_t> rb);
  NodeId sdpa_fused(NodeId q, NodeId k, NodeId v, bool causal);
  // weight-only quantised matmul: act [M, K] x dequant(qweight) [N, K]^T -> [M, N] in act's dtype; `mins` absent = symmetric
  NodeId quant_matmul(NodeId act, NodeId qweight, NodeId scales, const NodeId* mins, uint8_t bits, size_t group_size);
  // decompositions
  NodeId scalar(NodeId like, float v);
  NodeId sub(NodeId a, NodeId b);
  NodeId div(NodeId a, NodeId b);
  NodeId abs(NodeId a);
  NodeId square(NodeId a);
  NodeId min(NodeId a, NodeId b);
  NodeId clamp_min(NodeId a, float lo);
  NodeId exp(NodeId a);
  NodeId ln(NodeId a);
  NodeId cos(NodeId a);
  NodeId sigmoid(NodeId a);
  NodeId tanh(NodeId a);
  NodeId relu(NodeId a);
  NodeId silu(NodeId a);
  NodeId gelu(NodeId a);
  NodeId logical_not(NodeId a);
  NodeId gt(NodeId a, NodeId b);
  NodeId ge(NodeId a, NodeId b);
  NodeId le(NodeId a, NodeId b);
  NodeId ne(NodeId a, NodeId b);
  NodeId mean(NodeId a, size_t axis);
  NodeId reduce_min(NodeId a, size_t axis);
  NodeId transpose(NodeId a, size_t i, size_t j);
  NodeId broadcast_to(NodeId a, Shape shape);
  NodeId slice(NodeId a, std::vector<std::array<size_t, 2>> ranges);
  NodeId randn(Shape shape, uint64_t seed);
  NodeId rand_range(Shape shape, uint64_t seed, float lo, float hi);
  NodeId sdpa(NodeId q, NodeId k, NodeId v, bool causal);
  NodeId sdpa_decomposed(NodeId q, NodeId k, NodeId v, bool causal);

  NodeId push(Op op, std::vector<NodeId> src);  // inference only, no checks (used by passes)

 private:
  void same_shape(const char* op, NodeId a, NodeId b) const;
  void same_dtype(const char* op, NodeId a, NodeId b) const;
  void require(const char* op, NodeId a, bool ok, const char* want) const;
  NodeId bin(const char* name, OpKind k, NodeId a, NodeId b);
  NodeId unary_float(const char* name, OpKind k, NodeId a, bool allow_complex);
  void reduce_axis_ok(const char* op, NodeId a, size_t axis) const;
  NodeId causal_bias(size_t s, const Shape& out_shape);
  DType infer_dtype(const Op& op, const std::vector<NodeId>& src) const;
  Shape derive_shape(const Op& op, const std::vector<NodeId>& src) const;

  std::vector<Node> nodes_;
  uint64_t id_;
};

std::vector<size_t> free_axes(size_t rank, const std::vector<size_t>& batch, const std::vector<size_t>& contract);
std::vector<NodeId> reachable(const Graph& g, const std::vector<NodeId>& roots);
std::string dump(const Graph& g, NodeId root);

// Mixed-precision rewrite. `amp(g, root)` is the reference pass: each F32 DotGeneral runs with
// operands cast to F16 and its result cast back to F32. `amp_to` generalises the target:
//  * F16 / BF16: same rewrite with that dtype.
//  * F8E4M3: every F32/BF16/F16 DotGeneral gets each operand quantised through
//    cast(cast(x, F8E4M3), dt) unless the operand already is a Cast from F8E4M3; the contraction
//    keeps its dtype (so the f32 accumulation and the result rounding are unchanged). A backend
//    that sees both operands as casts from F8E4M3 may feed the fp8 bytes to its tensor cores:
//    the products are the same numbers.
NodeId amp(Graph& g, NodeId root);
NodeId amp_to(Graph& g, NodeId root, DType target);

// Group-wise weight quantisation for quant_matmul (kurumi_core/src/quant.rs:38-88): w is [rows, cols] f32,
// packed receives rows * cols * bits / 8 bytes (fields of a byte fill from its low bits), scales and mins one
// f16 per [row, group]; symmetric: w ~ q * scale with q a signed field, else w ~ q * scale + min with q unsigned.
void quantize(const float* w, size_t rows, size_t cols, uint8_t bits, size_t group_size, bool symmetric, uint8_t* packed, uint16_t* scales, uint16_t* mins);
// The f32 weights a quantised operand stands for (kurumi_core/src/quant.rs:90-113).
std::vector<float> dequantize(const uint8_t* packed, const uint16_t* scales, const uint16_t* mins, size_t rows, size_t cols, uint8_t bits, size_t group_size);

// Cast a host buffer through f64 (kurumi_core/src/dtype/convert.rs:14-47).
Tensor cast_tensor(const Tensor& src, DType to);

using Feeds = std::unordered_map<NodeId, TensorPtr>;

// The evaluation seam (kurumi_core/src/backend.rs:14-31).
class Backend {
 public:
  virtual ~Backend() = default;
  virtual const char* name() const = 0;
  virtual Tensor eval_with(const Graph& g, NodeId id, const Feeds& feeds) = 0;
  virtual std::vector<Tensor> eval_many_with(const Graph& g, const std::vector<NodeId>& ids, const Feeds& feeds) {
    std::vector<Tensor> out;
    for (NodeId id : ids) out.push_back(eval_with(g, id, feeds));
    return out;
  }
  Tensor eval(const Graph& g, NodeId id) { return eval_with(g, id, Feeds{}); }
};

// Each library that embeds the C ABI defines this (the CUDA library accepts only KU_CUDA).
std::unique_ptr<Backend> make_backend(uint32_t kind);
// ... and this: the backend behind ku_plan_compile, which takes no backend argument (kurumi/src/capi/eval.rs:152-168):
// compiles whatever can be compiled ahead of the first run and returns the backend that replays it, or null (with the
// reason in the last-error string) when `root` is off this library's compile-once path.
std::shared_ptr<Backend> plan_backend(const Graph& g, NodeId root);

}  // namespace ku

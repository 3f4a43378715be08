// The fused-expression IR of the CUDA backend and the compiled form of a graph evaluation.
//
// A graph value is held as a `Fused`: a small DAG of elementwise nodes over leaves, where each
// leaf reads a device buffer (or an immediate, an iota, a counter-based random draw, or the
// accumulator of a pending GEMM) through a strided View of the value's logical shape. Movement
// ops only rewrite the leaf views; elementwise ops grow the DAG; a reduction, softmax,
// contraction, attention or the root turns the DAG into one generated kernel. This is the
// device counterpart of kurumi_core/src/realize/expr.rs:47-63 (`Expr` / `Repr`) and of the Metal
// backend's kurumi_metal/src/backend/fuse.rs:59-98 (`Val::Fused`, `Leaf`, `FExpr`), designed
// around sharing (the DAG is hash-consed, so gelu's repeated `x` is one register) rather than
// re-inlining trees.
#pragma once
#include <functional>
#include <string>
#include <vector>

#include "../lower/view.h"
#include "runtime.h"

namespace ku::cu {

enum class LeafKind : uint8_t { Buffer, Imm, Iota, Rand, Acc };

struct Leaf {
  LeafKind kind = LeafKind::Buffer;
  DType dtype = DType::F32;
  View view;
  int slot = -1;        // Buffer: data slot. Rand: slot of the seed tensor, or -1 for an immediate seed
  uint64_t imm = 0;     // Imm: element bit pattern. Rand: the seed
  DType seed_dtype = DType::I64;
  int64_t iota_stride = 1, iota_len = 1;  // Iota: value = (flat / iota_stride) % iota_len
  int gemm = -1;        // Acc: id of the pending contraction
  bool same(const Leaf& o) const {
    return kind == o.kind && dtype == o.dtype && slot == o.slot && imm == o.imm && iota_stride == o.iota_stride &&
           iota_len == o.iota_len && gemm == o.gemm && seed_dtype == o.seed_dtype && view == o.view;
  }
};

// op == OpKind::Input marks a leaf load; every other op is the graph primitive of that name.
struct FNode {
  OpKind op = OpKind::Input;
  DType dtype = DType::F32;
  int in[3] = {-1, -1, -1};
  int leaf = -1;
};

struct Fused {
  Shape shape;
  std::vector<FNode> nodes;  // topological: inputs precede users
  std::vector<Leaf> leaves;
  int root = -1;
  DType dtype() const { return nodes[root].dtype; }
  // A bare load of an unguarded buffer leaf (no arithmetic)?
  bool is_plain_buffer() const { return nodes[root].op == OpKind::Input && leaves[nodes[root].leaf].kind == LeafKind::Buffer; }
  const Leaf& root_leaf() const { return leaves[nodes[root].leaf]; }
};

int add_leaf(Fused& f, const Leaf& l);
int add_node(Fused& f, const FNode& n);                 // hash-consed
int import_expr(Fused& dst, const Fused& src, int node); // copy src's sub-DAG into dst, deduplicated
Fused fused_leaf(const Shape& shape, const Leaf& l);

// ---- compiled program ---------------------------------------------------------------------------
struct Slot {
  enum Kind : uint8_t { Const, Feed, Temp, Out } kind = Temp;
  size_t bytes = 0;
  NodeId node = 0;     // Const / Feed: the graph node
  DType dtype = DType::F32;
  Shape shape;
  bool zero_init = false;   // Temp: cleared once, when the slot's memory is allocated
};

struct TmapSpec {  // a tensor map over a slot, encoded once the slot's address is known
  int slot = -1;
  int64_t byte_offset = 0;
  CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_UINT8;
  unsigned rank = 0;
  uint64_t dims[5] = {0, 0, 0, 0, 0};
  uint64_t strides[5] = {0, 0, 0, 0, 0};
  uint32_t box[5] = {0, 0, 0, 0, 0};
  CUtensorMapSwizzle swz = CU_TENSOR_MAP_SWIZZLE_NONE;
};

struct Arg {
  // Status: the backend's device status word. Epoch: a 32-bit count of this launch's issues (1 on the first), for
  // kernels whose scratch words carry the parity of the launch that wrote them
  enum Kind : uint8_t { SlotPtr, Bytes, Tmap, Status, Epoch } kind = SlotPtr;
  int slot = -1;
  int64_t byte_offset = 0;
  std::vector<uint8_t> bytes;
  TmapSpec tm;
};

struct Launch {
  std::string name;      // kernel family, for stats and profiles
  Kernel kernel;
  unsigned grid[3] = {1, 1, 1}, block[3] = {1, 1, 1}, cluster[3] = {1, 1, 1};
  unsigned smem = 0;
  int persistent_clusters = 0;  // -1: cap grid[0] at the co-resident cluster count (x cluster size) on first launch; > 0: done
  unsigned grid_multiple = 1;   // with persistent_clusters: the capped grid is rounded down to a multiple of this (CTA groups)
  bool cooperative = false;     // launch with the cooperative attribute: all CTAs co-resident, or the launch fails
  bool status_arg = false;      // append the backend's device status word as the last kernel parameter
  // When set, the step is a precompiled (nvcc-built) kernel sequence: the backend resolves the SlotPtr
  // arguments and calls this instead of launching `kernel`.
  std::function<void(const std::vector<void*>& ptrs, cudaStream_t stream)> host_launch;
  std::vector<Arg> args;
  int zero_slot = -1;       // when >= 0: the first zero_bytes of this slot are set to fill_byte on the stream before the launch
  size_t zero_bytes = 0;
  int fill_byte = 0;
  double algo_bytes = 0, flops = 0;  // algorithmic traffic / work of this launch
  uint32_t epoch = 0;       // how many times this launch has been issued (Arg::Epoch)
};

struct Program {
  std::vector<Slot> slots;
  std::vector<Launch> launches;
  std::vector<int> out_slots;   // one per requested root
  size_t graph_nodes = 0;
};

// Compiles (or fetches from a cache) one entry point of a generated source.
using KernelLoader = std::function<Kernel(const std::string& source, const std::string& entry, bool fmad)>;

// ---- source emission (emit.cc, emit_index.cc) ------------------------------------------------------------------
struct Emitted {
  std::string source, entry;
  std::vector<int> leaf_args;  // kernel pointer parameters, in order: leaf indices (then the output pointer)
  unsigned grid = 1, block = 256, smem = 0;
  unsigned cluster = 1;
  bool fmad = false;
  std::string family;
};

// One pass writing `f` row-major into a contiguous output of f.dtype().
Emitted emit_pointwise(const Fused& f, int sm_count);
// Sum / Prod / ReduceMax over `axis` of `f`; output is row-major over the remaining axes.
Emitted emit_reduce(const Fused& f, OpKind kind, size_t axis, int sm_count);
// I64 index of the first maximum / minimum of `f` along `axis` (one thread per output, index order).
Emitted emit_arg_reduce(const Fused& f, size_t axis, bool arg_min, int sm_count);
// Softmax / RmsNorm over `axis` of `f`; output has f's shape, row-major.
Emitted emit_softmax(const Fused& f, OpKind kind, size_t axis, float eps, int sm_count);

// Indexing along one axis and per-line sorting over contiguous buffers (kernel parameters: see emit_index.cc).
Emitted emit_gather(DType d, DType idx_dt, int64_t pre, int64_t da, int64_t post, int64_t k, int sm_count);
Emitted emit_gather_along(DType d, DType idx_dt, int64_t outer, int64_t da, int64_t la, int64_t inner, int sm_count);
Emitted emit_scatter(DType d, DType idx_dt, bool along, uint8_t combine, int64_t pre, int64_t da, int64_t post, int64_t k, int sm_count);
// The same for longer lines: four entry points over a padded copy in global scratch (see emit_index.cc)
Emitted emit_argsort_long(DType d, bool descending, int64_t outer, int64_t len, int64_t inner, int64_t* lpad_out, size_t* key_bytes_out);
Emitted emit_argsort(DType d, bool descending, int64_t outer, int64_t len, int64_t inner, int sm_count);

struct GemmDesc {
  DType dtype = DType::F32;       // operand / result dtype of the DotGeneral
  int64_t batch = 1, m = 0, n = 0, k = 0;
  int64_t a_bs = 0, a_ms = 0, a_ks = 0, a_base = 0;  // element strides of A[batch, m, k]
  int64_t b_bs = 0, b_ks = 0, b_ns = 0, b_base = 0;  // element strides of B[batch, k, n]
  DType in_dtype = DType::F32;    // storage dtype of the operands actually read (F8E4M3 when both are casts from fp8)
};
// C[batch, m, n] = epilogue(round_to_dtype(sum_k A*B)); `epi` (may be null) is a Fused over shape
// [batch, m, n] (collapsed to 3-D) containing one Acc leaf. SIMT kernel, any numeric dtype.
Emitted emit_gemm_simt(const GemmDesc& g, const Fused* epi, int sm_count);

// For the hand-written line kernels: when `f` collapses to [R lines, C positions] with the softmax axis
// last, generates `float ku_src(i, j, pointers)` (the fused producer) plus the KU_SRC_* / KU_ENC glue
// and reports whether the reads are transposed (contiguous across lines, strided along a line).
// `big` (optional) receives the one dominant f32 leaf that a TMA pipeline can stream (leaf = -1 if
// there is none); then `ku_src_t(lval, i, j, pointers)` is generated too, taking that leaf's value.
struct LineLeaf { int leaf = -1; int64_t ld = 0, base = 0; bool identity = false; };
bool emit_line_source_fn(const Fused& f, size_t axis, std::string* src, std::vector<int>* leaf_args, int64_t* R, int64_t* C, bool* transposed, LineLeaf* big = nullptr);

// Shared pieces the hand-written kernel templates splice in (prelude + the per-element epilogue).
std::string device_prelude();
std::string emit_epilogue_fn(const Fused* epi, DType acc_dtype, std::vector<int>* leaf_args);
const char* ctype(DType d);     // register type of a value
const char* stype(DType d);     // storage type of a value

}  // namespace ku::cu

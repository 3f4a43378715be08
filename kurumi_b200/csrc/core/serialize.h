// KGPH v2 graph blobs: the wire format a host hands a backend so that it can run a recorded graph
// without re-recording it through the builders.
//
// Format (kurumi_core/src/graph/serialize/encode.rs:81-111, encode/op.rs:8-170, little-endian):
//   "KGPH" u8 version(=2) u32 node_count
//   per node: u8 op tag, the op's attributes, u32 src_count, src ids (u32, each < the node's own id)
//   u32 entry_count; per entry: str name, u32 n_out, out ids, u32 n_in, per input: u32 node, u8 role, str name
// with usize as u64, vectors as u32 length + items, str as u32 length + UTF-8, dtypes as the C ABI tags,
// Const storage as dtype, u64 byte count, bytes. Op tags are the reference's; the primitives this
// library does not evaluate (tags 41..54) are refused with a clear error on read.
// The reader mirrors kurumi_core/src/graph/serialize/decode.rs:23-88 (bad magic, version, truncated
// blobs, forward source references, under- or over-filled Const payloads are errors, never crashes).
#pragma once
#include <string>
#include <vector>

#include "graph.h"

namespace ku {

struct InputBinding {
  NodeId node = 0;
  uint8_t role = 1;   // 0 = weight (bound by name), 1 = runtime feed
  std::string name;
};
struct Entry {
  std::string name;
  std::vector<NodeId> outputs;
  std::vector<InputBinding> inputs;
};
struct Runnable {
  std::unique_ptr<Graph> graph;
  std::vector<Entry> entries;   // at least one; entry 0 is "the" entry of a single-entry blob
};

// the whole arena in id order, one entry named ""
std::vector<uint8_t> serialize_graph(const Graph& g, const std::vector<NodeId>& outputs, const std::vector<InputBinding>& inputs);
// only the nodes the outputs depend on, renumbered densely; bindings of dropped nodes are omitted
std::vector<uint8_t> serialize_reachable(const Graph& g, const std::vector<NodeId>& outputs, const std::vector<InputBinding>& inputs);
// several named entries over the union of their cones
std::vector<uint8_t> serialize_multi(const Graph& g, const std::vector<Entry>& entries);
// throws ku::Error on a malformed blob or one without entries
Runnable deserialize_graph(const uint8_t* bytes, size_t len);

}  // namespace ku

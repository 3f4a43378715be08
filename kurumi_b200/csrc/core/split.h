// Row splitting of an evaluation: the graph whose root yields rows [c, c + 1) * rows / parts of the original
// root, given the matching slices of the inputs it depends on row-wise and all of the others.
//
// Every benchmark graph of this backend is a set of independent output rows (rows of x and y for the fused
// reduce, softmax lines, rows of A for a contraction with B shared, batch x heads for attention). The
// analysis walks from the root down and asks of every node "which of your axes carries the root's row
// index?": elementwise ops pass the axis on, movement ops map it, a reduction / softmax / contraction along
// another axis keeps it, an Expand from extent 1 ends it (the operand below is needed whole). It fails, with
// the reason, on anything that mixes rows (a reduction or softmax along the split axis, a causal attention
// split over its queries, an iota or a random draw along it, a slice / flip / pad of it, a constant that would
// have to be cut). The same part graph serves every part: only the input slices differ.
//
// Used by the CUDA backend to pipeline host-buffer evaluations chunk by chunk (upload, kernels and download
// overlapped) and to shard one evaluation across the GPUs of a box. The reference evaluates a graph in one
// piece on one device (kurumi_core/src/backend.rs:14-31), so this file has no counterpart there.
#pragma once
#include <string>
#include <vector>

#include "graph.h"

namespace ku {

struct SplitInput {
  NodeId orig = 0;   // Input node of the original graph
  NodeId part = 0;   // the matching Input node of the part graph
  int axis = -1;     // axis cut into `parts` equal slices, or -1: every part needs all of it
};

struct SplitPlan {
  Graph graph;       // recorded at the part's shapes
  NodeId root = 0;
  size_t parts = 1;
  std::vector<SplitInput> inputs;   // in the original graph's node order
};

// Split `root` of `g` along its axis 0 into `parts` equal parts. Returns false (and the reason in *why) when the
// evaluation does not separate by rows or the extents do not divide.
bool row_split(const Graph& g, NodeId root, size_t parts, SplitPlan* out, std::string* why);

}  // namespace ku

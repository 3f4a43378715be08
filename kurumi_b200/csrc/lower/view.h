// Strided read patterns: the view-fused IR the CUDA emitter consumes.
//
// A View maps an output coordinate to a flat source index: base + sum(coord[d] * stride[d]),
// with optional per-axis validity guards produced by Pad (outside the guard the read yields 0).
// It plays the role of kurumi_core/src/lower/index.rs:20-36 (`View {shape, offset, guards}`) and
// its movement algebra kurumi_core/src/lower/index/movement.rs:10-118; where the reference keeps a
// symbolic offset and extracts affine coefficients later (lower/sym/expr.rs:93-107), this keeps
// the coefficients directly, which is all a device kernel needs.
#pragma once
#include <array>
#include <cstdint>
#include <vector>

#include "../core/graph.h"

namespace ku {

struct Guard {
  size_t axis;
  int64_t lo, hi;  // valid iff lo <= coord[axis] < hi
  bool operator==(const Guard& o) const { return axis == o.axis && lo == o.lo && hi == o.hi; }
};

struct View {
  Shape shape;
  std::vector<int64_t> stride;
  int64_t base = 0;
  std::vector<Guard> guards;

  static View source(const Shape& s);
  bool is_contiguous() const;  // base 0, row-major strides, no guards
  bool operator==(const View& o) const { return shape == o.shape && stride == o.stride && base == o.base && guards == o.guards; }

  // Movement algebra. All require an unguarded view except `pad` composing onto itself is not
  // supported either: callers materialise a guarded value first (as the reference does,
  // kurumi_core/src/realize/sched.rs:117-125).
  View permute(const std::vector<size_t>& perm) const;
  View expand(const Shape& to) const;
  View slice(const std::vector<std::array<size_t, 3>>& ranges) const;
  View flip(const std::vector<size_t>& axes) const;
  View pad(const std::vector<std::array<size_t, 3>>& pads) const;
  // False when the strides do not allow the regrouping (the caller then materialises).
  bool reshape(const Shape& to, View* out) const;

  // Smallest / largest flat index the view can touch (inside its guards), for bounds checks.
  void extent(int64_t* lo, int64_t* hi) const;
};

}  // namespace ku

#include "view.h"

#include <algorithm>

namespace ku {

View View::source(const Shape& s) {
  View v;
  v.shape = s;
  auto st = row_major_strides(s);
  v.stride.assign(st.begin(), st.end());
  return v;
}

bool View::is_contiguous() const {
  if (base != 0 || !guards.empty()) return false;
  int64_t expect = 1;
  for (size_t d = shape.size(); d-- > 0;) {
    if (shape[d] != 1 && stride[d] != expect) return false;
    expect *= static_cast<int64_t>(shape[d]);
  }
  return true;
}

View View::permute(const std::vector<size_t>& perm) const {
  View o;
  o.base = base;
  for (size_t p : perm) { o.shape.push_back(shape[p]); o.stride.push_back(stride[p]); }
  return o;
}

View View::expand(const Shape& to) const {
  View o = *this;
  o.shape = to;
  for (size_t d = 0; d < shape.size(); ++d)
    if (shape[d] == 1 && to[d] != 1) o.stride[d] = 0;  // a broadcast axis contributes nothing
  return o;
}

View View::slice(const std::vector<std::array<size_t, 3>>& r) const {
  View o;
  o.base = base;
  for (size_t d = 0; d < shape.size(); ++d) {
    o.shape.push_back((r[d][1] - r[d][0] + r[d][2] - 1) / r[d][2]);
    o.stride.push_back(stride[d] * static_cast<int64_t>(r[d][2]));
    o.base += stride[d] * static_cast<int64_t>(r[d][0]);
  }
  return o;
}

View View::flip(const std::vector<size_t>& axes) const {
  View o = *this;
  for (size_t ax : axes) {
    o.base += stride[ax] * (static_cast<int64_t>(shape[ax]) - 1);
    o.stride[ax] = -stride[ax];
  }
  return o;
}

View View::pad(const std::vector<std::array<size_t, 3>>& pads) const {
  View o;
  o.base = base;
  o.stride = stride;
  for (size_t d = 0; d < shape.size(); ++d) {
    const size_t lo = pads[d][0], hi = pads[d][1];
    o.shape.push_back(lo + shape[d] + hi);
    o.base -= stride[d] * static_cast<int64_t>(lo);
    if (lo || hi) o.guards.push_back({d, static_cast<int64_t>(lo), static_cast<int64_t>(lo + shape[d])});
  }
  return o;
}

bool View::reshape(const Shape& ns, View* out) const {
  std::vector<int64_t> nst(ns.size(), 0);
  const size_t on = shape.size(), nn = ns.size();
  if (numel(shape) == 0) { *out = View::source(ns); return true; }
  size_t oi = 0, ni = 0;
  while (oi < on && ni < nn) {
    size_t op = shape[oi], np = ns[ni];
    size_t oj = oi + 1, nj = ni + 1;
    while (op != np) {
      if (op < np) { if (oj >= on) return false; op *= shape[oj++]; }
      else { if (nj >= nn) return false; np *= ns[nj++]; }
    }
    // the old axes [oi, oj) must form one evenly strided run (size-1 axes are free)
    int64_t run_stride = 0;
    bool have = false;
    int64_t expect = 0;
    for (size_t k = oj; k-- > oi;) {
      if (shape[k] == 1) continue;
      if (!have) { run_stride = stride[k]; expect = run_stride * static_cast<int64_t>(shape[k]); have = true; }
      else { if (stride[k] != expect) return false; expect *= static_cast<int64_t>(shape[k]); }
    }
    int64_t s = have ? run_stride : 0;
    for (size_t k = nj; k-- > ni;) { nst[k] = ns[k] == 1 ? 0 : s; s *= static_cast<int64_t>(ns[k]); }
    oi = oj; ni = nj;
  }
  while (oi < on) if (shape[oi++] != 1) return false;
  while (ni < nn) { if (ns[ni] != 1) return false; nst[ni++] = 0; }
  out->shape = ns;
  out->stride = nst;
  out->base = base;
  out->guards.clear();
  return true;
}

void View::extent(int64_t* lo, int64_t* hi) const {
  int64_t mn = base, mx = base;
  for (size_t d = 0; d < shape.size(); ++d) {
    int64_t c_lo = 0, c_hi = static_cast<int64_t>(shape[d]) - 1;
    for (const Guard& g : guards)
      if (g.axis == d) { c_lo = std::max(c_lo, g.lo); c_hi = std::min(c_hi, g.hi - 1); }
    if (c_hi < c_lo) continue;
    const int64_t a = stride[d] * c_lo, b = stride[d] * c_hi;
    mn += std::min(a, b);
    mx += std::max(a, b);
  }
  *lo = mn;
  *hi = mx;
}

}  // namespace ku

// TEST INFRASTRUCTURE, NOT PRODUCT CODE. Nothing under kurumi_b200/ may call into this file.
//
// CPU restatement of kurumi_core's reference interpreter (the correctness oracle of the
// reference) for the primitives the CUDA backend evaluates. Each function cites the reference
// file:line it follows. Two modes:
//   * native: every tensor is held in its own dtype and every primitive rounds like the
//     reference does (f32 arithmetic without FMA contraction, low-precision floats computed
//     in f32 and rounded after every primitive, integers wrapping).
//   * wide ("f64 interpreter run"): every float tensor is held in f64 and all float arithmetic
//     is f64; only an explicit Cast to a narrower float dtype rounds (to that format). This is
//     the yardstick the bf16 / fp8 GEMM and attention tolerances are stated against.
//
// Arithmetic that lives in third-party crates absent from the reference tree:
//   half 2.7.1 (bf16/f16 conversions)  -> restated as IEEE round-to-nearest-even
//   float8 0.7.0 (fp8 conversions)     -> restated as RNE + saturate-to-finite (e4m3 "fn")
//   gemm 0.19.0 (f32 sgemm)            -> stand-in: plain f32 loop, k ascending
// The reference's own tests pin those only at exactly representable values and through
// tolerances, so for rounding mode / summation order: parity unpinned.
#include "interp.h"

#include <algorithm>
#include <cmath>
#include <limits>
#include <unordered_map>

namespace ko {
using namespace ku;

// kurumi_core/src/rng.rs:10-26 (threefry2x32, 20 rounds, key injection every 4)
uint64_t threefry2x32(uint64_t key, uint64_t counter) {
  static const uint32_t ROT[8] = {13, 15, 26, 6, 17, 29, 16, 24};
  uint32_t k0 = static_cast<uint32_t>(key), k1 = static_cast<uint32_t>(key >> 32);
  uint32_t ks[3] = {k0, k1, 0x1BD11BDAu ^ k0 ^ k1};
  uint32_t x0 = static_cast<uint32_t>(counter) + ks[0], x1 = static_cast<uint32_t>(counter >> 32) + ks[1];
  for (uint32_t r = 0; r < 20; ++r) {
    x0 += x1;
    uint32_t s = ROT[r % 8];
    x1 = (x1 << s) | (x1 >> (32 - s));
    x1 ^= x0;
    if (r % 4 == 3) {
      uint32_t inj = r / 4 + 1;
      x0 += ks[inj % 3];
      x1 += ks[(inj + 1) % 3] + inj;
    }
  }
  return static_cast<uint64_t>(x0) | (static_cast<uint64_t>(x1) << 32);
}
// kurumi_core/src/rng.rs:29-31
float uniform_f32(uint64_t bits) { return static_cast<float>(static_cast<uint32_t>(bits) >> 8) / 16777216.0f; }

namespace {

// kurumi_core/src/layout.rs:18-27
inline void inc(std::vector<size_t>& coord, const Shape& shape) {
  for (size_t i = coord.size(); i-- > 0;) {
    if (++coord[i] < shape[i]) return;
    coord[i] = 0;
  }
}

size_t esize(const Val& v) { return v.wide ? 8 : dtype_width(v.dtype); }

Val make_val(DType dt, Shape shape, bool wide) {
  Val v;
  v.dtype = dt;
  v.wide = wide;
  v.shape = std::move(shape);
  v.bytes.assign(std::max<size_t>(numel(v.shape), 0) * (wide ? 8 : dtype_width(dt)), 0);
  return v;
}

// ---- per-dtype element traits: S = storage type, C = compute type -----------------------------
template <DType D> struct E;
#define KO_PLAIN(D, T) \
  template <> struct E<DType::D> { using S = T; using C = T; static C ld(S s) { return s; } static S st(C c) { return c; } };
KO_PLAIN(U8, uint8_t) KO_PLAIN(U16, uint16_t) KO_PLAIN(U32, uint32_t) KO_PLAIN(U64, uint64_t)
KO_PLAIN(I8, int8_t) KO_PLAIN(I16, int16_t) KO_PLAIN(I32, int32_t) KO_PLAIN(I64, int64_t)
KO_PLAIN(F32, float) KO_PLAIN(F64, double)
template <> struct E<DType::BOOL> { using S = uint8_t; using C = uint8_t; static C ld(S s) { return s; } static S st(C c) { return c; } };
// kurumi_core/src/dtype/traits/float.rs:134-161: upcast to f32, compute, round back
template <> struct E<DType::BF16> { using S = uint16_t; using C = float; static C ld(S s) { return bf16_to_f32(s); } static S st(C c) { return f32_to_bf16(c); } };
template <> struct E<DType::F16> { using S = uint16_t; using C = float; static C ld(S s) { return f16_to_f32(s); } static S st(C c) { return f32_to_f16(c); } };
template <> struct E<DType::F8E4M3> { using S = uint8_t; using C = float; static C ld(S s) { return e4m3_to_f32(s); } static S st(C c) { return f32_to_e4m3(c); } };
template <> struct E<DType::F8E5M2> { using S = uint8_t; using C = float; static C ld(S s) { return e5m2_to_f32(s); } static S st(C c) { return f32_to_e5m2(c); } };

#define KO_CASE(D, ...) case DType::D: { constexpr DType DT = DType::D; (void)DT; __VA_ARGS__; break; }
#define KO_FLOATS(dt, ...) \
  switch (dt) { KO_CASE(F8E4M3, __VA_ARGS__) KO_CASE(F8E5M2, __VA_ARGS__) KO_CASE(F16, __VA_ARGS__) KO_CASE(BF16, __VA_ARGS__) \
    KO_CASE(F32, __VA_ARGS__) KO_CASE(F64, __VA_ARGS__) default: throw Error("oracle: float dtype required"); }
#define KO_INTS(dt, ...) \
  switch (dt) { KO_CASE(U8, __VA_ARGS__) KO_CASE(U16, __VA_ARGS__) KO_CASE(U32, __VA_ARGS__) KO_CASE(U64, __VA_ARGS__) \
    KO_CASE(I8, __VA_ARGS__) KO_CASE(I16, __VA_ARGS__) KO_CASE(I32, __VA_ARGS__) KO_CASE(I64, __VA_ARGS__) \
    default: throw Error("oracle: integer dtype required"); }
#define KO_NUMERIC(dt, ...) \
  switch (dt) { KO_CASE(U8, __VA_ARGS__) KO_CASE(U16, __VA_ARGS__) KO_CASE(U32, __VA_ARGS__) KO_CASE(U64, __VA_ARGS__) \
    KO_CASE(I8, __VA_ARGS__) KO_CASE(I16, __VA_ARGS__) KO_CASE(I32, __VA_ARGS__) KO_CASE(I64, __VA_ARGS__) \
    KO_CASE(F8E4M3, __VA_ARGS__) KO_CASE(F8E5M2, __VA_ARGS__) KO_CASE(F16, __VA_ARGS__) KO_CASE(BF16, __VA_ARGS__) \
    KO_CASE(F32, __VA_ARGS__) KO_CASE(F64, __VA_ARGS__) default: throw Error("oracle: numeric dtype required"); }
#define KO_ALL(dt, ...) \
  switch (dt) { KO_CASE(BOOL, __VA_ARGS__) KO_CASE(U8, __VA_ARGS__) KO_CASE(U16, __VA_ARGS__) KO_CASE(U32, __VA_ARGS__) KO_CASE(U64, __VA_ARGS__) \
    KO_CASE(I8, __VA_ARGS__) KO_CASE(I16, __VA_ARGS__) KO_CASE(I32, __VA_ARGS__) KO_CASE(I64, __VA_ARGS__) \
    KO_CASE(F8E4M3, __VA_ARGS__) KO_CASE(F8E5M2, __VA_ARGS__) KO_CASE(F16, __VA_ARGS__) KO_CASE(BF16, __VA_ARGS__) \
    KO_CASE(F32, __VA_ARGS__) KO_CASE(F64, __VA_ARGS__) default: throw Error("oracle: complex dtypes are outside this oracle"); }

// ---- scalar semantics ---------------------------------------------------------------------------
// kurumi_core/src/dtype/traits/float.rs:10-37 (f32::max = IEEE maxNum), int.rs:10-42
template <typename C> C op_add(C a, C b) {
  if constexpr (std::is_integral_v<C>) { using U = std::make_unsigned_t<C>; return static_cast<C>(static_cast<U>(static_cast<U>(a) + static_cast<U>(b))); }
  else return a + b;
}
template <typename C> C op_mul(C a, C b) {
  if constexpr (std::is_integral_v<C>) { using U = std::make_unsigned_t<C>; return static_cast<C>(static_cast<U>(static_cast<U>(a) * static_cast<U>(b))); }
  else return a * b;
}
template <typename C> C op_max(C a, C b) {
  if constexpr (std::is_same_v<C, float>) return std::fmax(a, b);
  else if constexpr (std::is_same_v<C, double>) return std::fmax(a, b);
  else return a > b ? a : b;
}
template <typename C> C op_neg(C a) {
  if constexpr (std::is_integral_v<C>) { using U = std::make_unsigned_t<C>; return static_cast<C>(static_cast<U>(0) - static_cast<U>(a)); }
  else return -a;
}
template <typename C> C op_idiv(C a, C b) {
  if (b == 0) return 0;
  if constexpr (std::is_signed_v<C>) { if (a == std::numeric_limits<C>::min() && b == static_cast<C>(-1)) return a; }
  return static_cast<C>(a / b);
}
template <typename C> C op_shl(C a, C b) {
  using U = std::make_unsigned_t<C>;
  unsigned s = static_cast<unsigned>(static_cast<uint32_t>(b)) & (sizeof(C) * 8 - 1);
  return static_cast<C>(static_cast<U>(static_cast<U>(a) << s));
}
template <typename C> C op_shr(C a, C b) {
  unsigned s = static_cast<unsigned>(static_cast<uint32_t>(b)) & (sizeof(C) * 8 - 1);
  return static_cast<C>(a >> s);  // arithmetic for signed, logical for unsigned
}
template <typename C> C op_float1(OpKind k, C x) {
  switch (k) {
    case OpKind::Recip: return static_cast<C>(1) / x;
    case OpKind::Sqrt: return std::sqrt(x);
    case OpKind::Exp2: return std::exp2(x);
    case OpKind::Log2: return std::log2(x);
    case OpKind::Sin: return std::sin(x);
    case OpKind::Floor: return std::floor(x);
    default: throw Error("oracle: not a float unary");
  }
}

const double* wd(const Val& v) { return reinterpret_cast<const double*>(v.bytes.data()); }
double* wd(Val& v) { return reinterpret_cast<double*>(v.bytes.data()); }

// ---- elementwise (kurumi_core/src/interp/elementwise.rs:7-118) -----------------------------------
Val ew_binary(OpKind k, const Val& a, const Val& b) {
  const size_t n = numel(a.shape);
  if (a.wide) {  // wide float arithmetic
    const double *x = wd(a), *y = wd(b);
    if (k == OpKind::CmpLt || k == OpKind::CmpEq) {
      Val o = make_val(DType::BOOL, a.shape, false);
      for (size_t i = 0; i < n; ++i) o.bytes[i] = k == OpKind::CmpLt ? (x[i] < y[i]) : (x[i] == y[i]);
      return o;
    }
    Val o = make_val(a.dtype, a.shape, true);
    double* z = wd(o);
    for (size_t i = 0; i < n; ++i) z[i] = k == OpKind::Add ? x[i] + y[i] : k == OpKind::Mul ? x[i] * y[i] : std::fmax(x[i], y[i]);
    return o;
  }
  if (k == OpKind::CmpLt || k == OpKind::CmpEq) {
    Val o = make_val(DType::BOOL, a.shape, false);
    KO_ALL(a.dtype, {
      using T = E<DT>;
      auto* x = reinterpret_cast<const typename T::S*>(a.bytes.data());
      auto* y = reinterpret_cast<const typename T::S*>(b.bytes.data());
      for (size_t i = 0; i < n; ++i) { auto p = T::ld(x[i]); auto q = T::ld(y[i]); o.bytes[i] = k == OpKind::CmpLt ? (p < q) : (p == q); }
    })
    return o;
  }
  Val o = make_val(a.dtype, a.shape, false);
  if (k == OpKind::And || k == OpKind::Or || k == OpKind::Xor) {
    if (a.dtype == DType::BOOL) {
      for (size_t i = 0; i < n; ++i) {
        bool p = a.bytes[i], q = b.bytes[i];
        o.bytes[i] = k == OpKind::And ? (p && q) : k == OpKind::Or ? (p || q) : (p != q);
      }
      return o;
    }
    for (size_t i = 0; i < a.bytes.size(); ++i)
      o.bytes[i] = k == OpKind::And ? (a.bytes[i] & b.bytes[i]) : k == OpKind::Or ? (a.bytes[i] | b.bytes[i]) : (a.bytes[i] ^ b.bytes[i]);
    return o;
  }
  if (k == OpKind::IDiv || k == OpKind::Shl || k == OpKind::Shr) {
    KO_INTS(a.dtype, {
      using T = E<DT>;
      auto* x = reinterpret_cast<const typename T::S*>(a.bytes.data());
      auto* y = reinterpret_cast<const typename T::S*>(b.bytes.data());
      auto* z = reinterpret_cast<typename T::S*>(o.bytes.data());
      for (size_t i = 0; i < n; ++i) z[i] = k == OpKind::IDiv ? op_idiv(x[i], y[i]) : k == OpKind::Shl ? op_shl(x[i], y[i]) : op_shr(x[i], y[i]);
    })
    return o;
  }
  KO_NUMERIC(a.dtype, {
    using T = E<DT>;
    auto* x = reinterpret_cast<const typename T::S*>(a.bytes.data());
    auto* y = reinterpret_cast<const typename T::S*>(b.bytes.data());
    auto* z = reinterpret_cast<typename T::S*>(o.bytes.data());
    if (k == OpKind::Add) for (size_t i = 0; i < n; ++i) z[i] = T::st(op_add(T::ld(x[i]), T::ld(y[i])));
    else if (k == OpKind::Mul) for (size_t i = 0; i < n; ++i) z[i] = T::st(op_mul(T::ld(x[i]), T::ld(y[i])));
    else for (size_t i = 0; i < n; ++i) z[i] = T::st(op_max(T::ld(x[i]), T::ld(y[i])));
  })
  return o;
}

Val ew_unary(OpKind k, const Val& a) {
  const size_t n = numel(a.shape);
  Val o = make_val(a.dtype, a.shape, a.wide);
  if (a.wide) {
    const double* x = wd(a);
    double* z = wd(o);
    for (size_t i = 0; i < n; ++i) z[i] = k == OpKind::Neg ? -x[i] : op_float1(k, x[i]);
    return o;
  }
  if (k == OpKind::Neg) {
    KO_NUMERIC(a.dtype, {
      using T = E<DT>;
      auto* x = reinterpret_cast<const typename T::S*>(a.bytes.data());
      auto* z = reinterpret_cast<typename T::S*>(o.bytes.data());
      for (size_t i = 0; i < n; ++i) z[i] = T::st(op_neg(T::ld(x[i])));
    })
    return o;
  }
  KO_FLOATS(a.dtype, {
    using T = E<DT>;
    auto* x = reinterpret_cast<const typename T::S*>(a.bytes.data());
    auto* z = reinterpret_cast<typename T::S*>(o.bytes.data());
    for (size_t i = 0; i < n; ++i) z[i] = T::st(op_float1(k, T::ld(x[i])));
  })
  return o;
}

Val ew_where(const Val& c, const Val& a, const Val& b) {
  Val o = make_val(a.dtype, a.shape, a.wide);
  const size_t n = numel(a.shape), w = esize(a);
  for (size_t i = 0; i < n; ++i) std::memcpy(o.bytes.data() + i * w, (c.bytes[i] ? a.bytes.data() : b.bytes.data()) + i * w, w);
  return o;
}

// Round a wide value to a float format and widen it again.
double round_to(DType dt, double x) {
  if (dt == DType::F64) return x;
  uint8_t tmp[8];
  f64_to_elem(dt, x, tmp);
  return elem_to_f64(dt, tmp);
}

// kurumi_core/src/dtype/convert.rs:14-47: every cast goes through f64
Val cast_val(const Val& a, DType to, bool wide_mode) {
  const size_t n = numel(a.shape);
  const bool out_wide = wide_mode && is_float(to);
  Val o = make_val(to, a.shape, out_wide);
  const size_t ws = esize(a), wo = esize(o);
  if (!a.wide && !out_wide && a.dtype == to) { o.bytes = a.bytes; return o; }
  for (size_t i = 0; i < n; ++i) {
    double x = a.wide ? wd(a)[i] : elem_to_f64(a.dtype, a.bytes.data() + i * ws);
    if (out_wide) wd(o)[i] = round_to(to, x);
    else f64_to_elem(to, x, o.bytes.data() + i * wo);
  }
  return o;
}

Val narrow(const Val& a) {  // wide -> the logical dtype's own bytes
  if (!a.wide) return a;
  Val o = make_val(a.dtype, a.shape, false);
  const size_t n = numel(a.shape), w = dtype_width(a.dtype);
  for (size_t i = 0; i < n; ++i) f64_to_elem(a.dtype, wd(a)[i], o.bytes.data() + i * w);
  return o;
}
Val widen(const Val& a) {
  if (a.wide || !is_float(a.dtype)) return a;
  Val o = make_val(a.dtype, a.shape, true);
  const size_t n = numel(a.shape), w = dtype_width(a.dtype);
  for (size_t i = 0; i < n; ++i) wd(o)[i] = elem_to_f64(a.dtype, a.bytes.data() + i * w);
  return o;
}

// kurumi_core/src/dtype/convert.rs:150-152
Val bitcast_val(const Val& a0, DType to, bool wide_mode) {
  Val a = narrow(a0);
  Val o = make_val(to, a.shape, false);
  o.bytes = a.bytes;
  if (to == DType::BOOL) for (auto& b : o.bytes) b = b ? 1 : 0;
  return (wide_mode && is_float(to)) ? widen(o) : o;
}

// ---- reductions (kurumi_core/src/interp/reduce.rs:67-106) ---------------------------------------
template <typename T, typename F>
void reduce_fold(const T* data, const Shape& shape, size_t axis, T init, F f, T* out) {
  auto st = row_major_strides(shape);
  const size_t axis_len = shape[axis], axis_stride = st[axis];
  Shape out_shape;
  std::vector<size_t> base_strides;
  for (size_t i = 0; i < shape.size(); ++i)
    if (i != axis) { out_shape.push_back(shape[i]); base_strides.push_back(st[i]); }
  const size_t out_len = numel(out_shape);  // 1 for a rank-0 result, 0 when any kept axis is empty
  std::vector<size_t> coord(out_shape.size(), 0);
  for (size_t o = 0; o < out_len; ++o) {
    size_t base = 0;
    for (size_t i = 0; i < coord.size(); ++i) base += coord[i] * base_strides[i];
    T acc = init;
    for (size_t k = 0; k < axis_len; ++k) acc = f(acc, data[base + k * axis_stride]);  // strict left fold
    out[o] = acc;
    inc(coord, out_shape);
  }
}

// ---- indexing and sorting (kurumi_core/src/interp/indexing.rs:23-36, indexing/gather.rs, indexing/scatter.rs, sort.rs) ----
std::vector<int64_t> indices_i64(const Val& ix) {
  const size_t n = numel(ix.shape);
  std::vector<int64_t> out(n);
  KO_INTS(ix.dtype, {
    using T = E<DT>;
    auto* p = reinterpret_cast<const typename T::S*>(ix.bytes.data());
    for (size_t i = 0; i < n; ++i) out[i] = static_cast<int64_t>(p[i]);
  })
  return out;
}

// indexing/gather.rs:55-77: operand laid out [pre, axis, post]; the post-slice at each clamped index; out = [pre, idx.shape, post]
Val gather_val(const Val& a, const Val& ix, size_t axis) {
  const std::vector<int64_t> idx = indices_i64(ix);
  Shape out(a.shape.begin(), a.shape.begin() + static_cast<long>(axis));
  out.insert(out.end(), ix.shape.begin(), ix.shape.end());
  out.insert(out.end(), a.shape.begin() + static_cast<long>(axis) + 1, a.shape.end());
  Val o = make_val(a.dtype, out, a.wide);
  const size_t w = esize(a), da = a.shape[axis];
  size_t pre = 1, post = 1;
  for (size_t d = 0; d < axis; ++d) pre *= a.shape[d];
  for (size_t d = axis + 1; d < a.shape.size(); ++d) post *= a.shape[d];
  const size_t k = numel(ix.shape);
  if (numel(out) == 0) return o;
  size_t dst = 0;
  for (size_t p = 0; p < pre; ++p)
    for (size_t ki = 0; ki < k; ++ki) {
      const int64_t j = std::min<int64_t>(std::max<int64_t>(idx[ki], 0), static_cast<int64_t>(da) - 1);   // out of range: clamped
      std::memcpy(o.bytes.data() + dst * w, a.bytes.data() + ((p * da + static_cast<size_t>(j)) * post) * w, post * w);
      dst += post;
    }
  return o;
}

// indexing/gather.rs:31-51: out[c] = operand[c with axis <- clamp(idx[c])]; out and idx share a shape
Val gather_along_val(const Val& a, const Val& ix, size_t axis) {
  const std::vector<int64_t> idx = indices_i64(ix);
  Val o = make_val(a.dtype, ix.shape, a.wide);
  const size_t w = esize(a), n = numel(ix.shape);
  const auto st = row_major_strides(a.shape);
  const int64_t da = static_cast<int64_t>(a.shape[axis]);
  std::vector<size_t> coord(ix.shape.size(), 0);
  for (size_t f = 0; f < n; ++f) {
    const size_t j = static_cast<size_t>(std::min<int64_t>(std::max<int64_t>(idx[f], 0), da - 1));
    size_t src = 0;
    for (size_t d = 0; d < a.shape.size(); ++d) src += (d == axis ? j : coord[d]) * st[d];
    std::memcpy(o.bytes.data() + f * w, a.bytes.data() + src * w, w);
    inc(coord, ix.shape);
  }
  return o;
}

// fold element `src` of `up` into element `dst` of `out`: 0 set, 1 add, 2 max, 3 min, with the dtype's own arithmetic
// (low-precision floats: upcast to f32, combine, round back; integers wrap)
void combine_elem(Val& out, size_t dst, const Val& up, size_t src, uint8_t combine) {
  if (combine == 0) { const size_t w = esize(out); std::memcpy(out.bytes.data() + dst * w, up.bytes.data() + src * w, w); return; }
  if (out.wide) {
    double& x = wd(out)[dst];
    const double y = wd(up)[src];
    x = combine == 1 ? x + y : combine == 2 ? std::fmax(x, y) : std::fmin(x, y);
    return;
  }
  KO_NUMERIC(out.dtype, {
    using T = E<DT>;
    auto* z = reinterpret_cast<typename T::S*>(out.bytes.data());
    auto* u = reinterpret_cast<const typename T::S*>(up.bytes.data());
    const typename T::C x = T::ld(z[dst]), y = T::ld(u[src]);
    typename T::C r;
    if (combine == 1) r = op_add(x, y);
    else if (combine == 2) r = op_max(x, y);
    else { if constexpr (std::is_floating_point_v<typename T::C>) r = std::fmin(x, y); else r = x < y ? x : y; }
    z[dst] = T::st(r);
  })
}

// indexing/scatter.rs:180-207: a copy of the operand; each update post-slice folds into [.., idx, ..] in index order, out-of-range dropped
Val scatter_val(const Val& a, const Val& ix, const Val& up, size_t axis, uint8_t combine) {
  const std::vector<int64_t> idx = indices_i64(ix);
  Val o = a;
  size_t pre = 1, post = 1;
  for (size_t d = 0; d < axis; ++d) pre *= a.shape[d];
  for (size_t d = axis + 1; d < a.shape.size(); ++d) post *= a.shape[d];
  const size_t k = numel(ix.shape), da = a.shape[axis];
  if (numel(a.shape) == 0) return o;
  for (size_t p = 0; p < pre; ++p)
    for (size_t ki = 0; ki < k; ++ki) {
      const int64_t raw = idx[ki];
      if (raw < 0 || raw >= static_cast<int64_t>(da)) continue;
      const size_t dst = (p * da + static_cast<size_t>(raw)) * post, src = (p * k + ki) * post;
      for (size_t j = 0; j < post; ++j) combine_elem(o, dst + j, up, src + j, combine);
    }
  return o;
}

// indexing/scatter.rs:142-166: per-position index along the axis; idx and updates share a shape
Val scatter_along_val(const Val& a, const Val& ix, const Val& up, size_t axis, uint8_t combine) {
  const std::vector<int64_t> idx = indices_i64(ix);
  Val o = a;
  const auto st = row_major_strides(a.shape);
  const int64_t da = static_cast<int64_t>(a.shape[axis]);
  const size_t n = numel(ix.shape);
  std::vector<size_t> coord(ix.shape.size(), 0);
  for (size_t f = 0; f < n; ++f) {
    const int64_t j = idx[f];
    if (j >= 0 && j < da) {
      size_t dst = 0;
      for (size_t d = 0; d < a.shape.size(); ++d) dst += (d == axis ? static_cast<size_t>(j) : coord[d]) * st[d];
      combine_elem(o, dst, up, f, combine);
    }
    inc(coord, ix.shape);
  }
  return o;
}

// sort.rs:41-68: per line, the stable permutation that sorts it (ties keep the lower original index); elements compare
// by value, `descending` reverses the comparison of the keys only. A line holding a NaN has no defined order in the
// reference (partial_cmp falls back to Equal, which is not a consistent ordering): not pinned here either.
Val argsort_val(const Val& a, size_t axis, bool descending) {
  Val o = make_val(DType::I64, a.shape, false);
  auto* out = reinterpret_cast<int64_t*>(o.bytes.data());
  const auto st = row_major_strides(a.shape);
  const size_t len = a.shape[axis], stride = st[axis], total = numel(a.shape);
  if (total == 0) return o;
  auto run = [&](auto key) {   // key(flat) -> comparable value
    std::vector<size_t> perm(len);
    for (size_t f = 0; f < total; ++f) {
      if ((f / stride) % len != 0) continue;   // f is the first element of a line
      for (size_t i = 0; i < len; ++i) perm[i] = i;
      std::stable_sort(perm.begin(), perm.end(), [&](size_t i, size_t j) {
        const auto vi = key(f + i * stride), vj = key(f + j * stride);
        return descending ? vi > vj : vi < vj;
      });
      for (size_t r = 0; r < len; ++r) out[f + r * stride] = static_cast<int64_t>(perm[r]);
    }
  };
  if (a.wide) { const double* p = wd(a); run([&](size_t i) { return p[i]; }); return o; }
  KO_NUMERIC(a.dtype, {
    using T = E<DT>;
    auto* p = reinterpret_cast<const typename T::S*>(a.bytes.data());
    run([&](size_t i) { return T::ld(p[i]); });
  })
  return o;
}

// kurumi_core/src/interp/reduce.rs:16-66: I64 index of the maximum / minimum along `axis`; the first element is the
// starting best and a later one replaces it only when strictly greater / smaller, so ties keep the lowest index
// and a NaN never replaces anything (nor is a leading NaN ever replaced). Elements compare by value.
Val arg_reduce_val(const Val& a, size_t axis, bool arg_min) {
  Shape out_shape = a.shape;
  out_shape.erase(out_shape.begin() + static_cast<long>(axis));
  Val o = make_val(DType::I64, out_shape, false);
  auto* out = reinterpret_cast<int64_t*>(o.bytes.data());
  const size_t len = a.shape[axis];
  size_t inner = 1, outer = 1;
  for (size_t d = axis + 1; d < a.shape.size(); ++d) inner *= a.shape[d];
  for (size_t d = 0; d < axis; ++d) outer *= a.shape[d];
  if (len == 0 && outer * inner > 0) throw Error("panic: index out of bounds: argreduce over an empty axis");
  const bool integral = !is_float(a.dtype);
  const size_t w = a.wide ? 8 : dtype_width(a.dtype);
  // integers compare as integers (u64 / i64 do not fit a double), floats by value
  auto as_f = [&](size_t i) { return a.wide ? wd(a)[i] : elem_to_f64(a.dtype, a.bytes.data() + i * w); };
  auto as_i = [&](size_t i) -> std::pair<bool, uint64_t> {   // (negative, magnitude-ordered key)
    int64_t sv = 0; uint64_t uv = 0;
    const uint8_t* p = a.bytes.data() + i * w;
    switch (a.dtype) {
      case DType::I8: sv = *reinterpret_cast<const int8_t*>(p); break;
      case DType::I16: { int16_t t; std::memcpy(&t, p, 2); sv = t; break; }
      case DType::I32: { int32_t t; std::memcpy(&t, p, 4); sv = t; break; }
      case DType::I64: std::memcpy(&sv, p, 8); break;
      case DType::U8: case DType::BOOL: uv = *p; return {false, uv};
      case DType::U16: { uint16_t t; std::memcpy(&t, p, 2); return {false, t}; }
      case DType::U32: { uint32_t t; std::memcpy(&t, p, 4); return {false, t}; }
      default: std::memcpy(&uv, p, 8); return {false, uv};
    }
    return {sv < 0, static_cast<uint64_t>(sv)};
  };
  auto less_i = [](std::pair<bool, uint64_t> x, std::pair<bool, uint64_t> y) {
    if (x.first != y.first) return x.first;   // negative < non-negative
    return x.second < y.second;                // two's complement order holds within a sign
  };
  for (size_t oo = 0; oo < outer; ++oo)
    for (size_t oi = 0; oi < inner; ++oi) {
      const size_t base = oo * len * inner + oi;
      size_t best = 0;
      for (size_t k = 1; k < len; ++k) {
        const size_t i = base + k * inner, b = base + best * inner;
        bool better;
        if (integral) better = arg_min ? less_i(as_i(i), as_i(b)) : less_i(as_i(b), as_i(i));
        else better = arg_min ? as_f(i) < as_f(b) : as_f(i) > as_f(b);
        if (better) best = k;
      }
      out[oo * inner + oi] = static_cast<int64_t>(best);
    }
  return o;
}

Val reduce_val(OpKind k, const Val& a, size_t axis, bool wide_mode) {
  Shape out_shape = a.shape;
  out_shape.erase(out_shape.begin() + static_cast<long>(axis));
  if (a.wide) {
    Val o = make_val(a.dtype, out_shape, true);
    if (k == OpKind::Sum) reduce_fold<double>(wd(a), a.shape, axis, 0.0, [](double p, double q) { return p + q; }, wd(o));
    else if (k == OpKind::Prod) reduce_fold<double>(wd(a), a.shape, axis, 1.0, [](double p, double q) { return p * q; }, wd(o));
    else reduce_fold<double>(wd(a), a.shape, axis, -std::numeric_limits<double>::infinity(), [](double p, double q) { return std::fmax(p, q); }, wd(o));
    return o;
  }
  (void)wide_mode;
  if (is_low_float(a.dtype) && k != OpKind::ReduceMax) {  // promote to f32, fold, round once
    Val f = cast_val(a, DType::F32, false);
    Val r = reduce_val(k, f, axis, false);
    return cast_val(r, a.dtype, false);
  }
  Val o = make_val(a.dtype, out_shape, false);
  KO_NUMERIC(a.dtype, {
    using T = E<DT>;
    using C = typename T::C;
    if constexpr (std::is_same_v<typename T::S, C>) {
      auto* x = reinterpret_cast<const C*>(a.bytes.data());
      auto* z = reinterpret_cast<C*>(o.bytes.data());
      if (k == OpKind::Sum) reduce_fold<C>(x, a.shape, axis, C(0), [](C p, C q) { return op_add(p, q); }, z);
      else if (k == OpKind::Prod) reduce_fold<C>(x, a.shape, axis, C(1), [](C p, C q) { return op_mul(p, q); }, z);
      else {
        C lowest = std::is_floating_point_v<C> ? -std::numeric_limits<C>::infinity() : std::numeric_limits<C>::lowest();
        reduce_fold<C>(x, a.shape, axis, lowest, [](C p, C q) { return op_max(p, q); }, z);
      }
    } else {  // low-precision ReduceMax: identity is the format's lowest (float.rs:38-72), max is exact
      using S = typename T::S;
      auto* x = reinterpret_cast<const S*>(a.bytes.data());
      auto* z = reinterpret_cast<S*>(o.bytes.data());
      S lowest = (DT == DType::F16 || DT == DType::BF16) ? T::st(-std::numeric_limits<float>::infinity()) : T::st(std::numeric_limits<float>::lowest());
      reduce_fold<S>(x, a.shape, axis, lowest, [](S p, S q) { return T::st(std::fmax(T::ld(p), T::ld(q))); }, z);
    }
  })
  return o;
}

}  // namespace
void reduce_f32(OpKind k, const float* data, const Shape& shape, size_t axis, float* out) {
  if (k == OpKind::Sum) reduce_fold<float>(data, shape, axis, 0.0f, [](float p, float q) { return p + q; }, out);
  else reduce_fold<float>(data, shape, axis, -std::numeric_limits<float>::infinity(), [](float p, float q) { return std::fmax(p, q); }, out);
}
namespace {
// ---- movement (kurumi_core/src/interp/movement.rs:37-118): per-output-element gathers -----------
Val movement_val(const Op& op, const Val& a) {
  const size_t w = esize(a);
  const Shape& in_shape = a.shape;
  auto in_st = row_major_strides(in_shape);
  if (op.kind == OpKind::Reshape) { Val o = a; o.shape = op.shape; return o; }
  Shape out_shape;
  switch (op.kind) {
    case OpKind::Permute: for (size_t p : op.perm) out_shape.push_back(in_shape[p]); break;
    case OpKind::Expand: out_shape = op.shape; break;
    case OpKind::Slice: for (auto& r : op.ranges) out_shape.push_back((r[1] - r[0] + r[2] - 1) / r[2]); break;
    case OpKind::Flip: out_shape = in_shape; break;
    case OpKind::Pad: for (size_t d = 0; d < in_shape.size(); ++d) out_shape.push_back(op.ranges[d][0] + in_shape[d] + op.ranges[d][1]); break;
    default: throw Error("oracle: not a movement op");
  }
  Val o = make_val(a.dtype, out_shape, a.wide);
  const size_t out_len = numel(out_shape);
  std::vector<size_t> coord(out_shape.size(), 0);
  std::vector<bool> flipped(in_shape.size(), false);
  if (op.kind == OpKind::Flip) for (size_t ax : op.perm) flipped[ax] = true;
  for (size_t idx = 0; idx < out_len; ++idx) {
    size_t in_flat = 0;
    bool valid = true;
    switch (op.kind) {
      case OpKind::Permute: for (size_t i = 0; i < coord.size(); ++i) in_flat += coord[i] * in_st[op.perm[i]]; break;
      case OpKind::Expand: for (size_t d = 0; d < coord.size(); ++d) in_flat += in_shape[d] == 1 ? 0 : coord[d] * in_st[d]; break;
      case OpKind::Slice: for (size_t d = 0; d < coord.size(); ++d) in_flat += (op.ranges[d][0] + coord[d] * op.ranges[d][2]) * in_st[d]; break;
      case OpKind::Flip: for (size_t d = 0; d < coord.size(); ++d) in_flat += (flipped[d] ? in_shape[d] - 1 - coord[d] : coord[d]) * in_st[d]; break;
      case OpKind::Pad:
        for (size_t d = 0; d < coord.size(); ++d) {
          size_t lo = op.ranges[d][0];
          if (coord[d] < lo || coord[d] >= lo + in_shape[d]) { valid = false; break; }
          in_flat += (coord[d] - lo) * in_st[d];
        }
        break;
      default: break;
    }
    if (valid) std::memcpy(o.bytes.data() + idx * w, a.bytes.data() + in_flat * w, w);  // else stays 0
    inc(coord, out_shape);
  }
  return o;
}

// ---- contraction (kurumi_core/src/interp/contract.rs:26-166, contract/gemm.rs:8-113) -----------
template <typename T>
void dot_num(const T* a, const Shape& as, const T* b, const Shape& bs, const Op& op, T* out) {
  auto a_st = row_major_strides(as), b_st = row_major_strides(bs);
  auto a_free = free_axes(as.size(), op.lb, op.lc), b_free = free_axes(bs.size(), op.rb, op.rc);
  Shape out_shape, c_sizes;
  for (size_t i : op.lb) out_shape.push_back(as[i]);
  for (size_t i : a_free) out_shape.push_back(as[i]);
  for (size_t i : b_free) out_shape.push_back(bs[i]);
  for (size_t i : op.lc) c_sizes.push_back(as[i]);
  const size_t nb = op.lb.size(), nlf = a_free.size();
  const size_t out_len = numel(out_shape);
  const size_t c_len = c_sizes.empty() ? 1 : numel(c_sizes);
  std::vector<size_t> oc(out_shape.size(), 0), cc(c_sizes.size(), 0);
  for (size_t o = 0; o < out_len; ++o) {
    size_t abase = 0, bbase = 0;
    for (size_t i = 0; i < nb; ++i) { abase += oc[i] * a_st[op.lb[i]]; bbase += oc[i] * b_st[op.rb[i]]; }
    for (size_t i = 0; i < a_free.size(); ++i) abase += oc[nb + i] * a_st[a_free[i]];
    for (size_t i = 0; i < b_free.size(); ++i) bbase += oc[nb + nlf + i] * b_st[b_free[i]];
    T acc = T(0);
    std::fill(cc.begin(), cc.end(), 0);
    for (size_t c = 0; c < c_len; ++c) {
      size_t ai = abase, bi = bbase;
      for (size_t j = 0; j < cc.size(); ++j) { ai += cc[j] * a_st[op.lc[j]]; bi += cc[j] * b_st[op.rc[j]]; }
      acc = op_add(acc, op_mul(a[ai], b[bi]));
      inc(cc, c_sizes);
    }
    out[o] = acc;
    inc(oc, out_shape);
  }
}

// f32 2-D single-contract fast path. Stand-in for the un-vendored `gemm` crate: f32 multiply,
// f32 add, k ascending per output element (row-panel order so it vectorises over n).
void sgemm_2d(size_t m, size_t n, size_t k, float* out, const float* a, size_t a_fs, size_t a_cs, const float* b, size_t b_fs, size_t b_cs) {
  std::fill(out, out + m * n, 0.0f);
  if (b_fs == 1) {
    for (size_t i = 0; i < m; ++i)
      for (size_t kk = 0; kk < k; ++kk) {
        const float av = a[i * a_fs + kk * a_cs];
        const float* brow = b + kk * b_cs;
        float* orow = out + i * n;
        for (size_t j = 0; j < n; ++j) orow[j] += av * brow[j];
      }
  } else {
    for (size_t i = 0; i < m; ++i)
      for (size_t j = 0; j < n; ++j) {
        float acc = 0.0f;
        for (size_t kk = 0; kk < k; ++kk) acc += a[i * a_fs + kk * a_cs] * b[j * b_fs + kk * b_cs];
        out[i * n + j] = acc;
      }
  }
}

Shape dot_out_shape(const Shape& as, const Shape& bs, const Op& op) {
  Shape o;
  for (size_t i : op.lb) o.push_back(as[i]);
  for (size_t i : free_axes(as.size(), op.lb, op.lc)) o.push_back(as[i]);
  for (size_t i : free_axes(bs.size(), op.rb, op.rc)) o.push_back(bs[i]);
  return o;
}

Val dot_f32(const Val& a, const Val& b, const Op& op) {
  Val o = make_val(DType::F32, dot_out_shape(a.shape, b.shape, op), false);
  auto* x = reinterpret_cast<const float*>(a.bytes.data());
  auto* y = reinterpret_cast<const float*>(b.bytes.data());
  auto* z = reinterpret_cast<float*>(o.bytes.data());
  if (a.shape.size() == 2 && b.shape.size() == 2 && op.lb.empty() && op.lc.size() == 1) {
    size_t lc = op.lc[0], rc = op.rc[0], lf = 1 - lc, rf = 1 - rc;
    size_t m = a.shape[lf], k = a.shape[lc], n = b.shape[rf];
    auto a_st = row_major_strides(a.shape), b_st = row_major_strides(b.shape);
    if (m && n && k) sgemm_2d(m, n, k, z, x, a_st[lf], a_st[lc], y, b_st[rf], b_st[rc]);
    return o;
  }
  dot_num<float>(x, a.shape, y, b.shape, op, z);
  return o;
}

// The f64 run of a GEMM-shaped contraction (leading batch axes in order, one contract axis per operand): the same
// sums as dot_num<double> - per output element, products added in ascending k - walked in a cache-friendly order
// (rows of B streamed, or eight output columns at a time), so that the full-size parity samples finish in seconds.
// The f64 run is this test suite's tolerance reference, not a timed path.
bool dgemm_shaped(const double* a, const Shape& as, const double* b, const Shape& bs, const Op& op, double* out) {
  const size_t ra = as.size(), rb = bs.size(), nb = op.lb.size();
  if (ra != nb + 2 || rb != nb + 2 || op.lc.size() != 1 || op.rc.size() != 1 || op.rb.size() != nb) return false;
  for (size_t i = 0; i < nb; ++i) if (op.lb[i] != i || op.rb[i] != i) return false;
  const size_t lc = op.lc[0], rc = op.rc[0];
  if (lc < nb || rc < nb) return false;
  const size_t lf = lc == nb ? nb + 1 : nb, rf = rc == nb ? nb + 1 : nb;
  const auto a_st = row_major_strides(as), b_st = row_major_strides(bs);
  const size_t m = as[lf], k = as[lc], n = bs[rf];
  size_t batch = 1;
  for (size_t i = 0; i < nb; ++i) batch *= as[i];
  const size_t a_fs = a_st[lf], a_cs = a_st[lc], b_fs = b_st[rf], b_cs = b_st[rc];
  for (size_t bi = 0; bi < batch; ++bi) {
    const double* A = a + bi * m * k;
    const double* B = b + bi * k * n;
    double* O = out + bi * m * n;
    if (b_fs == 1) {   // B is [k][n]: stream its rows
      std::fill(O, O + m * n, 0.0);
      for (size_t i = 0; i < m; ++i)
        for (size_t kk = 0; kk < k; ++kk) {
          const double av = A[i * a_fs + kk * a_cs];
          const double* brow = B + kk * b_cs;
          double* orow = O + i * n;
          for (size_t j = 0; j < n; ++j) orow[j] += av * brow[j];
        }
    } else {           // B is [n][k]: eight independent dot products at a time
      for (size_t i = 0; i < m; ++i) {
        size_t j = 0;
        for (; j + 8 <= n; j += 8) {
          double acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
          for (size_t kk = 0; kk < k; ++kk) {
            const double av = A[i * a_fs + kk * a_cs];
            for (size_t u = 0; u < 8; ++u) acc[u] += av * B[(j + u) * b_fs + kk * b_cs];
          }
          for (size_t u = 0; u < 8; ++u) O[i * n + j + u] = acc[u];
        }
        for (; j < n; ++j) {
          double acc = 0;
          for (size_t kk = 0; kk < k; ++kk) acc += A[i * a_fs + kk * a_cs] * B[j * b_fs + kk * b_cs];
          O[i * n + j] = acc;
        }
      }
    }
  }
  return true;
}

Val dot_val(const Val& a, const Val& b, const Op& op) {
  if (a.wide) {
    Val o = make_val(a.dtype, dot_out_shape(a.shape, b.shape, op), true);
    if (!(numel(o.shape) && dgemm_shaped(wd(a), a.shape, wd(b), b.shape, op, wd(o))))
      dot_num<double>(wd(a), a.shape, wd(b), b.shape, op, wd(o));
    return o;
  }
  if (a.dtype == DType::F32) return dot_f32(a, b, op);
  if (is_low_float(a.dtype)) {  // dot_promoted: f32 GEMM, one rounding of the result
    Val r = dot_f32(cast_val(a, DType::F32, false), cast_val(b, DType::F32, false), op);
    return cast_val(r, a.dtype, false);
  }
  Val o = make_val(a.dtype, dot_out_shape(a.shape, b.shape, op), false);
  KO_NUMERIC(a.dtype, {
    using T = E<DT>;
    if constexpr (std::is_same_v<typename T::S, typename T::C>) {
      using C = typename T::C;
      dot_num<C>(reinterpret_cast<const C*>(a.bytes.data()), a.shape, reinterpret_cast<const C*>(b.bytes.data()), b.shape, op, reinterpret_cast<C*>(o.bytes.data()));
    }
  })
  return o;
}

// ---- nn oracles (kurumi_core/src/interp/nn.rs:18-172) -------------------------------------------
template <typename T>
void softmax_lines(const T* data, const Shape& shape, size_t axis, T* out) {
  auto st = row_major_strides(shape);
  const size_t axis_len = shape[axis], axis_stride = st[axis];
  Shape out_shape;
  std::vector<size_t> base_strides;
  for (size_t i = 0; i < shape.size(); ++i)
    if (i != axis) { out_shape.push_back(shape[i]); base_strides.push_back(st[i]); }
  const size_t out_len = numel(out_shape);
  std::vector<size_t> coord(out_shape.size(), 0);
  for (size_t o = 0; o < out_len; ++o) {
    size_t base = 0;
    for (size_t i = 0; i < coord.size(); ++i) base += coord[i] * base_strides[i];
    T m = -std::numeric_limits<T>::infinity();
    for (size_t k = 0; k < axis_len; ++k) m = std::fmax(m, data[base + k * axis_stride]);
    T sum = 0;
    for (size_t k = 0; k < axis_len; ++k) {
      T e = std::exp(data[base + k * axis_stride] - m);
      out[base + k * axis_stride] = e;
      sum += e;
    }
    for (size_t k = 0; k < axis_len; ++k) out[base + k * axis_stride] /= sum;
    inc(coord, out_shape);
  }
}

Val softmax_val(const Val& a, size_t axis) {
  if (a.wide || a.dtype == DType::F64) {
    Val o = make_val(a.dtype, a.shape, a.wide);
    softmax_lines<double>(reinterpret_cast<const double*>(a.bytes.data()), a.shape, axis, reinterpret_cast<double*>(o.bytes.data()));
    return o;
  }
  Val f = cast_val(a, DType::F32, false);
  Val r = make_val(DType::F32, a.shape, false);
  softmax_lines<float>(reinterpret_cast<const float*>(f.bytes.data()), a.shape, axis, reinterpret_cast<float*>(r.bytes.data()));
  return a.dtype == DType::F32 ? r : cast_val(r, a.dtype, false);
}

template <typename T>
void rmsnorm_lines(const T* data, const Shape& shape, size_t axis, T eps, T* out) {
  auto st = row_major_strides(shape);
  const size_t axis_len = shape[axis], axis_stride = st[axis];
  Shape out_shape;
  std::vector<size_t> base_strides;
  for (size_t i = 0; i < shape.size(); ++i)
    if (i != axis) { out_shape.push_back(shape[i]); base_strides.push_back(st[i]); }
  const size_t out_len = numel(out_shape);
  std::vector<size_t> coord(out_shape.size(), 0);
  for (size_t o = 0; o < out_len; ++o) {
    size_t base = 0;
    for (size_t i = 0; i < coord.size(); ++i) base += coord[i] * base_strides[i];
    T ss = 0;
    for (size_t k = 0; k < axis_len; ++k) { T x = data[base + k * axis_stride]; ss += x * x; }
    T rms = std::sqrt(ss / static_cast<T>(axis_len) + eps);
    for (size_t k = 0; k < axis_len; ++k) out[base + k * axis_stride] = data[base + k * axis_stride] / rms;
    inc(coord, out_shape);
  }
}

Val rmsnorm_val(const Val& a, size_t axis, float eps) {
  if (a.wide || a.dtype == DType::F64) {
    Val o = make_val(a.dtype, a.shape, a.wide);
    rmsnorm_lines<double>(reinterpret_cast<const double*>(a.bytes.data()), a.shape, axis, static_cast<double>(eps), reinterpret_cast<double*>(o.bytes.data()));
    return o;
  }
  Val f = cast_val(a, DType::F32, false);
  Val r = make_val(DType::F32, a.shape, false);
  rmsnorm_lines<float>(reinterpret_cast<const float*>(f.bytes.data()), a.shape, axis, eps, reinterpret_cast<float*>(r.bytes.data()));
  return a.dtype == DType::F32 ? r : cast_val(r, a.dtype, false);
}

template <typename T>
void scale_causal(const T* data, size_t total, size_t s, T scale, bool causal, T* out) {
  const size_t block = s * s;
  for (size_t base = 0; base < total; base += std::max<size_t>(block, 1))
    for (size_t i = 0; i < s; ++i)
      for (size_t j = 0; j < s; ++j) {
        size_t idx = base + i * s + j;
        out[idx] = (causal && j > i) ? -std::numeric_limits<T>::infinity() : data[idx] * scale;
      }
}

Val sdpa_val(const Val& q, const Val& k, const Val& v, bool causal) {
  const size_t r = q.shape.size();
  const size_t s = q.shape[r - 2], dh = q.shape[r - 1];
  Op qk; qk.kind = OpKind::DotGeneral; qk.lc = {r - 1}; qk.rc = {r - 1};
  for (size_t i = 0; i + 2 < r; ++i) { qk.lb.push_back(i); qk.rb.push_back(i); }
  Val raw = dot_val(q, k, qk);
  const float scale = 1.0f / std::sqrt(static_cast<float>(dh));
  Val scores;
  if (raw.wide || raw.dtype == DType::F64) {
    scores = make_val(raw.dtype, raw.shape, raw.wide);
    scale_causal<double>(reinterpret_cast<const double*>(raw.bytes.data()), numel(raw.shape), s, static_cast<double>(scale), causal, reinterpret_cast<double*>(scores.bytes.data()));
  } else {
    Val f = cast_val(raw, DType::F32, false);
    Val o = make_val(DType::F32, raw.shape, false);
    scale_causal<float>(reinterpret_cast<const float*>(f.bytes.data()), numel(raw.shape), s, scale, causal, reinterpret_cast<float*>(o.bytes.data()));
    scores = raw.dtype == DType::F32 ? o : cast_val(o, raw.dtype, false);
  }
  Val attn = softmax_val(scores, r - 1);
  Op av; av.kind = OpKind::DotGeneral; av.lc = {r - 1}; av.rc = {r - 2}; av.lb = qk.lb; av.rb = qk.rb;
  return dot_val(attn, v, av);
}

// ---- generation (kurumi_core/src/interp/random.rs:10-28, dtype/convert.rs:72-80) ----------------
// kurumi_core/src/interp/contract.rs:69-99 with kurumi_core/src/quant.rs:90-113: dequantise the packed weight
// [N, K] to f32 (raw * scale + min, or the sign-extended field * scale), then act [M, K] x W^T as an f32
// contraction, rounded once to act's dtype. The wide run does the same in f64.
Val quant_matmul_val(const Val& act, const Val& qw, const Val& scales, const Val* mins, const Op& op) {
  const size_t m = act.shape[0], k = act.shape[1], n = qw.shape[0];
  const size_t ng = k / op.group_size, rb = k * op.bits / 8, per = 8 / op.bits;
  auto half_at = [](const Val& v, size_t i) -> double {
    if (v.wide) return wd(v)[i];
    return elem_to_f64(DType::F16, v.bytes.data() + 2 * i);
  };
  Op dot;
  dot.kind = OpKind::DotGeneral;
  dot.lc = {1};
  dot.rc = {1};
  if (act.wide) {
    Val w = make_val(DType::F64, {n, k}, true);
    double* wp = wd(w);
    for (size_t r = 0; r < n; ++r)
      for (size_t c = 0; c < k; ++c) {
        const size_t gi = r * ng + c / op.group_size;
        const unsigned raw = (qw.bytes[r * rb + c / per] >> ((c % per) * op.bits)) & ((1u << op.bits) - 1);
        if (mins) wp[r * k + c] = static_cast<double>(raw) * half_at(scales, gi) + half_at(*mins, gi);
        else { const int sh = 32 - op.bits; wp[r * k + c] = static_cast<double>(static_cast<int>(raw << sh) >> sh) * half_at(scales, gi); }
      }
    Val o = make_val(act.dtype, {m, n}, true);
    dot_num<double>(wd(act), act.shape, wp, w.shape, dot, wd(o));
    return o;
  }
  std::vector<uint16_t> sc(n * ng), mn(mins ? n * ng : 0);
  for (size_t i = 0; i < n * ng; ++i) {
    f64_to_elem(DType::F16, half_at(scales, i), &sc[i]);
    if (mins) f64_to_elem(DType::F16, half_at(*mins, i), &mn[i]);
  }
  std::vector<float> wf = ku::dequantize(qw.bytes.data(), sc.data(), mins ? mn.data() : nullptr, n, k, op.bits, op.group_size);
  Val w = make_val(DType::F32, {n, k}, false);
  std::memcpy(w.bytes.data(), wf.data(), wf.size() * 4);
  Val r = dot_f32(cast_val(act, DType::F32, false), w, dot);
  return cast_val(r, act.dtype, false);
}

Val iota_val(const Op& op, bool wide_mode) {
  const size_t len = numel(op.shape);
  size_t stride = 1;
  for (size_t i = op.axis + 1; i < op.shape.size(); ++i) stride *= op.shape[i];
  const size_t axis_len = op.shape[op.axis];
  Val o = make_val(op.to, op.shape, false);
  const size_t w = dtype_width(op.to);
  for (size_t flat = 0; flat < len; ++flat) f64_to_elem(op.to, static_cast<double>((flat / stride) % axis_len), o.bytes.data() + flat * w);
  return (wide_mode && is_float(op.to)) ? widen(o) : o;
}

Val rand_val(const Op& op, const Val& seed_v, bool wide_mode) {
  Val sv = narrow(seed_v);
  uint64_t seed = static_cast<uint64_t>(static_cast<int64_t>(0));
  switch (sv.dtype) {  // read the first element as i64 (sign-extending signed types), then as u64
    case DType::U8: seed = *reinterpret_cast<const uint8_t*>(sv.bytes.data()); break;
    case DType::U16: seed = *reinterpret_cast<const uint16_t*>(sv.bytes.data()); break;
    case DType::U32: seed = *reinterpret_cast<const uint32_t*>(sv.bytes.data()); break;
    case DType::U64: seed = *reinterpret_cast<const uint64_t*>(sv.bytes.data()); break;
    case DType::I8: seed = static_cast<uint64_t>(static_cast<int64_t>(*reinterpret_cast<const int8_t*>(sv.bytes.data()))); break;
    case DType::I16: seed = static_cast<uint64_t>(static_cast<int64_t>(*reinterpret_cast<const int16_t*>(sv.bytes.data()))); break;
    case DType::I32: seed = static_cast<uint64_t>(static_cast<int64_t>(*reinterpret_cast<const int32_t*>(sv.bytes.data()))); break;
    case DType::I64: seed = static_cast<uint64_t>(*reinterpret_cast<const int64_t*>(sv.bytes.data())); break;
    default: throw Error("oracle: rand_uniform seed must be an integer tensor");
  }
  const size_t n = numel(op.shape);
  Val o = make_val(DType::F32, op.shape, false);
  auto* z = reinterpret_cast<float*>(o.bytes.data());
  for (size_t i = 0; i < n; ++i) z[i] = uniform_f32(threefry2x32(seed, i));
  return wide_mode ? widen(o) : o;
}

Val from_tensor(const Tensor& t, bool wide_mode) {
  Val v;
  v.shape = t.shape; v.dtype = t.dtype; v.wide = false; v.bytes.assign(t.bytes.begin(), t.bytes.end());
  return (wide_mode && is_float(t.dtype)) ? widen(v) : v;
}

}  // namespace

// kurumi_core/src/interp.rs:62-112: one primitive given its materialised inputs
Val eval_op(const Node& n, const std::vector<const Val*>& in, bool wide_mode) {
  const Op& op = n.op;
  switch (op.kind) {
    case OpKind::Const: return from_tensor(*op.data, wide_mode);
    case OpKind::Input: throw Error("panic: Input must be resolved from feeds before eval_op");
    case OpKind::Detach: return *in[0];
    case OpKind::Iota: return iota_val(op, wide_mode);
    case OpKind::RandUniform: return rand_val(op, *in[0], wide_mode);
    case OpKind::Cast: return cast_val(*in[0], op.to, wide_mode);
    case OpKind::Bitcast: return bitcast_val(*in[0], op.to, wide_mode);
    case OpKind::Add: case OpKind::Mul: case OpKind::Max: case OpKind::IDiv: case OpKind::And: case OpKind::Or:
    case OpKind::Xor: case OpKind::Shl: case OpKind::Shr: case OpKind::CmpLt: case OpKind::CmpEq:
      return ew_binary(op.kind, *in[0], *in[1]);
    case OpKind::Where: return ew_where(*in[0], *in[1], *in[2]);
    case OpKind::Neg: case OpKind::Recip: case OpKind::Sqrt: case OpKind::Exp2: case OpKind::Log2: case OpKind::Sin:
    case OpKind::Floor:
      return ew_unary(op.kind, *in[0]);
    case OpKind::Sum: case OpKind::Prod: case OpKind::ReduceMax: return reduce_val(op.kind, *in[0], op.axis, wide_mode);
    case OpKind::ArgReduce: return arg_reduce_val(*in[0], op.axis, op.arg_min);
    case OpKind::Gather: return gather_val(*in[0], *in[1], op.axis);
    case OpKind::GatherAlong: return gather_along_val(*in[0], *in[1], op.axis);
    case OpKind::Scatter: return scatter_val(*in[0], *in[1], *in[2], op.axis, op.combine);
    case OpKind::ScatterAlong: return scatter_along_val(*in[0], *in[1], *in[2], op.axis, op.combine);
    case OpKind::Argsort: return argsort_val(*in[0], op.axis, op.descending);
    case OpKind::Softmax: return softmax_val(*in[0], op.axis);
    case OpKind::RmsNorm: return rmsnorm_val(*in[0], op.axis, op.eps);
    case OpKind::Sdpa: return sdpa_val(*in[0], *in[1], *in[2], op.causal);
    case OpKind::Reshape: case OpKind::Permute: case OpKind::Expand: case OpKind::Slice: case OpKind::Flip: case OpKind::Pad:
      return movement_val(op, *in[0]);
    case OpKind::DotGeneral: return dot_val(*in[0], *in[1], op);
    case OpKind::QuantMatmul: return quant_matmul_val(*in[0], *in[1], *in[2], in.size() > 3 ? in[3] : nullptr, op);
  }
  throw Error("oracle: unknown op");
}

Tensor to_tensor(const Val& v) {
  Tensor t;
  t.shape = v.shape;
  t.dtype = v.wide ? DType::F64 : v.dtype;
  t.bytes.assign(v.bytes.begin(), v.bytes.end());
  return t;
}

// kurumi_core/src/interp.rs:25-56: memoised walk; a missing feed is an error
std::vector<Tensor> interpret_many(const Graph& g, const std::vector<NodeId>& ids, const Feeds& feeds, bool wide_mode) {
  std::unordered_map<NodeId, Val> memo;
  for (NodeId id : reachable(g, ids)) {  // topological order: every source is evaluated first
    const Node& n = g.node(id);
    if (n.op.kind == OpKind::Input) {
      auto it = feeds.find(id);
      if (it == feeds.end()) throw Error("panic: interpret: missing feed for an Input node");
      memo.emplace(id, from_tensor(*it->second, wide_mode));
      continue;
    }
    std::vector<const Val*> in;
    for (NodeId s : n.src) in.push_back(&memo.at(s));
    memo.emplace(id, eval_op(n, in, wide_mode));
  }
  std::vector<Tensor> out;
  for (NodeId id : ids) out.push_back(to_tensor(memo.at(id)));
  return out;
}

}  // namespace ko

// Element dtypes and host-side value conversions.
//
// Mirrors kurumi_core/src/dtype.rs:24-87 (the 17 dtype tags, in declaration order, and their
// byte widths) and the conversion rules of kurumi_core/src/dtype/convert.rs:14-47 and
// kurumi_core/src/dtype/traits/elem.rs:31-45: every cast goes through an f64 intermediate,
// float->int is truncate + saturate with NaN -> 0, anything -> BOOL is `x != 0`.
//
// The narrow float formats live in third-party crates in the reference (`half` 2.7.1 for
// bf16/f16, `float8` 0.7.0 for the two fp8 formats). Their published behaviour is restated
// here: round-to-nearest-even, NaN stays NaN, fp8 conversions saturate to the largest finite
// value (the reference relies on that for its reduce-max identity,
// kurumi_core/src/dtype/traits/float.rs:54-56).
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <stdexcept>
#include <string>

namespace ku {

enum class DType : uint32_t {
  BOOL = 0, U8, U16, U32, U64, I8, I16, I32, I64, F8E4M3, F8E5M2, F16, BF16, F32, F64, C64, C128
};
constexpr uint32_t kNumDTypes = 17;

inline const char* dtype_name(DType d) {
  static const char* n[] = {"BOOL", "U8",  "U16",  "U32", "U64", "I8",  "I16", "I32", "I64",
                            "F8E4M3", "F8E5M2", "F16", "BF16", "F32", "F64", "C64", "C128"};
  return n[static_cast<uint32_t>(d)];
}
inline bool is_float(DType d) { return d >= DType::F8E4M3 && d <= DType::F64; }
inline bool is_int(DType d) { return d >= DType::U8 && d <= DType::I64; }
inline bool is_complex(DType d) { return d == DType::C64 || d == DType::C128; }
inline bool is_numeric(DType d) { return is_int(d) || is_float(d); }
inline bool is_arith(DType d) { return is_numeric(d) || is_complex(d); }
inline bool is_signed(DType d) { return is_float(d) || (d >= DType::I8 && d <= DType::I64); }
inline bool is_low_float(DType d) { return d >= DType::F8E4M3 && d <= DType::BF16; }
inline size_t dtype_width(DType d) {
  switch (d) {
    case DType::BOOL: case DType::U8: case DType::I8: case DType::F8E4M3: case DType::F8E5M2: return 1;
    case DType::U16: case DType::I16: case DType::F16: case DType::BF16: return 2;
    case DType::U32: case DType::I32: case DType::F32: return 4;
    case DType::U64: case DType::I64: case DType::F64: case DType::C64: return 8;
    case DType::C128: return 16;
  }
  return 0;
}

// ---- narrow IEEE-like formats (sign, ebits exponent, mbits mantissa, inf + NaN) ----------
// One rounding from f64, ties to even; used for bf16 (8,7) and f16 (5,10).
inline uint32_t f64_to_ieee_small(double x, int ebits, int mbits) {
  const int bias = (1 << (ebits - 1)) - 1;
  const uint32_t sign = std::signbit(x) ? (1u << (ebits + mbits)) : 0u;
  const uint32_t exp_all = ((1u << ebits) - 1u) << mbits;
  if (std::isnan(x)) return sign | exp_all | (1u << (mbits - 1));
  double a = std::fabs(x);
  if (std::isinf(a)) return sign | exp_all;
  if (a == 0.0) return sign;
  int e;
  std::frexp(a, &e);
  int E = e - 1;  // a = 1.f * 2^E
  const int emin = 1 - bias, emax = bias;
  if (E < emin) {
    double q = std::nearbyint(std::ldexp(a, mbits - emin));  // multiples of the subnormal quantum
    return sign | static_cast<uint32_t>(q);                  // q == 2^mbits encodes the least normal
  }
  double q = std::nearbyint(std::ldexp(a, mbits - E));  // in [2^mbits, 2^(mbits+1)]
  if (q >= std::ldexp(1.0, mbits + 1)) { E += 1; q = std::ldexp(1.0, mbits); }
  if (E > emax) return sign | exp_all;
  return sign | (static_cast<uint32_t>(E + bias) << mbits) | (static_cast<uint32_t>(q) - (1u << mbits));
}
inline double ieee_small_to_f64(uint32_t bits, int ebits, int mbits) {
  const int bias = (1 << (ebits - 1)) - 1;
  const bool neg = (bits >> (ebits + mbits)) & 1u;
  const uint32_t ef = (bits >> mbits) & ((1u << ebits) - 1u);
  const uint32_t mf = bits & ((1u << mbits) - 1u);
  double v;
  if (ef == (1u << ebits) - 1u) v = mf ? std::numeric_limits<double>::quiet_NaN() : std::numeric_limits<double>::infinity();
  else if (ef == 0) v = std::ldexp(static_cast<double>(mf), 1 - bias - mbits);
  else v = std::ldexp(static_cast<double>(mf | (1u << mbits)), static_cast<int>(ef) - bias - mbits);
  return neg ? -v : v;
}
inline uint16_t f64_to_bf16(double x) { return static_cast<uint16_t>(f64_to_ieee_small(x, 8, 7)); }
inline uint16_t f64_to_f16(double x) { return static_cast<uint16_t>(f64_to_ieee_small(x, 5, 10)); }
inline double bf16_to_f64(uint16_t b) { return ieee_small_to_f64(b, 8, 7); }
inline double f16_to_f64(uint16_t b) { return ieee_small_to_f64(b, 5, 10); }
inline float bf16_to_f32(uint16_t b) { uint32_t u = static_cast<uint32_t>(b) << 16; float f; std::memcpy(&f, &u, 4); return f; }
inline uint16_t f32_to_bf16(float x) { return f64_to_bf16(static_cast<double>(x)); }  // f32->f64 is exact
inline uint16_t f32_to_f16(float x) { return f64_to_f16(static_cast<double>(x)); }
inline float f16_to_f32(uint16_t b) { return static_cast<float>(f16_to_f64(b)); }

// ---- fp8 -----------------------------------------------------------------------------------
// e4m3 ("fn" flavour): bias 7, no infinity, S.1111.111 is NaN, largest finite 448.
// e5m2: bias 15; conversions here saturate to the largest finite 57344 (no inf is produced).
inline uint8_t f32_to_f8(float xf, int ebits, int mbits, double max_finite, uint8_t nan_bits) {
  const double x = static_cast<double>(xf);
  const int bias = (1 << (ebits - 1)) - 1;
  const uint8_t sign = std::signbit(x) ? 0x80 : 0x00;
  if (std::isnan(x)) return sign | nan_bits;
  double a = std::fabs(x);
  if (a == 0.0) return sign;
  if (std::isinf(a)) a = max_finite;
  int e;
  std::frexp(a, &e);
  int E = e - 1;
  const int emin = 1 - bias;
  double q;
  uint32_t bits;
  if (E < emin) {
    q = std::nearbyint(std::ldexp(a, mbits - emin));
    bits = static_cast<uint32_t>(q);
  } else {
    q = std::nearbyint(std::ldexp(a, mbits - E));
    if (q >= std::ldexp(1.0, mbits + 1)) { E += 1; q = std::ldexp(1.0, mbits); }
    double val = std::ldexp(q, E - mbits);
    if (val > max_finite) { val = max_finite; std::frexp(val, &e); E = e - 1; q = std::ldexp(val, mbits - E); }
    bits = (static_cast<uint32_t>(E + bias) << mbits) | (static_cast<uint32_t>(q) - (1u << mbits));
  }
  return sign | static_cast<uint8_t>(bits);
}
inline uint8_t f32_to_e4m3(float x) { return f32_to_f8(x, 4, 3, 448.0, 0x7f); }
inline uint8_t f32_to_e5m2(float x) { return f32_to_f8(x, 5, 2, 57344.0, 0x7f); }
inline float e4m3_to_f32(uint8_t b) {
  if ((b & 0x7f) == 0x7f) return std::numeric_limits<float>::quiet_NaN();
  const uint32_t ef = (b >> 3) & 0xf, mf = b & 7;
  double v = ef == 0 ? std::ldexp(static_cast<double>(mf), -9) : std::ldexp(static_cast<double>(mf | 8), static_cast<int>(ef) - 10);
  return static_cast<float>((b & 0x80) ? -v : v);
}
inline float e5m2_to_f32(uint8_t b) { return static_cast<float>(ieee_small_to_f64(b, 5, 2)); }

// ---- f64 <-> element (kurumi_core/src/dtype/traits/elem.rs:31-45) --------------------------
template <typename I>
inline I sat_cast(double x) {  // Rust `as`: truncate toward zero, saturate, NaN -> 0
  if (std::isnan(x)) return 0;
  const double lo = static_cast<double>(std::numeric_limits<I>::lowest());
  const double hi = static_cast<double>(std::numeric_limits<I>::max());  // rounds up to 2^N for 64-bit
  if (x <= lo) return std::numeric_limits<I>::lowest();
  if (x >= hi) return std::numeric_limits<I>::max();
  return static_cast<I>(x);
}

inline double elem_to_f64(DType d, const void* p) {
  switch (d) {
    case DType::BOOL: return *static_cast<const uint8_t*>(p) ? 1.0 : 0.0;
    case DType::U8: return *static_cast<const uint8_t*>(p);
    case DType::U16: { uint16_t v; std::memcpy(&v, p, 2); return v; }
    case DType::U32: { uint32_t v; std::memcpy(&v, p, 4); return v; }
    case DType::U64: { uint64_t v; std::memcpy(&v, p, 8); return static_cast<double>(v); }
    case DType::I8: return *static_cast<const int8_t*>(p);
    case DType::I16: { int16_t v; std::memcpy(&v, p, 2); return v; }
    case DType::I32: { int32_t v; std::memcpy(&v, p, 4); return v; }
    case DType::I64: { int64_t v; std::memcpy(&v, p, 8); return static_cast<double>(v); }
    case DType::F8E4M3: return e4m3_to_f32(*static_cast<const uint8_t*>(p));
    case DType::F8E5M2: return e5m2_to_f32(*static_cast<const uint8_t*>(p));
    case DType::F16: { uint16_t v; std::memcpy(&v, p, 2); return f16_to_f64(v); }
    case DType::BF16: { uint16_t v; std::memcpy(&v, p, 2); return bf16_to_f64(v); }
    case DType::F32: { float v; std::memcpy(&v, p, 4); return v; }
    case DType::F64: { double v; std::memcpy(&v, p, 8); return v; }
    case DType::C64: { float v; std::memcpy(&v, p, 4); return v; }   // real part
    case DType::C128: { double v; std::memcpy(&v, p, 8); return v; }
  }
  return 0.0;
}

inline void f64_to_elem(DType d, double x, void* p) {
  switch (d) {
    case DType::BOOL: *static_cast<uint8_t*>(p) = (x != 0.0) ? 1 : 0; return;  // NaN != 0 -> true
    case DType::U8: *static_cast<uint8_t*>(p) = sat_cast<uint8_t>(x); return;
    case DType::U16: { uint16_t v = sat_cast<uint16_t>(x); std::memcpy(p, &v, 2); return; }
    case DType::U32: { uint32_t v = sat_cast<uint32_t>(x); std::memcpy(p, &v, 4); return; }
    case DType::U64: { uint64_t v = sat_cast<uint64_t>(x); std::memcpy(p, &v, 8); return; }
    case DType::I8: *static_cast<int8_t*>(p) = sat_cast<int8_t>(x); return;
    case DType::I16: { int16_t v = sat_cast<int16_t>(x); std::memcpy(p, &v, 2); return; }
    case DType::I32: { int32_t v = sat_cast<int32_t>(x); std::memcpy(p, &v, 4); return; }
    case DType::I64: { int64_t v = sat_cast<int64_t>(x); std::memcpy(p, &v, 8); return; }
    case DType::F8E4M3: *static_cast<uint8_t*>(p) = f32_to_e4m3(static_cast<float>(x)); return;
    case DType::F8E5M2: *static_cast<uint8_t*>(p) = f32_to_e5m2(static_cast<float>(x)); return;
    case DType::F16: { uint16_t v = f64_to_f16(x); std::memcpy(p, &v, 2); return; }
    case DType::BF16: { uint16_t v = f64_to_bf16(x); std::memcpy(p, &v, 2); return; }
    case DType::F32: { float v = static_cast<float>(x); std::memcpy(p, &v, 4); return; }
    case DType::F64: std::memcpy(p, &x, 8); return;
    case DType::C64: { float v[2] = {static_cast<float>(x), 0.f}; std::memcpy(p, v, 8); return; }
    case DType::C128: { double v[2] = {x, 0.0}; std::memcpy(p, v, 16); return; }
  }
}

struct Error : std::runtime_error {
  using std::runtime_error::runtime_error;
  static Error shape(const std::string& op, const std::string& msg) { return Error("Shape { op: \"" + op + "\", msg: \"" + msg + "\" }"); }
  static Error backend(const std::string& msg) { return Error("Backend(\"" + msg + "\")"); }
};

}  // namespace ku

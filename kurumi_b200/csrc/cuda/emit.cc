// CUDA source emitter: turns a Fused expression into the body of a hand-written kernel template
// (pointwise, reduce, softmax / rmsnorm, GEMM epilogue) that NVRTC compiles for sm_100a.
//
// Value semantics follow the reference interpreter exactly (kurumi_core/src/interp/elementwise.rs,
// kurumi_core/src/dtype/traits/{float,int,elem}.rs, kurumi_core/src/dtype/convert.rs):
//   * no FMA contraction (kernels are compiled with --fmad=false), IEEE division and sqrt;
//   * f16 / bf16 / fp8 values live in registers as already-rounded f32 and are rounded again
//     after every primitive;
//   * integers wrap, x/0 = 0, MIN/-1 = MIN, shift counts are masked to the bit width;
//   * casts go through f64: float->int truncates and saturates with NaN -> 0, ->BOOL is x != 0.
// The reference's device backend generates one thread per element with per-leaf div/mod index
// math (kurumi_metal/src/backend/fuse/emit.rs:46-142); here the iteration space is collapsed
// first, shapes and strides are baked in as constants, and loads/stores are 128-bit wide
// wherever the innermost axis allows.
#include <algorithm>
#include <cmath>
#include <functional>
#include <sstream>

#include "emit_util.h"
#include "fuse.h"

namespace ku::cu {

const char* ctype(DType d) {
  switch (d) {
    case DType::BOOL: case DType::U8: return "u8";
    case DType::U16: return "u16";
    case DType::U32: return "u32";
    case DType::U64: return "u64";
    case DType::I8: return "i8";
    case DType::I16: return "i16";
    case DType::I32: return "i32";
    case DType::I64: return "i64";
    case DType::F64: return "double";
    case DType::F8E4M3: case DType::F8E5M2: case DType::F16: case DType::BF16: case DType::F32: return "float";
    default: throw Error::backend("complex dtypes are not supported by the CUDA backend");
  }
}
const char* stype(DType d) {
  switch (d) {
    case DType::F8E4M3: case DType::F8E5M2: return "u8";
    case DType::F16: case DType::BF16: return "u16";
    default: return ctype(d);
  }
}
static std::string lname(DType d) {
  std::string s = dtype_name(d);
  for (auto& c : s) c = static_cast<char>(std::tolower(c));
  return s;
}

std::string device_prelude() {
  return R"KU(
typedef unsigned char u8; typedef signed char i8; typedef unsigned short u16; typedef short i16;
typedef unsigned int u32; typedef int i32; typedef unsigned long long u64; typedef long long i64;
#define KU_INF __int_as_float(0x7f800000)
__device__ __forceinline__ float ku_dec_bf16(u16 b) { return __uint_as_float(((u32)b) << 16); }
__device__ __forceinline__ u16 ku_enc_bf16(float f) { u16 r; asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(r) : "f"(f)); return r; }
__device__ __forceinline__ float ku_dec_f16(u16 b) { float f; asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(b)); return f; }
__device__ __forceinline__ u16 ku_enc_f16(float f) { u16 r; asm("cvt.rn.f16.f32 %0, %1;" : "=h"(r) : "f"(f)); return r; }
__device__ __forceinline__ u8 ku_enc_f8e4m3(float f) { u16 r; asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.0f), "f"(f)); return (u8)(r & 0xff); }
__device__ __forceinline__ float ku_dec_f8e4m3(u8 b) { u32 h2; u16 s = b; asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(s)); return ku_dec_f16((u16)(h2 & 0xffffu)); }
__device__ __forceinline__ u8 ku_enc_f8e5m2(float f) { u16 r; asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.0f), "f"(f)); return (u8)(r & 0xff); }
__device__ __forceinline__ float ku_dec_f8e5m2(u8 b) { u32 h2; u16 s = b; asm("cvt.rn.f16x2.e5m2x2 %0, %1;" : "=r"(h2) : "h"(s)); return ku_dec_f16((u16)(h2 & 0xffffu)); }
__device__ __forceinline__ float ku_rnd_bf16(float f) { return ku_dec_bf16(ku_enc_bf16(f)); }
__device__ __forceinline__ float ku_rnd_f16(float f) { return ku_dec_f16(ku_enc_f16(f)); }
__device__ __forceinline__ float ku_rnd_f8e4m3(float f) { return ku_dec_f8e4m3(ku_enc_f8e4m3(f)); }
__device__ __forceinline__ float ku_rnd_f8e5m2(float f) { return ku_dec_f8e5m2(ku_enc_f8e5m2(f)); }
// f64 -> f32 with round-to-odd, so that a following round-to-nearest to a narrower format is a single rounding
__device__ __forceinline__ float ku_d2f_odd(double d) {
  float f = __double2float_rz(d);
  if (d == d && (double)f != d) f = __uint_as_float(__float_as_uint(f) | 1u);
  return f;
}
// float -> integer: truncate toward zero, saturate, NaN -> 0. The range tests are explicit: a bare
// float-to-int conversion of an out-of-range value is undefined to the optimiser, which may fold
// int -> double -> int round trips into a move.
__device__ __forceinline__ i32 ku_f2i_i32(double d) { if (!(d == d)) return 0; if (d <= -2147483648.0) return (i32)0x80000000u; if (d >= 2147483647.0) return 2147483647; return (i32)d; }
__device__ __forceinline__ u32 ku_f2i_u32(double d) { if (!(d == d)) return 0u; if (d <= 0.0) return 0u; if (d >= 4294967295.0) return 0xffffffffu; return (u32)d; }
__device__ __forceinline__ i64 ku_f2i_i64(double d) { if (!(d == d)) return 0ll; if (d <= -9223372036854775808.0) return (i64)0x8000000000000000ull; if (d >= 9223372036854775808.0) return 0x7fffffffffffffffll; return (i64)d; }
__device__ __forceinline__ u64 ku_f2i_u64(double d) { if (!(d == d)) return 0ull; if (d <= 0.0) return 0ull; if (d >= 18446744073709551616.0) return 0xffffffffffffffffull; return (u64)d; }
__device__ __forceinline__ i8 ku_f2i_i8(double d) { i32 v = ku_f2i_i32(d); return (i8)(v < -128 ? -128 : (v > 127 ? 127 : v)); }
__device__ __forceinline__ u8 ku_f2i_u8(double d) { i32 v = ku_f2i_i32(d); return (u8)(v < 0 ? 0 : (v > 255 ? 255 : v)); }
__device__ __forceinline__ i16 ku_f2i_i16(double d) { i32 v = ku_f2i_i32(d); return (i16)(v < -32768 ? -32768 : (v > 32767 ? 32767 : v)); }
__device__ __forceinline__ u16 ku_f2i_u16(double d) { i32 v = ku_f2i_i32(d); return (u16)(v < 0 ? 0 : (v > 65535 ? 65535 : v)); }
__device__ __forceinline__ u8 ku_f2i_bool(double d) { return (u8)(d != 0.0); }
// threefry2x32-20 keyed by a 64-bit seed, counter = flat element index
__device__ __forceinline__ u64 ku_threefry(u64 key, u64 ctr) {
  const u32 k0 = (u32)key, k1 = (u32)(key >> 32), k2 = 0x1BD11BDAu ^ k0 ^ k1;
  u32 x0 = (u32)ctr + k0, x1 = (u32)(ctr >> 32) + k1;
#define KU_R(s) x0 += x1; x1 = (x1 << s) | (x1 >> (32 - s)); x1 ^= x0;
  KU_R(13) KU_R(15) KU_R(26) KU_R(6)  x0 += k1; x1 += k2 + 1u;
  KU_R(17) KU_R(29) KU_R(16) KU_R(24) x0 += k2; x1 += k0 + 2u;
  KU_R(13) KU_R(15) KU_R(26) KU_R(6)  x0 += k0; x1 += k1 + 3u;
  KU_R(17) KU_R(29) KU_R(16) KU_R(24) x0 += k1; x1 += k2 + 4u;
  KU_R(13) KU_R(15) KU_R(26) KU_R(6)  x0 += k2; x1 += k0 + 5u;
#undef KU_R
  return (u64)x0 | ((u64)x1 << 32);
}
__device__ __forceinline__ float ku_uniform(u64 bits) { return (float)(((u32)bits) >> 8) / 16777216.0f; }
)KU";
}

namespace emitutil {   // shared with emit_index.cc (emit_util.h)
bool is_lowf(DType d) { return is_low_float(d); }
std::string rnd(DType d, const std::string& e) { return is_lowf(d) ? "ku_rnd_" + lname(d) + "(" + e + ")" : e; }
std::string dec(DType d, const std::string& e) { return is_lowf(d) ? "ku_dec_" + lname(d) + "(" + e + ")" : e; }
std::string enc(DType d, const std::string& e) { return is_lowf(d) ? "ku_enc_" + lname(d) + "(" + e + ")" : e; }
int bits_of(DType d) { return static_cast<int>(dtype_width(d)) * 8; }
const char* wrap_utype(DType d) { return dtype_width(d) == 8 ? "u64" : "u32"; }
unsigned pick_grid(int64_t work_items, unsigned per_block, int sm_count, unsigned blocks_per_sm) {
  int64_t blocks = (work_items + per_block - 1) / per_block;
  int64_t cap = static_cast<int64_t>(sm_count) * blocks_per_sm;
  return static_cast<unsigned>(std::max<int64_t>(1, std::min(blocks, cap)));
}
// Grid of a kernel whose CTAs loop over `items` lines, `cap` of them resident at once. Up to eight residencies' worth
// get a CTA per line: the hardware hands the next line to whichever SM has room, which measured better than a resident
// grid whose CTAs take 3 or 4 turns each (4096 lines on 1184 CTAs: 0.87 -> 0.90 of the copy rate), and better than
// fewer CTAs with equal turns (0.78). Beyond that a resident grid loops; the uneven last turn is then under an eighth.
unsigned line_grid(int64_t items, int64_t cap) {
  if (items <= cap * 8) return static_cast<unsigned>(std::max<int64_t>(1, items));
  return static_cast<unsigned>(cap);
}
}  // namespace emitutil
using namespace emitutil;

namespace {

std::string imm_literal(DType d, uint64_t bits) {
  std::ostringstream o;
  switch (d) {
    case DType::F32: o << "__uint_as_float(0x" << std::hex << (bits & 0xffffffffu) << "u)"; break;
    case DType::F64: o << "__longlong_as_double((i64)0x" << std::hex << bits << "ull)"; break;
    case DType::F16: case DType::BF16: o << "ku_dec_" << lname(d) << "((u16)0x" << std::hex << (bits & 0xffff) << "u)"; break;
    case DType::F8E4M3: case DType::F8E5M2: o << "ku_dec_" << lname(d) << "((u8)0x" << std::hex << (bits & 0xff) << "u)"; break;
    case DType::BOOL: o << "(u8)" << ((bits & 0xff) ? 1 : 0); break;
    default: o << "(" << ctype(d) << ")0x" << std::hex << bits << "ull"; break;
  }
  return o.str();
}

// value `e` of dtype `from` -> dtype `to`, through f64
std::string cast_expr(DType from, DType to, const std::string& e) {
  if (from == to) return e;
  const bool exact_in_f32 = is_lowf(from) || from == DType::F32 || from == DType::BOOL || dtype_width(from) <= 2;
  switch (to) {
    case DType::BOOL: return "(u8)((" + e + ") != 0)";
    case DType::U8: case DType::U16: case DType::U32: case DType::U64: case DType::I8: case DType::I16: case DType::I32: case DType::I64:
      return "ku_f2i_" + lname(to) + "((double)(" + e + "))";
    case DType::F64: return "(double)(" + e + ")";
    case DType::F32: return (is_lowf(from) || from == DType::F32) ? e : "(float)(double)(" + e + ")";
    case DType::F16: case DType::BF16:
      return exact_in_f32 ? "ku_rnd_" + lname(to) + "((float)(" + e + "))" : "ku_rnd_" + lname(to) + "(ku_d2f_odd((double)(" + e + ")))";
    case DType::F8E4M3: case DType::F8E5M2:
      return "ku_rnd_" + lname(to) + "((float)(double)(" + e + "))";
    default: throw Error::backend("cast to a complex dtype is not supported by the CUDA backend");
  }
}

std::string to_bits(DType d, const std::string& e) {
  switch (d) {
    case DType::F32: return "__float_as_uint(" + e + ")";
    case DType::F64: return "(u64)__double_as_longlong(" + e + ")";
    case DType::F16: case DType::BF16: case DType::F8E4M3: case DType::F8E5M2: return enc(d, e);
    default: return std::string("(") + (dtype_width(d) == 8 ? "u64" : dtype_width(d) == 4 ? "u32" : dtype_width(d) == 2 ? "u16" : "u8") + ")(" + e + ")";
  }
}
std::string from_bits(DType d, const std::string& b) {
  switch (d) {
    case DType::F32: return "__uint_as_float(" + b + ")";
    case DType::F64: return "__longlong_as_double((i64)(" + b + "))";
    case DType::F16: case DType::BF16: case DType::F8E4M3: case DType::F8E5M2: return dec(d, "(" + std::string(stype(d)) + ")(" + b + ")");
    case DType::BOOL: return "(u8)((" + b + ") != 0)";
    default: return std::string("(") + ctype(d) + ")(" + b + ")";
  }
}

// one primitive on register values
std::string op_expr(const FNode& n, DType in_dt, const std::string& a, const std::string& b, const std::string& c) {
  const DType d = n.dtype;
  const bool flt = is_float(d);
  auto wrap = [&](const std::string& x) { return std::string("(") + ctype(d) + ")(" + x + ")"; };
  const std::string U = wrap_utype(d);
  switch (n.op) {
    case OpKind::Add: return flt ? rnd(d, a + " + " + b) : wrap("(" + U + ")" + a + " + (" + U + ")" + b);
    case OpKind::Mul: return flt ? rnd(d, a + " * " + b) : wrap("(" + U + ")" + a + " * (" + U + ")" + b);
    case OpKind::Max:
      if (d == DType::F64) return "fmax(" + a + ", " + b + ")";
      return flt ? "fmaxf(" + a + ", " + b + ")" : "(" + a + " > " + b + " ? " + a + " : " + b + ")";
    case OpKind::Neg: return flt ? "(-" + a + ")" : wrap("(" + U + ")0 - (" + U + ")" + a);
    case OpKind::IDiv: {
      std::string s = "(" + b + " == 0 ? (" + ctype(d) + ")0 : ";
      if (is_signed(d)) {
        std::string mn = dtype_width(d) == 8 ? "(i64)0x8000000000000000ull" : "(" + std::string(ctype(d)) + ")(-(1ll << " + std::to_string(bits_of(d) - 1) + "))";
        s += "((" + a + " == " + mn + " && " + b + " == (" + ctype(d) + ")-1) ? " + a + " : " + wrap(a + " / " + b) + "))";
      } else {
        s += wrap(a + " / " + b) + ")";
      }
      return s;
    }
    case OpKind::Shl: return wrap("(" + U + ")" + a + " << ((u32)" + b + " & " + std::to_string(bits_of(d) - 1) + "u)");
    case OpKind::Shr: return wrap(a + " >> ((u32)" + b + " & " + std::to_string(bits_of(d) - 1) + "u)");
    case OpKind::And: return d == DType::BOOL ? "(u8)(" + a + " & " + b + ")" : wrap(a + " & " + b);
    case OpKind::Or: return d == DType::BOOL ? "(u8)(" + a + " | " + b + ")" : wrap(a + " | " + b);
    case OpKind::Xor: return d == DType::BOOL ? "(u8)(" + a + " ^ " + b + ")" : wrap(a + " ^ " + b);
    case OpKind::CmpLt: return "(u8)(" + a + " < " + b + ")";
    case OpKind::CmpEq: return "(u8)(" + a + " == " + b + ")";
    case OpKind::Where: return "(" + a + " ? " + b + " : " + c + ")";
    case OpKind::Recip: return d == DType::F64 ? "(1.0 / " + a + ")" : rnd(d, "1.0f / " + a);
    case OpKind::Sqrt: return d == DType::F64 ? "sqrt(" + a + ")" : rnd(d, "sqrtf(" + a + ")");
    case OpKind::Exp2: return d == DType::F64 ? "exp2(" + a + ")" : rnd(d, "exp2f(" + a + ")");
    case OpKind::Log2: return d == DType::F64 ? "log2(" + a + ")" : rnd(d, "log2f(" + a + ")");
    case OpKind::Sin: return d == DType::F64 ? "sin(" + a + ")" : rnd(d, "sinf(" + a + ")");
    case OpKind::Floor: return d == DType::F64 ? "floor(" + a + ")" : "floorf(" + a + ")";
    case OpKind::Cast: return cast_expr(in_dt, d, a);
    case OpKind::Bitcast: return from_bits(d, to_bits(in_dt, a));
    case OpKind::Detach: return a;
    default: throw Error::backend(std::string("op ") + op_name(n.op) + " cannot appear inside a fused expression");
  }
}

// ---- collapsed iteration space ------------------------------------------------------------------
struct Space {
  std::vector<int64_t> dims;
  std::vector<std::vector<int64_t>> ls;  // [leaf][dim] element strides
  std::vector<int> axis_dim;             // original axis -> dim, -1 when dropped
  int special = -1;                      // dim of the reduce / softmax axis
};

Space collapse(const Fused& f, int special_axis) {
  const size_t rank = f.shape.size();
  std::vector<bool> guarded(rank, false);
  for (auto& l : f.leaves) for (auto& g : l.view.guards) guarded[g.axis] = true;
  Space s;
  s.axis_dim.assign(rank, -1);
  s.ls.assign(f.leaves.size(), {});
  bool cur_locked = true;  // may the current last dim absorb the next axis?
  for (size_t ax = 0; ax < rank; ++ax) {
    const bool sp = static_cast<int>(ax) == special_axis;
    const bool locked = sp || guarded[ax];
    if (f.shape[ax] == 1 && !locked) continue;  // contributes nothing
    bool merge = !s.dims.empty() && !cur_locked && !locked;
    for (size_t li = 0; merge && li < f.leaves.size(); ++li)
      if (s.ls[li].back() != f.leaves[li].view.stride[ax] * static_cast<int64_t>(f.shape[ax])) merge = false;
    if (merge) {
      s.dims.back() *= static_cast<int64_t>(f.shape[ax]);
      for (size_t li = 0; li < f.leaves.size(); ++li) s.ls[li].back() = f.leaves[li].view.stride[ax];
    } else {
      s.dims.push_back(static_cast<int64_t>(f.shape[ax]));
      for (size_t li = 0; li < f.leaves.size(); ++li) s.ls[li].push_back(f.leaves[li].view.stride[ax]);
      cur_locked = locked;
      if (sp) s.special = static_cast<int>(s.dims.size()) - 1;
    }
    s.axis_dim[ax] = static_cast<int>(s.dims.size()) - 1;
  }
  return s;
}

bool needs_i64(const Fused& f) {
  int64_t mx = static_cast<int64_t>(numel(f.shape));
  for (auto& l : f.leaves) { int64_t lo, hi; l.view.extent(&lo, &hi); mx = std::max({mx, hi, -lo}); }
  return mx >= (int64_t(1) << 31) - 1;
}

struct Gen {
  const Fused& f;
  const Space& sp;
  std::string idx_t;
  std::vector<int> ptr_arg;  // leaf -> pointer parameter index (-1 none)
  std::vector<int> args;     // pointer parameters: leaf indices

  Gen(const Fused& f_, const Space& sp_) : f(f_), sp(sp_) {
    idx_t = needs_i64(f) ? "i64" : "i32";
    ptr_arg.assign(f.leaves.size(), -1);
    for (size_t li = 0; li < f.leaves.size(); ++li) {
      const Leaf& l = f.leaves[li];
      if (l.kind == LeafKind::Buffer || (l.kind == LeafKind::Rand && l.slot >= 0)) {
        ptr_arg[li] = static_cast<int>(args.size());
        args.push_back(static_cast<int>(li));
      }
    }
  }
  std::string params() const {
    std::string s;
    for (size_t i = 0; i < args.size(); ++i) s += "const void* __restrict__ p" + std::to_string(i) + ", ";
    return s;
  }
  // flat source index of leaf li given coordinate variable names per dim ("" = coordinate is 0)
  std::string offset(size_t li, const std::vector<std::string>& c) const {
    std::ostringstream o;
    o << "(" << idx_t << ")" << f.leaves[li].view.base;
    for (size_t d = 0; d < sp.dims.size(); ++d) {
      const int64_t st = sp.ls[li][d];
      if (st == 0 || c[d].empty()) continue;
      o << " + (" << idx_t << ")" << c[d] << " * (" << idx_t << ")" << st;
    }
    return o.str();
  }
  std::string guard(size_t li, const std::vector<std::string>& c) const {
    std::string g;
    for (auto& gd : f.leaves[li].view.guards) {
      const int d = sp.axis_dim[gd.axis];
      const std::string cv = c[static_cast<size_t>(d)].empty() ? "0" : c[static_cast<size_t>(d)];
      if (!g.empty()) g += " && ";
      g += "(" + cv + " >= " + std::to_string(gd.lo) + " && " + cv + " < " + std::to_string(gd.hi) + ")";
    }
    return g;
  }
  // register value of leaf li at the coordinates; `acc` names the GEMM accumulator value
  std::string leaf_value(size_t li, const std::vector<std::string>& c, const std::string& acc = "") const {
    const Leaf& l = f.leaves[li];
    std::string v;
    switch (l.kind) {
      case LeafKind::Buffer:
        v = dec(l.dtype, "((const " + std::string(stype(l.dtype)) + "*)p" + std::to_string(ptr_arg[li]) + ")[" + offset(li, c) + "]");
        break;
      case LeafKind::Imm: v = imm_literal(l.dtype, l.imm); break;
      case LeafKind::Iota: {
        std::string flat = "(i64)(" + offset(li, c) + ")";
        v = cast_expr(DType::I64, l.dtype, "((" + flat + " / " + std::to_string(l.iota_stride) + "ll) % " + std::to_string(l.iota_len) + "ll)");
        break;
      }
      case LeafKind::Rand: {
        std::string seed = l.slot >= 0 ? "(u64)(i64)(((const " + std::string(stype(l.seed_dtype)) + "*)p" + std::to_string(ptr_arg[li]) + ")[0])"
                                       : "0x" + [&] { std::ostringstream h; h << std::hex << l.imm; return h.str(); }() + "ull";
        v = "ku_uniform(ku_threefry(" + seed + ", (u64)(i64)(" + offset(li, c) + ")))";
        break;
      }
      case LeafKind::Acc: v = acc; break;
    }
    std::string g = guard(li, c);
    if (!g.empty()) v = "((" + g + ") ? " + v + " : " + imm_literal(l.dtype, 0) + ")";
    return v;
  }
  // storage bits of a buffer leaf at the coordinates ("" when the leaf has no storage to read)
  std::string leaf_raw(size_t li, const std::vector<std::string>& c) const {
    const Leaf& l = f.leaves[li];
    if (l.kind != LeafKind::Buffer || !is_lowf(l.dtype)) return "";  // wider types hold their own bits in registers
    std::string v = "((const " + std::string(stype(l.dtype)) + "*)p" + std::to_string(ptr_arg[li]) + ")[" + offset(li, c) + "]";
    std::string g = guard(li, c);
    if (!g.empty()) v = "((" + g + ") ? " + v + " : (" + std::string(stype(l.dtype)) + ")0)";
    return v;
  }
  // Is the root a bare load of a buffer leaf (pure movement)? Then the stored element is the loaded
  // bit pattern itself, so NaN payloads of the narrow float formats survive a copy.
  bool root_is_copy() const { return f.nodes[static_cast<size_t>(f.root)].op == OpKind::Input && f.leaves[static_cast<size_t>(f.nodes[static_cast<size_t>(f.root)].leaf)].kind == LeafKind::Buffer; }
  // storage-typed expression to store for the root
  std::string root_store(const std::vector<std::string>& leaf_raws) const {
    const FNode& r = f.nodes[static_cast<size_t>(f.root)];
    if (root_is_copy() && !leaf_raws[static_cast<size_t>(r.leaf)].empty()) return leaf_raws[static_cast<size_t>(r.leaf)];
    if (r.op == OpKind::Bitcast && is_lowf(r.dtype)) {  // reinterpretation: store the source bits, do not round-trip them through a float
      const FNode& src = f.nodes[static_cast<size_t>(r.in[0])];
      const std::string raw = src.op == OpKind::Input ? leaf_raws[static_cast<size_t>(src.leaf)] : std::string();
      return "(" + std::string(stype(r.dtype)) + ")(" + (raw.empty() ? to_bits(src.dtype, "v" + std::to_string(r.in[0])) : raw) + ")";
    }
    return enc(r.dtype, "v" + std::to_string(f.root));
  }
  // statements computing every node; the root value is left in `v<root>`. `leaf_raws` (optional)
  // gives the storage bits of buffer leaves, used by a Bitcast that sits directly on a load.
  std::string body(const std::vector<std::string>& leaf_vals, const std::string& ind, const std::vector<std::string>* leaf_raws = nullptr) const {
    std::vector<bool> need(f.nodes.size(), false);
    need[static_cast<size_t>(f.root)] = true;
    for (size_t i = f.nodes.size(); i-- > 0;)
      if (need[i]) for (int k = 0; k < 3; ++k) if (f.nodes[i].in[k] >= 0) need[static_cast<size_t>(f.nodes[i].in[k])] = true;
    std::ostringstream o;
    for (size_t i = 0; i < f.nodes.size(); ++i) {
      if (!need[i]) continue;
      const FNode& n = f.nodes[i];
      o << ind << "const " << ctype(n.dtype) << " v" << i << " = ";
      if (n.op == OpKind::Input) o << leaf_vals[static_cast<size_t>(n.leaf)];
      else if (n.op == OpKind::Bitcast && leaf_raws && f.nodes[static_cast<size_t>(n.in[0])].op == OpKind::Input &&
               !(*leaf_raws)[static_cast<size_t>(f.nodes[static_cast<size_t>(n.in[0])].leaf)].empty()) {
        o << from_bits(n.dtype, (*leaf_raws)[static_cast<size_t>(f.nodes[static_cast<size_t>(n.in[0])].leaf)]);
      } else {
        auto nm = [&](int k) { return n.in[k] >= 0 ? "v" + std::to_string(n.in[k]) : std::string(); };
        o << op_expr(n, n.in[0] >= 0 ? f.nodes[static_cast<size_t>(n.in[0])].dtype : n.dtype, nm(0), nm(1), nm(2));
      }
      o << ";\n";
    }
    return o.str();
  }
};

// decompose a linear index into coordinates over dims[first..last)
std::string decompose(const std::string& lin, const std::vector<int64_t>& dims, size_t first, size_t last, const std::string& idx_t,
                      const std::string& prefix, const std::string& ind) {
  std::ostringstream o;
  const std::string t = "t_" + prefix + std::to_string(first);
  if (last <= first) return "";
  o << ind << idx_t << " " << t << " = " << lin << ";\n";
  for (size_t d = last; d-- > first;) {
    if (d == first) o << ind << "const " << idx_t << " " << prefix << d << " = " << t << ";\n";
    else {
      o << ind << "const " << idx_t << " " << prefix << d << " = " << t << " % " << dims[d] << ";\n";
      o << ind << t << " /= " << dims[d] << ";\n";
    }
  }
  return o.str();
}

// can leaf li be read with one aligned vector of `vec` elements along the innermost dim?
bool vec_ok(const Fused& f, const Space& sp, size_t li, int vec) {
  const Leaf& l = f.leaves[li];
  if (l.kind != LeafKind::Buffer || !l.view.guards.empty()) return false;
  if (sp.ls[li].back() != 1) return false;
  if (l.view.base % vec) return false;
  for (size_t d = 0; d + 1 < sp.dims.size(); ++d) if (sp.ls[li][d] % vec) return false;
  return true;
}

const char* block_reduce_helpers() {
  return R"KU(
// warp shuffle tree, then one shared-memory stage across the warps of the CTA
template <typename T, typename F> __device__ __forceinline__ T ku_block_reduce(T v, F f, T* smem) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = f(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if ((threadIdx.x & 31) == 0) smem[w] = v;
  __syncthreads();
  T r = smem[0];
  for (int i = 1; i < nw; ++i) r = f(r, smem[i]);
  return r;
}
)KU";
}

}  // namespace

// ---- pointwise ------------------------------------------------------------------------------------
namespace {
// Dim along which the leaves that are strided along the output's innermost dim are contiguous instead (a transposed
// operand), or -1. Such a leaf read at the output's coordinates touches one element per 32-byte sector.
int transposed_dim(const Fused& f, const Space& sp) {
  const size_t nd = sp.dims.size();
  if (nd < 2 || sp.dims.back() < 32) return -1;
  for (size_t li = 0; li < f.leaves.size(); ++li) {
    const Leaf& l = f.leaves[li];
    if (l.kind != LeafKind::Buffer || !l.view.guards.empty()) continue;
    const int64_t sl = sp.ls[li].back();
    if (sl == 0 || sl == 1) continue;
    for (size_t d = 0; d + 1 < nd; ++d)
      if (sp.ls[li][d] == 1 && sp.dims[d] >= 32) return static_cast<int>(d);
  }
  return -1;
}

// Pointwise pass with transposed operands: a CTA takes a T x T tile over (dim a, innermost dim b). The leaves that are
// contiguous along a are read along a (coalesced) into shared memory and read back transposed; every other leaf is read
// at the output's coordinates; the stores run along b. Same expression body as ku_pointwise, so the same values.
Emitted emit_pointwise_transposed(const Fused& f, const Space& sp, const Gen& g, int a_dim, int sm_count) {
  const size_t nd = sp.dims.size(), a = static_cast<size_t>(a_dim), b = nd - 1;
  const DType od = f.dtype();
  std::vector<bool> staged(f.leaves.size(), false);
  size_t min_w = dtype_width(od);
  for (size_t li = 0; li < f.leaves.size(); ++li) {
    const Leaf& l = f.leaves[li];
    const int64_t sl = sp.ls[li].back();
    if (l.kind == LeafKind::Buffer && l.view.guards.empty() && sl != 0 && sl != 1 && sp.ls[li][a] == 1) {
      staged[li] = true;
      min_w = std::min(min_w, dtype_width(l.dtype));
    }
  }
  const int T = min_w <= 2 ? 64 : 32, RS = 256 / T;
  std::vector<int64_t> tdims(sp.dims);
  tdims[a] = (sp.dims[a] + T - 1) / T;
  tdims[b] = (sp.dims[b] + T - 1) / T;
  int64_t ntiles = 1;
  for (int64_t d : tdims) ntiles *= d;
  std::ostringstream o;
  o << device_prelude();
  o << "extern \"C\" __global__ void __launch_bounds__(256) ku_pointwise_t(" << g.params() << "void* __restrict__ out) {\n";
  for (size_t li = 0; li < f.leaves.size(); ++li)
    if (staged[li]) o << "  __shared__ " << stype(f.leaves[li].dtype) << " s" << li << "[" << T << "][" << T + std::max<size_t>(1, 4 / dtype_width(f.leaves[li].dtype)) << "];\n";
  o << "  const int tx = threadIdx.x % " << T << ", ty = threadIdx.x / " << T << ";\n";
  o << "  for (" << g.idx_t << " tile = blockIdx.x; tile < " << ntiles << "; tile += gridDim.x) {\n";
  o << decompose("tile", tdims, 0, nd, g.idx_t, "q", "    ");
  o << "    const " << g.idx_t << " a0 = q" << a << " * " << T << ", b0 = q" << b << " * " << T << ";\n";
  std::vector<std::string> coords(nd);
  for (size_t d = 0; d < nd; ++d) coords[d] = "q" + std::to_string(d);
  coords[a] = "ca"; coords[b] = "cb";
  o << "    __syncthreads();   // the tile before has been read out\n";
  o << "#pragma unroll\n    for (int r = 0; r < " << T << "; r += " << RS << ") {\n";
  o << "      const " << g.idx_t << " ca = a0 + tx, cb = b0 + ty + r;\n";
  o << "      if (ca < " << sp.dims[a] << " && cb < " << sp.dims[b] << ") {\n";
  for (size_t li = 0; li < f.leaves.size(); ++li)
    if (staged[li]) o << "        s" << li << "[ty + r][tx] = ((const " << stype(f.leaves[li].dtype) << "*)p" << g.ptr_arg[li] << ")[" << g.offset(li, coords) << "];\n";
  o << "      }\n    }\n    __syncthreads();\n";
  o << "#pragma unroll\n    for (int r = 0; r < " << T << "; r += " << RS << ") {\n";
  o << "      const " << g.idx_t << " ca = a0 + ty + r, cb = b0 + tx;\n";
  o << "      if (ca < " << sp.dims[a] << " && cb < " << sp.dims[b] << ") {\n";
  std::vector<std::string> lv(f.leaves.size()), lr(f.leaves.size());
  for (size_t li = 0; li < f.leaves.size(); ++li) {
    const std::string raw = "s" + std::to_string(li) + "[tx][ty + r]";
    lv[li] = staged[li] ? dec(f.leaves[li].dtype, raw) : g.leaf_value(li, coords);
    lr[li] = !is_lowf(f.leaves[li].dtype) ? std::string() : staged[li] ? raw : g.leaf_raw(li, coords);
  }
  o << g.body(lv, "        ", &lr);
  std::ostringstream lin;
  int64_t stride = 1;
  std::vector<int64_t> ostr(nd);
  for (size_t d = nd; d-- > 0;) { ostr[d] = stride; stride *= sp.dims[d]; }
  for (size_t d = 0; d < nd; ++d) lin << (d ? " + " : "") << "(" << g.idx_t << ")" << coords[d] << " * (" << g.idx_t << ")" << ostr[d];
  o << "        ((" << stype(od) << "*)out)[" << lin.str() << "] = " << g.root_store(lr) << ";\n";
  o << "      }\n    }\n  }\n}\n";
  Emitted e;
  e.source = o.str();
  e.entry = "ku_pointwise_t";
  e.leaf_args = g.args;
  e.block = 256;
  e.grid = line_grid(ntiles, static_cast<int64_t>(sm_count) * 8);   // (larger grids measured the same or slower here)
  e.family = "pointwise_tiled";
  return e;
}
}  // namespace

Emitted emit_pointwise(const Fused& f, int sm_count) {
  Space sp = collapse(f, -1);
  if (sp.dims.empty()) { sp.dims.push_back(1); for (auto& v : sp.ls) v.push_back(0); }
  Gen g(f, sp);
  if (const int a = transposed_dim(f, sp); a >= 0) return emit_pointwise_transposed(f, sp, g, a, sm_count);
  const DType od = f.dtype();
  const int64_t total = static_cast<int64_t>(numel(f.shape));
  const int64_t inner = sp.dims.back();
  int vec = static_cast<int>(16 / dtype_width(od));
  while (vec > 1 && inner % vec) vec >>= 1;
  const size_t nd = sp.dims.size();
  std::ostringstream o;
  o << device_prelude();
  o << "extern \"C\" __global__ void __launch_bounds__(256) ku_pointwise(" << g.params() << "void* __restrict__ out) {\n";
  o << "  const " << g.idx_t << " NV = " << total / vec << ";\n";
  o << "  for (" << g.idx_t << " v = blockIdx.x * 256 + threadIdx.x; v < NV; v += (" << g.idx_t << ")gridDim.x * 256) {\n";
  o << "    const " << g.idx_t << " e0 = v * " << vec << ";\n";
  o << decompose("e0", sp.dims, 0, nd, g.idx_t, "c", "    ");
  std::vector<std::string> coords(nd);
  for (size_t d = 0; d < nd; ++d) coords[d] = "c" + std::to_string(d);
  // vector pre-loads
  std::vector<bool> pre(f.leaves.size(), false);
  for (size_t li = 0; li < f.leaves.size(); ++li) {
    if (vec > 1 && vec_ok(f, sp, li, vec)) {
      pre[li] = true;
      const std::string st = stype(f.leaves[li].dtype);
      const size_t bytes = dtype_width(f.leaves[li].dtype) * static_cast<size_t>(vec);
      o << "    " << st << " b" << li << "[" << vec << "];\n";
      const std::string src = "((const " + st + "*)p" + std::to_string(g.ptr_arg[li]) + " + (" + g.offset(li, coords) + "))";
      if (bytes % 16 == 0) for (size_t q = 0; q < bytes / 16; ++q) o << "    ((uint4*)b" << li << ")[" << q << "] = ((const uint4*)" << src << ")[" << q << "];\n";
      else if (bytes == 8) o << "    *(uint2*)b" << li << " = *(const uint2*)" << src << ";\n";
      else if (bytes == 4) o << "    *(u32*)b" << li << " = *(const u32*)" << src << ";\n";
      else o << "    *(u16*)b" << li << " = *(const u16*)" << src << ";\n";
    }
  }
  o << "    " << stype(od) << " r[" << vec << "];\n";
  o << "#pragma unroll\n    for (int l = 0; l < " << vec << "; ++l) {\n";
  std::vector<std::string> lc = coords;
  lc.back() = "(c" + std::to_string(nd - 1) + " + l)";
  std::vector<std::string> lv(f.leaves.size()), lr(f.leaves.size());
  for (size_t li = 0; li < f.leaves.size(); ++li) {
    lv[li] = pre[li] ? dec(f.leaves[li].dtype, "b" + std::to_string(li) + "[l]") : g.leaf_value(li, lc);
    lr[li] = !is_lowf(f.leaves[li].dtype) ? std::string() : pre[li] ? "b" + std::to_string(li) + "[l]" : g.leaf_raw(li, lc);
  }
  o << g.body(lv, "      ", &lr);
  o << "      r[l] = " << g.root_store(lr) << ";\n    }\n";
  const size_t obytes = dtype_width(od) * static_cast<size_t>(vec);
  const std::string dst = "((" + std::string(stype(od)) + "*)out + e0)";
  if (obytes == 16) o << "    *(uint4*)" << dst << " = *(const uint4*)r;\n";
  else if (obytes == 8) o << "    *(uint2*)" << dst << " = *(const uint2*)r;\n";
  else if (obytes == 4) o << "    *(u32*)" << dst << " = *(const u32*)r;\n";
  else if (obytes == 2) o << "    *(u16*)" << dst << " = *(const u16*)r;\n";
  else o << "    *" << dst << " = r[0];\n";
  o << "  }\n}\n";
  Emitted e;
  e.source = o.str();
  e.entry = "ku_pointwise";
  e.leaf_args = g.args;
  e.block = 256;
  // Eight CTAs of 256 threads fill an SM, but a grid of only the resident CTAs, each looping far, measured 0.83-0.90 of the
  // copy rate on [8192, 8192] f32 passes against 0.95-1.0 with eight times as many CTAs and shorter loops
  e.grid = pick_grid(total / vec, 256, sm_count, kStreamCtasPerSm);
  e.family = "pointwise";
  return e;
}

// ---- reductions -----------------------------------------------------------------------------------
namespace {
struct RedOps { std::string acc_t, identity, combine; };
RedOps red_ops(OpKind k, DType d) {
  RedOps r;
  r.acc_t = ctype(d);
  const bool flt = is_float(d);
  const std::string U = wrap_utype(d);
  if (k == OpKind::Sum) {
    r.identity = flt ? (d == DType::F64 ? "0.0" : "0.0f") : "0";
    r.combine = flt ? "(a + b)" : "(" + r.acc_t + ")((" + U + ")a + (" + U + ")b)";
  } else if (k == OpKind::Prod) {
    r.identity = flt ? (d == DType::F64 ? "1.0" : "1.0f") : "1";
    r.combine = flt ? "(a * b)" : "(" + r.acc_t + ")((" + U + ")a * (" + U + ")b)";
  } else {
    if (d == DType::F64) { r.identity = "-__longlong_as_double(0x7ff0000000000000ll)"; r.combine = "fmax(a, b)"; }
    else if (d == DType::F8E4M3) { r.identity = "-448.0f"; r.combine = "fmaxf(a, b)"; }
    else if (d == DType::F8E5M2) { r.identity = "-57344.0f"; r.combine = "fmaxf(a, b)"; }
    else if (flt) { r.identity = "-KU_INF"; r.combine = "fmaxf(a, b)"; }
    else {
      r.combine = "(a > b ? a : b)";
      if (is_signed(d)) r.identity = dtype_width(d) == 8 ? "(i64)0x8000000000000000ull" : "(" + r.acc_t + ")(-(1ll << " + std::to_string(bits_of(d) - 1) + "))";
      else r.identity = "0";
    }
  }
  return r;
}
}  // namespace

Emitted emit_reduce(const Fused& f, OpKind kind, size_t axis, int sm_count) {
  Space sp = collapse(f, static_cast<int>(axis));
  Gen g(f, sp);
  const DType d = f.dtype();
  RedOps ro = red_ops(kind, d);
  const size_t nd = sp.dims.size();
  const size_t ax = static_cast<size_t>(sp.special);
  const int64_t len = sp.dims[ax];
  int64_t outer = 1, inner = 1;
  for (size_t q = 0; q < ax; ++q) outer *= sp.dims[q];
  for (size_t q = ax + 1; q < nd; ++q) inner *= sp.dims[q];
  std::vector<std::string> coords(nd);
  for (size_t q = 0; q < nd; ++q) coords[q] = "c" + std::to_string(q);
  coords[ax] = "k";
  std::ostringstream o;
  o << device_prelude() << block_reduce_helpers();
  o << "struct KuComb { __device__ __forceinline__ " << ro.acc_t << " operator()(" << ro.acc_t << " a, " << ro.acc_t << " b) const { return " << ro.combine << "; } };\n";
  Emitted e;
  e.leaf_args = g.args;
  const bool row_kernel = inner == 1 && len >= 128;
  if (row_kernel) {
    // one CTA per output row; each thread folds a strided set of vectors, then a shuffle / shared-memory tree
    int vec = 4;
    while (vec > 1 && len % vec) vec >>= 1;
    std::vector<bool> pre(f.leaves.size(), false);
    o << "extern \"C\" __global__ void __launch_bounds__(256) ku_reduce_rows(" << g.params() << "void* __restrict__ out) {\n";
    o << "  __shared__ " << ro.acc_t << " red[32];\n  const KuComb comb;\n";
    o << "  for (" << g.idx_t << " row = blockIdx.x; row < " << outer << "; row += gridDim.x) {\n";
    o << decompose("row", sp.dims, 0, ax, g.idx_t, "c", "    ");
    o << "    " << ro.acc_t << " acc[" << vec << "];\n#pragma unroll\n    for (int l = 0; l < " << vec << "; ++l) acc[l] = " << ro.identity << ";\n";
    o << "#pragma unroll 4\n    for (" << g.idx_t << " k0 = threadIdx.x * " << vec << "; k0 < " << len << "; k0 += 256 * " << vec << ") {\n";
    std::vector<std::string> c0 = coords;
    c0[ax] = "k0";
    for (size_t li = 0; li < f.leaves.size(); ++li) {
      if (vec > 1 && vec_ok(f, sp, li, vec)) {
        pre[li] = true;
        const std::string st = stype(f.leaves[li].dtype);
        const size_t bytes = dtype_width(f.leaves[li].dtype) * static_cast<size_t>(vec);
        o << "      " << st << " b" << li << "[" << vec << "];\n";
        const std::string src = "((const " + st + "*)p" + std::to_string(g.ptr_arg[li]) + " + (" + g.offset(li, c0) + "))";
        if (bytes % 16 == 0) for (size_t q = 0; q < bytes / 16; ++q) o << "      ((uint4*)b" << li << ")[" << q << "] = ((const uint4*)" << src << ")[" << q << "];\n";
        else if (bytes == 8) o << "      *(uint2*)b" << li << " = *(const uint2*)" << src << ";\n";
        else o << "      *(u32*)b" << li << " = *(const u32*)" << src << ";\n";
      }
    }
    o << "#pragma unroll\n      for (int l = 0; l < " << vec << "; ++l) {\n        const " << g.idx_t << " k = k0 + l;\n";
    std::vector<std::string> lv(f.leaves.size());
    for (size_t li = 0; li < f.leaves.size(); ++li) lv[li] = pre[li] ? dec(f.leaves[li].dtype, "b" + std::to_string(li) + "[l]") : g.leaf_value(li, coords);
    o << g.body(lv, "        ");
    o << "        acc[l] = comb(acc[l], v" << f.root << ");\n      }\n    }\n";
    o << "    " << ro.acc_t << " a = acc[0];\n#pragma unroll\n    for (int l = 1; l < " << vec << "; ++l) a = comb(a, acc[l]);\n";
    o << "    a = ku_block_reduce(a, comb, red);\n";
    o << "    if (threadIdx.x == 0) ((" << stype(d) << "*)out)[row] = " << enc(d, "a") << ";\n  }\n}\n";
    e.entry = "ku_reduce_rows";
    e.block = 256;
    e.grid = line_grid(outer, static_cast<int64_t>(sm_count) * 8);
    e.family = "reduce_rows";
  } else if (len >= 64 && outer * inner <= static_cast<int64_t>(sm_count) * 512) {
    // few outputs, a long axis (a reduction over rows, a short tensor's last axis): a CTA owns 32 neighbouring outputs and
    // cuts the axis into SEG contiguous segments, one per warp-row of threads; a thread folds its segment in index order,
    // then the segments combine in ascending order (a fixed order: results do not depend on the launch)
    const int64_t outs = outer * inner;
    const int threads = len >= 2048 ? 1024 : 256, seg = threads / 32;
    const int64_t chunk = (len + seg - 1) / seg;
    o << "extern \"C\" __global__ void __launch_bounds__(" << threads << ") ku_reduce_split(" << g.params() << "void* __restrict__ out) {\n  const KuComb comb;\n";
    o << "  __shared__ " << ro.acc_t << " part[" << seg << "][33];\n";
    o << "  const int col = threadIdx.x & 31, sg = threadIdx.x >> 5;\n";
    o << "  for (" << g.idx_t << " o0 = (" << g.idx_t << ")blockIdx.x * 32; o0 < " << outs << "; o0 += (" << g.idx_t << ")gridDim.x * 32) {\n";
    o << "    const " << g.idx_t << " o = o0 + col;\n";
    o << "    " << ro.acc_t << " acc = " << ro.identity << ";\n";
    o << "    if (o < " << outs << ") {\n";
    o << "      const " << g.idx_t << " oi = o % " << inner << ", oo = o / " << inner << ";\n";
    if (ax > 0) o << decompose("oo", sp.dims, 0, ax, g.idx_t, "c", "      ");
    if (ax + 1 < nd) {
      std::vector<int64_t> tail(sp.dims);
      o << decompose("oi", tail, ax + 1, nd, g.idx_t, "c", "      ");
    }
    o << "      const " << g.idx_t << " k1 = (" << g.idx_t << ")(sg + 1) * " << chunk << " < " << len << " ? (" << g.idx_t << ")(sg + 1) * " << chunk << " : " << len << ";\n";
    o << "      for (" << g.idx_t << " k = (" << g.idx_t << ")sg * " << chunk << "; k < k1; ++k) {\n";
    {
      std::vector<std::string> lv(f.leaves.size());
      for (size_t li = 0; li < f.leaves.size(); ++li) lv[li] = g.leaf_value(li, coords);
      o << g.body(lv, "        ");
    }
    o << "        acc = comb(acc, v" << f.root << ");\n      }\n    }\n";
    o << "    part[sg][col] = acc;\n    __syncthreads();\n";
    o << "    if (sg == 0 && o < " << outs << ") {\n      " << ro.acc_t << " a = part[0][col];\n";
    o << "      for (int q = 1; q < " << seg << "; ++q) a = comb(a, part[q][col]);\n";
    o << "      ((" << stype(d) << "*)out)[o] = " << enc(d, "a") << ";\n    }\n    __syncthreads();\n  }\n}\n";
    e.entry = "ku_reduce_split";
    e.block = static_cast<unsigned>(threads);
    e.grid = static_cast<unsigned>(std::max<int64_t>(1, std::min<int64_t>((outs + 31) / 32, static_cast<int64_t>(sm_count) * 4)));
    e.family = "reduce_split";
  } else {
    // one thread per output element, folding the axis in index order (the interpreter's own order);
    // adjacent threads walk adjacent inner positions, so loads coalesce when the axis is not innermost
    const int64_t outs = outer * inner;
    o << "extern \"C\" __global__ void __launch_bounds__(256) ku_reduce_fold(" << g.params() << "void* __restrict__ out) {\n  const KuComb comb;\n";
    o << "  for (" << g.idx_t << " o = blockIdx.x * 256 + threadIdx.x; o < " << outs << "; o += (" << g.idx_t << ")gridDim.x * 256) {\n";
    o << "    const " << g.idx_t << " oi = o % " << inner << ", oo = o / " << inner << ";\n";
    if (ax > 0) o << decompose("oo", sp.dims, 0, ax, g.idx_t, "c", "    ");
    if (ax + 1 < nd) {
      std::vector<int64_t> tail(sp.dims);
      o << decompose("oi", tail, ax + 1, nd, g.idx_t, "c", "    ");
    }
    o << "    " << ro.acc_t << " acc = " << ro.identity << ";\n";
    o << "    for (" << g.idx_t << " k = 0; k < " << len << "; ++k) {\n";
    std::vector<std::string> lv(f.leaves.size());
    for (size_t li = 0; li < f.leaves.size(); ++li) lv[li] = g.leaf_value(li, coords);
    o << g.body(lv, "      ");
    o << "      acc = comb(acc, v" << f.root << ");\n    }\n";
    o << "    ((" << stype(d) << "*)out)[o] = " << enc(d, "acc") << ";\n  }\n}\n";
    e.entry = "ku_reduce_fold";
    e.block = 256;
    e.grid = pick_grid(outs, 256, sm_count, 8);
    e.family = "reduce_fold";
  }
  e.source = o.str();
  return e;
}

// Index of the first maximum / minimum along an axis (kurumi_core/src/interp/reduce.rs:41-66): one thread per output
// element walks the axis in index order, starting from element 0 and replacing the best only on a strict
// comparison, which is also what keeps a NaN from ever replacing anything. Output is I64.
Emitted emit_arg_reduce(const Fused& f, size_t axis, bool arg_min, int sm_count) {
  Space sp = collapse(f, static_cast<int>(axis));
  Gen g(f, sp);
  const DType d = f.dtype();
  const size_t nd = sp.dims.size();
  const size_t ax = static_cast<size_t>(sp.special);
  const int64_t len = sp.dims[ax];
  int64_t outer = 1, inner = 1;
  for (size_t q = 0; q < ax; ++q) outer *= sp.dims[q];
  for (size_t q = ax + 1; q < nd; ++q) inner *= sp.dims[q];
  std::vector<std::string> coords(nd);
  for (size_t q = 0; q < nd; ++q) coords[q] = "c" + std::to_string(q);
  coords[ax] = "k";
  const int64_t outs = outer * inner;
  std::ostringstream o;
  o << device_prelude();
  Emitted e;
  e.leaf_args = g.args;
  if (inner == 1 && len >= 256) {
    // The axis is the innermost one and long: a CTA per line. A thread walks positions t, t + 256, ... in index order with
    // the interpreter's rule among the elements it sees (a NaN never becomes the best; strict comparison, so the first of
    // equal values stays); partial results merge by value, then by lower index, which is the same first-maximum; a NaN in
    // position 0 is never replaced, so that line answers 0.
    const std::string T = ctype(d);
    o << "template <class T> __device__ __forceinline__ T ku_shfl_down_any(T v, int dlt) {\n"
         "  union { T t; unsigned long long u; } x; x.u = 0ull; x.t = v; x.u = __shfl_down_sync(0xffffffffu, x.u, dlt); return x.t;\n}\n";
    o << "#define KU_BETTER(av, ak, bv, bk) ((av) " << (arg_min ? "<" : ">") << " (bv) || ((av) == (bv) && (ak) < (bk)))\n";
    o << "extern \"C\" __global__ void __launch_bounds__(256) ku_arg_rows(" << g.params() << "void* __restrict__ out) {\n";
    o << "  __shared__ " << T << " s_v[8];\n  __shared__ i64 s_k[8];\n  __shared__ int s_h[8];\n";
    o << "  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;\n";
    o << "  for (" << g.idx_t << " o = blockIdx.x; o < " << outs << "; o += gridDim.x) {\n";
    o << "    const " << g.idx_t << " oo = o;\n";
    if (ax > 0) o << decompose("oo", sp.dims, 0, ax, g.idx_t, "c", "    ");
    o << "    " << T << " best = 0;\n    i64 best_k = 0;\n    int has = 0, first_nan = 0;\n";
    // A thread takes `vec` neighbouring positions per turn (one 128-bit load where a leaf allows it), still in rising
    // order. Eight turns' loads are issued together before the first comparison: the comparisons form one dependent chain
    // and the compiler does not lift the loads over it by itself.
    int vec = 4;
    while (vec > 1 && len % vec) vec >>= 1;
    const int turns = 8;
    std::vector<bool> pre(f.leaves.size(), false);
    for (size_t li = 0; li < f.leaves.size(); ++li) pre[li] = vec > 1 && vec_ok(f, sp, li, vec);
    o << "    for (" << g.idx_t << " kk = threadIdx.x * " << vec << "; kk < " << len << "; kk += " << 256 * vec * turns << ") {\n";
    for (size_t li = 0; li < f.leaves.size(); ++li)
      if (pre[li]) o << "      " << stype(f.leaves[li].dtype) << " b" << li << "[" << turns << "][" << vec << "];\n";
    o << "#pragma unroll\n      for (int u = 0; u < " << turns << "; ++u) {\n";
    o << "        const " << g.idx_t << " k0 = kk + u * " << 256 * vec << ";\n        if (k0 < " << len << ") {\n";
    std::vector<std::string> c0 = coords;
    c0[ax] = "k0";
    for (size_t li = 0; li < f.leaves.size(); ++li) {
      if (!pre[li]) continue;
      const std::string st = stype(f.leaves[li].dtype);
      const size_t bytes = dtype_width(f.leaves[li].dtype) * static_cast<size_t>(vec);
      const std::string src = "((const " + st + "*)p" + std::to_string(g.ptr_arg[li]) + " + (" + g.offset(li, c0) + "))";
      if (bytes % 16 == 0) for (size_t q = 0; q < bytes / 16; ++q) o << "          ((uint4*)b" << li << "[u])[" << q << "] = ((const uint4*)" << src << ")[" << q << "];\n";
      else if (bytes == 8) o << "          *(uint2*)b" << li << "[u] = *(const uint2*)" << src << ";\n";
      else o << "          *(u32*)b" << li << "[u] = *(const u32*)" << src << ";\n";
    }
    o << "        }\n      }\n";
    o << "#pragma unroll\n      for (int u = 0; u < " << turns << "; ++u) {\n";
    o << "        const " << g.idx_t << " k0 = kk + u * " << 256 * vec << ";\n        if (k0 >= " << len << ") break;\n";
    o << "#pragma unroll\n        for (int l = 0; l < " << vec << "; ++l) {\n          const " << g.idx_t << " k = k0 + l;\n";
    {
      std::vector<std::string> lv(f.leaves.size());
      for (size_t li = 0; li < f.leaves.size(); ++li) lv[li] = pre[li] ? dec(f.leaves[li].dtype, "b" + std::to_string(li) + "[u][l]") : g.leaf_value(li, coords);
      o << g.body(lv, "          ");
    }
    o << "          const " << T << " v = v" << f.root << ";\n";
    o << "          if (k == 0 && v != v) first_nan = 1;\n";
    o << "          if (v == v && (!has || v " << (arg_min ? "<" : ">") << " best)) { best = v; best_k = (i64)k; has = 1; }\n        }\n      }\n    }\n";
    o << "    for (int dlt = 16; dlt > 0; dlt >>= 1) {\n";
    o << "      const " << T << " ov = ku_shfl_down_any(best, dlt); const i64 ok = ku_shfl_down_any(best_k, dlt); const int oh = __shfl_down_sync(0xffffffffu, has, dlt);\n";
    o << "      if (oh && (!has || KU_BETTER(ov, ok, best, best_k))) { best = ov; best_k = ok; has = 1; }\n    }\n";
    o << "    if (lane == 0) { s_v[warp] = best; s_k[warp] = best_k; s_h[warp] = has; }\n    __syncthreads();\n";
    o << "    if (threadIdx.x == 0) {\n";
    o << "      for (int w = 1; w < 8; ++w) if (s_h[w] && (!has || KU_BETTER(s_v[w], s_k[w], best, best_k))) { best = s_v[w]; best_k = s_k[w]; has = 1; }\n";
    o << "      ((i64*)out)[o] = (first_nan || !has) ? (i64)0 : best_k;\n    }\n    __syncthreads();\n  }\n}\n";
    e.entry = "ku_arg_rows";
    e.block = 256;
    e.grid = line_grid(outs, static_cast<int64_t>(sm_count) * 8);
    e.family = "arg_rows";
    e.source = o.str();
    return e;
  }
  o << "extern \"C\" __global__ void __launch_bounds__(256) ku_arg_fold(" << g.params() << "void* __restrict__ out) {\n";
  o << "  for (" << g.idx_t << " o = blockIdx.x * 256 + threadIdx.x; o < " << outs << "; o += (" << g.idx_t << ")gridDim.x * 256) {\n";
  o << "    const " << g.idx_t << " oi = o % " << inner << ", oo = o / " << inner << ";\n";
  if (ax > 0) o << decompose("oo", sp.dims, 0, ax, g.idx_t, "c", "    ");
  if (ax + 1 < nd) {
    std::vector<int64_t> tail(sp.dims);
    o << decompose("oi", tail, ax + 1, nd, g.idx_t, "c", "    ");
  }
  o << "    " << ctype(d) << " best = 0;\n    i64 best_k = 0;\n";
  o << "    for (" << g.idx_t << " k = 0; k < " << len << "; ++k) {\n";
  std::vector<std::string> lv(f.leaves.size());
  for (size_t li = 0; li < f.leaves.size(); ++li) lv[li] = g.leaf_value(li, coords);
  o << g.body(lv, "      ");
  o << "      if (k == 0 || v" << f.root << (arg_min ? " < " : " > ") << "best) { best = v" << f.root << "; best_k = (i64)k; }\n    }\n";
  o << "    ((i64*)out)[o] = best_k;\n  }\n}\n";
  e.entry = "ku_arg_fold";
  e.block = 256;
  e.grid = pick_grid(outs, 256, sm_count, 8);
  e.family = "arg_fold";
  e.source = o.str();
  return e;
}

// ---- softmax / rmsnorm ----------------------------------------------------------------------------
// Softmax follows kurumi_core/src/interp/nn.rs:35-69: line max, e = exp(x - max) (exp, not exp2),
// sum of e, e / sum (a division). RmsNorm follows nn.rs:88-116: x / sqrt(sum(x*x)/n + eps).
Emitted emit_softmax(const Fused& f, OpKind kind, size_t axis, float eps, int sm_count) {
  Space sp = collapse(f, static_cast<int>(axis));
  Gen g(f, sp);
  const DType d = f.dtype();
  const bool dbl = d == DType::F64;
  const std::string T = dbl ? "double" : "float";
  const size_t nd = sp.dims.size();
  const size_t ax = static_cast<size_t>(sp.special);
  const int64_t len = sp.dims[ax];
  int64_t outer = 1, inner = 1;
  for (size_t q = 0; q < ax; ++q) outer *= sp.dims[q];
  for (size_t q = ax + 1; q < nd; ++q) inner *= sp.dims[q];
  std::vector<std::string> coords(nd);
  for (size_t q = 0; q < nd; ++q) coords[q] = "c" + std::to_string(q);
  coords[ax] = "k";
  const bool sm = kind == OpKind::Softmax;
  std::ostringstream epsl;
  epsl.precision(9);
  epsl << std::scientific << eps;
  const std::string EXP = dbl ? "exp" : "expf", SQRT = dbl ? "sqrt" : "sqrtf", MAXF = dbl ? "fmax" : "fmaxf";
  const std::string NEG_INF = dbl ? "-__longlong_as_double(0x7ff0000000000000ll)" : "-KU_INF";
  const std::string EPS = dbl ? "(double)" + epsl.str() + "f" : epsl.str() + "f";
  std::ostringstream o;
  o << device_prelude() << block_reduce_helpers();
  o << "struct KuMax { __device__ __forceinline__ " << T << " operator()(" << T << " a, " << T << " b) const { return " << MAXF << "(a, b); } };\n";
  o << "struct KuAdd { __device__ __forceinline__ " << T << " operator()(" << T << " a, " << T << " b) const { return a + b; } };\n";
  Emitted e;
  e.leaf_args = g.args;
  const int NT = 256;
  const int64_t per = (len + NT - 1) / NT;
  if (inner == 1 && !dbl && len >= 64 && per > 64) {
    // a line too long for registers: one CTA per line, three passes over the (L2-resident) line with
    // block-wide reductions in between
    std::vector<std::string> lv(f.leaves.size());
    for (size_t li = 0; li < f.leaves.size(); ++li) lv[li] = g.leaf_value(li, coords);
    const std::string body = g.body(lv, "      ");
    const std::string X = "v" + std::to_string(f.root);
    o << "extern \"C\" __global__ void __launch_bounds__(256) ku_line_passes(" << g.params() << "void* __restrict__ out) {\n";
    o << "  __shared__ float red[32];\n";
    o << "  for (" << g.idx_t << " row = blockIdx.x; row < " << outer << "; row += gridDim.x) {\n";
    o << decompose("row", sp.dims, 0, ax, g.idx_t, "c", "    ");
    if (sm) {
      o << "    float m = -KU_INF;\n    for (" << g.idx_t << " k = threadIdx.x; k < " << len << "; k += 256) {\n" << body << "      m = fmaxf(m, " << X << ");\n    }\n";
      o << "    m = ku_block_reduce(m, KuMax(), red);\n";
      o << "    float s = 0.0f;\n    for (" << g.idx_t << " k = threadIdx.x; k < " << len << "; k += 256) {\n" << body << "      s += expf(" << X << " - m);\n    }\n";
      o << "    s = ku_block_reduce(s, KuAdd(), red);\n";
    } else {
      o << "    float s = 0.0f;\n    for (" << g.idx_t << " k = threadIdx.x; k < " << len << "; k += 256) {\n" << body << "      s += " << X << " * " << X << ";\n    }\n";
      o << "    s = ku_block_reduce(s, KuAdd(), red);\n    s = sqrtf(s / " << len << ".0f + " << EPS << ");\n";
    }
    o << "    for (" << g.idx_t << " k = threadIdx.x; k < " << len << "; k += 256) {\n" << body;
    o << "      ((" << stype(d) << "*)out)[row * " << len << " + k] = " << enc(d, sm ? "(expf(" + X + " - m) / s)" : "(" + X + " / s)") << ";\n    }\n  }\n}\n";
    e.entry = "ku_line_passes";
    e.block = 256;
    e.grid = line_grid(outer, static_cast<int64_t>(sm_count) * 8);
    e.family = sm ? "softmax_passes" : "rmsnorm_passes";
  } else if (inner == 1 && !dbl && len >= 64 && per <= 64) {
    // one CTA per line; the line lives in registers between the passes: one read, one write
    int vec = 4;
    while (vec > 1 && (len % vec)) vec >>= 1;
    const int64_t chunks = (len / vec + NT - 1) / NT;  // vectors per thread
    std::vector<bool> pre(f.leaves.size(), false);
    o << "extern \"C\" __global__ void __launch_bounds__(256) ku_line_regs(" << g.params() << "void* __restrict__ out) {\n";
    o << "  __shared__ float red[32];\n";
    o << "  for (" << g.idx_t << " row = blockIdx.x; row < " << outer << "; row += gridDim.x) {\n";
    o << decompose("row", sp.dims, 0, ax, g.idx_t, "c", "    ");
    o << "    float x[" << chunks * vec << "];\n";
    o << "#pragma unroll\n    for (int q = 0; q < " << chunks << "; ++q) {\n";
    o << "      const " << g.idx_t << " k0 = ((" << g.idx_t << ")q * " << NT << " + threadIdx.x) * " << vec << ";\n";
    o << "      if (k0 < " << len << ") {\n";
    std::vector<std::string> c0 = coords;
    c0[ax] = "k0";
    for (size_t li = 0; li < f.leaves.size(); ++li) {
      if (vec > 1 && vec_ok(f, sp, li, vec)) {
        pre[li] = true;
        const std::string st = stype(f.leaves[li].dtype);
        const size_t bytes = dtype_width(f.leaves[li].dtype) * static_cast<size_t>(vec);
        o << "        " << st << " b" << li << "[" << vec << "];\n";
        const std::string src = "((const " + st + "*)p" + std::to_string(g.ptr_arg[li]) + " + (" + g.offset(li, c0) + "))";
        if (bytes % 16 == 0) for (size_t q = 0; q < bytes / 16; ++q) o << "        ((uint4*)b" << li << ")[" << q << "] = ((const uint4*)" << src << ")[" << q << "];\n";
        else if (bytes == 8) o << "        *(uint2*)b" << li << " = *(const uint2*)" << src << ";\n";
        else o << "        *(u32*)b" << li << " = *(const u32*)" << src << ";\n";
      }
    }
    o << "#pragma unroll\n        for (int l = 0; l < " << vec << "; ++l) {\n          const " << g.idx_t << " k = k0 + l;\n";
    std::vector<std::string> lv(f.leaves.size());
    for (size_t li = 0; li < f.leaves.size(); ++li) lv[li] = pre[li] ? dec(f.leaves[li].dtype, "b" + std::to_string(li) + "[l]") : g.leaf_value(li, coords);
    o << g.body(lv, "          ");
    o << "          x[q * " << vec << " + l] = v" << f.root << ";\n        }\n";
    o << "      } else {\n#pragma unroll\n        for (int l = 0; l < " << vec << "; ++l) x[q * " << vec << " + l] = " << (sm ? "-KU_INF" : "0.0f") << ";\n      }\n    }\n";
    if (sm) {
      o << "    float m = -KU_INF;\n#pragma unroll\n    for (int i = 0; i < " << chunks * vec << "; ++i) m = fmaxf(m, x[i]);\n";
      o << "    m = ku_block_reduce(m, KuMax(), red);\n";
      o << "    float s = 0.0f;\n#pragma unroll\n    for (int i = 0; i < " << chunks * vec << "; ++i) { x[i] = expf(x[i] - m); s += x[i]; }\n";
      o << "    s = ku_block_reduce(s, KuAdd(), red);\n";
    } else {
      o << "    float s = 0.0f;\n#pragma unroll\n    for (int i = 0; i < " << chunks * vec << "; ++i) s += x[i] * x[i];\n";
      o << "    s = ku_block_reduce(s, KuAdd(), red);\n    s = sqrtf(s / " << len << ".0f + " << EPS << ");\n";
    }
    o << "#pragma unroll\n    for (int q = 0; q < " << chunks << "; ++q) {\n";
    o << "      const " << g.idx_t << " k0 = ((" << g.idx_t << ")q * " << NT << " + threadIdx.x) * " << vec << ";\n";
    o << "      if (k0 < " << len << ") {\n        " << stype(d) << " r[" << vec << "];\n";
    o << "#pragma unroll\n        for (int l = 0; l < " << vec << "; ++l) r[l] = " << enc(d, "(x[q * " + std::to_string(vec) + " + l] / s)") << ";\n";
    const size_t obytes = dtype_width(d) * static_cast<size_t>(vec);
    const std::string dst = "((" + std::string(stype(d)) + "*)out + row * " + std::to_string(len) + " + k0)";
    if (obytes == 16) o << "        *(uint4*)" << dst << " = *(const uint4*)r;\n";
    else if (obytes == 8) o << "        *(uint2*)" << dst << " = *(const uint2*)r;\n";
    else if (obytes == 4) o << "        *(u32*)" << dst << " = *(const u32*)r;\n";
    else if (obytes == 2) o << "        *(u16*)" << dst << " = *(const u16*)r;\n";
    else o << "        *" << dst << " = r[0];\n";
    o << "      }\n    }\n  }\n}\n";
    e.entry = "ku_line_regs";
    e.block = NT;
    e.grid = line_grid(outer, static_cast<int64_t>(sm_count) * 8);
    e.family = sm ? "softmax_rows" : "rmsnorm_rows";
  } else {
    // one thread per line, three passes; adjacent threads take adjacent inner positions
    const int64_t lines = outer * inner;
    o << "extern \"C\" __global__ void __launch_bounds__(256) ku_line_fold(" << g.params() << "void* __restrict__ out) {\n";
    o << "  for (" << g.idx_t << " o = blockIdx.x * 256 + threadIdx.x; o < " << lines << "; o += (" << g.idx_t << ")gridDim.x * 256) {\n";
    o << "    const " << g.idx_t << " oi = o % " << inner << ", oo = o / " << inner << ";\n";
    if (ax > 0) o << decompose("oo", sp.dims, 0, ax, g.idx_t, "c", "    ");
    if (ax + 1 < nd) o << decompose("oi", sp.dims, ax + 1, nd, g.idx_t, "c", "    ");
    std::vector<std::string> lv(f.leaves.size());
    for (size_t li = 0; li < f.leaves.size(); ++li) lv[li] = g.leaf_value(li, coords);
    const std::string body = g.body(lv, "      ");
    const std::string X = "(" + T + ")v" + std::to_string(f.root);
    if (sm) {
      o << "    " << T << " m = " << NEG_INF << ";\n    for (" << g.idx_t << " k = 0; k < " << len << "; ++k) {\n" << body << "      m = " << MAXF << "(m, " << X << ");\n    }\n";
      // compensated (Kahan) running sum: one thread folds the whole line, so plain f32 accumulation
      // would lose up to len * 2^-24 of relative accuracy
      o << "    " << T << " s = 0, comp = 0;\n    for (" << g.idx_t << " k = 0; k < " << len << "; ++k) {\n" << body << "      const " << T << " y = " << EXP << "(" << X << " - m) - comp; const " << T << " t = s + y; comp = (t - s) - y; s = t;\n    }\n";
    } else {
      o << "    " << T << " s = 0, comp = 0;\n    for (" << g.idx_t << " k = 0; k < " << len << "; ++k) {\n" << body << "      const " << T << " y = " << X << " * " << X << " - comp; const " << T << " t = s + y; comp = (t - s) - y; s = t;\n    }\n";
      o << "    s = " << SQRT << "(s / (" << T << ")" << len << " + " << EPS << ");\n";
    }
    o << "    for (" << g.idx_t << " k = 0; k < " << len << "; ++k) {\n" << body;
    const std::string val = sm ? "(" + EXP + "(" + X + " - m) / s)" : "(" + X + " / s)";
    o << "      ((" << stype(d) << "*)out)[(oo * " << len << " + k) * " << inner << " + oi] = " << enc(d, val) << ";\n    }\n  }\n}\n";
    e.entry = "ku_line_fold";
    e.block = 256;
    e.grid = pick_grid(lines, 256, sm_count, 8);
    e.family = sm ? "softmax_fold" : "rmsnorm_fold";
  }
  e.source = o.str();
  return e;
}

// ---- producer function for the hand-written line kernels -------------------------------------------------
bool emit_line_source_fn(const Fused& f, size_t axis, std::string* src, std::vector<int>* leaf_args, int64_t* R, int64_t* C, bool* transposed, LineLeaf* big) {
  Space sp = collapse(f, static_cast<int>(axis));
  if (sp.dims.size() != 2 || sp.special != 1) return false;
  *R = sp.dims[0];
  *C = sp.dims[1];
  Gen g(f, sp);
  *leaf_args = g.args;
  // the transposed pattern: the dominant buffers are contiguous along the line index and strided
  // along the line, and nothing large is contiguous along the line
  bool has_t = false, has_n = false;
  for (size_t li = 0; li < f.leaves.size(); ++li) {
    if (f.leaves[li].kind != LeafKind::Buffer) continue;
    const int64_t s0 = sp.ls[li][0], s1 = sp.ls[li][1];
    if ((s0 == 1 || s0 == -1) && s1 != 0 && s1 != 1 && s1 != -1) has_t = true;
    else if (s0 != 0 && (s1 == 1 || s1 == -1)) has_n = true;
    else if (s0 != 0 && s1 != 0) has_n = true;
  }
  *transposed = has_t && !has_n;
  // the single dominant leaf a TMA pipeline can stream: plain f32, unit stride across lines, 16-byte aligned rows
  int big_leaf = -1;
  if (big) {
    big->leaf = -1;
    int count = 0;
    for (size_t li = 0; li < f.leaves.size(); ++li) {
      const Leaf& l = f.leaves[li];
      if (l.kind != LeafKind::Buffer) continue;
      const int64_t s0 = sp.ls[li][0], s1 = sp.ls[li][1];
      if (s0 == 1 && s1 > 1) {
        ++count;
        if (l.dtype == DType::F32 && l.view.guards.empty() && l.view.base % 4 == 0 && s1 % 4 == 0 && l.view.base >= 0) { big_leaf = static_cast<int>(li); big->ld = s1; big->base = l.view.base; }
      }
    }
    if (count != 1) big_leaf = -1;
    big->leaf = big_leaf;
    if (big_leaf >= 0) {
      const FNode& r = f.nodes[static_cast<size_t>(f.root)];
      big->identity = r.op == OpKind::Input && r.leaf == big_leaf;
    }
  }
  std::ostringstream o;
  std::string params, args;
  for (size_t i = 0; i < g.args.size(); ++i) { params += ", const void* __restrict__ p" + std::to_string(i); args += ", p" + std::to_string(i); }
  o << "#define KU_SRC_PARAMS " << params << "\n#define KU_SRC_ARGS " << args << "\n";
  std::string lead;
  for (size_t i = 0; i < g.args.size(); ++i) lead += "const void* __restrict__ p" + std::to_string(i) + ", ";
  o << "#define KU_SRC_PARAMS_LEAD " << lead << "\n";
  o << "typedef " << stype(f.dtype()) << " ku_out_t;\n#define KU_ENC(x) " << enc(f.dtype(), "(x)") << "\n";
  o << "__device__ __forceinline__ float ku_src(" << g.idx_t << " i, " << g.idx_t << " j" << params << ") {\n";
  std::vector<std::string> coords = {"i", "j"};
  std::vector<std::string> lv(f.leaves.size());
  for (size_t li = 0; li < f.leaves.size(); ++li) lv[li] = g.leaf_value(li, coords);
  o << g.body(lv, "  ");
  o << "  return (float)v" << f.root << ";\n}\n";
  if (big_leaf >= 0) {  // same producer with the dominant leaf's value handed in (it was staged in shared memory)
    o << "__device__ __forceinline__ float ku_src_t(float lval, " << g.idx_t << " i, " << g.idx_t << " j" << params << ") {\n";
    std::vector<std::string> lv2 = lv;
    lv2[static_cast<size_t>(big_leaf)] = "lval";
    o << g.body(lv2, "  ");
    o << "  return (float)v" << f.root << ";\n}\n";
  }
  *src = o.str();
  return true;
}

// ---- GEMM epilogue + SIMT GEMM ----------------------------------------------------------------------
// Generates `ku_epilogue(acc, b, m, n, pointers...)`: the pointwise chain that consumes the rounded
// contraction result at output coordinate (b, m, n) and returns the stored element.
std::string emit_epilogue_fn(const Fused* epi, DType acc_dtype, std::vector<int>* leaf_args) {
  std::ostringstream o;
  if (!epi) {
    o << "#define KU_EPI_PARAMS\n#define KU_EPI_ARGS\n";
    o << "typedef " << stype(acc_dtype) << " ku_out_t;\n";
    o << "__device__ __forceinline__ ku_out_t ku_epilogue(" << ctype(acc_dtype) << " acc, i64 b, i64 m, i64 n) { return " << enc(acc_dtype, "acc") << "; }\n";
    return o.str();
  }
  Space sp;  // no collapsing: dims are exactly (b, m, n)
  for (size_t d = 0; d < 3; ++d) sp.dims.push_back(static_cast<int64_t>(epi->shape[d]));
  sp.axis_dim = {0, 1, 2};
  for (auto& l : epi->leaves) sp.ls.push_back(l.view.stride);
  Gen g(*epi, sp);
  g.idx_t = "i64";
  *leaf_args = g.args;
  std::string params, args;
  for (size_t i = 0; i < g.args.size(); ++i) { params += ", const void* __restrict__ p" + std::to_string(i); args += ", p" + std::to_string(i); }
  o << "#define KU_EPI_PARAMS " << params << "\n#define KU_EPI_ARGS " << args << "\n";
  o << "typedef " << stype(epi->dtype()) << " ku_out_t;\n";
  o << "__device__ __forceinline__ ku_out_t ku_epilogue(" << ctype(acc_dtype) << " acc, i64 b, i64 m, i64 n" << params << ") {\n";
  std::vector<std::string> coords = {"b", "m", "n"};
  std::vector<std::string> lv(epi->leaves.size());
  for (size_t li = 0; li < epi->leaves.size(); ++li) lv[li] = g.leaf_value(li, coords, "acc");
  o << g.body(lv, "  ");
  o << "  return " << enc(epi->dtype(), "v" + std::to_string(epi->root)) << ";\n}\n";
  return o.str();
}

// Plain tiled SIMT contraction for every numeric dtype (f32 / f64 / integers run here; the
// low-precision float types use it only when the tensor-core kernel's layout rules are not met).
// Accumulates like the interpreter: f32 for f32 and low-precision floats (then one rounding to
// the operand dtype, kurumi_core/src/interp/contract.rs:58-64), own type for f64 and integers.
Emitted emit_gemm_simt(const GemmDesc& gd, const Fused* epi, int sm_count) {
  const DType d = gd.dtype;
  const std::string A = ctype(d);  // accumulator register type
  std::ostringstream o;
  o << device_prelude();
  Emitted e;
  o << emit_epilogue_fn(epi, d, &e.leaf_args);
  const std::string ST = stype(gd.in_dtype);
  const bool flt = is_float(d);
  const std::string U = wrap_utype(d);
  const std::string mac = flt ? "acc[i][j] = acc[i][j] + a[i] * b[j];" : "acc[i][j] = (" + A + ")((" + U + ")acc[i][j] + (" + U + ")a[i] * (" + U + ")b[j]);";
  o << "#define TM 64\n#define TN 64\n#define TK 16\n";
  o << "extern \"C\" __global__ void __launch_bounds__(256) ku_gemm_simt(const void* __restrict__ Ap, const void* __restrict__ Bp, void* __restrict__ Cp KU_EPI_PARAMS) {\n";
  o << "  __shared__ " << A << " As[TK][TM + 1];\n  __shared__ " << A << " Bs[TK][TN + 1];\n";
  o << "  const i64 M = " << gd.m << ", N = " << gd.n << ", K = " << gd.k << ";\n";
  o << "  const i64 bz = blockIdx.z, m0 = (i64)blockIdx.y * TM, n0 = (i64)blockIdx.x * TN;\n";
  o << "  const " << ST << "* Ag = (const " << ST << "*)Ap + " << gd.a_base << "ll + bz * " << gd.a_bs << "ll;\n";
  o << "  const " << ST << "* Bg = (const " << ST << "*)Bp + " << gd.b_base << "ll + bz * " << gd.b_bs << "ll;\n";
  o << "  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;\n";
  o << "  " << A << " acc[4][4];\n#pragma unroll\n  for (int i = 0; i < 4; ++i)\n#pragma unroll\n    for (int j = 0; j < 4; ++j) acc[i][j] = 0;\n";
  o << "  for (i64 k0 = 0; k0 < K; k0 += TK) {\n";
  o << "    for (int t = threadIdx.x; t < TM * TK; t += 256) {\n";
  o << "      const int kk = t % TK, mm = t / TK; const i64 gm = m0 + mm, gk = k0 + kk;\n";
  o << "      As[kk][mm] = (gm < M && gk < K) ? " << dec(gd.in_dtype, "Ag[gm * " + std::to_string(gd.a_ms) + "ll + gk * " + std::to_string(gd.a_ks) + "ll]") << " : (" << A << ")0;\n    }\n";
  o << "    for (int t = threadIdx.x; t < TN * TK; t += 256) {\n";
  o << "      const int nn = t % TN, kk = t / TN; const i64 gn = n0 + nn, gk = k0 + kk;\n";
  o << "      Bs[kk][nn] = (gn < N && gk < K) ? " << dec(gd.in_dtype, "Bg[gk * " + std::to_string(gd.b_ks) + "ll + gn * " + std::to_string(gd.b_ns) + "ll]") << " : (" << A << ")0;\n    }\n";
  o << "    __syncthreads();\n#pragma unroll\n    for (int kk = 0; kk < TK; ++kk) {\n      " << A << " a[4], b[4];\n";
  o << "#pragma unroll\n      for (int i = 0; i < 4; ++i) { a[i] = As[kk][ty * 4 + i]; b[i] = Bs[kk][tx * 4 + i]; }\n";
  o << "#pragma unroll\n      for (int i = 0; i < 4; ++i)\n#pragma unroll\n        for (int j = 0; j < 4; ++j) " << mac << "\n    }\n    __syncthreads();\n  }\n";
  o << "#pragma unroll\n  for (int i = 0; i < 4; ++i)\n#pragma unroll\n    for (int j = 0; j < 4; ++j) {\n";
  o << "      const i64 gm = m0 + ty * 4 + i, gn = n0 + tx * 4 + j;\n";
  o << "      if (gm < M && gn < N) ((ku_out_t*)Cp)[(bz * M + gm) * N + gn] = ku_epilogue(" << rnd(d, "acc[i][j]") << ", bz, gm, gn KU_EPI_ARGS);\n    }\n}\n";
  e.source = o.str();
  e.entry = "ku_gemm_simt";
  e.block = 256;
  e.family = "gemm_simt";
  (void)sm_count;
  return e;
}

}  // namespace ku::cu

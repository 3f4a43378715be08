// CUDA source emitters for indexing along one axis (gather, scatter and their per-line forms) and per-line sorting.
#include <algorithm>
#include <sstream>

#include "emit_util.h"
#include "fuse.h"

namespace ku::cu {

using namespace emitutil;

// Kernels over contiguous row-major buffers (the scheduler writes operands out first). The semantics are the
// interpreter's, kurumi_core/src/interp/indexing/{gather,scatter}.rs and interp/sort.rs: gathers clamp an out-of-range
// index, scatters drop it, updates fold into the copy of the operand in index order (so results are bit-exact and
// deterministic: every destination element is owned by one thread, which walks the indices in order), sorting is stable.
namespace {
std::string combine_expr(uint8_t combine, DType d) {   // old value `a`, update `b`, both in the dtype's register type
  const std::string C = ctype(d), U = wrap_utype(d);
  const bool flt = is_float(d);
  switch (combine) {
    case 0: return "b";
    case 1: return flt ? "(a + b)" : "(" + C + ")((" + U + ")a + (" + U + ")b)";
    case 2: return flt ? (d == DType::F64 ? "fmax(a, b)" : "fmaxf(a, b)") : "(a > b ? a : b)";
    default: return flt ? (d == DType::F64 ? "fmin(a, b)" : "fminf(a, b)") : "(a < b ? a : b)";
  }
}
}  // namespace

Emitted emit_gather(DType d, DType idx_dt, int64_t pre, int64_t da, int64_t post, int64_t k, int sm_count) {
  std::ostringstream o;
  o << device_prelude();
  const int64_t total = pre * k * post;
  o << "extern \"C\" __global__ void __launch_bounds__(256) ku_gather(const void* __restrict__ src, const void* __restrict__ idx, void* __restrict__ out) {\n";
  o << "  for (i64 e = (i64)blockIdx.x * 256 + threadIdx.x; e < " << total << "ll; e += (i64)gridDim.x * 256) {\n";
  o << "    const i64 j = e % " << post << "ll, ki = (e / " << post << "ll) % " << k << "ll, p = e / " << (post * k) << "ll;\n";
  o << "    i64 a = (i64)((const " << stype(idx_dt) << "*)idx)[ki];\n";
  o << "    a = a < 0 ? 0 : (a > " << (da - 1) << "ll ? " << (da - 1) << "ll : a);\n";
  o << "    ((" << stype(d) << "*)out)[e] = ((const " << stype(d) << "*)src)[(p * " << da << "ll + a) * " << post << "ll + j];\n  }\n}\n";
  Emitted e;
  e.source = o.str(); e.entry = "ku_gather"; e.block = 256; e.grid = pick_grid(total, 256, sm_count, kStreamCtasPerSm); e.family = "gather";
  return e;
}

Emitted emit_gather_along(DType d, DType idx_dt, int64_t outer, int64_t da, int64_t la, int64_t inner, int sm_count) {
  std::ostringstream o;
  o << device_prelude();
  const int64_t total = outer * la * inner;
  o << "extern \"C\" __global__ void __launch_bounds__(256) ku_gather_along(const void* __restrict__ src, const void* __restrict__ idx, void* __restrict__ out) {\n";
  o << "  for (i64 e = (i64)blockIdx.x * 256 + threadIdx.x; e < " << total << "ll; e += (i64)gridDim.x * 256) {\n";
  o << "    const i64 pi = e % " << inner << "ll, po = e / " << (la * inner) << "ll;\n";
  o << "    i64 a = (i64)((const " << stype(idx_dt) << "*)idx)[e];\n";
  o << "    a = a < 0 ? 0 : (a > " << (da - 1) << "ll ? " << (da - 1) << "ll : a);\n";
  o << "    ((" << stype(d) << "*)out)[e] = ((const " << stype(d) << "*)src)[(po * " << da << "ll + a) * " << inner << "ll + pi];\n  }\n}\n";
  Emitted e;
  e.source = o.str(); e.entry = "ku_gather_along"; e.block = 256; e.grid = pick_grid(total, 256, sm_count, kStreamCtasPerSm); e.family = "gather_along";
  return e;
}

// `out` already holds the copy of the operand. Scatter: thread per (p, j) walks the k indices; ScatterAlong (along = true):
// thread per line (po, pi) walks the la positions of the index tensor. [pre | outer, da, post | inner] is the operand.
Emitted emit_scatter(DType d, DType idx_dt, bool along, uint8_t combine, int64_t pre, int64_t da, int64_t post, int64_t k, int sm_count) {
  std::ostringstream o;
  o << device_prelude();
  const int64_t total = pre * post;
  // A destination element belongs to exactly one thread, which walks the indices in order: bit-exact and deterministic
  // whatever the combine. With few columns and many indices that is too few threads, so the destination axis is cut
  // into NB blocks as well: thread (column, block) scans all of the column's indices, four at a time, and applies those
  // that fall into its block. The scan is cheap next to the dependent update-row / destination-row accesses it skips.
  const int64_t want = static_cast<int64_t>(sm_count) * 2048 * 2;
  const int64_t nb = std::max<int64_t>(1, std::min<int64_t>({(want + total - 1) / std::max<int64_t>(total, 1), da, k / 64 > 0 ? k / 64 : 1, 256}));
  const int64_t rbs = (da + nb - 1) / nb;
  const std::string S = stype(d), C = ctype(d), I = stype(idx_dt);
  auto apply = [&](const std::string& raw, const std::string& ki, const std::string& ind) {
    o << ind << "const i64 u = (p * " << k << "ll + " << ki << ") * " << post << "ll + j;\n";
    o << ind << S << "* dst = (" << S << "*)out + (p * " << da << "ll + " << raw << ") * " << post << "ll + j;\n";
    if (combine == 0) {
      o << ind << "*dst = ((const " << S << "*)upd)[u];\n";
    } else {
      o << ind << "const " << C << " a = " << dec(d, "*dst") << ", b = " << dec(d, "((const " + S + "*)upd)[u]") << ";\n";
      o << ind << "*dst = (" << S << ")" << enc(d, combine_expr(combine, d)) << ";\n";
    }
  };
  o << "extern \"C\" __global__ void __launch_bounds__(128) ku_scatter(const void* __restrict__ idx, const void* __restrict__ upd, void* __restrict__ out) {\n";
  if (!along) {
    // One index list for every column. A CTA is 128 columns of one destination block, so its threads all want the same
    // indices: a tile of 512 is tested by the CTA once (four indices per thread), the matching positions are packed in
    // index order (ballot + prefix sums) and every thread applies just those, in that order.
    const int64_t cchunks = (total + 127) / 128;
    o << "  __shared__ int s_pos[512];\n  __shared__ i64 s_row[512];\n  __shared__ int s_wsum[4];\n";
    o << "  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;\n";
    o << "  for (i64 unit = blockIdx.x; unit < " << nb * cchunks << "ll; unit += gridDim.x) {\n";
    o << "    const i64 rb = unit / " << cchunks << "ll, t = (unit % " << cchunks << "ll) * 128 + threadIdx.x;\n";
    o << "    const bool live = t < " << total << "ll;\n";
    o << "    const i64 lo = rb * " << rbs << "ll, hi = (lo + " << rbs << "ll) < " << da << "ll ? (lo + " << rbs << "ll) : " << da << "ll;\n";
    o << "    const i64 j = t % " << post << "ll, p = t / " << post << "ll;\n";
    o << "    for (i64 k0 = 0; k0 < " << k << "ll; k0 += 512) {\n";
    o << "      i64 raw[4];\n      int cnt = 0;\n";
    o << "#pragma unroll\n      for (int q = 0; q < 4; ++q) {\n";
    o << "        const i64 ki = k0 + threadIdx.x * 4 + q;\n";
    o << "        raw[q] = ki < " << k << "ll ? (i64)((const " << I << "*)idx)[ki] : (i64)-1;\n";
    o << "        cnt += (raw[q] >= lo && raw[q] < hi) ? 1 : 0;\n      }\n";
    o << "      int pre = cnt;\n";
    o << "#pragma unroll\n      for (int dlt = 1; dlt < 32; dlt <<= 1) { const int v = __shfl_up_sync(0xffffffffu, pre, dlt); if (lane >= dlt) pre += v; }\n";
    o << "      __syncthreads();   // the list of the tile before has been applied\n";
    o << "      if (lane == 31) s_wsum[warp] = pre;\n      __syncthreads();\n";
    o << "      int base = pre - cnt;\n      for (int w = 0; w < warp; ++w) base += s_wsum[w];\n";
    o << "      const int n = s_wsum[0] + s_wsum[1] + s_wsum[2] + s_wsum[3];\n";
    o << "#pragma unroll\n      for (int q = 0; q < 4; ++q)\n";
    o << "        if (raw[q] >= lo && raw[q] < hi) { s_pos[base] = threadIdx.x * 4 + q; s_row[base] = raw[q]; ++base; }\n";
    o << "      __syncthreads();\n";
    o << "      if (live) {\n        for (int q = 0; q < n; ++q) {\n          const i64 row = s_row[q];\n";
    apply("row", "(k0 + s_pos[q])", "          ");
    o << "        }\n      }\n    }\n    __syncthreads();\n  }\n}\n";
  } else {
    o << "  for (i64 tt = (i64)blockIdx.x * 128 + threadIdx.x; tt < " << total * nb << "ll; tt += (i64)gridDim.x * 128) {\n";
    o << "    const i64 t = tt % " << total << "ll, rb = tt / " << total << "ll;\n";
    o << "    const i64 lo = rb * " << rbs << "ll, hi = (lo + " << rbs << "ll) < " << da << "ll ? (lo + " << rbs << "ll) : " << da << "ll;\n";
    o << "    const i64 j = t % " << post << "ll, p = t / " << post << "ll;\n";
    o << "    for (i64 k0 = 0; k0 < " << k << "ll; k0 += 4) {\n";
    o << "      i64 raw[4];\n";
    o << "#pragma unroll\n      for (int q = 0; q < 4; ++q) {\n";
    o << "        const i64 ki = k0 + q;\n";
    o << "        raw[q] = ki < " << k << "ll ? (i64)((const " << I << "*)idx)[(p * " << k << "ll + ki) * " << post << "ll + j] : (i64)-1;\n";
    o << "      }\n";
    o << "#pragma unroll\n      for (int q = 0; q < 4; ++q) {\n";
    o << "        if (raw[q] < lo || raw[q] >= hi) continue;\n";
    apply("raw[q]", "(k0 + q)", "        ");
    o << "      }\n    }\n  }\n}\n";
  }
  Emitted e;
  e.source = o.str(); e.entry = "ku_scatter"; e.block = 128;
  e.grid = along ? pick_grid(total * nb, 128, sm_count, 8)
                 : static_cast<unsigned>(std::max<int64_t>(1, std::min<int64_t>(nb * ((total + 127) / 128), static_cast<int64_t>(sm_count) * 16)));
  e.family = along ? "scatter_along" : "scatter";
  return e;
}

// One CTA per line: a bitonic network over (key, original index) pairs in shared memory. The pairs are totally ordered
// (equal keys order by index), so the network's result is the stable permutation; padding sorts last.
// A stage's compare-exchange steps are taken three at a time: a thread loads the eight pairs whose positions differ in
// the three step bits, runs the three steps on them in registers and stores them back, one barrier per three steps
// (35 passes over the line instead of 91 for 8192 elements). Positions are skewed by one per 32 so that the strided
// loads of the low steps spread over the banks.
Emitted emit_argsort(DType d, bool descending, int64_t outer, int64_t len, int64_t inner, int sm_count) {
  int64_t lpad = 1;
  while (lpad < len) lpad <<= 1;
  // keys are held in at least 32 bits (the index array behind them stays aligned)
  const size_t key_bytes = d == DType::F64 || dtype_width(d) == 8 ? 8 : 4;
  const std::string S = stype(d), C = is_float(d) ? (d == DType::F64 ? "double" : "float") : key_bytes == 8 ? ctype(d) : is_signed(d) ? "i32" : "u32";
  const int64_t slots = lpad + lpad / 32;
  std::ostringstream o;
  o << device_prelude();
  o << "#define LEN " << len << "\n#define LPAD " << lpad << "\n#define SLOTS " << slots << "\n#define INNER " << inner << "ll\n#define KU_AT(i) ((i) + ((i) >> 5))\n";
  o << "typedef " << C << " key_t;\n";
  o << "__device__ __forceinline__ bool ku_before(key_t ka, int ia, key_t kb, int ib) {\n";
  o << "  if (ia >= LEN || ib >= LEN) return ia < ib;\n";
  o << "  const bool lt = " << (descending ? "ka > kb" : "ka < kb") << ", gt = " << (descending ? "ka < kb" : "ka > kb") << ";\n";
  o << "  return lt || (!gt && ia < ib);\n}\n";
  // the steps j = 2^(sh+G-1) .. 2^sh of stage k on the 2^G pairs base + m * 2^sh; bit k of a position is above all of them
  o << "template <int G> __device__ __forceinline__ void ku_steps(key_t* keys, int* ids, int k, int sh) {\n";
  o << "  constexpr int E = 1 << G;\n";
  o << "  for (int w = threadIdx.x; w < (LPAD >> G); w += blockDim.x) {\n";
  o << "    const int base = ((w >> sh) << (sh + G)) | (w & ((1 << sh) - 1));\n";
  o << "    key_t kv[E];\n    int iv[E];\n";
  o << "#pragma unroll\n    for (int m = 0; m < E; ++m) { const int a = KU_AT(base + (m << sh)); kv[m] = keys[a]; iv[m] = ids[a]; }\n";
  o << "    const bool up = (base & k) == 0;\n";
  o << "#pragma unroll\n    for (int b = G - 1; b >= 0; --b) {\n";
  o << "#pragma unroll\n      for (int m = 0; m < E; ++m) {\n";
  o << "        if (m & (1 << b)) continue;\n        const int n = m | (1 << b);\n";
  o << "        if (ku_before(kv[n], iv[n], kv[m], iv[m]) == up) { const key_t tk = kv[m]; kv[m] = kv[n]; kv[n] = tk; const int ti = iv[m]; iv[m] = iv[n]; iv[n] = ti; }\n";
  o << "      }\n    }\n";
  o << "#pragma unroll\n    for (int m = 0; m < E; ++m) { const int a = KU_AT(base + (m << sh)); keys[a] = kv[m]; ids[a] = iv[m]; }\n";
  o << "  }\n  __syncthreads();\n}\n";
  o << "extern \"C\" __global__ void ku_argsort(const void* __restrict__ src, void* __restrict__ out) {\n";
  o << "  extern __shared__ __align__(16) unsigned char raw[];\n";
  o << "  key_t* keys = (key_t*)raw;\n  int* ids = (int*)(raw + (size_t)SLOTS * sizeof(key_t));\n";
  o << "  const i64 line = blockIdx.x, po = line / INNER, pi = line % INNER;\n";
  o << "  const " << S << "* base = (const " << S << "*)src + po * LEN * INNER + pi;\n";
  o << "  for (int i = threadIdx.x; i < LPAD; i += blockDim.x) {\n";
  o << "    ids[KU_AT(i)] = i;\n    keys[KU_AT(i)] = i < LEN ? (key_t)" << dec(d, "base[(i64)i * INNER]") << " : (key_t)0;\n  }\n";
  o << "  __syncthreads();\n";
  o << "  for (int s = 1; (1 << s) <= LPAD; ++s) {\n";
  o << "    const int k = 1 << s;\n    int hi = s;   // the step bits [0, hi) of this stage are still to do, highest first\n";
  o << "    if (hi % 3 == 1) { ku_steps<1>(keys, ids, k, hi - 1); hi -= 1; }\n";
  o << "    else if (hi % 3 == 2) { ku_steps<2>(keys, ids, k, hi - 2); hi -= 2; }\n";
  o << "    for (; hi > 0; hi -= 3) ku_steps<3>(keys, ids, k, hi - 3);\n  }\n";
  o << "  i64* dst = (i64*)out + po * LEN * INNER + pi;\n";
  o << "  for (int r = threadIdx.x; r < LEN; r += blockDim.x) dst[(i64)r * INNER] = (i64)ids[KU_AT(r)];\n}\n";
  Emitted e;
  e.source = o.str(); e.entry = "ku_argsort";
  e.block = static_cast<unsigned>(std::max<int64_t>(32, std::min<int64_t>(1024, lpad / 8)));
  e.grid = static_cast<unsigned>(outer * inner);
  e.smem = static_cast<unsigned>(slots * (key_bytes + 4));
  e.family = "argsort";
  (void)sm_count;
  return e;
}

// Argsort along an axis longer than one CTA's shared memory holds: the same bitonic network over (key, original index)
// pairs, run on a padded copy in global scratch. Chunks of ASL_CH pairs are sorted in shared memory (all stages up to
// k = ASL_CH); for the larger k the steps with j >= ASL_CH are one global compare-exchange launch each and the steps
// below are finished per chunk in shared memory again. The direction of a compare depends on the pair's position in
// the whole line, so the pieces compose to the one network, and the result is the same stable permutation.
// Entry points: ku_asl_chunks(src, keys, ids), ku_asl_global(keys, ids, k, j), ku_asl_local(keys, ids, k), ku_asl_out(ids, out).
Emitted emit_argsort_long(DType d, bool descending, int64_t outer, int64_t len, int64_t inner, int64_t* lpad_out, size_t* key_bytes_out) {
  int64_t lpad = 1;
  while (lpad < len) lpad <<= 1;
  const size_t key_bytes = d == DType::F64 || dtype_width(d) == 8 ? 8 : 4;
  const std::string S = stype(d), C = is_float(d) ? (d == DType::F64 ? "double" : "float") : key_bytes == 8 ? ctype(d) : is_signed(d) ? "i32" : "u32";
  std::ostringstream o;
  o << device_prelude();
  o << "#define LEN " << len << "ll\n#define LPAD " << lpad << "ll\n#define INNER " << inner << "ll\n#define LINES " << outer * inner << "ll\n#define ASL_CH 4096\n#define ASL_LOG 12\n";
  o << "typedef " << C << " key_t;\n";
  o << "__device__ __forceinline__ bool ku_before(key_t ka, int ia, key_t kb, int ib) {\n";
  o << "  if (ia >= LEN || ib >= LEN) return ia < ib;\n";
  o << "  const bool lt = " << (descending ? "ka > kb" : "ka < kb") << ", gt = " << (descending ? "ka < kb" : "ka > kb") << ";\n";
  o << "  return lt || (!gt && ia < ib);\n}\n";
  // the steps j = 2^(nbits-1) .. 1 of stage k on one chunk in shared memory, three steps per pass in registers as in
  // ku_argsort; gi0 = position of the chunk's first pair in its line (the direction depends on the position in the line)
  o << "template <int G> __device__ __forceinline__ void ku_asl_pass(key_t* keys, int* ids, i64 gi0, i64 k, int sh) {\n";
  o << "  constexpr int E = 1 << G;\n";
  o << "  for (int w = threadIdx.x; w < (ASL_CH >> G); w += blockDim.x) {\n";
  o << "    const int base = ((w >> sh) << (sh + G)) | (w & ((1 << sh) - 1));\n";
  o << "    key_t kv[E];\n    int iv[E];\n";
  o << "#pragma unroll\n    for (int m = 0; m < E; ++m) { kv[m] = keys[base + (m << sh)]; iv[m] = ids[base + (m << sh)]; }\n";
  o << "    const bool up = ((gi0 + base) & k) == 0;\n";
  o << "#pragma unroll\n    for (int b = G - 1; b >= 0; --b) {\n";
  o << "#pragma unroll\n      for (int m = 0; m < E; ++m) {\n";
  o << "        if (m & (1 << b)) continue;\n        const int n = m | (1 << b);\n";
  o << "        if (ku_before(kv[n], iv[n], kv[m], iv[m]) == up) { const key_t tk = kv[m]; kv[m] = kv[n]; kv[n] = tk; const int ti = iv[m]; iv[m] = iv[n]; iv[n] = ti; }\n";
  o << "      }\n    }\n";
  o << "#pragma unroll\n    for (int m = 0; m < E; ++m) { keys[base + (m << sh)] = kv[m]; ids[base + (m << sh)] = iv[m]; }\n";
  o << "  }\n  __syncthreads();\n}\n";
  o << "__device__ __forceinline__ void ku_asl_steps(key_t* keys, int* ids, i64 gi0, i64 k, int nbits) {\n";
  o << "  int hi = nbits;\n";
  o << "  if (hi % 3 == 1) { ku_asl_pass<1>(keys, ids, gi0, k, hi - 1); hi -= 1; }\n";
  o << "  else if (hi % 3 == 2) { ku_asl_pass<2>(keys, ids, gi0, k, hi - 2); hi -= 2; }\n";
  o << "  for (; hi > 0; hi -= 3) ku_asl_pass<3>(keys, ids, gi0, k, hi - 3);\n}\n";
  o << "extern \"C\" __global__ void __launch_bounds__(1024) ku_asl_chunks(const void* __restrict__ src, key_t* __restrict__ gkeys, int* __restrict__ gids) {\n";
  o << "  __shared__ key_t keys[ASL_CH];\n  __shared__ int ids[ASL_CH];\n";
  o << "  const i64 cpl = LPAD / ASL_CH, line = blockIdx.x / cpl, gi0 = (blockIdx.x % cpl) * ASL_CH;\n";
  o << "  const i64 po = line / INNER, pi = line % INNER;\n";
  o << "  const " << S << "* base = (const " << S << "*)src + po * LEN * INNER + pi;\n";
  o << "  for (int i = threadIdx.x; i < ASL_CH; i += blockDim.x) {\n";
  o << "    const i64 gi = gi0 + i;\n    ids[i] = (int)gi;\n    keys[i] = gi < LEN ? (key_t)" << dec(d, "base[gi * INNER]") << " : (key_t)0;\n  }\n";
  o << "  __syncthreads();\n";
  o << "  for (int s = 1; s <= ASL_LOG; ++s) ku_asl_steps(keys, ids, gi0, (i64)1 << s, s);\n";
  o << "  for (int i = threadIdx.x; i < ASL_CH; i += blockDim.x) { gkeys[line * LPAD + gi0 + i] = keys[i]; gids[line * LPAD + gi0 + i] = ids[i]; }\n}\n";
  o << "extern \"C\" __global__ void __launch_bounds__(256) ku_asl_global(key_t* __restrict__ gkeys, int* __restrict__ gids, long long k, long long j) {\n";
  o << "  const i64 pairs = LINES * (LPAD / 2);\n";
  o << "  for (i64 q = (i64)blockIdx.x * 256 + threadIdx.x; q < pairs; q += (i64)gridDim.x * 256) {\n";
  o << "    const i64 line = q / (LPAD / 2), pq = q % (LPAD / 2);\n";
  o << "    const i64 i = (pq / j) * 2 * j + (pq % j), l = i + j;\n";
  o << "    key_t* kk = gkeys + line * LPAD;\n    int* ii = gids + line * LPAD;\n";
  o << "    const key_t ka = kk[i], kb = kk[l];\n    const int ia = ii[i], ib = ii[l];\n";
  o << "    const bool up = (i & k) == 0;\n";
  o << "    if (ku_before(kb, ib, ka, ia) == up) { kk[i] = kb; kk[l] = ka; ii[i] = ib; ii[l] = ia; }\n  }\n}\n";
  o << "extern \"C\" __global__ void __launch_bounds__(1024) ku_asl_local(key_t* __restrict__ gkeys, int* __restrict__ gids, long long k) {\n";
  o << "  __shared__ key_t keys[ASL_CH];\n  __shared__ int ids[ASL_CH];\n";
  o << "  const i64 cpl = LPAD / ASL_CH, line = blockIdx.x / cpl, gi0 = (blockIdx.x % cpl) * ASL_CH;\n";
  o << "  for (int i = threadIdx.x; i < ASL_CH; i += blockDim.x) { keys[i] = gkeys[line * LPAD + gi0 + i]; ids[i] = gids[line * LPAD + gi0 + i]; }\n";
  o << "  __syncthreads();\n";
  o << "  ku_asl_steps(keys, ids, gi0, k, ASL_LOG);\n";
  o << "  for (int i = threadIdx.x; i < ASL_CH; i += blockDim.x) { gkeys[line * LPAD + gi0 + i] = keys[i]; gids[line * LPAD + gi0 + i] = ids[i]; }\n}\n";
  o << "extern \"C\" __global__ void __launch_bounds__(256) ku_asl_out(const int* __restrict__ gids, void* __restrict__ out) {\n";
  o << "  const i64 total = LINES * LEN;\n";
  o << "  for (i64 q = (i64)blockIdx.x * 256 + threadIdx.x; q < total; q += (i64)gridDim.x * 256) {\n";
  o << "    const i64 line = q / LEN, r = q % LEN, po = line / INNER, pi = line % INNER;\n";
  o << "    ((i64*)out)[po * LEN * INNER + r * INNER + pi] = (i64)gids[line * LPAD + r];\n  }\n}\n";
  Emitted e;
  e.source = o.str(); e.entry = "ku_asl_chunks"; e.family = "argsort";
  *lpad_out = lpad; *key_bytes_out = key_bytes;
  return e;
}

}  // namespace ku::cu

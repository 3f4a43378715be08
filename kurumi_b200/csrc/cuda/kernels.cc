#include "kernels.h"

#include <cstdio>
#include <cstdlib>

namespace ku::cu {

namespace {
std::string defines(std::initializer_list<std::pair<const char*, int64_t>> kv) {
  std::string s;
  for (auto& p : kv) s += std::string("#define ") + p.first + " " + std::to_string(p.second) + "\n";
  return s;
}
}  // namespace

extern const std::string kSrc_gemm_tc;
extern const std::string kSrc_gemm_tc2;

static std::string lower(std::string s) { for (auto& c : s) c = static_cast<char>(std::tolower(c)); return s; }

bool build_gemm_tc(const KernelLoader& load, const GemmDesc& d, const Fused* epi, int sm_count, Launch* out, std::vector<int>* epi_leaf_args) {
  if (std::getenv("KURUMI_NO_TC")) return false;
  const DType in = d.in_dtype;
  const bool f8 = in == DType::F8E4M3;
  if (!(d.dtype == DType::BF16 || d.dtype == DType::F16)) return false;
  if (!(in == d.dtype || f8)) return false;
  const int64_t es = f8 ? 1 : 2, al = 16 / es;  // element size, elements per 16 bytes
  if (d.m < 1 || d.n < 1 || d.k < 1 || d.m >= (int64_t(1) << 31) || d.n >= (int64_t(1) << 31) || d.k >= (int64_t(1) << 31)) return false;
  // each operand must be K-major or MN-major with 16-byte aligned rows, base and batch stride
  auto major = [&](int64_t row_stride, int64_t k_stride, int64_t rows, int64_t base, int64_t bs, int* mn) {
    if (base % al || base < 0 || (d.batch > 1 && (bs % al || bs <= 0))) return false;
    if (k_stride == 1 && (rows == 1 || (row_stride % al == 0 && row_stride >= d.k))) { *mn = 0; return true; }
    if (row_stride == 1 && (d.k == 1 || (k_stride % al == 0 && k_stride >= rows))) { *mn = 1; return true; }
    return false;
  };
  int a_mn = 0, b_mn = 0;
  if (!major(d.a_ms, d.a_ks, d.m, d.a_base, d.a_bs, &a_mn) || !major(d.b_ns, d.b_ks, d.n, d.b_base, d.b_bs, &b_mn)) return false;
  const int64_t bm = 128, bn = d.n > 128 ? 256 : d.n > 64 ? 128 : 64, bkb = 128, bk = bkb / es;
  // wide outputs with at least two row blocks run on SM pairs (cta_group::2): 256 x 256 tiles, half of B per CTA
  const bool pair = bn == 256 && d.m > 128 && sm_count >= 2 && !std::getenv("KURUMI_NO_TC2");
  const int64_t stage = (bm + (pair ? bn / 2 : bn)) * bkb;
  const int64_t stages = std::min<int64_t>(8, (200 * 1024) / stage);
  const int64_t tiles_m = pair ? (d.m + 255) / 256 : (d.m + bm - 1) / bm, tiles_n = (d.n + bn - 1) / bn;
  if (d.batch * tiles_m * tiles_n >= (int64_t(1) << 31)) return false;
  // instruction descriptor: f32 accumulate, operand formats, major-ness, N >> 3, M >> 4
  const uint32_t fmt = f8 ? 0u : (d.dtype == DType::BF16 ? 1u : 0u);
  const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(a_mn) << 15) | (static_cast<uint32_t>(b_mn) << 16) |
                         (static_cast<uint32_t>(bn >> 3) << 17) | (static_cast<uint32_t>((pair ? 256 : bm) >> 4) << 24);
  std::string src = device_prelude() + emit_epilogue_fn(epi, d.dtype, epi_leaf_args) +
                    defines({{"M", d.m}, {"N", d.n}, {"K", d.k}, {"BATCH", d.batch}, {"BM", bm}, {"BN", bn}, {"BKB", bkb}, {"ESIZE", es}, {"STAGES", stages},
                             {"A_MN", a_mn}, {"B_MN", b_mn}, {"IDESC", static_cast<int64_t>(idesc)}, {"TILES_M", tiles_m}, {"TILES_N", tiles_n}}) +
                    "#define KU_ROUND(x) ku_rnd_" + lower(dtype_name(d.dtype)) + "(x)\n" + (pair ? kSrc_gemm_tc2 : kSrc_gemm_tc);
  out->name = f8 ? "gemm_tc_f8" : "gemm_tc";
  out->kernel = load(src, pair ? "ku_gemm_tc2" : "ku_gemm_tc", true);
  out->grid[0] = static_cast<unsigned>(pair ? 2 * std::min<int64_t>(d.batch * tiles_m * tiles_n, sm_count / 2) : std::min<int64_t>(d.batch * tiles_m * tiles_n, sm_count));
  if (pair) { out->cluster[0] = 2; out->persistent_clusters = -1; }   // cap at the co-resident pair count on first launch
  out->block[0] = 320;   // TMA warp, MMA warp, 8 epilogue warps
  out->smem = static_cast<unsigned>(std::max<int64_t>(stages * stage + 1024, 120 * 1024));  // > half an SM: one CTA per SM owns all of tensor memory
  auto tmap = [&](int slot, int mn, int64_t rows, int64_t row_stride, int64_t k_stride, int64_t base, int64_t bs, int64_t tile_rows) {
    Arg a;
    a.kind = Arg::Tmap;
    a.tm.slot = slot;
    a.tm.byte_offset = base * es;
    a.tm.dt = f8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : (d.dtype == DType::BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
    a.tm.rank = 3;
    a.tm.swz = CU_TENSOR_MAP_SWIZZLE_128B;
    const int64_t batch_stride = d.batch > 1 ? bs : std::max<int64_t>(al, ((mn ? d.k * std::max<int64_t>(k_stride, 1) : rows * std::max<int64_t>(row_stride, 1)) + al - 1) / al * al);
    if (!mn) {  // K-major: dims (K, rows, batch), box (BK, tile rows, 1)
      a.tm.dims[0] = static_cast<uint64_t>(d.k); a.tm.dims[1] = static_cast<uint64_t>(rows); a.tm.dims[2] = static_cast<uint64_t>(d.batch);
      a.tm.strides[0] = static_cast<uint64_t>((rows == 1 ? std::max<int64_t>(d.k, al) : row_stride) * es);
      a.tm.box[0] = static_cast<uint32_t>(bk); a.tm.box[1] = static_cast<uint32_t>(tile_rows); a.tm.box[2] = 1;
    } else {    // MN-major: dims (rows, K, batch), box (128 bytes of rows, BK, 1)
      a.tm.dims[0] = static_cast<uint64_t>(rows); a.tm.dims[1] = static_cast<uint64_t>(d.k); a.tm.dims[2] = static_cast<uint64_t>(d.batch);
      a.tm.strides[0] = static_cast<uint64_t>((d.k == 1 ? std::max<int64_t>(rows, al) : k_stride) * es);
      a.tm.box[0] = static_cast<uint32_t>(128 / es); a.tm.box[1] = static_cast<uint32_t>(bk); a.tm.box[2] = 1;
    }
    a.tm.strides[0] = (a.tm.strides[0] + 15) / 16 * 16;
    a.tm.strides[1] = static_cast<uint64_t>(batch_stride * es);
    return a;
  };
  out->args.push_back(tmap(-1, a_mn, d.m, d.a_ms, d.a_ks, d.a_base, d.a_bs, bm));
  out->args.push_back(tmap(-2, b_mn, d.n, d.b_ns, d.b_ks, d.b_base, d.b_bs, pair ? bn / 2 : bn));
  Arg c; c.kind = Arg::SlotPtr; c.slot = -3; out->args.push_back(c);
  Arg st; st.kind = Arg::Status; out->args.push_back(st);
  return true;
}
extern const std::string kSrc_softmax_transposed;


size_t softmax_two_pass_scratch_bytes(size_t lines, size_t len);
void softmax_two_pass_launch(const float* in, const float* bias, float* out, size_t lines, size_t len, size_t ld, void* scratch, cudaStream_t stream);

bool build_softmax_two_pass(const Fused& f, size_t axis, Launch* out, size_t* scratch_bytes) {
  if (std::getenv("KURUMI_SMT_NO_TWO_PASS")) return false;
  if (f.dtype() != DType::F32 || f.shape.size() != 2 || axis != 1) return false;
  const int64_t lines = static_cast<int64_t>(f.shape[0]), len = static_cast<int64_t>(f.shape[1]);
  // lines of 2048 positions and more go to the single-pass cluster kernel, which measured faster there
  if (len >= 2048 && !std::getenv("KURUMI_SMT_TWO_PASS")) return false;
  if (lines < 64 || len < 256 || lines >= (int64_t(1) << 31) || len >= (int64_t(1) << 31)) return false;
  auto is_big = [&](const Leaf& l) {
    return l.kind == LeafKind::Buffer && l.dtype == DType::F32 && l.view.guards.empty() && l.view.stride[0] == 1 && l.view.stride[1] >= lines && l.view.base >= 0;
  };
  auto is_bias = [&](const Leaf& l) {
    return l.kind == LeafKind::Buffer && l.dtype == DType::F32 && l.view.guards.empty() && l.view.stride[0] == 0 && l.view.stride[1] == 1 && l.view.base >= 0;
  };
  const FNode& r = f.nodes[static_cast<size_t>(f.root)];
  const Leaf *big = nullptr, *bias = nullptr;
  if (r.op == OpKind::Input) {
    big = &f.leaves[static_cast<size_t>(r.leaf)];
  } else if (r.op == OpKind::Add && r.dtype == DType::F32) {
    const FNode &a = f.nodes[static_cast<size_t>(r.in[0])], &b = f.nodes[static_cast<size_t>(r.in[1])];
    if (a.op != OpKind::Input || b.op != OpKind::Input) return false;
    const Leaf &la = f.leaves[static_cast<size_t>(a.leaf)], &lb = f.leaves[static_cast<size_t>(b.leaf)];
    if (is_big(la) && is_bias(lb)) { big = &la; bias = &lb; }
    else if (is_big(lb) && is_bias(la)) { big = &lb; bias = &la; }
    else return false;
  } else {
    return false;
  }
  if (!is_big(*big)) return false;
  const size_t ld = static_cast<size_t>(big->view.stride[1]);
  const bool has_bias = bias != nullptr;
  *scratch_bytes = softmax_two_pass_scratch_bytes(static_cast<size_t>(lines), static_cast<size_t>(len));
  out->name = "softmax_two_pass";
  Arg in; in.kind = Arg::SlotPtr; in.slot = big->slot; in.byte_offset = big->view.base * 4; out->args.push_back(in);
  Arg bi = in;
  if (has_bias) { bi.slot = bias->slot; bi.byte_offset = bias->view.base * 4; }
  out->args.push_back(bi);
  Arg o; o.kind = Arg::SlotPtr; o.slot = -3; out->args.push_back(o);
  Arg sc; sc.kind = Arg::SlotPtr; sc.slot = -1; out->args.push_back(sc);
  out->host_launch = [=](const std::vector<void*>& p, cudaStream_t stream) {
    softmax_two_pass_launch(static_cast<const float*>(p[0]), has_bias ? static_cast<const float*>(p[1]) : nullptr, static_cast<float*>(p[2]), static_cast<size_t>(lines),
                            static_cast<size_t>(len), ld, p[3], stream);
  };
  return true;
}

extern const std::string kSrc_quant_gemv;
extern const std::string kSrc_quant_gemv_mma;

bool quant_gemv_supported(DType act, int64_t m, int64_t n, int64_t k, int bits, int64_t group) {
  if (std::getenv("KURUMI_NO_QUANT_GEMV")) return false;
  if (!(act == DType::F32 || act == DType::BF16 || act == DType::F16)) return false;
  const int64_t piece = 128 / bits;
  return m >= 1 && m <= 8 && n >= 1 && k >= piece && (k * bits / 8) % 16 == 0 && (group % piece == 0 || piece % group == 0) && n < (int64_t(1) << 31) && k < (int64_t(1) << 31);
}

// slots are symbolic: -1 qweight, -2 scales, -3 mins (or scales again when symmetric), -4 act, -5 out
bool build_quant_gemv(const KernelLoader& load, DType act, int64_t m, int64_t n, int64_t k, int bits, int64_t group, bool symmetric, int sm_count, Launch* out) {
  if (!quant_gemv_supported(act, m, n, k, bits, group)) return false;
  const int64_t piece = 128 / bits;
  // 16-bit activations against 2- or 4-bit weights whose groups hold whole runs of four 16-byte pieces: the products run on
  // mma.sync with the raw field values as one operand (kernels/quant_gemv_mma.cuh)
  if (act != DType::F32 && (bits == 2 || bits == 4) && group % (4 * piece) == 0 && k % (4 * piece) == 0 && n * (k / group) < (int64_t(1) << 31)) {
    const int64_t run = 4 * piece, depth = 3, res = 4;
    // a CTA is 8 warps: 8 / ks tiles of 16 rows, ks warps per tile. The largest split whose CTAs make up at most two waves:
    // CTAs that start as others finish overlap their staging and final sums with the others' weight stream (28672 x 8192,
    // 4 bits: 896 CTAs of 32 rows 49.6 us, 448 of 64 rows in exactly one wave 55.7 us, 1792 of 16 rows 51.3 us); past
    // that the CTAs of one wave loop over blocks of rows.
    const int64_t tiles = (n + 15) / 16, wave = static_cast<int64_t>(sm_count) * res;
    int64_t ks = 8;
    while (ks > 1 && ((tiles + 8 / ks - 1) / (8 / ks) > 2 * wave || k / run < ks * depth)) ks /= 2;
    // all K columns of the activations staged once when that leaves room for res CTAs per SM, else in chunks that the
    // ring's slots line up with
    const int64_t budget = (200 * 1024) / res - 4096, unit = run * ks * depth;
    int64_t kc = k;
    if (m * (k + 16) * 2 + m * (k / run) * 4 > budget) kc = std::max<int64_t>(unit, (budget / (2 * m) - 16) / unit * unit);
    std::string src = device_prelude() +
                      defines({{"M", m}, {"N", n}, {"K", k}, {"BITS", bits}, {"GROUP", group}, {"SYM", symmetric ? 1 : 0}, {"ACT", act == DType::BF16 ? 1 : 2},
                               {"KC", kc}, {"KS", ks}, {"D", depth}, {"RES", res}}) +
                      kSrc_quant_gemv_mma;
    out->name = "quant_gemv";
    out->kernel = load(src, "ku_quant_gemv_mma", true);
    const int64_t rows_per_cta = (8 / ks) * 16;
    const int64_t row_blocks = (n + rows_per_cta - 1) / rows_per_cta;
    out->grid[0] = static_cast<unsigned>(row_blocks <= 2 * wave ? row_blocks : wave);
    out->block[0] = 256;
    out->smem = static_cast<unsigned>(m * (kc + 16) * 2 + m * ((kc + run - 1) / run) * 4);
    for (int sidx = 1; sidx <= 5; ++sidx) { Arg a; a.kind = Arg::SlotPtr; a.slot = -sidx; out->args.push_back(a); }
    out->algo_bytes = static_cast<double>(n * k * bits / 8 + n * (k / group) * 2 * (symmetric ? 1 : 2) + m * k * dtype_width(act) + m * n * dtype_width(act));
    out->flops = 2.0 * static_cast<double>(m) * static_cast<double>(n) * static_cast<double>(k);
    return true;
  }
  // a chunk of activation columns in shared memory: whole warp-wide strides of 32 pieces (the kernel's layout
  // permutes columns inside such a stride), about 96 KB at most, never more than K rounded up to a stride
  const int64_t stride = 32 * piece;
  int64_t kc = std::max<int64_t>(stride, (96 * 1024) / (4 * m) / stride * stride);
  kc = std::min<int64_t>(kc, (k + stride - 1) / stride * stride);
  const int64_t rpw = m <= 2 ? 4 : 2;
  std::string src = device_prelude() +
                    defines({{"M", m}, {"N", n}, {"K", k}, {"BITS", bits}, {"GROUP", group}, {"SYM", symmetric ? 1 : 0},
                             {"ACT", act == DType::F32 ? 0 : act == DType::BF16 ? 1 : 2}, {"KC", kc}, {"RPW", rpw}}) +
                    kSrc_quant_gemv;
  out->name = "quant_gemv";
  out->kernel = load(src, "ku_quant_gemv", true);
  const int64_t blocks = (n + 8 * rpw - 1) / (8 * rpw);
  out->grid[0] = static_cast<unsigned>(std::min<int64_t>(blocks, static_cast<int64_t>(sm_count) * 4));
  out->block[0] = 256;
  out->smem = static_cast<unsigned>(m * kc * 4);
  for (int sidx = 1; sidx <= 5; ++sidx) { Arg a; a.kind = Arg::SlotPtr; a.slot = -sidx; out->args.push_back(a); }
  out->algo_bytes = static_cast<double>(n * k * bits / 8 + n * (k / group) * 2 * (symmetric ? 1 : 2) + m * k * dtype_width(act) + m * n * dtype_width(act));
  out->flops = 2.0 * static_cast<double>(m) * static_cast<double>(n) * static_cast<double>(k);
  return true;
}

extern const std::string kSrc_softmax_groups_tma;

bool build_softmax_groups(const KernelLoader& load, const Fused& f, size_t axis, int sm_count, Launch* out, std::vector<int>* leaf_args, size_t* scratch_bytes) {
  if (f.dtype() != DType::F32 || std::getenv("KURUMI_SMT_NO_GROUPS")) return false;
  std::string src_fn;
  int64_t R = 0, C = 0;
  bool transposed = false;
  LineLeaf big;
  if (!emit_line_source_fn(f, axis, &src_fn, leaf_args, &R, &C, &transposed, &big) || !transposed || big.leaf < 0) return false;
  // A group of P CTAs shares a slab of 32 lines; a CTA keeps CJ positions of it, eight float4 values per thread at most,
  // in registers, for two slabs at a time (128 registers per thread). Two CTAs of 256 threads per SM (CJ <= 256) while a
  // group then has at most 32 CTAs, else one CTA of 512 threads (CJ <= 512); lines beyond 32 * 512 positions take the
  // panel kernel.
  const int64_t lw = 32;
  const int64_t nt = (C + 255) / 256 <= 32 ? 256 : 512, span = nt;   // positions per CTA at eight values per thread
  const int64_t p = std::max<int64_t>(2, (C + span - 1) / span), per_sm = 512 / nt, unit = nt / 8;
  if (p > 32 || sm_count * per_sm < p || R < lw * 8 || C < 1024 || R * C < (int64_t(1) << 22) || R >= (int64_t(1) << 30) || (big.base * 4) % 16 != 0) return false;
  const int64_t cj = ((C + p - 1) / p + unit - 1) / unit * unit;
  const int64_t boxj = cj % 256 == 0 ? 256 : cj % 128 == 0 ? 128 : cj % 64 == 0 ? 64 : 32;
  const int64_t slabs = (R + lw - 1) / lw;
  const int64_t nbuf = std::min<int64_t>(3, (200 * 1024 / per_sm) / (cj * lw * 4));   // tiles in flight per CTA
  std::string src = device_prelude() + src_fn +
                    defines({{"R", R}, {"C", C}, {"P", p}, {"CJ", cj}, {"BOXJ", boxj}, {"NBUF", nbuf}, {"NT", nt}, {"NSLABS", slabs}, {"KU_OUT_F32", 1}, {"KU_SRC_IDENTITY", big.identity ? 1 : 0}}) +
                    kSrc_softmax_groups_tma;
  out->name = "softmax_groups_tma";
  out->kernel = load(src, "ku_softmax_groups_tma", false);
  out->grid[0] = static_cast<unsigned>(std::min<int64_t>(slabs, per_sm * sm_count / p) * p);
  out->block[0] = static_cast<unsigned>(nt);
  out->smem = static_cast<unsigned>(nbuf * cj * lw * 4 + 1024);   // 1024 bytes of slack: the ring is placed on a 1024-byte boundary
  out->persistent_clusters = -1;                               // cap the grid at the co-resident CTA count on first launch,
  out->grid_multiple = static_cast<unsigned>(p);               // in whole groups,
  out->cooperative = true;                                     // and have the driver hold the launch to it
  Arg tm;
  tm.kind = Arg::Tmap;
  tm.tm.slot = f.leaves[static_cast<size_t>(big.leaf)].slot;
  tm.tm.byte_offset = big.base * 4;
  tm.tm.dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  tm.tm.rank = 2;
  tm.tm.dims[0] = static_cast<uint64_t>(R); tm.tm.dims[1] = static_cast<uint64_t>(C);
  tm.tm.strides[0] = static_cast<uint64_t>(big.ld) * 4;
  tm.tm.box[0] = static_cast<uint32_t>(lw); tm.tm.box[1] = static_cast<uint32_t>(boxj);
  tm.tm.swz = CU_TENSOR_MAP_SWIZZLE_128B;
  out->args.push_back(tm);
  *scratch_bytes = static_cast<size_t>(slabs * (nt / 256) * p * lw * 8);   // one 64-bit (max, sum, parity) word per slab, CTA, warp of a chunk and line
  return true;
}

extern const std::string kSrc_softmax_panels_tma;

size_t softmax_panels_scratch_bytes(int64_t R, int64_t C, int64_t jt, int64_t npb) {
  const int64_t nj = (C + jt - 1) / jt;
  return static_cast<size_t>(16384 + (R * 4 + 255) / 256 * 256 + npb * nj * 256 * 8);   // control block, c, partials [npb][nj][256 lines]
}

bool build_softmax_panels(const KernelLoader& load, const Fused& f, size_t axis, int sm_count, Launch* out, std::vector<int>* leaf_args, size_t* scratch_bytes) {
  if (f.dtype() != DType::F32 || std::getenv("KURUMI_SMT_NO_PANELS")) return false;
  std::string src_fn;
  int64_t R = 0, C = 0;
  bool transposed = false;
  LineLeaf big;
  if (!emit_line_source_fn(f, axis, &src_fn, leaf_args, &R, &C, &transposed, &big) || !transposed || big.leaf < 0) return false;
  if (R < 64 || C < 256 || R * C < (int64_t(1) << 20) || (R + 255) / 256 > 1024 || C >= (int64_t(1) << 30)) return false;
  // tile height, ring depth, how far statistics (la) and merges (lc) run ahead of the output tiles: the measured best
  const int64_t jt = 256, nbuf = 2, la = 4, lc = 2;
  const int64_t npb = la + 2;
  std::string src = device_prelude() + src_fn +
                    defines({{"R", R}, {"C", C}, {"JT", jt}, {"NBUF", nbuf}, {"LA", la}, {"LC", lc}, {"NPB", npb}, {"KU_L2_HINTS", 1}, {"KU_OUT_F32", 1}, {"KU_SRC_IDENTITY", big.identity ? 1 : 0}}) +
                    kSrc_softmax_panels_tma;
  out->name = "softmax_panels_tma";
  out->kernel = load(src, "ku_softmax_panels_tma", false);
  out->grid[0] = static_cast<unsigned>(sm_count * 8);
  out->block[0] = 256;
  out->smem = static_cast<unsigned>(nbuf * jt * 128 + 1024);   // 1024 bytes of slack: the ring is placed on a 1024-byte boundary
  out->persistent_clusters = -1;                               // cap the grid at the co-resident CTA count on first launch
  Arg tm;
  tm.kind = Arg::Tmap;
  tm.tm.slot = f.leaves[static_cast<size_t>(big.leaf)].slot;
  tm.tm.byte_offset = big.base * 4;
  tm.tm.dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  tm.tm.rank = 2;
  tm.tm.dims[0] = static_cast<uint64_t>(R); tm.tm.dims[1] = static_cast<uint64_t>(C);
  tm.tm.strides[0] = static_cast<uint64_t>(big.ld) * 4;
  tm.tm.box[0] = 32; tm.tm.box[1] = static_cast<uint32_t>(jt);
  tm.tm.swz = CU_TENSOR_MAP_SWIZZLE_128B;
  out->args.push_back(tm);
  *scratch_bytes = softmax_panels_scratch_bytes(R, C, jt, npb);
  return true;
}

bool build_softmax_transposed(const KernelLoader& load, const Fused& f, size_t axis, int sm_count, Launch* out, std::vector<int>* leaf_args) {
  if (f.dtype() == DType::F64 || !is_float(f.dtype())) return false;
  std::string src_fn;
  int64_t R = 0, C = 0;
  bool transposed = false;
  LineLeaf big;
  if (!emit_line_source_fn(f, axis, &src_fn, leaf_args, &R, &C, &transposed, &big) || !transposed) return false;
  if (R < 32 || C < 256) return false;
  // cluster size: the smallest power of two whose per-CTA share of a line fits shared memory
  const int64_t max_cj = (200 * 1024) / (33 * 4);
  int64_t cl = 1;
  while (cl < 16 && (C + cl - 1) / cl > max_cj) cl *= 2;
  while (cl < 8 && (C + cl - 1) / cl > 1024) cl *= 2;   // spread a slab over more SMs: more loads in flight per line
  const int64_t cj = (C + cl - 1) / cl;
  if (cj > max_cj) return false;
  const int64_t nt = cj >= 512 ? 1024 : 256, unr = 8;
  std::string src = device_prelude() + src_fn + defines({{"R", R}, {"C", C}, {"CL", cl}, {"CJ", cj}, {"NT", nt}, {"UNR", unr}}) + kSrc_softmax_transposed;
  out->name = "softmax_transposed";
  out->kernel = load(src, "ku_softmax_transposed", false);
  const int64_t slabs = (R + 31) / 32;
  out->grid[0] = static_cast<unsigned>(slabs * cl);
  out->block[0] = static_cast<unsigned>(nt);
  out->cluster[0] = static_cast<unsigned>(cl);
  out->smem = static_cast<unsigned>(cj * 33 * 4);
  (void)sm_count;
  return true;
}
extern const std::string kSrc_attention_tc;

bool attention_supported(DType dt, const Shape& shape) {
  if (std::getenv("KURUMI_NO_TC_ATTENTION")) return false;
  if (!(dt == DType::BF16 || dt == DType::F16) || shape.size() < 2) return false;
  const size_t r = shape.size(), dh = shape[r - 1], s = shape[r - 2];
  size_t bh = 1;
  for (size_t i = 0; i + 2 < r; ++i) bh *= shape[i];
  return (dh == 64 || dh == 128) && s >= 1 && s < (size_t(1) << 24) && bh >= 1 && bh < 65536;
}

bool build_attention(const KernelLoader& load, DType dt, const Shape& shape, bool causal, float scale, int sm_count, Launch* out) {
  if (!attention_supported(dt, shape)) return false;
  const size_t r = shape.size();
  const int64_t dh = static_cast<int64_t>(shape[r - 1]), s = static_cast<int64_t>(shape[r - 2]);
  int64_t bh = 1;
  for (size_t i = 0; i + 2 < r; ++i) bh *= static_cast<int64_t>(shape[i]);
  const uint32_t fmt = dt == DType::BF16 ? 1u : 0u;
  if (!(scale > 0.0f)) return false;   // the kernel scales the block maximum instead of every score
  // K and V rings of two 32 KB stages each (DH = 128): three-stage rings measured the same on the causal 4096-key
  // configuration, the loads are not what the MMA thread waits for
  const int64_t nks = 2, nvs = 2, tk = 128;
  const uint32_t idesc_s = (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(tk >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
  const uint32_t idesc_o = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | (static_cast<uint32_t>(dh >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
  char lit[64];
  std::snprintf(lit, sizeof(lit), "%.9gf", static_cast<double>(scale * 1.4426950408889634f));
  std::string src = device_prelude() +
                    defines({{"BH", bh}, {"S", s}, {"DH", dh}, {"CAUSAL", causal ? 1 : 0}, {"IDESC_S", static_cast<int64_t>(idesc_s)}, {"IDESC_O", static_cast<int64_t>(idesc_o)},
                             {"KU_IS_BF16", dt == DType::BF16 ? 1 : 0}, {"NKS", nks}, {"NVS", nvs}}) +
                    "#define SCALE_LOG2E " + lit + "\n" + kSrc_attention_tc;
  out->name = "attention_tc";
  out->kernel = load(src, "ku_attention_tc_duo", true);
  out->grid[0] = static_cast<unsigned>((s + 255) / 256);
  out->grid[1] = static_cast<unsigned>(bh);
  const int64_t tile = 128 * 128 * (dh / 64);
  out->block[0] = 320;   // TMA warp, MMA warp, a softmax warpgroup per query tile
  // two Q tiles, two K and two V stages, barriers; at least 120 KB so that an SM (512 columns of tensor memory) holds one CTA
  out->smem = static_cast<unsigned>(std::max<int64_t>((2 + nks + nvs) * tile + 256, 120 * 1024));
  for (int slot = -1; slot >= -3; --slot) {
    Arg a;
    a.kind = Arg::Tmap;
    a.tm.slot = slot;
    a.tm.dt = dt == DType::BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    a.tm.rank = 3;
    a.tm.swz = CU_TENSOR_MAP_SWIZZLE_128B;
    a.tm.dims[0] = static_cast<uint64_t>(dh); a.tm.dims[1] = static_cast<uint64_t>(s); a.tm.dims[2] = static_cast<uint64_t>(bh);
    a.tm.strides[0] = static_cast<uint64_t>(dh * 2); a.tm.strides[1] = static_cast<uint64_t>(s * dh * 2);
    a.tm.box[0] = 64; a.tm.box[1] = (slot == -1) ? 128 : static_cast<uint32_t>(tk); a.tm.box[2] = 1;   // slot -1 is Q
    out->args.push_back(a);
  }
  Arg o; o.kind = Arg::SlotPtr; o.slot = -4; out->args.push_back(o);
  Arg st; st.kind = Arg::Status; out->args.push_back(st);
  (void)sm_count;
  return true;
}
std::vector<std::pair<std::string, std::string>> representative_kernel_sources() { return {}; }

}  // namespace ku::cu

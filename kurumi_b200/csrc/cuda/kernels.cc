#include "kernels.h"

#include <cstdlib>

namespace ku::cu {

bool build_gemm_tc(const KernelLoader&, const GemmDesc&, const Fused*, int, Launch*, std::vector<int>*) { return false; }
extern const std::string kSrc_softmax_transposed;
extern const std::string kSrc_softmax_transposed_tma;

namespace {
std::string defines(std::initializer_list<std::pair<const char*, int64_t>> kv) {
  std::string s;
  for (auto& p : kv) s += std::string("#define ") + p.first + " " + std::to_string(p.second) + "\n";
  return s;
}
}  // namespace

bool build_softmax_transposed(const KernelLoader& load, const Fused& f, size_t axis, int sm_count, Launch* out, std::vector<int>* leaf_args) {
  if (f.dtype() == DType::F64 || !is_float(f.dtype())) return false;
  std::string src_fn;
  int64_t R = 0, C = 0;
  bool transposed = false;
  LineLeaf big;
  if (!emit_line_source_fn(f, axis, &src_fn, leaf_args, &R, &C, &transposed, &big) || !transposed) return false;
  if (R < 32 || C < 256) return false;
  // fast path: persistent clusters of 16 fed by TMA, when one plain f32 buffer dominates the reads
  if (big.leaf >= 0 && C >= 2048 && f.dtype() == DType::F32 && !std::getenv("KURUMI_SMT_NO_TMA")) {
    const int64_t cl = 16;
    int64_t cj = (C + cl - 1) / cl;
    cj = (cj + 31) / 32 * 32;
    const int64_t boxj = cj % 256 == 0 ? 256 : cj % 128 == 0 ? 128 : cj % 64 == 0 ? 64 : 32;
    int64_t nbuf = std::min<int64_t>(3, (200 * 1024) / (cj * 128));
    if (const char* e = std::getenv("KURUMI_SMT_NBUF")) nbuf = std::atoi(e);
    if (nbuf >= 2 && R < (int64_t(1) << 30) && C < (int64_t(1) << 30)) {
      const int64_t nt = 512, slabs = (R + 31) / 32;
      std::string src = device_prelude() + src_fn +
                        defines({{"R", R}, {"C", C}, {"CL", cl}, {"CJ", cj}, {"BOXJ", boxj}, {"NBUF", nbuf}, {"NT", nt}, {"NSLABS", slabs}, {"KU_SRC_IDENTITY", big.identity ? 1 : 0}}) +
                        kSrc_softmax_transposed_tma;
      out->name = "softmax_transposed_tma";
      out->kernel = load(src, "ku_softmax_transposed_tma", false);
      out->grid[0] = static_cast<unsigned>(slabs * cl);
      out->block[0] = static_cast<unsigned>(nt);
      out->cluster[0] = static_cast<unsigned>(cl);
      out->smem = static_cast<unsigned>(nbuf * cj * 128 + 1024);  // + slack for the 1024-byte alignment of the tile ring
      out->persistent_clusters = -1;                              // cap the grid at the co-resident cluster count on first launch
      Arg tm;
      tm.kind = Arg::Tmap;
      tm.tm.slot = f.leaves[static_cast<size_t>(big.leaf)].slot;
      tm.tm.byte_offset = big.base * 4;
      tm.tm.dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
      tm.tm.rank = 2;
      tm.tm.dims[0] = static_cast<uint64_t>(R); tm.tm.dims[1] = static_cast<uint64_t>(C);
      tm.tm.strides[0] = static_cast<uint64_t>(big.ld) * 4;
      tm.tm.box[0] = 32; tm.tm.box[1] = static_cast<uint32_t>(boxj);
      tm.tm.swz = CU_TENSOR_MAP_SWIZZLE_128B;
      out->args.push_back(tm);
      out->status_arg = true;   // the kernel's last parameter is the device status word
      return true;
    }
  }
  // cluster size: the smallest power of two whose per-CTA share of a line fits shared memory
  const int64_t max_cj = (200 * 1024) / (33 * 4);
  int64_t cl = 1;
  while (cl < 16 && (C + cl - 1) / cl > max_cj) cl *= 2;
  while (cl < 8 && (C + cl - 1) / cl > 1024) cl *= 2;   // spread a slab over more SMs: more loads in flight per line
  if (const char* e = std::getenv("KURUMI_SMT_CL")) cl = std::atoi(e);
  const int64_t cj = (C + cl - 1) / cl;
  if (cj > max_cj) return false;
  int64_t nt = cj >= 512 ? 1024 : 256;
  int64_t unr = 8;
  if (const char* e = std::getenv("KURUMI_SMT_NT")) nt = std::atoi(e);
  if (const char* e = std::getenv("KURUMI_SMT_UNR")) unr = std::atoi(e);
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
bool attention_supported(DType, const Shape&) { return false; }
bool build_attention(const KernelLoader&, DType, const Shape&, bool, float, int, Launch*) { return false; }
std::vector<std::pair<std::string, std::string>> representative_kernel_sources() { return {}; }

}  // namespace ku::cu

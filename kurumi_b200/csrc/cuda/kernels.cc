#include "kernels.h"

namespace ku::cu {

bool build_gemm_tc(const KernelLoader&, const GemmDesc&, const Fused*, int, Launch*, std::vector<int>*) { return false; }
bool build_softmax_transposed(const KernelLoader&, const Fused&, size_t, int, Launch*, std::vector<int>*) { return false; }
bool attention_supported(DType, const Shape&) { return false; }
bool build_attention(const KernelLoader&, DType, const Shape&, bool, float, int, Launch*) { return false; }
std::vector<std::pair<std::string, std::string>> representative_kernel_sources() { return {}; }

}  // namespace ku::cu

// Hand-written sm_100a kernel templates (sources under kernels/) and the host code that
// instantiates them: picks tiles, builds TMA tensor maps, fills in the launch.
#pragma once
#include "fuse.h"

namespace ku::cu {

// Tensor-core contraction (tcgen05 + TMEM, TMA-fed) with the generated epilogue. Returns false
// when the operand layout / dtype is outside what the kernel takes (the caller then uses the SIMT
// kernel). Operand slots in the returned launch are symbolic: -1 = A, -2 = B, -3 = C.
bool build_gemm_tc(const KernelLoader& load, const GemmDesc& d, const Fused* epi, int sm_count, Launch* out, std::vector<int>* epi_leaf_args);

// Single-pass softmax for lines that are strided in memory while the previous axis is contiguous
// (a softmax consumed through a transpose view). Returns false when the pattern does not apply.
bool build_softmax_transposed(const KernelLoader& load, const Fused& f, size_t axis, int sm_count, Launch* out, std::vector<int>* leaf_args);

// The same softmax in a single pass: groups of P co-resident CTAs hold a 32-line slab on chip (the tile goes from
// shared memory into registers) and exchange per-line (max, sum) pairs through global scratch
// (kernels/softmax_groups_tma.cuh). After the leaf arguments the kernel takes {output, scratch, launch counter,
// status}; the caller creates the scratch slot of `*scratch_bytes` bytes, zero when allocated and never cleared
// again (the words carry the parity of the launch counter).
bool build_softmax_groups(const KernelLoader& load, const Fused& f, size_t axis, int sm_count, Launch* out, std::vector<int>* leaf_args, size_t* scratch_bytes);

// The same softmax as two passes inside one persistent TMA-fed kernel whose second pass reads from L2
// (kernels/softmax_panels_tma.cuh). After the leaf arguments the kernel takes {output, scratch, status};
// the caller creates the scratch slot of `*scratch_bytes` bytes and has its first 16 KB cleared before each launch.
bool build_softmax_panels(const KernelLoader& load, const Fused& f, size_t axis, int sm_count, Launch* out, std::vector<int>* leaf_args, size_t* scratch_bytes);

// The streaming two-pass form of the same softmax (precompiled kernels, softmax_two_pass.cu) for the
// plain case: one f32 buffer read transposed, optionally plus a bias that broadcasts along the lines.
// On success `out->args` is {input, bias (or input again when absent), output, scratch} with the
// scratch slot symbolic (-1) and `*scratch_bytes` set; the caller creates that slot.
bool build_softmax_two_pass(const Fused& f, size_t axis, Launch* out, size_t* scratch_bytes);

// Quantised matmul for at most 8 activation rows, reading the packed weight directly (kernels/quant_gemv.cuh).
// Slots are symbolic: -1 qweight, -2 scales, -3 mins (scales again when symmetric), -4 act, -5 out.
bool quant_gemv_supported(DType act, int64_t m, int64_t n, int64_t k, int bits, int64_t group);
bool build_quant_gemv(const KernelLoader& load, DType act, int64_t m, int64_t n, int64_t k, int bits, int64_t group, bool symmetric, int sm_count, Launch* out);

// Fused causal / full attention with online softmax. Slots are symbolic: -1 q, -2 k, -3 v, -4 out.
bool attention_supported(DType dt, const Shape& shape);
bool build_attention(const KernelLoader& load, DType dt, const Shape& shape, bool causal, float scale, int sm_count, Launch* out);

// Every template instantiated once with representative parameters, for the no-GPU build check.
std::vector<std::pair<std::string, std::string>> representative_kernel_sources();

}  // namespace ku::cu

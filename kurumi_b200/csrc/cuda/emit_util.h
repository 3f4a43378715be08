// Small helpers shared by the emitter files (defined in emit.cc).
#pragma once
#include <cstdint>
#include <string>

#include "../core/dtype.h"

namespace ku::cu::emitutil {

bool is_lowf(DType d);                                     // f16 / bf16 / fp8: held in registers as rounded f32
std::string rnd(DType d, const std::string& e);           // round a register value to the dtype's grid
std::string dec(DType d, const std::string& e);           // storage bits -> register value
std::string enc(DType d, const std::string& e);           // register value -> storage bits
int bits_of(DType d);
const char* wrap_utype(DType d);                           // unsigned type integer arithmetic wraps in
constexpr unsigned kStreamCtasPerSm = 64;                  // grid cap of the streaming kernels, in CTAs of 256 threads per SM (measured; see emit_pointwise)
unsigned pick_grid(int64_t work_items, unsigned per_block, int sm_count, unsigned blocks_per_sm);
unsigned line_grid(int64_t items, int64_t cap);          // CTAs of a kernel that loops over `items` lines, `cap` resident at once

}  // namespace ku::cu::emitutil

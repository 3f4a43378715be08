// Softmax over lines that are strided in memory, as a streaming two-pass algorithm with a small
// scratch buffer: out[i][j] = softmax_j(in[j * ld + i] + bias[j]) for i < lines, j < len, f32.
// This is the shape a softmax takes when it is consumed through a transpose view with a bias that
// broadcasts along the lines (kurumi_core/src/interp/nn.rs:35-69 gives the math; the view comes
// from kurumi_core/src/lower/index/movement.rs:18-30).
//
//   pass 1  ku_sm2_stats    every CTA streams a block of JT positions (whole rows of `in`, fully
//                           coalesced) and keeps, per line, a running (max, sum of exp2) in the
//                           log2 domain; one partial per (position block, line) goes to scratch
//   pass 1b ku_sm2_combine  per line: merge the partials into c = max + log2(sum)
//   pass 2  ku_sm2_apply    64 x 64 tiles: read rows of `in` coalesced, out = exp2(x*log2e - c),
//                           transpose through shared memory, write rows of `out` coalesced; tiles
//                           run from the last positions back to the first so that what pass 1
//                           left in L2 is read before it is evicted
// HBM traffic: `in` is read twice at most (less by what L2 keeps), `out` written once.
//
// Two host entry points share the kernels: ku_cuda_softmax_lines_f32 takes its scratch from the
// backend's device pool; ku_cuda_softmax_lines_f32_noalloc uses a fixed array that lives in the
// library's device image and therefore allocates nothing.
#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>

#include "../../../include/kurumi_cuda.h"
#include "../capi/handles.h"
#include "backend.h"

namespace {

constexpr int JT = 128;       // positions per statistics block
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }

// partial[(jb * lines + i)] = (max_t, sum_j exp2(t_j - max_t)) over the block's positions, t = (x + bias) * log2e
template <int VEC>
__global__ void __launch_bounds__(256) ku_sm2_stats(const float* __restrict__ in, const float* __restrict__ bias, float2* __restrict__ partial, int lines, int len,
                                                    long long ld) {
  const int i = (blockIdx.x * 256 + threadIdx.x) * VEC;
  const int j0 = blockIdx.y * JT, j1 = min(j0 + JT, len);
  if (i >= lines) return;
  float m[VEC], s[VEC];
#pragma unroll
  for (int v = 0; v < VEC; ++v) { m[v] = -INFINITY; s[v] = 0.0f; }
  for (int j = j0; j < j1; j += 8) {
    float t[8][VEC];
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const int jj = j + r;
      if (jj < j1) {
        const float b = bias ? bias[jj] : 0.0f;
        if (VEC == 4) {
          const float4 x = *reinterpret_cast<const float4*>(in + (long long)jj * ld + i);
          t[r][0] = (x.x + b) * kLog2e; t[r][1 % VEC] = (x.y + b) * kLog2e; t[r][2 % VEC] = (x.z + b) * kLog2e; t[r][3 % VEC] = (x.w + b) * kLog2e;
        } else {
#pragma unroll
          for (int v = 0; v < VEC; ++v) t[r][v] = (in[(long long)jj * ld + i + v] + b) * kLog2e;
        }
      } else {
#pragma unroll
        for (int v = 0; v < VEC; ++v) t[r][v] = -INFINITY;
      }
    }
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      float m8 = t[0][v];
#pragma unroll
      for (int r = 1; r < 8; ++r) m8 = fmaxf(m8, t[r][v]);
      const float mn = fmaxf(m[v], m8);
      // all -inf so far: keep the sum at 0 instead of producing inf - inf
      float acc = (mn == -INFINITY) ? 0.0f : s[v] * ex2(m[v] - mn);
#pragma unroll
      for (int r = 0; r < 8; ++r) acc += (mn == -INFINITY && !(t[r][v] != t[r][v])) ? 0.0f : ex2(t[r][v] - mn);
      m[v] = mn;
      s[v] = acc;
    }
  }
#pragma unroll
  for (int v = 0; v < VEC; ++v) partial[(long long)blockIdx.y * lines + i + v] = make_float2(m[v], s[v]);
}

// c[i] = max_t + log2(sum): exp(x - max) / sum == exp2(t - c)
__global__ void __launch_bounds__(256) ku_sm2_combine(const float2* __restrict__ partial, float* __restrict__ c, int lines, int blocks) {
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (i >= lines) return;
  float m = -INFINITY;
  for (int b = 0; b < blocks; ++b) m = fmaxf(m, partial[(long long)b * lines + i].x);
  float s = 0.0f;
  for (int b = 0; b < blocks; ++b) {
    const float2 p = partial[(long long)b * lines + i];
    s += (p.x == -INFINITY) ? ((p.y != p.y) ? p.y : 0.0f) : p.y * ex2(p.x - m);
  }
  // a line of -inf only: the interpreter computes exp(-inf - -inf) = NaN everywhere
  c[i] = (m == -INFINITY) ? __int_as_float(0x7fc00000) : m + log2f(s);
}

__global__ void __launch_bounds__(256) ku_sm2_apply(const float* __restrict__ in, const float* __restrict__ bias, const float* __restrict__ c, float* __restrict__ out,
                                                    int lines, int len, long long ld) {
  __shared__ float tile[64][65];
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
  const int i0 = blockIdx.x * 64;
  const int j0 = (gridDim.y - 1 - blockIdx.y) * 64;  // last positions first: they are the freshest in L2
  const int i = i0 + tx;
  const float ci = i < lines ? c[i] : 0.0f;
#pragma unroll 4
  for (int r = 0; r < 16; ++r) {
    const int jl = ty + 4 * r, j = j0 + jl;
    float v = 0.0f;
    if (i < lines && j < len) {
      const float b = bias ? bias[j] : 0.0f;
      v = ex2(__fmaf_rn(in[(long long)j * ld + i] + b, kLog2e, -ci));
    }
    tile[jl][tx] = v;
  }
  __syncthreads();
#pragma unroll 4
  for (int r = 0; r < 16; ++r) {
    const int il = ty + 4 * r;
    if (i0 + il < lines && j0 + tx < len) out[(long long)(i0 + il) * len + j0 + tx] = tile[tx][il];
  }
}

// scratch layout: partials [blocks][lines] float2, then c [lines] float
size_t scratch_bytes(size_t lines, size_t len) {
  const size_t blocks = (len + JT - 1) / JT;
  return blocks * lines * sizeof(float2) + lines * sizeof(float);
}

cudaError_t launch_two_pass(const float* in, const float* bias, float* out, size_t lines, size_t len, size_t ld, void* scratch, cudaStream_t stream) {
  if (lines == 0 || len == 0) return cudaSuccess;
  const int blocks = static_cast<int>((len + JT - 1) / JT);
  float2* partial = static_cast<float2*>(scratch);
  float* c = reinterpret_cast<float*>(partial + static_cast<size_t>(blocks) * lines);
  const bool vec = lines % 4 == 0 && ld % 4 == 0 && (reinterpret_cast<uintptr_t>(in) & 15) == 0;
  if (vec) {
    dim3 grid(static_cast<unsigned>((lines / 4 + 255) / 256), static_cast<unsigned>(blocks));
    ku_sm2_stats<4><<<grid, 256, 0, stream>>>(in, bias, partial, static_cast<int>(lines), static_cast<int>(len), static_cast<long long>(ld));
  } else {
    dim3 grid(static_cast<unsigned>((lines + 255) / 256), static_cast<unsigned>(blocks));
    ku_sm2_stats<1><<<grid, 256, 0, stream>>>(in, bias, partial, static_cast<int>(lines), static_cast<int>(len), static_cast<long long>(ld));
  }
  ku_sm2_combine<<<static_cast<unsigned>((lines + 255) / 256), 256, 0, stream>>>(partial, c, static_cast<int>(lines), blocks);
  dim3 grid2(static_cast<unsigned>((lines + 63) / 64), static_cast<unsigned>((len + 63) / 64));
  ku_sm2_apply<<<grid2, 256, 0, stream>>>(in, bias, c, out, static_cast<int>(lines), static_cast<int>(len), static_cast<long long>(ld));
  return cudaGetLastError();
}

bool args_ok(const float* in, const float* out, size_t lines, size_t len, size_t ld) {
  if ((!in || !out) && lines && len) { ku::set_err("softmax_lines: null input / output pointer"); return false; }
  if (ld < lines) { ku::set_err("softmax_lines: ld is smaller than the number of lines"); return false; }
  if (lines >= (size_t(1) << 31) || len >= (size_t(1) << 31)) { ku::set_err("softmax_lines: extent does not fit 31 bits"); return false; }
  // the position blocks of a line (64 positions each in the write-out pass) are the launch grid's second dimension
  if (len > size_t(65535) * 64) { ku::set_err("softmax_lines: lines longer than 65535 * 64 = 4194240 positions are not supported by this entry point"); return false; }
  return true;
}

}  // namespace

namespace ku::cu {
// used by the graph scheduler when a softmax has exactly this shape
size_t softmax_two_pass_scratch_bytes(size_t lines, size_t len) { return scratch_bytes(lines, len); }
void softmax_two_pass_launch(const float* in, const float* bias, float* out, size_t lines, size_t len, size_t ld, void* scratch, cudaStream_t stream) {
  cuda_check(launch_two_pass(in, bias, out, lines, len, ld, scratch, stream), "softmax two-pass launch");
}
}  // namespace ku::cu

extern "C" int32_t ku_cuda_softmax_lines_f32(const KuBackend* b, const float* in, const float* bias, float* out, size_t lines, size_t len, size_t ld) {
  if (!b) { ku::set_err("ku_cuda_softmax_lines_f32: null backend handle"); return -1; }
  if (!args_ok(in, out, lines, len, ld)) return -1;
  return ku::guard<int32_t>(-1, [&]() -> int32_t {
    auto* cb = dynamic_cast<ku::cu::CudaBackend*>(b->b.get());
    if (!cb) throw ku::Error::backend("not a CUDA backend");
    ku::cu::Runtime& rt = cb->runtime();
    rt.make_current();
    void* scratch = rt.alloc(scratch_bytes(lines, len));
    cudaError_t e = launch_two_pass(in, bias, out, lines, len, ld, scratch, rt.stream());
    rt.free(scratch);  // stream-ordered reuse: the pool hands it only to later work on the same stream
    ku::cu::cuda_check(e, "ku_cuda_softmax_lines_f32");
    ++rt.stats.launches;
    return 0;
  });
}

// ---- the entry point that allocates nothing -------------------------------------------------------
// Some callers may not allocate device memory at the moment they need this softmax: a serving loop
// whose latency budget has no room for the device-wide synchronisation cudaMalloc / cudaFree can
// imply, a host application that has handed all of HBM to its own arena so the CUDA allocator has
// nothing left to give, or code that runs where entering the CUDA allocator is not allowed (another
// library's allocation hook). For them the scratch of the two-pass algorithm lives in a fixed array
// inside the library's device image. The FIRST call on a device is different: it looks up the array's
// device address, and with the CUDA runtime's lazy loading it is also the moment the device image - the
// kernels and the 8 MiB array itself - is placed on that GPU. So a process makes one small real call per
// device at start-up (a few lines, so that all three kernels load), before it hands HBM away and before
// any stream capture; the calls after it touch neither the allocator nor the loader.
namespace {
constexpr size_t kNoAllocScratchBytes = size_t(8) << 20;  // 8 MiB per GPU that loads the library, held until the process exits
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

constexpr int kMaxDevices = 64;
void* g_noalloc_ptr[kMaxDevices] = {nullptr};
std::mutex g_noalloc_mutex;

// In host code `g_noalloc_scratch` is only a handle for the symbol, not a device address: the address
// this device gave the array has to be asked for, once per device, with that device current.
void* noalloc_scratch_for_current_device() {
  int dev = -1;
  ku::cu::cuda_check(cudaGetDevice(&dev), "cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices) throw ku::Error::backend("ku_cuda_softmax_lines_f32_noalloc: device index out of range");
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (!g_noalloc_ptr[dev]) {
    void* p = nullptr;
    ku::cu::cuda_check(cudaGetSymbolAddress(&p, g_noalloc_scratch), "cudaGetSymbolAddress(scratch)");
    g_noalloc_ptr[dev] = p;
  }
  return g_noalloc_ptr[dev];
}
}  // namespace

extern "C" int32_t ku_cuda_softmax_lines_f32_noalloc(const float* in, const float* bias, float* out, size_t lines, size_t len, size_t ld, void* stream) {
  if (!args_ok(in, out, lines, len, ld)) return -1;
  return ku::guard<int32_t>(-1, [&]() -> int32_t {
    const size_t need = scratch_bytes(lines, len);
    if (need > kNoAllocScratchBytes)
      throw ku::Error::backend("ku_cuda_softmax_lines_f32_noalloc: lines * ceil(len / 128) * 8 + lines * 4 = " + std::to_string(need) +
                               " bytes of scratch exceed the fixed " + std::to_string(kNoAllocScratchBytes) + "; use ku_cuda_softmax_lines_f32");
    void* scratch = noalloc_scratch_for_current_device();
    // every scratch entry the kernels read is written earlier in the same call, so nothing needs clearing
    ku::cu::cuda_check(launch_two_pass(in, bias, out, lines, len, ld, scratch, static_cast<cudaStream_t>(stream)), "ku_cuda_softmax_lines_f32_noalloc");
    return 0;
  });
}

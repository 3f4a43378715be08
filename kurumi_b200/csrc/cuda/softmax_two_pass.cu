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

#include <algorithm>
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

// ---- the same two passes as ONE persistent kernel, panel by panel, so that pass 2 reads from L2 -------
// The lines are cut into panels of PW = 256 lines (a panel of an 8192-position input is 8 MB, a small
// part of L2). Work items are handed out from one global counter, group after group; group g holds
//   A(g + LA)  statistics of JT2 positions of panel g + LA: one partial (max, sum) per line
//   C(g + LC)  merges of 16 lines of panel g + LC: partials -> c[], once every A item of that panel is done
//   B(g)       64 x 64 output tiles of panel g; they wait for the panel's merges
// so a panel's statistics are handed out LA groups, and its merges LC groups, before its output tiles,
// which find their input still in L2. HBM traffic is then the algorithmic minimum: every input byte
// read once, every output byte written once.
// Every wait is on items that were claimed earlier, by CTAs that are therefore already running, so the
// kernel needs no co-residency guarantee; all waits are bounded and raise a sticky error when they give up.
constexpr int PW = 256;          // lines per panel
constexpr int JT2 = 64;          // positions per statistics item
constexpr int LA = 3;            // groups by which statistics run ahead of the output tiles
constexpr int LC = 2;            // groups by which merges run ahead of the output tiles
constexpr int NBUFS = 4;         // partial buffers in rotation (must exceed LA - LC)
constexpr int NC = PW / 16;      // merge items per panel
constexpr int kMaxPanels = 1024;
constexpr unsigned kSpinLimit = 1u << 24;
struct FusedCtl { unsigned next_item; unsigned error; unsigned cnt_a[kMaxPanels]; unsigned cnt_c[kMaxPanels]; };
constexpr size_t kCtlBytes = 16384;
static_assert(sizeof(FusedCtl) <= kCtlBytes, "control block");

// statistics of JT2 positions of a panel: each thread folds RG positions of VEC lines, the G row groups
// are merged through shared memory, and partial row jb of the panel's buffer is written
template <int VEC>
__device__ __forceinline__ void sm2_stats_item(const float* __restrict__ in, const float* __restrict__ bias, float2* __restrict__ partial, int lines, int len,
                                               long long ld, int i_base, int jb, float2 (*s_part)[PW]) {
  constexpr int TX = PW / VEC, G = 256 / TX, RG = JT2 / G;
  const int tx = threadIdx.x % TX, g = threadIdx.x / TX;
  const int il = tx * VEC, i = i_base + il;
  const int j0 = jb * JT2 + g * RG, j1 = min(j0 + RG, len);
  float m[VEC], s[VEC];
#pragma unroll
  for (int v = 0; v < VEC; ++v) { m[v] = -INFINITY; s[v] = 0.0f; }
  for (int j = j0; j < j1 && i < lines; j += 8) {
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
      float acc = (mn == -INFINITY) ? s[v] : s[v] * ex2(m[v] - mn);
#pragma unroll
      for (int r = 0; r < 8; ++r) acc += (mn == -INFINITY && !(t[r][v] != t[r][v])) ? 0.0f : ex2(t[r][v] - mn);
      m[v] = mn;
      s[v] = acc;
    }
  }
  if (G == 1) {
    if (i < lines) partial[(long long)jb * PW + il] = make_float2(m[0], s[0]);
  } else {
#pragma unroll
    for (int v = 0; v < VEC; ++v) s_part[g % 4][il + v] = make_float2(m[v], s[v]);
    __syncthreads();
    const int l = threadIdx.x;
    if (i_base + l < lines) {
      float mm = -INFINITY;
#pragma unroll
      for (int k = 0; k < G; ++k) mm = fmaxf(mm, s_part[k % 4][l].x);
      float tot = 0.0f;
#pragma unroll
      for (int k = 0; k < G; ++k) {
        const float2 q2 = s_part[k % 4][l];
        tot += (q2.x == -INFINITY) ? q2.y : q2.y * ex2(q2.x - mm);
      }
      partial[(long long)jb * PW + l] = make_float2(mm, tot);
    }
  }
}

__device__ __forceinline__ unsigned sm2_ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// one thread publishes the CTA's earlier writes (ordered before it by the CTA barrier) and counts the item as done
__device__ __forceinline__ void sm2_signal(unsigned* counter) {
  __syncthreads();
  if (threadIdx.x == 0) asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(counter) : "memory");
}
// bounded wait of a whole CTA until *counter reaches target; on giving up it raises the sticky error.
// Only thread 0 polls (acquire); the CTA barrier orders the other threads' later L2 loads after it.
__device__ __forceinline__ void sm2_wait(unsigned* counter, unsigned target, FusedCtl* ctl, int* status) {
  if (threadIdx.x == 0) {
    unsigned spins = 0;
    while (sm2_ld_acquire(counter) < target) {
      if (++spins > kSpinLimit || sm2_ld_acquire(&ctl->error) != 0u) {
        atomicExch(&ctl->error, 1u);
        if (status) atomicExch(status, 7);
        break;
      }
      __nanosleep(32);
    }
  }
  __syncthreads();
}

template <int VEC>
__global__ void __launch_bounds__(256) ku_sm2_fused(const float* __restrict__ in, const float* __restrict__ bias, float* __restrict__ out, float2* __restrict__ partials,
                                                    float* __restrict__ c, FusedCtl* __restrict__ ctl, int* __restrict__ status, int lines, int len, long long ld) {
  __shared__ float tile[64][65];
  __shared__ float2 s_part[4][PW];
  __shared__ unsigned s_item;
  const int panels = (lines + PW - 1) / PW;
  const int na = (len + JT2 - 1) / JT2;                       // statistics items per panel = partial rows per panel
  const int tiles_j = (len + 63) / 64;
  const int nbt = (PW / 64) * tiles_j;                        // output tiles per panel
  const int per = na + NC + nbt;
  const long long total = (long long)panels * per;
  const int nfull = max(panels - LA, 0);                      // groups that hold all three kinds
  if (threadIdx.x == 0) s_item = atomicAdd(&ctl->next_item, 1u);
  __syncthreads();
  for (;;) {
    const long long t = s_item;
    if (t >= total) break;
    // claim the following item now; the answer is only needed when this one is finished
    unsigned following = 0;
    if (threadIdx.x == 0) following = atomicAdd(&ctl->next_item, 1u);
    // find the group g and the offset inside it
    long long rem = t;
    int g = -LA;
    bool found = false;
    for (; g < 0; ++g) {
      const int sz = (g + LA < panels ? na : 0) + ((g + LC >= 0 && g + LC < panels) ? NC : 0);
      if (rem < sz) { found = true; break; }
      rem -= sz;
    }
    if (!found) {
      if (rem < (long long)nfull * per) { g = (int)(rem / per); rem -= (long long)g * per; }
      else {
        rem -= (long long)nfull * per;
        for (g = nfull; g < panels; ++g) {
          const int sz = (g + LA < panels ? na : 0) + (g + LC < panels ? NC : 0) + nbt;
          if (rem < sz) break;
          rem -= sz;
        }
      }
    }
    const int a_sz = (g + LA < panels) ? na : 0;
    const int c_sz = (g + LC >= 0 && g + LC < panels) ? NC : 0;
    int p, r, kind;   // kind 0 = statistics, 1 = merge, 2 = output tile
    if (rem < a_sz) { p = g + LA; r = (int)rem; kind = 0; }
    else if (rem < a_sz + c_sz) { p = g + LC; r = (int)rem - a_sz; kind = 1; }
    else { p = g; r = (int)rem - a_sz - c_sz; kind = 2; }
    const int i_base = p * PW;
    float2* part = partials + (long long)(p % NBUFS) * na * PW;
    if (kind == 0) {
      // this panel's partials reuse the buffer of panel p - NBUFS: its merge must be over (it nearly always is)
      if (p >= NBUFS) sm2_wait(&ctl->cnt_c[p - NBUFS], NC, ctl, status);
      sm2_stats_item<VEC>(in, bias, part, lines, len, ld, i_base, r, s_part);
      sm2_signal(&ctl->cnt_a[p]);
    } else if (kind == 1) {
      sm2_wait(&ctl->cnt_a[p], (unsigned)na, ctl, status);
      // 16 lines x 16 slices of the partial rows; one batch of 8 loads per thread for 128 partial rows
      const int ln = threadIdx.x & 15, sl = threadIdx.x >> 4;
      const int il = r * 16 + ln;
      float m = -INFINITY, sum = 0.0f;
      for (int b0 = sl; b0 < na; b0 += 128) {
        float2 q2[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const int b = b0 + 16 * k;
          q2[k] = b < na ? __ldcg(part + (long long)b * PW + il) : make_float2(-INFINITY, 0.0f);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float mn = fmaxf(m, q2[k].x);
          const float a0 = (m == -INFINITY) ? sum : sum * ex2(m - mn);                 // sum is 0 or NaN while m is -inf
          const float a1 = (q2[k].x == -INFINITY) ? q2[k].y : q2[k].y * ex2(q2[k].x - mn);
          sum = a0 + a1;
          m = mn;
        }
      }
      float2* s_merge = &s_part[0][0];   // [16 slices][16 lines]
      s_merge[sl * 16 + ln] = make_float2(m, sum);
      __syncthreads();
      if (sl == 0 && i_base + il < lines) {
        float mm = -INFINITY;
#pragma unroll
        for (int k = 0; k < 16; ++k) mm = fmaxf(mm, s_merge[k * 16 + ln].x);
        float tot = 0.0f;
#pragma unroll
        for (int k = 0; k < 16; ++k) {
          const float2 q2 = s_merge[k * 16 + ln];
          tot += (q2.x == -INFINITY) ? q2.y : q2.y * ex2(q2.x - mm);
        }
        c[i_base + il] = (mm == -INFINITY) ? __int_as_float(0x7fc00000) : mm + log2f(tot);
      }
      sm2_signal(&ctl->cnt_c[p]);
    } else {
      // the panel's merges were handed out LC groups ago; normally no wait at all
      sm2_wait(&ctl->cnt_c[p], NC, ctl, status);
      const int ti = r / tiles_j, tj = r - ti * tiles_j;
      const int i0 = i_base + ti * 64, j0 = tj * 64;
      if (VEC == 4) {
        // 16 threads x float4 cover the 64 lines of a position; all four loads of a thread are in flight together
        const int lq = threadIdx.x & 15, jr = threadIdx.x >> 4;
        const int i = i0 + 4 * lq;
        float4 x[4];
        float bj[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int j = j0 + jr + 16 * q;
          const bool ok = i < lines && j < len;
          x[q] = ok ? *reinterpret_cast<const float4*>(in + (long long)j * ld + i) : make_float4(0.f, 0.f, 0.f, 0.f);
          bj[q] = (ok && bias) ? bias[j] : 0.0f;
        }
        const float4 ci = i < lines ? __ldcg(reinterpret_cast<const float4*>(c + i)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float* row = &tile[jr + 16 * q][4 * lq];
          row[0] = ex2(__fmaf_rn(x[q].x + bj[q], kLog2e, -ci.x));
          row[1] = ex2(__fmaf_rn(x[q].y + bj[q], kLog2e, -ci.y));
          row[2] = ex2(__fmaf_rn(x[q].z + bj[q], kLog2e, -ci.z));
          row[3] = ex2(__fmaf_rn(x[q].w + bj[q], kLog2e, -ci.w));
        }
        __syncthreads();
        // 16 threads x float4 cover the 64 positions of a line
        const bool vec_out = (len & 3) == 0;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int il = jr + 16 * q, jl = 4 * lq;
          if (i0 + il < lines) {
            float* dst = out + (long long)(i0 + il) * len + j0 + jl;
            const float v0 = tile[jl][il], v1 = tile[jl + 1][il], v2 = tile[jl + 2][il], v3 = tile[jl + 3][il];
            if (vec_out && j0 + jl + 3 < len) *reinterpret_cast<float4*>(dst) = make_float4(v0, v1, v2, v3);
            else {
              if (j0 + jl < len) dst[0] = v0;
              if (j0 + jl + 1 < len) dst[1] = v1;
              if (j0 + jl + 2 < len) dst[2] = v2;
              if (j0 + jl + 3 < len) dst[3] = v3;
            }
          }
        }
      } else {
        const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
        const int i = i0 + tx;
        const float ci = i < lines ? __ldcg(c + i) : 0.0f;
#pragma unroll
        for (int q = 0; q < 16; ++q) {
          const int jl = ty + 4 * q, j = j0 + jl;
          float v = 0.0f;
          if (i < lines && j < len) {
            const float b = bias ? bias[j] : 0.0f;
            v = ex2(__fmaf_rn(in[(long long)j * ld + i] + b, kLog2e, -ci));
          }
          tile[jl][tx] = v;
        }
        __syncthreads();
#pragma unroll 4
        for (int q = 0; q < 16; ++q) {
          const int il = ty + 4 * q;
          if (i0 + il < lines && j0 + tx < len) out[(long long)(i0 + il) * len + j0 + tx] = tile[tx][il];
        }
      }
    }
    __syncthreads();   // every thread is done with s_item and the shared tiles
    if (threadIdx.x == 0) s_item = following;
    __syncthreads();
  }
}

// scratch of the fused kernel: control block, c [lines], partials [NBUFS][partial rows][PW]
size_t fused_scratch_bytes(size_t lines, size_t len) {
  const size_t na = (len + JT2 - 1) / JT2;
  return kCtlBytes + ((lines * sizeof(float) + 255) / 256) * 256 + size_t(NBUFS) * na * PW * sizeof(float2);
}

cudaError_t launch_fused(const float* in, const float* bias, float* out, size_t lines, size_t len, size_t ld, void* scratch, cudaStream_t stream, int sm_count, int* status) {
  if (lines == 0 || len == 0) return cudaSuccess;
  auto* ctl = static_cast<FusedCtl*>(scratch);
  float* c = reinterpret_cast<float*>(static_cast<char*>(scratch) + kCtlBytes);
  float2* partials = reinterpret_cast<float2*>(static_cast<char*>(scratch) + kCtlBytes + ((lines * sizeof(float) + 255) / 256) * 256);
  const size_t panels = (lines + PW - 1) / PW;
  cudaError_t e = cudaMemsetAsync(ctl, 0, 8 + 2 * sizeof(unsigned) * kMaxPanels, stream);
  (void)panels;
  if (e != cudaSuccess) return e;
  const bool vec = lines % 4 == 0 && ld % 4 == 0 && (reinterpret_cast<uintptr_t>(in) & 15) == 0;
  static int per_sm[2] = {0, 0};   // resident CTAs per SM of the two instantiations
  int& occ = per_sm[vec ? 1 : 0];
  if (occ == 0) {
    e = vec ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, ku_sm2_fused<4>, 256, 0) : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, ku_sm2_fused<1>, 256, 0);
    if (e != cudaSuccess) return e;
    if (occ < 1) occ = 1;
  }
  const unsigned grid = static_cast<unsigned>(sm_count) * static_cast<unsigned>(occ);
  int li = static_cast<int>(lines), le = static_cast<int>(len);
  long long lld = static_cast<long long>(ld);
  if (vec) ku_sm2_fused<4><<<grid, 256, 0, stream>>>(in, bias, out, partials, c, ctl, status, li, le, lld);
  else ku_sm2_fused<1><<<grid, 256, 0, stream>>>(in, bias, out, partials, c, ctl, status, li, le, lld);
  return cudaGetLastError();
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
  return true;
}

}  // namespace

namespace ku::cu {
// used by the graph scheduler when a softmax has exactly this shape
// the fused persistent kernel serves up to kMaxPanels panels of 256 lines; beyond that the three-kernel form runs
static bool use_fused(size_t lines, size_t, const float*) { return (lines + PW - 1) / PW <= size_t(kMaxPanels); }
size_t softmax_two_pass_scratch_bytes(size_t lines, size_t len) { return std::max(scratch_bytes(lines, len), fused_scratch_bytes(lines, len)); }
void softmax_two_pass_launch(const float* in, const float* bias, float* out, size_t lines, size_t len, size_t ld, void* scratch, cudaStream_t stream, int sm_count, int* status) {
  if (use_fused(lines, ld, in)) cuda_check(launch_fused(in, bias, out, lines, len, ld, scratch, stream, sm_count, status), "softmax fused two-pass launch");
  else cuda_check(launch_two_pass(in, bias, out, lines, len, ld, scratch, stream), "softmax two-pass launch");
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
    void* scratch = rt.alloc(ku::cu::softmax_two_pass_scratch_bytes(lines, len));
    try {
      ku::cu::softmax_two_pass_launch(in, bias, out, lines, len, ld, scratch, rt.stream(), rt.sm_count(), rt.status_word());
    } catch (...) { rt.free(scratch); throw; }
    rt.free(scratch);  // stream-ordered reuse: the pool hands it only to later work on the same stream
    ++rt.stats.launches;
    return 0;
  });
}

// ---- the entry point that allocates nothing -------------------------------------------------------
// Some callers may not allocate device memory at the moment they need this softmax: a serving loop
// whose latency budget has no room for the device-wide synchronisation cudaMalloc / cudaFree can
// imply, a host application that has handed all of HBM to its own arena so the CUDA allocator has
// nothing left to give, or code that runs where entering the CUDA allocator is not allowed (a
// host callback, another library's allocation hook). For them the scratch of the two-pass algorithm
// lives in a fixed array inside the library's device image.
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

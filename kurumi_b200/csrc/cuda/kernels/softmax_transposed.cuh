// Single-pass softmax over lines that are strided in memory while the neighbouring axis is
// contiguous: softmax consumed through a transpose view. Output is [R, C] row-major with the
// softmax along C; the dominant input is read as in[j * ld + i], so a warp reads 32 consecutive
// lines i at one position j (one coalesced 128-byte segment) and the transposition happens in
// shared memory.
//
// A cluster of CL CTAs owns a slab of 32 lines. CTA `rank` holds positions [rank*CJ, rank*CJ+CJ) of
// all 32 lines in shared memory (pitch 33 floats: both the row-wise fill and the column-wise drain
// are bank-conflict free). Per-line max and sum are combined across the cluster through
// distributed shared memory, so every element is read from HBM once and written once.
//
// The math is the interpreter's (kurumi_core/src/interp/nn.rs:47-61): line max, e = exp(x - max),
// sum of e, e / sum. It is evaluated as exp2((x - max) * log2 e) for the sum and as
// exp2(x * log2 e - (max * log2 e + log2 sum)) for the output, one fused multiply-add and one
// ex2.approx per element and pass: at 8 bytes of HBM traffic per element the kernel has about 25
// instructions per element to spend, which rules out a full-precision expf plus an IEEE division.
// The result stays within rel 1e-5 of the f64 run (ex2.approx is good to 2 ulp; the exponent
// argument carries about 1e-6 of absolute rounding for |x| up to 100).
//
// Spliced in by the host: R, C, CL, CJ, NT (threads, multiple of 32), and
//   float ku_src(i64 i, i64 j KU_SRC_PARAMS)  - the fused producer at line i, position j.
#define PITCH 33
#define NW (NT / 32)
#define KU_LOG2E 1.4426950408889634f

__device__ __forceinline__ float ku_ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }

__device__ __forceinline__ unsigned ku_cluster_rank() { unsigned r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void ku_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// read a float from the same shared-memory offset in CTA `rank` of this cluster
__device__ __forceinline__ float ku_ld_peer(const float* p, unsigned rank) {
  unsigned a = (unsigned)__cvta_generic_to_shared(p), ra;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(a), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(ra));
  return v;
}

extern "C" __global__ void __launch_bounds__(NT) ku_softmax_transposed(KU_SRC_PARAMS_LEAD void* __restrict__ out) {
  extern __shared__ float tile[];  // [CJ][PITCH]
  __shared__ float part[NW][32];
  __shared__ float cta_max[32], cta_sum[32], line_max[32], line_sum[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned rank = ku_cluster_rank();
  const int i0 = (int)(blockIdx.x / CL) * 32, j0 = (int)rank * CJ;
  const bool line_ok = i0 + lane < R;

  // fill: one 128-byte row segment per warp iteration; running max per line
  float m = -KU_INF;
#pragma unroll UNR
  for (int jj = warp; jj < CJ; jj += NW) {
    const int j = j0 + jj;
    const float v = (line_ok && j < C) ? ku_src(i0 + lane, j KU_SRC_ARGS) : -KU_INF;
    tile[jj * PITCH + lane] = v;
    m = fmaxf(m, v);
  }
  part[warp][lane] = m;
  __syncthreads();
  if (warp == 0) {
    float r = part[0][lane];
    for (int w = 1; w < NW; ++w) r = fmaxf(r, part[w][lane]);
    cta_max[lane] = r;
  }
  ku_cluster_sync();
  if (warp == 0) {
    float r = ku_ld_peer(&cta_max[lane], 0);
    for (unsigned c = 1; c < CL; ++c) r = fmaxf(r, ku_ld_peer(&cta_max[lane], c));
    line_max[lane] = r;
  }
  __syncthreads();

  // sum of exponentials per line (each thread revisits exactly the elements it wrote)
  const float m2 = line_max[lane] * KU_LOG2E;
  float s = 0.0f;
#pragma unroll UNR
  for (int jj = warp; jj < CJ; jj += NW) {
    const float e = ku_ex2(__fmaf_rn(tile[jj * PITCH + lane], KU_LOG2E, -m2));   // padding holds -inf: contributes 0
    s += e;
  }
  part[warp][lane] = s;
  __syncthreads();
  if (warp == 0) {
    float r = part[0][lane];
    for (int w = 1; w < NW; ++w) r += part[w][lane];
    cta_sum[lane] = r;
  }
  ku_cluster_sync();
  if (warp == 0) {
    float r = ku_ld_peer(&cta_sum[lane], 0);
    for (unsigned c = 1; c < CL; ++c) r += ku_ld_peer(&cta_sum[lane], c);
    line_sum[lane] = m2 + log2f(r);   // exp(x - max) / sum == exp2(x * log2e - (max * log2e + log2 sum))
  }
  __syncthreads();

  // drain: a warp writes 32 consecutive positions of one line (one 128-byte segment)
  constexpr int JB = (CJ + 31) / 32;
  for (int t = warp; t < 32 * JB; t += NW) {
    const int ii = t / JB, jb = t - ii * JB;
    const int jj = jb * 32 + lane;
    const int i = i0 + ii, j = j0 + jj;
    if (i < R && jj < CJ && j < C) ((ku_out_t*)out)[(i64)i * C + j] = KU_ENC(ku_ex2(__fmaf_rn(tile[jj * PITCH + ii], KU_LOG2E, -line_sum[ii])));
  }
  // a peer may still be reading this CTA's partials: do not exit before everyone has them
  ku_cluster_sync();
}

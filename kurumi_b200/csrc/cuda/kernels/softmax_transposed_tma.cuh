// Single-pass softmax through a transpose view, TMA-fed and persistent (the fast path of
// softmax_transposed.cuh, same data flow and same math; see that file for both).
//
// Persistent clusters of CL CTAs walk the 32-line slabs. CTA `rank` owns positions
// [rank*CJ, rank*CJ+CJ) of every slab its cluster processes. The dominant input is a plain f32
// buffer read as in[j * ld + i]: one elected thread streams [BOXJ positions x 32 lines] boxes
// (128-byte rows, SWIZZLE_128B) into a ring of NBUF shared-memory tiles with cp.async.bulk.tensor
// (no multicast), completing on an mbarrier, so HBM reads for the next slabs are in flight while
// the current slab is reduced and drained. In the swizzled tile a warp reads a row (32 lines at one
// position) conflict-free with 4-byte loads, and reads a 32-position column strip of 4 lines
// conflict-free with 16-byte loads, which is what makes the transposed drain coalesced.
//
// Every wait is bounded: a thread that gives up records it in *status and carries on, so the
// cluster barriers are still reached and the kernel ends; the host reports the error.
//
// Spliced in by the host: R, C, CL, CJ, BOXJ, NBUF, NT, NSLABS, KU_SRC_IDENTITY, and
//   float ku_src_t(float lval, idx i, idx j KU_SRC_PARAMS) - the fused producer given the loaded value.
#define NW (NT / 32)
#define KU_LOG2E 1.4426950408889634f
#define TILE_BYTES (CJ * 128)
#define SPIN_LIMIT (1u << 22)

struct alignas(64) KuTmap { unsigned long long opaque[16]; };

__device__ __forceinline__ float ku_ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ unsigned ku_cluster_rank() { unsigned r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void ku_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ku_ld_peer(const float* p, unsigned rank) {
  unsigned a = (unsigned)__cvta_generic_to_shared(p), ra;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(a), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(ra) : "memory");
  return v;
}
// per-line partials travel between the CTAs of a cluster as asynchronous remote stores that complete
// on the receiver's mbarrier: no cluster-wide barrier, and no release fence that would have to wait
// for the drain's global stores
__device__ __forceinline__ unsigned ku_mapa(unsigned a, unsigned rank) { unsigned ra; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(a), "r"(rank)); return ra; }
__device__ __forceinline__ void ku_st_async(unsigned remote_addr, float v, unsigned remote_mbar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];" ::"r"(remote_addr), "r"(__float_as_uint(v)), "r"(remote_mbar) : "memory");
}
__device__ __forceinline__ unsigned ku_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ku_mbar_init(unsigned a, unsigned n) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(a), "r"(n)); }
__device__ __forceinline__ void ku_mbar_expect(unsigned a, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(a), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool ku_mbar_try(unsigned a, unsigned parity) {
  unsigned ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(a), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ void ku_tma_2d(unsigned dst, const KuTmap* map, int x, int y, unsigned mbar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(mbar) : "memory");
}
// byte offset of (position jj, line ii) inside a swizzled tile
__device__ __forceinline__ unsigned ku_tile_off(int jj, int ii) { return (unsigned)(jj * 128 + ((((ii >> 2) ^ (jj & 7))) << 4) + ((ii & 3) << 2)); }

extern "C" __global__ void __launch_bounds__(NT, 1)
ku_softmax_transposed_tma(const __grid_constant__ KuTmap tmap, KU_SRC_PARAMS_LEAD void* __restrict__ out, int* __restrict__ status) {
  extern __shared__ __align__(1024) unsigned char tiles_raw[];  // NBUF tiles of [CJ][32] f32, 128-byte swizzled rows
  __shared__ __align__(8) unsigned long long full[NBUF];
  __shared__ float part[NW][32];
  __shared__ __align__(8) unsigned long long bar_max[2], bar_sum[2];
  __shared__ float cta_val[32], line_c[32];
  __shared__ float gather_max[2][CL][32], gather_sum[2][CL][32];   // [slab parity][sender rank][line]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned rank = ku_cluster_rank();
  const int cid = blockIdx.x / CL, nclusters = gridDim.x / CL;
  const int j0 = (int)rank * CJ;
  // the swizzle pattern is a function of the shared-memory address: tiles start on a 1024-byte boundary
  unsigned char* tiles = tiles_raw + ((1024u - (ku_smem(tiles_raw) & 1023u)) & 1023u);
  const unsigned tiles_s = ku_smem(tiles);
  if (tiles != tiles_raw) {  // the host sized the ring without slack: a misplaced ring is reported, not used
    if (threadIdx.x == 0) atomicExch(status, 5);
    return;
  }

  if (threadIdx.x == 0) {
    for (int b = 0; b < NBUF; ++b) ku_mbar_init(ku_smem(&full[b]), 1);
    for (int b = 0; b < 2; ++b) { ku_mbar_init(ku_smem(&bar_max[b]), 1); ku_mbar_init(ku_smem(&bar_sum[b]), 1); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  ku_cluster_sync();   // every CTA's barriers exist before any peer sends to them
  auto issue = [&](int slab, int b) {  // one thread: stream this CTA's share of a slab into tile b
    const unsigned mb = ku_smem(&full[b]);
    ku_mbar_expect(mb, TILE_BYTES);
    for (int k = 0; k < CJ / BOXJ; ++k) ku_tma_2d(tiles_s + b * TILE_BYTES + k * BOXJ * 128, &tmap, slab * 32, j0 + k * BOXJ, mb);
  };
  if (threadIdx.x == 0)
    for (int b = 0; b < NBUF; ++b)
      if (cid + b * nclusters < NSLABS) issue(cid + b * nclusters, b);

  int n = 0;
  for (int slab = cid; slab < NSLABS; slab += nclusters, ++n) {
    const int b = n % NBUF;
    const unsigned parity = (n / NBUF) & 1, mb = ku_smem(&full[b]);
    bool failed = false;
    unsigned spins = 0;
    while (!failed && !ku_mbar_try(mb, parity)) {
      ++spins;
      if ((spins & 1023u) == 0 && *(volatile int*)status != 0) failed = true;   // someone already gave up: stop waiting everywhere
      if (spins > SPIN_LIMIT) { atomicExch(status, 1); failed = true; }
    }
    unsigned char* tile = tiles + b * TILE_BYTES;
    const int i0 = slab * 32, pp = n & 1;

    // line max (and the fused producer, written back so the later passes read finished values)
    float m = -KU_INF;
#pragma unroll 8
    for (int jj = warp; jj < CJ; jj += NW) {
      float* p = (float*)(tile + ku_tile_off(jj, lane));
      const int j = j0 + jj;
      float v = *p;
#if !KU_SRC_IDENTITY
      v = ku_src_t(v, i0 + lane, j KU_SRC_ARGS);
#endif
      if (j >= C) v = -KU_INF;
#if !KU_SRC_IDENTITY
      *p = v;
#else
      if (j >= C) *p = v;
#endif
      m = fmaxf(m, v);
    }
    const unsigned xparity = (n >> 1) & 1;   // each exchange barrier is used every second slab
    part[warp][lane] = m;
    __syncthreads();
    if (warp == 0) {
      float r = part[0][lane];
      for (int w = 1; w < NW; ++w) r = fmaxf(r, part[w][lane]);
      cta_val[lane] = r;
      if (lane == 0) ku_mbar_expect(ku_smem(&bar_max[pp]), CL * 128);
    }
    __syncthreads();
    if (warp < CL)   // warp w delivers this CTA's 32 partial maxima to CTA w
      ku_st_async(ku_mapa(ku_smem(&gather_max[pp][rank][lane]), warp), cta_val[lane], ku_mapa(ku_smem(&bar_max[pp]), warp));
    {
      unsigned sp = 0;
      while (!failed && !ku_mbar_try(ku_smem(&bar_max[pp]), xparity)) { ++sp; if ((sp & 1023u) == 0 && *(volatile int*)status != 0) failed = true; if (sp > SPIN_LIMIT) { atomicExch(status, 3); failed = true; } }
    }
    float mx = gather_max[pp][0][lane];
#pragma unroll
    for (int c = 1; c < CL; ++c) mx = fmaxf(mx, gather_max[pp][c][lane]);

    const float m2 = mx * KU_LOG2E;
    float s = 0.0f;
#pragma unroll 8
    for (int jj = warp; jj < CJ; jj += NW) s += ku_ex2(__fmaf_rn(*(const float*)(tile + ku_tile_off(jj, lane)), KU_LOG2E, -m2));
    __syncthreads();   // cta_val and part are free again
    part[warp][lane] = s;
    __syncthreads();
    if (warp == 0) {
      float r = part[0][lane];
      for (int w = 1; w < NW; ++w) r += part[w][lane];
      cta_val[lane] = r;
      if (lane == 0) ku_mbar_expect(ku_smem(&bar_sum[pp]), CL * 128);
    }
    __syncthreads();
    if (warp < CL) ku_st_async(ku_mapa(ku_smem(&gather_sum[pp][rank][lane]), warp), cta_val[lane], ku_mapa(ku_smem(&bar_sum[pp]), warp));
    {
      unsigned sp = 0;
      while (!failed && !ku_mbar_try(ku_smem(&bar_sum[pp]), xparity)) { ++sp; if ((sp & 1023u) == 0 && *(volatile int*)status != 0) failed = true; if (sp > SPIN_LIMIT) { atomicExch(status, 4); failed = true; } }
    }
    if (warp == 0) {
      float r = gather_sum[pp][0][lane];
#pragma unroll
      for (int c = 1; c < CL; ++c) r += gather_sum[pp][c][lane];
      line_c[lane] = m2 + log2f(r);  // exp(x - max) / sum == exp2(x * log2e - (max * log2e + log2 sum))
    }
    __syncthreads();

    // drain: lane = position within a 32-position strip; one 16-byte load gives 4 lines at that position,
    // then 4 warp-wide stores of 128 contiguous bytes each
    for (int t = warp; t < 8 * (CJ / 32); t += NW) {
      const int q = t & 7, jb = t >> 3;
      const int jj = jb * 32 + lane, j = j0 + jj;
      const float4 v = *(const float4*)(tile + jj * 128 + ((q ^ (jj & 7)) << 4));
      const float c0 = line_c[q * 4 + 0], c1 = line_c[q * 4 + 1], c2 = line_c[q * 4 + 2], c3 = line_c[q * 4 + 3];
      if (j < C) {
        ku_out_t* o = (ku_out_t*)out + (i64)(i0 + q * 4) * C + j;
        if (i0 + q * 4 + 0 < R) o[0] = KU_ENC(ku_ex2(__fmaf_rn(v.x, KU_LOG2E, -c0)));
        if (i0 + q * 4 + 1 < R) o[(i64)C] = KU_ENC(ku_ex2(__fmaf_rn(v.y, KU_LOG2E, -c1)));
        if (i0 + q * 4 + 2 < R) o[2 * (i64)C] = KU_ENC(ku_ex2(__fmaf_rn(v.z, KU_LOG2E, -c2)));
        if (i0 + q * 4 + 3 < R) o[3 * (i64)C] = KU_ENC(ku_ex2(__fmaf_rn(v.w, KU_LOG2E, -c3)));
      }
    }
    __syncthreads();  // every thread is done with tile b
    if (threadIdx.x == 0 && slab + NBUF * nclusters < NSLABS) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy accesses to the tile precede the async refill
      issue(slab + NBUF * nclusters, b);
    }
  }
  ku_cluster_sync();  // peers may still be reading this CTA's partials
}

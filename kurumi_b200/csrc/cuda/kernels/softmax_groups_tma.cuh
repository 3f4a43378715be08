// Single-pass softmax through a transpose view: every input byte crosses HBM and L2 once, because a
// tile stays in shared memory between the statistics and the write-out.
//
// The dominant input is a plain f32 buffer read as in[j * ld + i] (i = line, j = position along the
// softmax axis). A slab is 32 lines. A GROUP of P co-resident CTAs shares a slab: CTA r keeps positions
// [r*CJ, r*CJ + CJ) of it as a [CJ][32] f32 tile (TMA, 128-byte swizzled rows) in a ring of NBUF tiles.
// Groups walk the slabs with a fixed stride; there are no clusters, so any number of groups up to
// (resident CTAs / P) runs, and the launch is cooperative so that a group's CTAs really are co-resident.
// Per slab a CTA
//   1. reduces its tile to one (max, sum) pair per line, writes the 32 pairs to global scratch and bumps
//      the slab's counter (release);
//   2. waits until the counter shows all P CTAs (acquire; one polling thread per CTA), merges the P x 32
//      pairs, and writes its tile out transposed: out[line][position] = exp2(x * log2e - (max * log2e + log2 sum)).
// With NBUF = 1 (one tile per CTA, several CTAs of different groups per SM) the steps follow each other
// and the neighbours on the SM fill the waits; with a deeper ring step 2 of a slab runs after step 1 of the next.
// Every wait is bounded: a CTA that gives up records it in *status and carries on.
//
// Spliced in by the host: R, C, LW (lines per slab: 32 or 16), P, CJ (multiple of (128 / LW) * NT / 32), BOXJ, NBUF, NT, NSLABS,
// KU_OUT_F32, KU_SRC_IDENTITY and
//   float ku_src_t(float lval, idx i, idx j KU_SRC_PARAMS) - the fused producer given the loaded value.
#define NW (NT / 32)
#define ROWB (LW * 4)          /* bytes of a tile row: LW lines at one position */
#define CHUNKS (LW / 4)        /* 16-byte chunks (4 lines) per tile row */
#define RSN (32 / CHUNKS)      /* tile rows a warp reads with one 16-byte load per lane */
#define KU_LOG2E 1.4426950408889634f
#define TILE_BYTES (CJ * ROWB)
#define SPIN_LIMIT (1u << 22)
#define RPW (CJ / NW)   /* tile rows per warp */
#if KU_OUT_F32
#define KU_STORE(p, v) __stcs((p), (v))   // the output is not read again: stream it through L2
#else
#define KU_STORE(p, v) (*(p) = (v))
#endif

struct alignas(64) KuTmap { unsigned long long opaque[16]; };

__device__ __forceinline__ float ku_ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ unsigned ku_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
// byte offset of 16-byte chunk q (lines 4q .. 4q+3) of tile row jj: rows are ROWB bytes, swizzled as the TMA wrote them
// (128-byte rows: chunk ^ (row & 7); 64-byte rows: chunk ^ ((row >> 1) & 3))
__device__ __forceinline__ unsigned ku_chunk_off(int jj, int q) {
#if LW == 32
  return (unsigned)(jj * ROWB + ((q ^ (jj & 7)) << 4));
#else
  return (unsigned)(jj * ROWB + ((q ^ ((jj >> 1) & 3)) << 4));
#endif
}
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
__device__ __forceinline__ unsigned ku_ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// (max, sum) pairs in log2 units: merge b into a
__device__ __forceinline__ void ku_merge(float& m, float& sum, float om, float osum) {
  const float mn = fmaxf(m, om);
  const float a0 = (m == -KU_INF) ? sum : sum * ku_ex2(m - mn);      // a sum is 0 or NaN while its max is -inf
  const float a1 = (om == -KU_INF) ? osum : osum * ku_ex2(om - mn);
  sum = a0 + a1;
  m = mn;
}

extern "C" __global__ void __launch_bounds__(NT)
ku_softmax_groups_tma(const __grid_constant__ KuTmap tmap, KU_SRC_PARAMS_LEAD void* __restrict__ out, void* __restrict__ scratch, int* __restrict__ status) {
  extern __shared__ __align__(1024) unsigned char tiles_raw[];  // NBUF tiles of [CJ][32] f32, 128-byte swizzled rows
  __shared__ __align__(8) unsigned long long full[NBUF];
  __shared__ __align__(16) float2 s_part[NW][LW];
  __shared__ __align__(16) float line_c[LW];
  __shared__ int s_failed;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int group = blockIdx.x / P, ngroups = gridDim.x / P, rank = blockIdx.x % P;
  const int j0 = rank * CJ;
  unsigned* counters = (unsigned*)scratch;                                  // [NSLABS], cleared by the host before the launch
  float2* partials = (float2*)((char*)scratch + (((size_t)NSLABS * 4 + 255) / 256) * 256);   // [NSLABS][P][LW]
  // the swizzle pattern is a function of the shared-memory address: tiles start on a 1024-byte boundary
  // (the host sizes the ring with 1024 bytes of slack)
  unsigned char* tiles = tiles_raw + ((1024u - (ku_smem(tiles_raw) & 1023u)) & 1023u);
  const unsigned tiles_s = ku_smem(tiles);
  if (blockIdx.x >= (unsigned)(ngroups * P)) return;   // CTAs beyond the last whole group have no work

  auto issue = [&](int slab, int b) {  // one thread: stream this CTA's share of a slab into tile b
    const unsigned mb = ku_smem(&full[b]);
    ku_mbar_expect(mb, TILE_BYTES);
    for (int k = 0; k < CJ / BOXJ; ++k) ku_tma_2d(tiles_s + b * TILE_BYTES + k * BOXJ * ROWB, &tmap, slab * LW, j0 + k * BOXJ, mb);
  };
  if (threadIdx.x == 0) {
    s_failed = 0;
    for (int b = 0; b < NBUF; ++b) ku_mbar_init(ku_smem(&full[b]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    for (int b = 0; b < NBUF; ++b)
      if (group + b * ngroups < NSLABS) issue(group + b * ngroups, b);
  }
  __syncthreads();

  // step 1 of the n-th slab of this CTA
  auto stats = [&](int n, int slab) {
    const int b = n % NBUF;
    const unsigned parity = (unsigned)((n / NBUF) & 1), mb = ku_smem(&full[b]);
    unsigned spins = 0;
    while (!ku_mbar_try(mb, parity)) {
      if (++spins > SPIN_LIMIT) { atomicExch(status, 1); break; }
    }
    const unsigned char* tile = tiles + b * TILE_BYTES;
    const int i0 = slab * LW;
    // thread = (4 lines: chunk q of the row, row group rs); a warp owns RPW consecutive rows of the tile
    const int q = lane % CHUNKS, rs = lane / CHUNKS;
    // two passes over the warp's rows of the tile (16-byte shared-memory loads are cheap; registers are not)
    auto load = [&](int it) {
      const int row = warp * RPW + it * RSN + rs, j = j0 + row;
      float4 v = *(const float4*)(tile + ku_chunk_off(row, q));
#if !KU_SRC_IDENTITY
      v.x = ku_src_t(v.x, i0 + q * 4 + 0, j KU_SRC_ARGS);
      v.y = ku_src_t(v.y, i0 + q * 4 + 1, j KU_SRC_ARGS);
      v.z = ku_src_t(v.z, i0 + q * 4 + 2, j KU_SRC_ARGS);
      v.w = ku_src_t(v.w, i0 + q * 4 + 3, j KU_SRC_ARGS);
#endif
      if ((C % CJ != 0) && j >= C) v = make_float4(-KU_INF, -KU_INF, -KU_INF, -KU_INF);
      return v;
    };
    float4 m = load(0);
#pragma unroll 4
    for (int it = 1; it < RPW / RSN; ++it) { const float4 v = load(it); m.x = fmaxf(m.x, v.x); m.y = fmaxf(m.y, v.y); m.z = fmaxf(m.z, v.z); m.w = fmaxf(m.w, v.w); }
#pragma unroll
    for (int o = CHUNKS; o <= 16; o <<= 1) {
      m.x = fmaxf(m.x, __shfl_xor_sync(0xffffffffu, m.x, o)); m.y = fmaxf(m.y, __shfl_xor_sync(0xffffffffu, m.y, o));
      m.z = fmaxf(m.z, __shfl_xor_sync(0xffffffffu, m.z, o)); m.w = fmaxf(m.w, __shfl_xor_sync(0xffffffffu, m.w, o));
    }
    // exp2(x*log2e - max*log2e); lines that are all -inf so far subtract 0 and sum zeros
    const float4 k = make_float4(m.x == -KU_INF ? 0.0f : m.x * KU_LOG2E, m.y == -KU_INF ? 0.0f : m.y * KU_LOG2E,
                                 m.z == -KU_INF ? 0.0f : m.z * KU_LOG2E, m.w == -KU_INF ? 0.0f : m.w * KU_LOG2E);
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int it = 0; it < RPW / RSN; ++it) {
      const float4 v = load(it);
      sum.x += ku_ex2(__fmaf_rn(v.x, KU_LOG2E, -k.x)); sum.y += ku_ex2(__fmaf_rn(v.y, KU_LOG2E, -k.y));
      sum.z += ku_ex2(__fmaf_rn(v.z, KU_LOG2E, -k.z)); sum.w += ku_ex2(__fmaf_rn(v.w, KU_LOG2E, -k.w));
    }
#pragma unroll
    for (int o = CHUNKS; o <= 16; o <<= 1) {
      sum.x += __shfl_xor_sync(0xffffffffu, sum.x, o); sum.y += __shfl_xor_sync(0xffffffffu, sum.y, o);
      sum.z += __shfl_xor_sync(0xffffffffu, sum.z, o); sum.w += __shfl_xor_sync(0xffffffffu, sum.w, o);
    }
    if (rs == 0) {   // the warp's pairs for lines 4q .. 4q+3, max in log2 units
      *(float4*)&s_part[warp][q * 4] = make_float4(m.x * KU_LOG2E, sum.x, m.y * KU_LOG2E, sum.y);
      *(float4*)&s_part[warp][q * 4 + 2] = make_float4(m.z * KU_LOG2E, sum.z, m.w * KU_LOG2E, sum.w);
    }
    __syncthreads();
    if (warp == 0) {
      if (lane < LW) {
        float mm = s_part[0][lane].x, tot = s_part[0][lane].y;
#pragma unroll
        for (int w = 1; w < NW; ++w) ku_merge(mm, tot, s_part[w][lane].x, s_part[w][lane].y);
        partials[((size_t)slab * P + rank) * LW + lane] = make_float2(mm, tot);
      }
      __syncwarp();
      // the warp's 32 stores are ordered before this release by the warp barrier above
      if (lane == 0) asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(counters + slab) : "memory");
    }
    __syncthreads();   // s_part is free again
  };

  // step 2 of the n-th slab of this CTA
  auto finish = [&](int n, int slab) {
    const int b = n % NBUF;
    const unsigned char* tile = tiles + b * TILE_BYTES;
    const int i0 = slab * LW;
    if (warp == 0) {
      if (lane == 0) {   // one poller per CTA: the counter is shared by the whole group
        unsigned spins = 0;
        bool bad = s_failed != 0;
        while (!bad && ku_ld_acquire(counters + slab) < (unsigned)P) {
          if (++spins > SPIN_LIMIT || *(volatile int*)status != 0) { atomicExch(status, 3); bad = true; }
          __nanosleep(20);
        }
        if (bad) s_failed = 1;
      }
      __syncwarp();   // orders the other lanes' loads of the pairs after lane 0's acquire
      if (lane < LW) {
        const float2* src = partials + (size_t)slab * P * LW + lane;
        float2 pr[P];
#pragma unroll
        for (int c = 0; c < P; ++c) pr[c] = __ldcg(src + c * LW);
        float mm = pr[0].x, tot = pr[0].y;
#pragma unroll
        for (int c = 1; c < P; ++c) ku_merge(mm, tot, pr[c].x, pr[c].y);
        line_c[lane] = (mm == -KU_INF) ? __int_as_float(0x7fc00000) : mm + log2f(tot);
      }
    }
    __syncthreads();
    // lane = position within a 32-position strip; one 16-byte load gives 4 lines at that position,
    // then 4 warp-wide stores of 128 contiguous bytes each
#pragma unroll 4
    for (int t = warp; t < CHUNKS * (CJ / 32); t += NW) {
      const int q = t % CHUNKS, js = t / CHUNKS;
      const int jj = js * 32 + lane, j = j0 + jj;
      float4 v = *(const float4*)(tile + ku_chunk_off(jj, q));
      const float4 c4 = *(const float4*)&line_c[q * 4];
      if ((C % CJ == 0) || j < C) {
#if !KU_SRC_IDENTITY
        v.x = ku_src_t(v.x, i0 + q * 4 + 0, j KU_SRC_ARGS);
        v.y = ku_src_t(v.y, i0 + q * 4 + 1, j KU_SRC_ARGS);
        v.z = ku_src_t(v.z, i0 + q * 4 + 2, j KU_SRC_ARGS);
        v.w = ku_src_t(v.w, i0 + q * 4 + 3, j KU_SRC_ARGS);
#endif
        ku_out_t* o = (ku_out_t*)out + (i64)(i0 + q * 4) * C + j;
        if ((R % LW == 0) || i0 + q * 4 + 0 < R) KU_STORE(&o[0], KU_ENC(ku_ex2(__fmaf_rn(v.x, KU_LOG2E, -c4.x))));
        if ((R % LW == 0) || i0 + q * 4 + 1 < R) KU_STORE(&o[(i64)C], KU_ENC(ku_ex2(__fmaf_rn(v.y, KU_LOG2E, -c4.y))));
        if ((R % LW == 0) || i0 + q * 4 + 2 < R) KU_STORE(&o[2 * (i64)C], KU_ENC(ku_ex2(__fmaf_rn(v.z, KU_LOG2E, -c4.z))));
        if ((R % LW == 0) || i0 + q * 4 + 3 < R) KU_STORE(&o[3 * (i64)C], KU_ENC(ku_ex2(__fmaf_rn(v.w, KU_LOG2E, -c4.w))));
      }
    }
    __syncthreads();  // every thread is done with tile b and with line_c
    const int next = slab + NBUF * ngroups;
    if (threadIdx.x == 0 && next < NSLABS) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy reads of the tile precede the async refill
      issue(next, b);
    }
  };

  int n = 0;
  for (int slab = group; slab < NSLABS; slab += ngroups, ++n) {
    stats(n, slab);
    if (NBUF == 1) finish(n, slab);                    // one tile: nothing to overlap inside the CTA, its neighbours on the SM do
    else if (n > 0) finish(n - 1, slab - ngroups);     // the previous slab's exchange has had a whole statistics pass to complete
  }
  if (NBUF > 1 && n > 0) finish(n - 1, group + (n - 1) * ngroups);
}

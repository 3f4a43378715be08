// Single-pass softmax through a transpose view: every input byte crosses HBM and L2 once, and every
// element is read from shared memory once: a tile is lifted into registers as soon as it lands, so the
// shared-memory ring only ever holds tiles in flight, and the exchange of line statistics between CTAs is
// hidden behind the next slab's work.
//
// The dominant input is a plain f32 buffer read as in[j * ld + i] (i = line, j = position along the
// softmax axis). A slab is 32 lines. A GROUP of P co-resident CTAs shares a slab: CTA r loads positions
// [r*CJ, r*CJ + CJ) of it as a [CJ][32] f32 tile (TMA, 128-byte swizzled rows) into a ring of NBUF tiles.
// Groups walk the slabs with a fixed stride; there are no clusters, so any number of groups up to
// (resident CTAs / P) runs, and the launch is cooperative so that a group's CTAs really are co-resident.
// 512 threads per SM at 128 registers each, as one CTA or as two CTAs of 256 (of different groups, so that one's
// exp2 phase overlaps the other's stores): a ring of NBUF tiles being filled by TMA per CTA, and two tiles per
// CTA held in registers.
//
// Thread layout (the same for the statistics and for the write-out, so the values never leave their
// registers): warp w owns the 16-byte chunk q = w % 8 of the tile rows (lines 4q .. 4q+3) and the
// 32-position strips h, h + HALVES, ... (h = w / 8, HALVES = warps / 8); lane = position inside a strip. A thread
// holds V = CJ / (32 HALVES) float4 values per tile: 4 lines at V positions. A warp-wide store then writes 128 contiguous
// bytes of one output line.
//
// Per slab a CTA
//   1. waits for its tile, copies it to registers (one conflict-free 16-byte shared-memory load per
//      float4, the fused producer applied on the way) and hands the tile's buffer to the next TMA load;
//   2. per warp: line maxima over its positions (redux.sync), e = exp2(x * log2e - k) in place with k the
//      WARP's maximum in log2 units, line sums by a 6-shuffle butterfly; the warp's (max, sum) pairs go
//      to global scratch as one 64-bit word each, whose top bit (the sign bit of the sum, which is never
//      negative) carries the launch parity: data and "ready" flag travel in one store, no fence, no counter;
//   3. one slab later (steps 1 and 2 of the next slab come first, into the other register tile): polls the HALVES x P
//      words of each of the 32 lines (every warp polls its share, bounded), merges them to
//      c = max + log2(sum) per line and writes out[line][position] = e * exp2(k - c).
// One exp2 per element, plus a handful per thread. Every wait is bounded: a CTA that gives up records it
// in *status and carries on (its results are then invalid, the host reports it).
//
// Spliced in by the host: R, C, P, CJ (multiple of NT / 8), BOXJ, NBUF, NT (256 or 512), NSLABS, KU_OUT_F32, KU_SRC_IDENTITY and
//   float ku_src_t(float lval, idx i, idx j KU_SRC_PARAMS) - the fused producer given the loaded value.
#define LW 32                  /* lines per slab: a tile row is 128 bytes */
#define NW (NT / 32)
#define HALVES (NW / 8)        /* warps that share a 16-byte chunk of the tile rows */
#define V (CJ / (32 * HALVES)) /* float4 values per thread and tile */
#define NPART (HALVES * P)     /* (max, sum) pairs per line and slab: one per CTA and warp of a chunk */
#define NE ((NPART + NW - 1) / NW)   /* pairs of a line a warp polls */
#define KU_LOG2E 1.4426950408889634f
#define TILE_BYTES (CJ * 128)
#define SPIN_LIMIT (1u << 22)
#define POLL_LIMIT (1u << 20)
#if KU_OUT_F32
#define KU_STORE(p, v) __stcs((p), (v))   // the output is not read again: stream it through L2
#else
#define KU_STORE(p, v) (*(p) = (v))
#endif

struct alignas(64) KuTmap { unsigned long long opaque[16]; };

__device__ __forceinline__ float ku_ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float ku_warp_max(float x) { float y; asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ unsigned ku_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
// byte offset of 16-byte chunk q (lines 4q .. 4q+3) of tile row jj: rows are 128 bytes, swizzled as the TMA wrote them
__device__ __forceinline__ unsigned ku_chunk_off(int jj, int q) { return (unsigned)(jj * 128 + ((q ^ (jj & 7)) << 4)); }
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
__device__ __forceinline__ unsigned long long ku_ld_relaxed(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.gpu.global.b64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void ku_st_relaxed(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// sums of four values over the warp with six shuffles: on return every lane holds the total of value (lane & 3)
__device__ __forceinline__ float ku_sum4(float a0, float a1, float a2, float a3, int lane) {
  const bool b1 = lane & 2, b0 = lane & 1;
  const float r0 = __shfl_xor_sync(0xffffffffu, b1 ? a0 : a2, 2), r1 = __shfl_xor_sync(0xffffffffu, b1 ? a1 : a3, 2);
  const float c0 = (b1 ? a2 : a0) + r0, c1 = (b1 ? a3 : a1) + r1;          // values 2*b1 and 2*b1 + 1 over the lane pair
  float s = (b0 ? c1 : c0) + __shfl_xor_sync(0xffffffffu, b0 ? c0 : c1, 1);   // value (lane & 3) over four lanes
  s += __shfl_xor_sync(0xffffffffu, s, 4);
  s += __shfl_xor_sync(0xffffffffu, s, 8);
  s += __shfl_xor_sync(0xffffffffu, s, 16);
  return s;
}

extern "C" __global__ void __launch_bounds__(NT, 512 / NT)
ku_softmax_groups_tma(const __grid_constant__ KuTmap tmap, KU_SRC_PARAMS_LEAD void* __restrict__ out, void* __restrict__ scratch, unsigned epoch, int* __restrict__ status) {
  extern __shared__ __align__(1024) unsigned char tiles_raw[];  // NBUF tiles of [CJ][32] f32, 128-byte swizzled rows
  __shared__ __align__(8) unsigned long long full[NBUF];
  // the slab's (max, sum) pairs, as polled. Rows are padded by four pairs (a row stride of 8 banks modulo 32): the
  // merge reads pairs e, e + 1, e + 2, e + 3 of four neighbouring lines in one half-warp access, conflict-free
  __shared__ __align__(16) float2 s_x[NPART][LW + 4];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int group = blockIdx.x / P, ngroups = gridDim.x / P, rank = blockIdx.x % P;
  const int j0 = rank * CJ;
  unsigned long long* partials = (unsigned long long*)scratch;   // [NSLABS][NPART][LW]; zero when allocated, parity flips per launch
  const unsigned par = epoch & 1u;
  // the swizzle pattern is a function of the shared-memory address: the tiles start on a 1024-byte boundary
  // (the host sizes the allocation with 1024 bytes of slack)
  unsigned char* tiles = tiles_raw + ((1024u - (ku_smem(tiles_raw) & 1023u)) & 1023u);
  const unsigned tiles_s = ku_smem(tiles);
  if (blockIdx.x >= (unsigned)(ngroups * P)) return;   // CTAs beyond the last whole group have no work

  auto issue = [&](int slab, int b) {  // one thread: stream this CTA's share of a slab into tile b
    const unsigned mb = ku_smem(&full[b]);
    ku_mbar_expect(mb, TILE_BYTES);
    for (int k = 0; k < CJ / BOXJ; ++k) ku_tma_2d(tiles_s + b * TILE_BYTES + k * BOXJ * 128, &tmap, slab * LW, j0 + k * BOXJ, mb);
  };
  if (threadIdx.x == 0) {
    for (int b = 0; b < NBUF; ++b) ku_mbar_init(ku_smem(&full[b]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    for (int b = 0; b < NBUF; ++b)
      if (group + b * ngroups < NSLABS) issue(group + b * ngroups, b);
  }
  __syncthreads();

  const int q = warp & 7, h = warp >> 3;
  const int ls = lane & 3, part = lane >> 2;

  // Steps 1 and 2 of the n-th slab of this CTA: tile -> registers x, the warp's statistics, e in place, pairs published.
  // kk receives the warp's line maxima in log2 units (0 where the warp saw only -inf, flagged in minf).
  auto take = [&](float4 (&x)[V], float4& kk, unsigned& minf, int n, int slab) {
    const int b = n % NBUF, i0 = slab * LW;
    const unsigned char* tile = tiles + b * TILE_BYTES;
    {
      const unsigned mb = ku_smem(&full[b]), parity = (unsigned)((n / NBUF) & 1);
      unsigned spins = 0;
      while (!ku_mbar_try(mb, parity)) {
        if (++spins > SPIN_LIMIT) { atomicExch(status, 1); break; }
      }
    }
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const int jj = (h + HALVES * k) * 32 + lane, j = j0 + jj;
      float4 v = *(const float4*)(tile + ku_chunk_off(jj, q));
#if !KU_SRC_IDENTITY
      {   // operands other than the staged one are read at coordinates clamped into the tensor: the padding is masked below
        const int jc = (C % CJ != 0 && j >= C) ? C - 1 : j, ic = i0 + q * 4;
        v.x = ku_src_t(v.x, (R % LW != 0 && ic + 0 >= R) ? R - 1 : ic + 0, jc KU_SRC_ARGS);
        v.y = ku_src_t(v.y, (R % LW != 0 && ic + 1 >= R) ? R - 1 : ic + 1, jc KU_SRC_ARGS);
        v.z = ku_src_t(v.z, (R % LW != 0 && ic + 2 >= R) ? R - 1 : ic + 2, jc KU_SRC_ARGS);
        v.w = ku_src_t(v.w, (R % LW != 0 && ic + 3 >= R) ? R - 1 : ic + 3, jc KU_SRC_ARGS);
      }
#endif
      if ((C % CJ != 0) && j >= C) v = make_float4(-KU_INF, -KU_INF, -KU_INF, -KU_INF);
      x[k] = v;
    }
    __syncthreads();   // every thread has its part of the tile; s_x of the slab finished before is no longer read
    {
      const int next = slab + NBUF * ngroups;
      if (threadIdx.x == 0 && next < NSLABS) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy reads of the tile precede the async refill
        issue(next, b);
      }
    }
    float4 m = x[0];
#pragma unroll
    for (int k = 1; k < V; ++k) { m.x = fmaxf(m.x, x[k].x); m.y = fmaxf(m.y, x[k].y); m.z = fmaxf(m.z, x[k].z); m.w = fmaxf(m.w, x[k].w); }
    m.x = ku_warp_max(m.x); m.y = ku_warp_max(m.y); m.z = ku_warp_max(m.z); m.w = ku_warp_max(m.w);
    minf = (m.x == -KU_INF ? 1u : 0u) | (m.y == -KU_INF ? 2u : 0u) | (m.z == -KU_INF ? 4u : 0u) | (m.w == -KU_INF ? 8u : 0u);
    // exp2(x*log2e - max*log2e); lines that are all -inf here subtract 0 and sum zeros
    kk = make_float4((minf & 1u) ? 0.0f : m.x * KU_LOG2E, (minf & 2u) ? 0.0f : m.y * KU_LOG2E, (minf & 4u) ? 0.0f : m.z * KU_LOG2E, (minf & 8u) ? 0.0f : m.w * KU_LOG2E);
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int k = 0; k < V; ++k) {
      x[k].x = ku_ex2(__fmaf_rn(x[k].x, KU_LOG2E, -kk.x)); sum.x += x[k].x;
      x[k].y = ku_ex2(__fmaf_rn(x[k].y, KU_LOG2E, -kk.y)); sum.y += x[k].y;
      x[k].z = ku_ex2(__fmaf_rn(x[k].z, KU_LOG2E, -kk.z)); sum.z += x[k].z;
      x[k].w = ku_ex2(__fmaf_rn(x[k].w, KU_LOG2E, -kk.w)); sum.w += x[k].w;
    }
    const float tot = ku_sum4(sum.x, sum.y, sum.z, sum.w, lane);   // line 4q + (lane & 3)
    if (lane < 4) {
      const float ml = (ls == 0 ? m.x : ls == 1 ? m.y : ls == 2 ? m.z : m.w) * KU_LOG2E;   // -inf stays -inf
      const unsigned long long w = ((unsigned long long)((__float_as_uint(tot) & 0x7fffffffu) | (par << 31)) << 32) | __float_as_uint(ml);
      ku_st_relaxed(partials + ((size_t)slab * NPART + (rank * HALVES + h)) * LW + q * 4 + lane, w);
    }
  };

  // Step 3 of a slab whose pairs this CTA published a whole slab earlier: gather, merge, write out from registers.
  // `guard`: no take() ran since the previous finish(), so its barrier has to be made up for before s_x is rewritten.
  auto finish = [&](const float4 (&x)[V], const float4& kk, unsigned minf, int slab, bool guard) {
    const int i0 = slab * LW;
    if (guard) __syncthreads();
    // warp w polls pairs w, w + NW, ... of every line (lane = line), two loads in flight at a time
#pragma unroll
    for (int t0 = 0; t0 < NE; t0 += 2) {
      const int e0 = warp + t0 * NW, e1 = e0 + NW;
      const unsigned long long* p0 = partials + ((size_t)slab * NPART + e0) * LW + lane;
      bool ok0 = e0 >= NPART, ok1 = (t0 + 1 >= NE) || e1 >= NPART;
      unsigned spins = 0;
      while (!(ok0 && ok1)) {
        unsigned long long w0 = 0, w1 = 0;
        if (!ok0) w0 = ku_ld_relaxed(p0);
        if (!ok1) w1 = ku_ld_relaxed(p0 + (size_t)NW * LW);
        if (!ok0 && (unsigned)(w0 >> 63) == par) { ok0 = true; s_x[e0][lane] = make_float2(__uint_as_float((unsigned)w0), __uint_as_float((unsigned)(w0 >> 32) & 0x7fffffffu)); }
        if (!ok1 && (unsigned)(w1 >> 63) == par) { ok1 = true; s_x[e1][lane] = make_float2(__uint_as_float((unsigned)w1), __uint_as_float((unsigned)(w1 >> 32) & 0x7fffffffu)); }
        if (ok0 && ok1) break;
        if (++spins > POLL_LIMIT) { atomicExch(status, 3); break; }
        __nanosleep(40);
      }
    }
    __syncthreads();
    // the warp merges the pairs of its four lines: lane = (line lane & 3, pairs part, part + 8, ...)
    float4 f;
    {
      const int line = q * 4 + ls;
      float M = -KU_INF;
#pragma unroll
      for (int e = part; e < NPART; e += 8) M = fmaxf(M, s_x[e][line].x);
      M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, 4));
      M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, 8));
      M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, 16));
      float t = 0.0f;
#pragma unroll
      for (int e = part; e < NPART; e += 8) {
        const float2 pr = s_x[e][line];
        t += (pr.x == -KU_INF) ? pr.y : pr.y * ku_ex2(pr.x - M);   // a sum is 0 or NaN while its max is -inf
      }
      t += __shfl_xor_sync(0xffffffffu, t, 4);
      t += __shfl_xor_sync(0xffffffffu, t, 8);
      t += __shfl_xor_sync(0xffffffffu, t, 16);
      const float c = (M == -KU_INF) ? __int_as_float(0x7fc00000) : M + log2f(t);
      const float4 c4 = make_float4(__shfl_sync(0xffffffffu, c, 0), __shfl_sync(0xffffffffu, c, 1), __shfl_sync(0xffffffffu, c, 2), __shfl_sync(0xffffffffu, c, 3));
      // e was taken against the warp's own maximum k <= c: the factor is at most 1. Where the warp saw only -inf, e is 0
      // and k is 0: the factor must not overflow (0 * inf), but a NaN line stays NaN.
      f.x = (minf & 1u) ? c4.x * 0.0f : ku_ex2(kk.x - c4.x);
      f.y = (minf & 2u) ? c4.y * 0.0f : ku_ex2(kk.y - c4.y);
      f.z = (minf & 4u) ? c4.z * 0.0f : ku_ex2(kk.z - c4.z);
      f.w = (minf & 8u) ? c4.w * 0.0f : ku_ex2(kk.w - c4.w);
    }
    // write-out: a warp-wide store is 128 contiguous bytes of one line
    ku_out_t* o = (ku_out_t*)out + (i64)(i0 + q * 4) * C + j0 + lane;
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const int jj = (h + HALVES * k) * 32;
      if ((C % CJ == 0) || j0 + jj + lane < C) {
        if ((R % LW == 0) || i0 + q * 4 + 0 < R) KU_STORE(&o[jj], KU_ENC(x[k].x * f.x));
        if ((R % LW == 0) || i0 + q * 4 + 1 < R) KU_STORE(&o[(i64)C + jj], KU_ENC(x[k].y * f.y));
        if ((R % LW == 0) || i0 + q * 4 + 2 < R) KU_STORE(&o[2 * (i64)C + jj], KU_ENC(x[k].z * f.z));
        if ((R % LW == 0) || i0 + q * 4 + 3 < R) KU_STORE(&o[3 * (i64)C + jj], KU_ENC(x[k].w * f.w));
      }
    }
  };

  // Two register tiles: while slab n waits for its group's pairs, slab n + 1 is lifted, reduced and published, so the
  // exchange has a whole slab's worth of time to complete and CTAs of a group may drift apart by that much.
  float4 xa[V], xb[V], ka, kb;
  unsigned fa = 0, fb = 0;
  int slab = group, n = 0;
  if (slab >= NSLABS) return;
  take(xa, ka, fa, 0, slab);
  for (;;) {
    const int s1 = slab + ngroups;
    if (s1 < NSLABS) take(xb, kb, fb, n + 1, s1);
    finish(xa, ka, fa, slab, s1 >= NSLABS && n > 0);
    if (s1 >= NSLABS) break;
    const int s2 = s1 + ngroups;
    if (s2 < NSLABS) take(xa, ka, fa, n + 2, s2);
    finish(xb, kb, fb, s1, s2 >= NSLABS);
    if (s2 >= NSLABS) break;
    slab = s2;
    n += 2;
  }
}

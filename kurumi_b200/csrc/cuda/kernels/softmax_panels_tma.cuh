// Softmax through a transpose view in two passes that share one persistent, TMA-fed kernel, ordered so
// that the second pass reads its input from L2: HBM sees every input byte once and every output byte
// once, and no cluster, no co-residency and no lockstep between CTAs is needed.
//
// The dominant input is a plain f32 buffer read as in[j * ld + i] (i = line, j = position along the
// softmax axis). Lines are cut into panels of PWL = 256 lines; a panel of 8192 positions is 8 MB.
// Work items are handed out from one global counter, group after group; group g holds
//   A(g + LA)  statistics: a [JT positions x 32 lines] tile of panel g + LA -> one (max, sum) partial per line
//   C(g + LC)  merges: the partials of 16 lines of panel g + LC -> c[line] = max*log2e + log2(sum)
//   B(g)       output: a [JT x 32] tile of panel g -> out[line][position] = exp2(x*log2e - c[line])
// A CTA keeps a ring of NBUF tiles: it claims items ahead of the one it is working on and starts the TMA
// load of a claimed tile at once (a B tile's load needs nothing but the input), so its loads are in
// flight while it works. While it works on one item, warp 0 already reads the counter the next item
// depends on (and an output tile's c values), so that in the steady state no wait is exposed.
// Tiles are [JT][32] f32 with 128-byte swizzled rows: a warp reads a row (32 lines at one position)
// conflict-free with 4-byte loads and a 32-position column strip of 4 lines with 16-byte loads, which
// makes the transposed write-out coalesced (128 contiguous bytes per warp store).
//
// Every wait is on items that were claimed earlier; each CTA works through its claimed items in claim
// order, so by induction over the claim index every item completes whatever the number of resident
// CTAs. Every wait is bounded: a CTA that gives up records it in *status and carries on.
//
// Spliced in by the host: R, C, JT, NBUF, LA, LC, NPB (partial buffers in rotation), KU_L2_HINTS, KU_OUT_F32, KU_SRC_IDENTITY, and
//   float ku_src_t(float lval, idx i, idx j KU_SRC_PARAMS) - the fused producer given the loaded value.
#define NT 256
#define NW 8
#define PWL 256
#define STRIPS (PWL / 32)
#define NCI (PWL / 16)
#define KU_LOG2E 1.4426950408889634f
// the fused producer reads its other operands at coordinates clamped into the tensor: tiles overhang the last
// lines / positions, and what is computed there is masked or never stored
#define KU_CI(i) ((R % PWL != 0 && (i) >= R) ? R - 1 : (i))
#define KU_CJ(j) ((C % JT != 0 && (j) >= C) ? C - 1 : (j))
#define TILE_BYTES (JT * 128)
#define SPIN_LIMIT (1u << 22)
#define NJ ((C + JT - 1) / JT)
#define PANELS ((R + PWL - 1) / PWL)
#define NA (STRIPS * NJ)
#define NB (STRIPS * NJ)
#define PER (NA + NCI + NB)
#define KU_MAX_PANELS 1024
#if KU_L2_HINTS && KU_OUT_F32
#define KU_STORE(p, v) __stcs((p), (v))   // the output is not read again: stream it through L2
#else
#define KU_STORE(p, v) (*(p) = (v))
#endif

struct alignas(64) KuTmap { unsigned long long opaque[16]; };
struct KuCtl { unsigned next_item; unsigned error; unsigned cnt_a[KU_MAX_PANELS]; unsigned cnt_c[KU_MAX_PANELS]; };

__device__ __forceinline__ float ku_ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
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
// the same load with an L2 eviction policy: statistics tiles are wanted again soon (evict last), output
// tiles are read for the last time (evict first)
__device__ __forceinline__ void ku_tma_2d_hint(unsigned dst, const KuTmap* map, int x, int y, unsigned mbar, unsigned long long policy) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(mbar), "l"(policy) : "memory");
}
__device__ __forceinline__ unsigned long long ku_policy_evict_last() { unsigned long long p; asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p)); return p; }
__device__ __forceinline__ unsigned long long ku_policy_evict_first() { unsigned long long p; asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p)); return p; }
__device__ __forceinline__ unsigned ku_ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// byte offset of (position jj, line ii) inside a swizzled tile
__device__ __forceinline__ unsigned ku_tile_off(int jj, int ii) { return (unsigned)(jj * 128 + ((((ii >> 2) ^ (jj & 7))) << 4) + ((ii & 3) << 2)); }

// bounded wait of the whole CTA until *counter reaches target; only thread 0 polls
__device__ __forceinline__ void ku_wait_count(unsigned* counter, unsigned target, KuCtl* ctl, int* status, int code) {
  if (threadIdx.x == 0) {
    unsigned spins = 0;
    while (ku_ld_acquire(counter) < target) {
      if (++spins > SPIN_LIMIT || ku_ld_acquire(&ctl->error) != 0u) {
        atomicExch(&ctl->error, 1u);
        atomicExch(status, code);
        break;
      }
      __nanosleep(32);
    }
  }
  __syncthreads();
}
// bounded wait on a shared-memory barrier phase
__device__ __forceinline__ void ku_wait_bar(unsigned mb, unsigned parity, KuCtl* ctl, int* status, int code) {
  unsigned spins = 0;
  while (!ku_mbar_try(mb, parity)) {
    if (++spins > SPIN_LIMIT) { atomicExch(status, code); atomicExch(&ctl->error, 1u); break; }
  }
}

// item index -> (kind, panel, index inside the panel's items of that kind); kind 0 = A, 1 = C, 2 = B, 3 = none
__device__ __forceinline__ void ku_decode(long long t, int* kind, int* p, int* r) {
  const long long total = (long long)PANELS * PER;
  if (t >= total) { *kind = 3; *p = 0; *r = 0; return; }
  long long rem = t;
  int g = -LA;
  bool found = false;
  for (; g < 0; ++g) {
    const int sz = (g + LA < PANELS ? NA : 0) + ((g + LC >= 0 && g + LC < PANELS) ? NCI : 0);
    if (rem < sz) { found = true; break; }
    rem -= sz;
  }
  if (!found) {
    const int nfull = PANELS > LA ? PANELS - LA : 0;   // groups that hold all three kinds
    if (rem < (long long)nfull * PER) { g = (int)(rem / PER); rem -= (long long)g * PER; }
    else {
      rem -= (long long)nfull * PER;
      for (g = nfull; g < PANELS - 1; ++g) {
        const int sz = (g + LA < PANELS ? NA : 0) + (g + LC < PANELS ? NCI : 0) + NB;
        if (rem < sz) break;
        rem -= sz;
      }
    }
  }
  const int a_sz = (g + LA < PANELS) ? NA : 0;
  const int c_sz = (g + LC >= 0 && g + LC < PANELS) ? NCI : 0;
  if (rem < a_sz) { *kind = 0; *p = g + LA; *r = (int)rem; }
  else if (rem < a_sz + c_sz) { *kind = 1; *p = g + LC; *r = (int)rem - a_sz; }
  else { *kind = 2; *p = g; *r = (int)rem - a_sz - c_sz; }
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
ku_softmax_panels_tma(const __grid_constant__ KuTmap tmap, KU_SRC_PARAMS_LEAD void* __restrict__ out, void* __restrict__ scratch, int* __restrict__ status) {
  extern __shared__ __align__(1024) unsigned char tiles_raw[];  // NBUF tiles of [JT][32] f32, 128-byte swizzled rows
  __shared__ __align__(8) unsigned long long full[NBUF];
  __shared__ int s_kind[NBUF], s_p[NBUF], s_r[NBUF];
  __shared__ __align__(16) float s_max[NW][32], s_sum[NW][32];
  __shared__ int s_ready[2];
  __shared__ __align__(16) float line_c[2][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  KuCtl* ctl = (KuCtl*)scratch;
  float* cvals = (float*)((char*)scratch + 16384);
  float2* partials = (float2*)((char*)scratch + 16384 + (((size_t)R * 4 + 255) / 256) * 256);
  // the swizzle pattern is a function of the shared-memory address: tiles start on a 1024-byte boundary
  // (the host sizes the ring with 1024 bytes of slack)
  unsigned char* tiles = tiles_raw + ((1024u - (ku_smem(tiles_raw) & 1023u)) & 1023u);
  const unsigned tiles_s = ku_smem(tiles);
#if KU_L2_HINTS
  const unsigned long long pol_keep = ku_policy_evict_last(), pol_drop = ku_policy_evict_first();
#endif
  // thread 0: record a claimed item in ring slot b and start its tile load
  auto place = [&](unsigned t, int b) {
    int kind, p, r;
    ku_decode((long long)t, &kind, &p, &r);
    s_kind[b] = kind; s_p[b] = p; s_r[b] = r;
    if (kind == 0 || kind == 2) {
      const int strip = r % STRIPS, jb = r / STRIPS;
      const unsigned mb = ku_smem(&full[b]);
      ku_mbar_expect(mb, TILE_BYTES);
#if KU_L2_HINTS
      ku_tma_2d_hint(tiles_s + b * TILE_BYTES, &tmap, p * PWL + strip * 32, jb * JT, mb, kind == 0 ? pol_keep : pol_drop);
#else
      ku_tma_2d(tiles_s + b * TILE_BYTES, &tmap, p * PWL + strip * 32, jb * JT, mb);
#endif
    }
  };
  unsigned pending = 0;   // thread 0: an item claimed one iteration ahead of the slot it will fill
  if (threadIdx.x == 0) {
    for (int b = 0; b < NBUF; ++b) ku_mbar_init(ku_smem(&full[b]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    for (int b = 0; b < NBUF; ++b) place(atomicAdd(&ctl->next_item, 1u), b);
    pending = atomicAdd(&ctl->next_item, 1u);
    s_ready[0] = 0;
  }
  __syncthreads();

  unsigned phase_bits = 0;   // parity of each ring slot's barrier
  for (int n = 0;; ++n) {
    const int b = n % NBUF;
    const int kind = s_kind[b], p = s_p[b], r = s_r[b];
    if (kind == 3) break;   // items are claimed in order: nothing later is pending either
    // Warp 0 looks ahead, with loads whose answers are only needed when this item is finished: it claims
    // one more item, reads the counter the NEXT item depends on and, for an output tile, that tile's c values.
    unsigned fresh = 0, dep_seen = 0, dep_target = 0;
    float c_next = 0.0f;
    if (warp == 0) {
      __syncwarp();   // lane 0 wrote the next slot's descriptor at the end of an earlier iteration
      if (lane == 0) fresh = atomicAdd(&ctl->next_item, 1u);
      if (NBUF > 1) {
        const int nb = (n + 1) % NBUF;
        const int nk = s_kind[nb], np = s_p[nb], nr = s_r[nb];
        const unsigned* dep = nullptr;
        if (nk == 0 && np >= NPB) { dep = &ctl->cnt_c[np - NPB]; dep_target = NCI; }
        else if (nk == 1) { dep = &ctl->cnt_a[np]; dep_target = NA; }
        else if (nk == 2) { dep = &ctl->cnt_c[np]; dep_target = NCI; }
        if (dep) dep_seen = ku_ld_acquire(dep);
        if (nk == 2) {
          const int li = np * PWL + (nr % STRIPS) * 32 + lane;
          if (li < R) c_next = __ldcg(cvals + li);   // valid if dep_seen reached the target: the load follows the acquire
        }
      }
    }
    const unsigned char* tile = tiles + b * TILE_BYTES;
    if (kind != 1) {
      const unsigned parity = (phase_bits >> b) & 1u;
      phase_bits ^= 1u << b;
      ku_wait_bar(ku_smem(&full[b]), parity, ctl, status, 1);
    }
    const bool ready = s_ready[n & 1] != 0;   // the look-ahead of the previous iteration found this item's dependency met
    const int i_base = p * PWL;
    float2* part = partials + (size_t)(p % NPB) * NJ * PWL;
    unsigned* done = nullptr;   // the counter this item bumps when it is finished
    if (kind == 0) {
      const int strip = r % STRIPS, jb = r / STRIPS;
      const int i0 = i_base + strip * 32, j0 = jb * JT;
      // this panel's partials reuse the buffer of panel p - NPB: its merges must be over (they nearly always are)
      if (!ready && p >= NPB) ku_wait_count(&ctl->cnt_c[p - NPB], NCI, ctl, status, 6);
      // thread = (4 lines: chunk q of the 32, row group rs of 4); it keeps its JT/32 x 4 values in registers
      const int q = lane & 7, rs = lane >> 3;
      float4 x[JT / 32];
#pragma unroll
      for (int it = 0; it < JT / 32; ++it) {
        const int row = it * 32 + warp * 4 + rs, j = j0 + row;
        float4 v = *(const float4*)(tile + row * 128 + ((q ^ (row & 7)) << 4));
#if !KU_SRC_IDENTITY
        v.x = ku_src_t(v.x, KU_CI(i0 + q * 4 + 0), KU_CJ(j) KU_SRC_ARGS);
        v.y = ku_src_t(v.y, KU_CI(i0 + q * 4 + 1), KU_CJ(j) KU_SRC_ARGS);
        v.z = ku_src_t(v.z, KU_CI(i0 + q * 4 + 2), KU_CJ(j) KU_SRC_ARGS);
        v.w = ku_src_t(v.w, KU_CI(i0 + q * 4 + 3), KU_CJ(j) KU_SRC_ARGS);
#endif
        if ((C % JT != 0) && j >= C) v = make_float4(-KU_INF, -KU_INF, -KU_INF, -KU_INF);
        x[it] = v;
      }
      float4 m = x[0];
#pragma unroll
      for (int it = 1; it < JT / 32; ++it) { m.x = fmaxf(m.x, x[it].x); m.y = fmaxf(m.y, x[it].y); m.z = fmaxf(m.z, x[it].z); m.w = fmaxf(m.w, x[it].w); }
#pragma unroll
      for (int o = 8; o <= 16; o <<= 1) {
        m.x = fmaxf(m.x, __shfl_xor_sync(0xffffffffu, m.x, o)); m.y = fmaxf(m.y, __shfl_xor_sync(0xffffffffu, m.y, o));
        m.z = fmaxf(m.z, __shfl_xor_sync(0xffffffffu, m.z, o)); m.w = fmaxf(m.w, __shfl_xor_sync(0xffffffffu, m.w, o));
      }
      if (rs == 0) *(float4*)&s_max[warp][q * 4] = m;
      __syncthreads();
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        const float4 o = *(const float4*)&s_max[w][q * 4];
        m.x = fmaxf(m.x, o.x); m.y = fmaxf(m.y, o.y); m.z = fmaxf(m.z, o.z); m.w = fmaxf(m.w, o.w);
      }
      // exp2(x*log2e - max*log2e); a line that is all -inf so far subtracts 0 and sums zeros
      const float4 k = make_float4(m.x == -KU_INF ? 0.0f : m.x * KU_LOG2E, m.y == -KU_INF ? 0.0f : m.y * KU_LOG2E,
                                   m.z == -KU_INF ? 0.0f : m.z * KU_LOG2E, m.w == -KU_INF ? 0.0f : m.w * KU_LOG2E);
      float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int it = 0; it < JT / 32; ++it) {
        sum.x += ku_ex2(__fmaf_rn(x[it].x, KU_LOG2E, -k.x)); sum.y += ku_ex2(__fmaf_rn(x[it].y, KU_LOG2E, -k.y));
        sum.z += ku_ex2(__fmaf_rn(x[it].z, KU_LOG2E, -k.z)); sum.w += ku_ex2(__fmaf_rn(x[it].w, KU_LOG2E, -k.w));
      }
#pragma unroll
      for (int o = 8; o <= 16; o <<= 1) {
        sum.x += __shfl_xor_sync(0xffffffffu, sum.x, o); sum.y += __shfl_xor_sync(0xffffffffu, sum.y, o);
        sum.z += __shfl_xor_sync(0xffffffffu, sum.z, o); sum.w += __shfl_xor_sync(0xffffffffu, sum.w, o);
      }
      if (rs == 0) *(float4*)&s_sum[warp][q * 4] = sum;
      __syncthreads();
      if (warp == 0 && i0 + lane < R) {
        float mm = s_max[0][lane], tot = s_sum[0][lane];
#pragma unroll
        for (int w = 1; w < NW; ++w) { mm = fmaxf(mm, s_max[w][lane]); tot += s_sum[w][lane]; }
        part[(size_t)jb * PWL + strip * 32 + lane] = make_float2(mm * KU_LOG2E, tot);   // (max in log2 units, sum relative to it)
      }
      done = &ctl->cnt_a[p];
    } else if (kind == 1) {
      if (!ready) ku_wait_count(&ctl->cnt_a[p], NA, ctl, status, 7);
      // the item is 16 lines; each warp takes two of them, 16 lanes each over the partial rows
      const int sl = lane & 15;
      const int il = r * 16 + warp * 2 + (lane >> 4);
      float m = -KU_INF, sum = 0.0f;
      for (int b0 = sl; b0 < NJ; b0 += 128) {
        float2 q2[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const int bb = b0 + 16 * k;
          q2[k] = bb < NJ ? __ldcg(part + (size_t)bb * PWL + il) : make_float2(-KU_INF, 0.0f);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) ku_merge(m, sum, q2[k].x, q2[k].y);
      }
#pragma unroll
      for (int o = 1; o <= 8; o <<= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, sum, o);
        ku_merge(m, sum, om, os);
      }
      if (sl == 0 && i_base + il < R) cvals[i_base + il] = (m == -KU_INF) ? __int_as_float(0x7fc00000) : m + log2f(sum);
      done = &ctl->cnt_c[p];
    } else {
      const int strip = r % STRIPS, jb = r / STRIPS;
      const int i0 = i_base + strip * 32, j0 = jb * JT;
      if (!ready) {   // the panel's merges were handed out LC groups ago; this path is rare
        ku_wait_count(&ctl->cnt_c[p], NCI, ctl, status, 8);
        if (warp == 0) line_c[n & 1][lane] = (i0 + lane < R) ? __ldcg(cvals + i0 + lane) : 0.0f;
        __syncthreads();
      }
      const int q = warp;   // this warp writes lines i0 + 4q .. i0 + 4q + 3
      const float4 c4 = *(const float4*)&line_c[n & 1][q * 4];
      // the last panel may hold fewer than its 8 strips of 32 lines: a strip past the last line has nothing to write
      // (its tile is zero fill, its item still counts)
      if ((R % PWL == 0) || i0 < R) {
      // lane = position within a 32-position strip; one 16-byte load gives 4 lines at that position,
      // then 4 warp-wide stores of 128 contiguous bytes each
#pragma unroll 4
      for (int js = 0; js < JT / 32; ++js) {
        const int jj = js * 32 + lane, j = j0 + jj;
        float4 v = *(const float4*)(tile + jj * 128 + ((q ^ (jj & 7)) << 4));
        if ((C % JT == 0) || j < C) {
#if !KU_SRC_IDENTITY
          v.x = ku_src_t(v.x, KU_CI(i0 + q * 4 + 0), KU_CJ(j) KU_SRC_ARGS);
          v.y = ku_src_t(v.y, KU_CI(i0 + q * 4 + 1), KU_CJ(j) KU_SRC_ARGS);
          v.z = ku_src_t(v.z, KU_CI(i0 + q * 4 + 2), KU_CJ(j) KU_SRC_ARGS);
          v.w = ku_src_t(v.w, KU_CI(i0 + q * 4 + 3), KU_CJ(j) KU_SRC_ARGS);
#endif
          ku_out_t* o = (ku_out_t*)out + (i64)(i0 + q * 4) * C + j;
          if ((R % 32 == 0) || i0 + q * 4 + 0 < R) KU_STORE(&o[0], KU_ENC(ku_ex2(__fmaf_rn(v.x, KU_LOG2E, -c4.x))));
          if ((R % 32 == 0) || i0 + q * 4 + 1 < R) KU_STORE(&o[(i64)C], KU_ENC(ku_ex2(__fmaf_rn(v.y, KU_LOG2E, -c4.y))));
          if ((R % 32 == 0) || i0 + q * 4 + 2 < R) KU_STORE(&o[2 * (i64)C], KU_ENC(ku_ex2(__fmaf_rn(v.z, KU_LOG2E, -c4.z))));
          if ((R % 32 == 0) || i0 + q * 4 + 3 < R) KU_STORE(&o[3 * (i64)C], KU_ENC(ku_ex2(__fmaf_rn(v.w, KU_LOG2E, -c4.w))));
        }
      }
      }
    }
    if (warp == 0) {   // hand the look-ahead to the next iteration
      if (lane == 0) s_ready[(n + 1) & 1] = (NBUF > 1 && dep_seen >= dep_target) ? 1 : 0;
      line_c[(n + 1) & 1][lane] = c_next;
    }
    __syncthreads();  // every thread is done with slot b: its tile, its descriptor, and the shared scratch
    if (threadIdx.x == 0) {
      // the CTA's global writes for this item are ordered before this release by the barrier above
      if (done) asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(done) : "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy accesses to the tile precede the async refill
      place(pending, b);
      pending = fresh;
    }
    if (NBUF == 1) __syncthreads();   // with a deeper ring the refilled slot is read again only after later barriers
  }
}

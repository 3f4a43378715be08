// Fused scaled-dot-product attention for sm_100a (Op::Sdpa, kurumi_core/src/graph/op.rs:55-58):
// out = softmax(q k^T / sqrt(dh) [+ causal mask]) v over the trailing [S, DH] of [BH, S, DH] bf16 / f16
// tensors, online softmax, no S x S buffer. The math is the interpreter's decomposition
// (kurumi_core/src/interp/nn.rs:125-172): scale = 1/sqrt(dh) as f32, key j > query i masked to -inf,
// softmax in f32; results stay within rel 2e-2 of the f64 run.
//
// One CTA per (head, block of 128 queries); key/value blocks of 128 stream through two-stage rings.
//   warp 0      TMA producer: Q once, then K_j / V_j (cp.async.bulk.tensor, SWIZZLE_128B, no multicast)
//   warp 1      tcgen05.mma issuer: S_j = Q K_j^T into one of two TMEM score buffers (so the scores of
//               block j+1 are computed while block j is in the softmax), then O += P_j V_j
//   warps 2..9  softmax, two threads per query row (one per half of the key block, so that two warps per
//               scheduler hide each other's latencies): tcgen05.ld the scores, maximum (exchanged through
//               shared memory inside the warp pair) / sum in the log2 domain, P_j as bf16 into shared
//               memory in the swizzled K-major layout the second MMA reads. O accumulates
//               in tensor memory across key blocks; the threads rescale it (tcgen05.ld / st) only when a
//               row's maximum has grown by more than 2^8 since the scale it was accumulated with
// Causal: key blocks above the diagonal are never loaded; the diagonal block is masked per element.
// Every mbarrier wait is bounded (status word + sticky failure), tensor memory is always released.
//
// Spliced in by the host: BH, S, DH (64 or 128), CAUSAL, SCALE_LOG2E (scale * log2 e as a float
// literal), IDESC_S, IDESC_O, KU_IS_BF16.
#define BQ 128
#define BKV 128
#define DCH (DH / 64)                    // 64-element (128-byte) chunks along the head dimension
#define TILE_BYTES (128 * 128 * DCH)     // one [128 rows][DH] bf16 tile: DCH chunks of [128][128 bytes]
#define P_BYTES (128 * 128 * 2)          // [128 queries][128 keys] bf16: 2 chunks of [128][128 bytes]
#define SPIN_LIMIT (1u << 24)

struct alignas(64) KuTmap { unsigned long long opaque[16]; };

__device__ __forceinline__ unsigned ku_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ku_mbar_init(unsigned a, unsigned n) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(a), "r"(n)); }
__device__ __forceinline__ void ku_mbar_expect(unsigned a, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(a), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ku_mbar_arrive(unsigned a) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(a) : "memory"); }
__device__ __forceinline__ bool ku_mbar_try(unsigned a, unsigned parity) {
  unsigned ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(a), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool ku_wait(unsigned a, unsigned parity, bool& failed, int* status) {
  if (failed) return false;
  unsigned spins = 0;
  while (!ku_mbar_try(a, parity)) {
    ++spins;
    if ((spins & 4095u) == 0 && *(volatile int*)status != 0) { failed = true; return false; }
    if (spins > SPIN_LIMIT) { failed = true; atomicExch(status, 6); return false; }
  }
  return true;
}
__device__ __forceinline__ void ku_tma_3d(unsigned dst, const KuTmap* map, int x, int y, int z, unsigned mbar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(mbar) : "memory");
}
__device__ __forceinline__ unsigned long long ku_smem_desc(unsigned addr, unsigned lbo, unsigned sbo) {
  return (unsigned long long)((addr & 0x3FFFFu) >> 4) | ((unsigned long long)(lbo >> 4) << 16) | ((unsigned long long)(sbo >> 4) << 32) |
         (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void ku_mma(unsigned d_tmem, unsigned long long adesc, unsigned long long bdesc, unsigned idesc, unsigned accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void ku_mma_commit(unsigned mbar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar) : "memory");
}
__device__ __forceinline__ void ku_tmem_ld32(unsigned taddr, float* v) {
  unsigned* r = (unsigned*)v;
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, "
      "%23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
        "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
        "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// the same load without the wait: several can be in flight before one tcgen05.wait::ld
__device__ __forceinline__ void ku_tmem_ld32_nowait(unsigned taddr, float* v) {
  unsigned* r = (unsigned*)v;
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, "
      "%23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
        "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
        "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void ku_tmem_st32(unsigned taddr, const float* v) {
  const unsigned* r = (const unsigned*)v;
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, "
      "%24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]),
        "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]),
        "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ float ku_ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ unsigned ku_pack2(float lo, float hi) {
#if KU_IS_BF16
  unsigned r; asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo)); return r;
#else
  unsigned r; asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo)); return r;
#endif
}

#if !KU_TWIN
extern "C" __global__ void __launch_bounds__(320, 1)
ku_attention_tc(const __grid_constant__ KuTmap tmap_q, const __grid_constant__ KuTmap tmap_k, const __grid_constant__ KuTmap tmap_v, void* __restrict__ Op,
                int* __restrict__ status) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], s_free[2], p_ready, o_full;
  __shared__ unsigned tmem_base_slot;
  __shared__ float x_max[2][2][128], x_sum[2][128];   // [block parity][column half][row], [column half][row]
  unsigned char* smem = smem_raw + ((1024u - (ku_smem(smem_raw) & 1023u)) & 1023u);
  const unsigned q_s = ku_smem(smem), k_s = q_s + TILE_BYTES, v_s = k_s + 2 * TILE_BYTES, p_s = v_s + 2 * TILE_BYTES;
  unsigned char* p_tile = smem + 5 * TILE_BYTES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qb = (int)gridDim.x - 1 - (int)blockIdx.x;   // long (late) query blocks first
  const int bh = blockIdx.y;
  const int kv_blocks = (S + BKV - 1) / BKV;
  const int nkv = CAUSAL ? ((qb + 1) < kv_blocks ? (qb + 1) : kv_blocks) : kv_blocks;

  if (threadIdx.x == 0) {
    ku_mbar_init(ku_smem(&q_full), 1);
    for (int i = 0; i < 2; ++i) {
      ku_mbar_init(ku_smem(&k_full[i]), 1); ku_mbar_init(ku_smem(&k_empty[i]), 1); ku_mbar_init(ku_smem(&v_full[i]), 1); ku_mbar_init(ku_smem(&v_empty[i]), 1);
      ku_mbar_init(ku_smem(&s_full[i]), 1); ku_mbar_init(ku_smem(&s_free[i]), 256);
    }
    ku_mbar_init(ku_smem(&p_ready), 256); ku_mbar_init(ku_smem(&o_full), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ku_smem(&tmem_base_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = tmem_base_slot;   // columns [0,128) and [128,256): score buffers; [256, 256+DH): O_j
  bool failed = false;

  if (warp == 0) {
    if (lane == 0) {  // ---- TMA producer ----
      ku_mbar_expect(ku_smem(&q_full), TILE_BYTES);
      for (int c = 0; c < DCH; ++c) ku_tma_3d(q_s + c * 16384, &tmap_q, c * 64, qb * BQ, bh, ku_smem(&q_full));
      // K runs a block ahead of V: K_{j+2} only needs S_j to have retired (early), V_j needs P_{j-2} V_{j-2} to have
      // retired (late); loading them in lock step would hold every K load back behind a V wait
      auto load_k = [&](int j) {
        const int st = j & 1;
        ku_wait(ku_smem(&k_empty[st]), ((j >> 1) & 1) ^ 1, failed, status);
        ku_mbar_expect(ku_smem(&k_full[st]), TILE_BYTES);
        for (int c = 0; c < DCH; ++c) ku_tma_3d(k_s + st * TILE_BYTES + c * 16384, &tmap_k, c * 64, j * BKV, bh, ku_smem(&k_full[st]));
      };
      if (nkv > 0) load_k(0);
      if (nkv > 1) load_k(1);
      for (int j = 0; j < nkv; ++j) {
        const int st = j & 1;
        ku_wait(ku_smem(&v_empty[st]), ((j >> 1) & 1) ^ 1, failed, status);
        ku_mbar_expect(ku_smem(&v_full[st]), TILE_BYTES);
        for (int c = 0; c < DCH; ++c) ku_tma_3d(v_s + st * TILE_BYTES + c * 16384, &tmap_v, c * 64, j * BKV, bh, ku_smem(&v_full[st]));
        if (j + 2 < nkv) load_k(j + 2);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {  // ---- MMA issuer ----
      auto issue_s = [&](int j) {   // S_j = Q K_j^T: both operands K-major over the head dimension
        const int st = j & 1;
        ku_wait(ku_smem(&k_full[st]), (j >> 1) & 1, failed, status);
        ku_wait(ku_smem(&s_free[st]), ((j >> 1) & 1) ^ 1, failed, status);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int kk = 0; kk < DH / 16; ++kk) {
          const unsigned off = (kk >> 2) * 16384 + (kk & 3) * 32;
          ku_mma(tmem_base + st * 128, ku_smem_desc(q_s + off, 16, 1024), ku_smem_desc(k_s + st * TILE_BYTES + off, 16, 1024), IDESC_S, kk != 0);
        }
        ku_mma_commit(ku_smem(&s_full[st]));
        ku_mma_commit(ku_smem(&k_empty[st]));
      };
      ku_wait(ku_smem(&q_full), 0, failed, status);
      issue_s(0);
      for (int j = 0; j < nkv; ++j) {
        if (j + 1 < nkv) issue_s(j + 1);
        const int st = j & 1;
        ku_wait(ku_smem(&v_full[st]), (j >> 1) & 1, failed, status);
        ku_wait(ku_smem(&p_ready), j & 1, failed, status);   // P_j is in shared memory and O has been rescaled if it had to be
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {   // O += P_j V_j: P K-major over keys, V MN-major (head dimension contiguous)
          const unsigned long long ad = ku_smem_desc(p_s + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
          const unsigned long long bd = ku_smem_desc(v_s + st * TILE_BYTES + kk * 16 * 128, 16384, 1024);
          ku_mma(tmem_base + 256, ad, bd, IDESC_O, (j | kk) != 0);
        }
        ku_mma_commit(ku_smem(&o_full));
        ku_mma_commit(ku_smem(&v_empty[st]));
      }
    }
  } else {  // ---- softmax: eight warps; a query row is shared by two threads, one per half of the key block ----
    const int q4 = warp & 3;                      // the TMEM lane quarter this warp may access
    const int half = (warp - 2) >> 2;             // key columns [64 half, 64 half + 64) of every block, head-dim columns [DH/2 half, ...) of O
    const int r = q4 * 32 + lane;                 // row of the tile == TMEM lane
    const int qrow = qb * BQ + r;
    const unsigned lane_addr = tmem_base + ((unsigned)(q4 * 32) << 16);
    const unsigned pair_bar = 1 + q4;             // named barrier of the two warps that share these 32 rows
    constexpr int HK = BKV / 2, HD = DH / 2;
    // m is the reference maximum the accumulator O (in tensor memory) and the sum l are scaled by. It follows
    // the running maximum lazily: only when a block's maximum exceeds it by more than 2^8 are O and l rescaled,
    // so most blocks touch O with the tensor core alone (probabilities stay below 2^8, accumulation is f32).
    float m = -KU_INF, l = 0.0f;   // l: this thread's share (its half of the keys)
    for (int j = 0; j < nkv; ++j) {
      const int st = j & 1;
      ku_wait(ku_smem(&s_full[st]), (j >> 1) & 1, failed, status);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const bool need_mask = (CAUSAL && j == qb) || (j * BKV + BKV > S);
      // this thread's half of the row's scores, in log2 units, masked keys at -inf
      float sc[HK];
#pragma unroll
      for (int c0 = 0; c0 < HK; c0 += 32) ku_tmem_ld32_nowait(lane_addr + st * 128 + half * HK + c0, sc + c0);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
      for (int c = 0; c < HK; ++c) asm volatile("" : "+f"(sc[c]));   // the values may only be read after the wait: tie every register to this point
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      ku_mbar_arrive(ku_smem(&s_free[st]));                          // the score buffer may be overwritten
      float bm = -KU_INF;
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < HK; ++c) {
          const int key = j * BKV + half * HK + c;
          sc[c] = ((CAUSAL && key > qrow) || key >= S) ? -KU_INF : sc[c] * SCALE_LOG2E;
          bm = fmaxf(bm, sc[c]);
        }
      } else {
#pragma unroll
        for (int c = 0; c < HK; ++c) { sc[c] *= SCALE_LOG2E; bm = fmaxf(bm, sc[c]); }
      }
      // the row maximum over both halves (double-buffered by block parity: a fast thread may be a block ahead)
      x_max[j & 1][half][r] = bm;
      asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
      bm = fmaxf(bm, x_max[j & 1][half ^ 1][r]);
      const bool grow = bm > m + 8.0f || (m == -KU_INF && bm != -KU_INF);
      const bool any_grow = __any_sync(0xffffffffu, grow);
      const float alpha = grow ? ku_ex2(m - bm) : 1.0f;   // 0 for a row's first finite block: O holds nothing for it yet
      if (grow) m = bm;
      const float mref = (m == -KU_INF) ? 0.0f : m;   // a row with nothing finite so far: exp2(-inf - 0) = 0
      // the probabilities, packed 8 keys = one 16-byte chunk at a time, while the previous block's P V product still runs
      float bs = 0.0f;
      uint4 pk[HK / 8];
#pragma unroll
      for (int c0 = 0; c0 < HK; c0 += 8) {
        float e[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) { e[c] = ku_ex2(sc[c0 + c] - mref); bs += e[c]; }
        pk[c0 >> 3].x = ku_pack2(e[0], e[1]); pk[c0 >> 3].y = ku_pack2(e[2], e[3]);
        pk[c0 >> 3].z = ku_pack2(e[4], e[5]); pk[c0 >> 3].w = ku_pack2(e[6], e[7]);
      }
      // that product must have retired before P is overwritten or O is touched
      if (j > 0) {
        ku_wait(ku_smem(&o_full), (j - 1) & 1, failed, status);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      }
      if (any_grow) {   // tensor-memory loads and stores are warp-wide: rows that keep their reference scale by 1
        if (j > 0) {
#pragma unroll 1
          for (int c0 = 0; c0 < HD; c0 += 32) {   // this thread's half of the head dimension
            float v[32];
            ku_tmem_ld32(lane_addr + 256 + half * HD + c0, v);
#pragma unroll
            for (int c = 0; c < 32; ++c) v[c] *= alpha;
            ku_tmem_st32(lane_addr + 256 + half * HD + c0, v);
          }
        }
        l *= alpha;
      }
      // as bf16 in the swizzled K-major tile; the half IS the 64-key (128-byte) chunk of the P tile
#pragma unroll
      for (int ch = 0; ch < HK / 8; ++ch) *(uint4*)(p_tile + half * 16384 + r * 128 + ((ch ^ (r & 7)) << 4)) = pk[ch];
      l += bs;
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P is read by the tensor core (async proxy)
      ku_mbar_arrive(ku_smem(&p_ready));
    }
    // the row's sum over both halves
    x_sum[half][r] = l;
    asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
    l += x_sum[half ^ 1][r];
    // the last product, then this thread's half of the row of O
    float o[HD];
    if (nkv > 0) {
      ku_wait(ku_smem(&o_full), (nkv - 1) & 1, failed, status);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (int c0 = 0; c0 < HD; c0 += 32) ku_tmem_ld32(lane_addr + 256 + half * HD + c0, o + c0);
    } else {
#pragma unroll
      for (int c = 0; c < HD; ++c) o[c] = 0.0f;
    }
    if (qrow < S) {
      const float inv = 1.0f / l;
      uint4* dst = (uint4*)((unsigned short*)Op + ((i64)bh * S + qrow) * DH + half * HD);
#pragma unroll
      for (int g = 0; g < HD / 8; ++g) {
        uint4 pk;
        pk.x = ku_pack2(o[g * 8 + 0] * inv, o[g * 8 + 1] * inv); pk.y = ku_pack2(o[g * 8 + 2] * inv, o[g * 8 + 3] * inv);
        pk.z = ku_pack2(o[g * 8 + 4] * inv, o[g * 8 + 5] * inv); pk.w = ku_pack2(o[g * 8 + 6] * inv, o[g * 8 + 7] * inv);
        dst[g] = pk;
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
}
#endif  // !KU_TWIN

#if KU_TWIN
// ---- Two CTAs per SM -------------------------------------------------------------------------------------
// The same algorithm with key blocks of 64, four softmax warps (one thread per query row) and half the
// tensor memory (two 64-column score buffers + O = 256 columns), so that two CTAs share an SM: while one
// CTA's softmax threads wait for scores, store P or wait for a product, the other CTA's exponentials keep
// the special-function unit busy and its MMAs keep the tensor core busy. Shared memory (DH = 128): Q 32 KB,
// K and V rings 2 x 16 KB each, P 16 KB, barriers: 112.25 KB per CTA, all of it dynamic (the swizzled tiles
// need 1024-byte alignment, which the start of dynamic shared memory has when nothing static precedes it).
#define TK 64
#ifndef KU_POLY
#define KU_POLY 0   // of every 8 exponentials, how many are computed on the FMA pipe instead of the special-function unit
#endif
// 2^x without the special-function unit: x = n + f with n = round(x), f in [-0.5, 0.5]; 2^f by a cubic (relative
// error 1.2e-4, below the 3.9e-3 rounding step of the bf16 probabilities it feeds), n added to the exponent field.
// x is clamped at -127, where the result is exactly 0 (masked keys arrive as -inf).
__device__ __forceinline__ float ku_ex2_fma(float x) {
  x = fmaxf(x, -127.0f);
  const float t = x + 12582912.0f;               // 1.5 * 2^23: the sum's low mantissa bits hold round(x)
  const float f = x - (t - 12582912.0f);
  const float p = fmaf(fmaf(fmaf(0.05459282547f, f, 0.24221783876f), f, 0.69336861372f), f, 1.0f);
  return __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
}
#ifndef KU_PTMEM
#define KU_PTMEM 1   // P_j goes to tensor memory (over the scores it was computed from) and is the MMA's A operand from there
#endif
// D += A B with A in tensor memory (row i of A in lane i, two 16-bit elements per 32-bit column) and B through a shared-memory descriptor
__device__ __forceinline__ void ku_mma_ts(unsigned d_tmem, unsigned a_tmem, unsigned long long bdesc, unsigned idesc, unsigned accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
               ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
#ifndef KU_PHASES
#define KU_PHASES 0   // 1: one CTA prints the clocks its softmax thread 0 and its MMA thread spent per phase (measurement builds only)
#endif
#if KU_PHASES
#define KU_TICK(i) { long long t_; asm volatile("mov.u64 %0, %%clock64;" : "=l"(t_)); ph[i] += t_ - t_prev; t_prev = t_; }
#else
#define KU_TICK(i)
#endif
#define Q_BYTES (128 * 128 * DCH)
#define KV_BYTES (TK * 128 * DCH)
#define KV_CHUNK (TK * 128)

#if KU_TWIN == 1
extern "C" __global__ void __launch_bounds__(192, 2)
ku_attention_tc_twin(const __grid_constant__ KuTmap tmap_q, const __grid_constant__ KuTmap tmap_k, const __grid_constant__ KuTmap tmap_v, void* __restrict__ Op,
                     int* __restrict__ status) {
  extern __shared__ __align__(1024) unsigned char smem[];
  const unsigned q_s = ku_smem(smem), k_s = q_s + Q_BYTES, v_s = k_s + 2 * KV_BYTES, p_s = v_s + 2 * KV_BYTES;
  if (q_s & 1023u) {   // never seen; a misplaced tile would corrupt the MMA operands silently
    if (threadIdx.x == 0) atomicExch(status, 7);
    return;
  }
  unsigned char* p_tile = smem + Q_BYTES + 4 * KV_BYTES;
  unsigned long long* bars = (unsigned long long*)(p_tile + 128 * 128);
  unsigned long long *q_full = bars, *k_full = bars + 1, *k_empty = bars + 3, *v_full = bars + 5, *v_empty = bars + 7, *s_full = bars + 9, *s_free = bars + 11,
                     *p_ready = bars + 13, *o_full = bars + 14;
  unsigned* tmem_base_slot = (unsigned*)(bars + 15);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qb = (int)gridDim.x - 1 - (int)blockIdx.x;   // long (late) query blocks first
  const int bh = blockIdx.y;
  const int kv_blocks = (S + TK - 1) / TK;
  const int nkv = CAUSAL ? ((qb + 1) * (BQ / TK) < kv_blocks ? (qb + 1) * (BQ / TK) : kv_blocks) : kv_blocks;

  if (threadIdx.x == 0) {
    ku_mbar_init(ku_smem(q_full), 1);
    for (int i = 0; i < 2; ++i) {
      ku_mbar_init(ku_smem(&k_full[i]), 1); ku_mbar_init(ku_smem(&k_empty[i]), 1); ku_mbar_init(ku_smem(&v_full[i]), 1); ku_mbar_init(ku_smem(&v_empty[i]), 1);
      ku_mbar_init(ku_smem(&s_full[i]), 1); ku_mbar_init(ku_smem(&s_free[i]), 128);
    }
    ku_mbar_init(ku_smem(p_ready), 128); ku_mbar_init(ku_smem(o_full), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ku_smem(tmem_base_slot)), "r"(256u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = *tmem_base_slot;   // columns [0,64) and [64,128): score buffers; [128, 128+DH): O
  bool failed = false;

  if (warp == 0) {
    if (lane == 0) {  // ---- TMA producer ----
      ku_mbar_expect(ku_smem(q_full), Q_BYTES);
      for (int c = 0; c < DCH; ++c) ku_tma_3d(q_s + c * 16384, &tmap_q, c * 64, qb * BQ, bh, ku_smem(q_full));
      auto load_k = [&](int j) {   // K runs a block ahead of V (see the one-CTA kernel)
        const int st = j & 1;
        ku_wait(ku_smem(&k_empty[st]), ((j >> 1) & 1) ^ 1, failed, status);
        ku_mbar_expect(ku_smem(&k_full[st]), KV_BYTES);
        for (int c = 0; c < DCH; ++c) ku_tma_3d(k_s + st * KV_BYTES + c * KV_CHUNK, &tmap_k, c * 64, j * TK, bh, ku_smem(&k_full[st]));
      };
      if (nkv > 0) load_k(0);
      if (nkv > 1) load_k(1);
      for (int j = 0; j < nkv; ++j) {
        const int st = j & 1;
        ku_wait(ku_smem(&v_empty[st]), ((j >> 1) & 1) ^ 1, failed, status);
        ku_mbar_expect(ku_smem(&v_full[st]), KV_BYTES);
        for (int c = 0; c < DCH; ++c) ku_tma_3d(v_s + st * KV_BYTES + c * KV_CHUNK, &tmap_v, c * 64, j * TK, bh, ku_smem(&v_full[st]));
        if (j + 2 < nkv) load_k(j + 2);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {  // ---- MMA issuer ----
      auto issue_s = [&](int j) {   // S_j = Q K_j^T, 128 x 64
        const int st = j & 1;
        ku_wait(ku_smem(&k_full[st]), (j >> 1) & 1, failed, status);
#if !KU_PTMEM
        ku_wait(ku_smem(&s_free[st]), ((j >> 1) & 1) ^ 1, failed, status);
#endif
        // with P in tensor memory the buffer last held P_{j-2}: P V_{j-2} was issued before this MMA and MMAs execute in
        // issue order, and that product was only issued once every softmax thread had read S_{j-2} and stored P_{j-2}
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int kk = 0; kk < DH / 16; ++kk) {
          ku_mma(tmem_base + st * TK, ku_smem_desc(q_s + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024),
                 ku_smem_desc(k_s + st * KV_BYTES + (kk >> 2) * KV_CHUNK + (kk & 3) * 32, 16, 1024), IDESC_S, kk != 0);
        }
        ku_mma_commit(ku_smem(&s_full[st]));
        ku_mma_commit(ku_smem(&k_empty[st]));
      };
      ku_wait(ku_smem(q_full), 0, failed, status);
      if (nkv > 0) issue_s(0);
#if KU_PHASES
      long long ph[4] = {0, 0, 0, 0}, t_prev;
      asm volatile("mov.u64 %0, %%clock64;" : "=l"(t_prev));
#endif
      for (int j = 0; j < nkv; ++j) {
        if (j + 1 < nkv) issue_s(j + 1);
        KU_TICK(0)
        const int st = j & 1;
        ku_wait(ku_smem(&v_full[st]), (j >> 1) & 1, failed, status);
        KU_TICK(1)
        ku_wait(ku_smem(p_ready), j & 1, failed, status);
        KU_TICK(2)
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int kk = 0; kk < TK / 16; ++kk) {   // O += P_j V_j: P K-major over its 64 keys, V MN-major (head dimension contiguous)
          const unsigned long long bd = ku_smem_desc(v_s + st * KV_BYTES + kk * 16 * 128, KV_CHUNK, 1024);
#if KU_PTMEM
          ku_mma_ts(tmem_base + 128, tmem_base + st * TK + kk * 8, bd, IDESC_O, (j | kk) != 0);   // 16 keys = 8 columns of packed P
#else
          ku_mma(tmem_base + 128, ku_smem_desc(p_s + kk * 32, 16, 1024), bd, IDESC_O, (j | kk) != 0);
#endif
        }
        ku_mma_commit(ku_smem(o_full));
        ku_mma_commit(ku_smem(&v_empty[st]));
        KU_TICK(3)
      }
#if KU_PHASES
      if (blockIdx.x == 0 && blockIdx.y == 40)
        printf("MMA thread, %d key blocks: issue S (incl. wait K) %lld, wait V %lld, wait P %lld, issue PV %lld\n", nkv, ph[0] / nkv, ph[1] / nkv, ph[2] / nkv, ph[3] / nkv);
#endif
    }
  } else {  // ---- softmax: four warps, one thread per query row ----
    const int q4 = warp & 3;                      // the TMEM lane quarter this warp may access
    const int r = q4 * 32 + lane;                 // row of the tile == TMEM lane
    const int qrow = qb * BQ + r;
    const unsigned lane_addr = tmem_base + ((unsigned)(q4 * 32) << 16);
    float m = -KU_INF, l = 0.0f;   // reference maximum (followed lazily, see the one-CTA kernel) and the row's sum
#if KU_PHASES
    long long ph[6] = {0, 0, 0, 0, 0, 0}, t_prev;
    asm volatile("mov.u64 %0, %%clock64;" : "=l"(t_prev));
#endif
    for (int j = 0; j < nkv; ++j) {
      const int st = j & 1;
      ku_wait(ku_smem(&s_full[st]), (j >> 1) & 1, failed, status);
      KU_TICK(0)
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const bool need_mask = (CAUSAL && j * TK + TK - 1 > qb * BQ) || (j * TK + TK > S);
      float sc[TK];
      ku_tmem_ld32_nowait(lane_addr + st * TK, sc);
      ku_tmem_ld32_nowait(lane_addr + st * TK + 32, sc + 32);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
      for (int c = 0; c < TK; ++c) asm volatile("" : "+f"(sc[c]));   // the values may only be read after the wait
      KU_TICK(1)
#if !KU_PTMEM
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      ku_mbar_arrive(ku_smem(&s_free[st]));
#endif
      // masked keys at -inf, then the block maximum over four independent chains (a single chain of 64 dependent
      // maxima would leave the two warps of a scheduler waiting on latency); the scale is applied to the maximum
      // and folded into the exponent's multiply-add (SCALE_LOG2E > 0)
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < TK; ++c) {
          const int key = j * TK + c;
          if ((CAUSAL && key > qrow) || key >= S) sc[c] = -KU_INF;
        }
      }
      float b4[4] = {sc[0], sc[1], sc[2], sc[3]};
#pragma unroll
      for (int c = 4; c < TK; ++c) b4[c & 3] = fmaxf(b4[c & 3], sc[c]);
      const float bm = fmaxf(fmaxf(b4[0], b4[1]), fmaxf(b4[2], b4[3])) * SCALE_LOG2E;
      const bool grow = bm > m + 8.0f || (m == -KU_INF && bm != -KU_INF);
      const bool any_grow = __any_sync(0xffffffffu, grow);
      const float alpha = grow ? ku_ex2(m - bm) : 1.0f;
      if (grow) m = bm;
      const float nref = (m == -KU_INF) ? 0.0f : -m;
      KU_TICK(2)
      float s4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      uint4 pk[TK / 8];
#pragma unroll
      for (int c0 = 0; c0 < TK; c0 += 8) {
        float e[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const float x = fmaf(sc[c0 + c], SCALE_LOG2E, nref);
          e[c] = (c >= 8 - KU_POLY) ? ku_ex2_fma(x) : ku_ex2(x);
          s4[c & 3] += e[c];
        }
        pk[c0 >> 3].x = ku_pack2(e[0], e[1]); pk[c0 >> 3].y = ku_pack2(e[2], e[3]);
        pk[c0 >> 3].z = ku_pack2(e[4], e[5]); pk[c0 >> 3].w = ku_pack2(e[6], e[7]);
      }
      const float bs = (s4[0] + s4[1]) + (s4[2] + s4[3]);
#if KU_PHASES
      asm volatile("" :: "f"(bs), "r"(pk[0].x), "r"(pk[7].w));
#endif
      KU_TICK(3)
#if KU_PTMEM
      // P_j overwrites the scores it came from (this lane's own columns), so only a rescale of O has to wait for the
      // previous product; o_full can be at most one phase ahead of this wait because P V_j needs this thread's arrival
      if (any_grow && j > 0) {
#else
      if (j > 0) {   // the previous product must have retired before P is overwritten or O is touched
#endif
        ku_wait(ku_smem(o_full), (j - 1) & 1, failed, status);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      }
      if (any_grow) {
        if (j > 0) {
#pragma unroll 1
          for (int c0 = 0; c0 < DH; c0 += 32) {
            float v[32];
            ku_tmem_ld32(lane_addr + 128 + c0, v);
#pragma unroll
            for (int c = 0; c < 32; ++c) v[c] *= alpha;
            ku_tmem_st32(lane_addr + 128 + c0, v);
          }
        }
        l *= alpha;
      }
      l += bs;
      KU_TICK(4)
#if KU_PTMEM
      ku_tmem_st32(lane_addr + st * TK, (const float*)pk);   // 64 bf16 = 32 columns, waits for the store
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
#else
#pragma unroll
      for (int ch = 0; ch < TK / 8; ++ch) *(uint4*)(p_tile + r * 128 + ((ch ^ (r & 7)) << 4)) = pk[ch];
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
#endif
      ku_mbar_arrive(ku_smem(p_ready));
      KU_TICK(5)
    }
#if KU_PHASES
    if (blockIdx.x == 0 && blockIdx.y == 40 && threadIdx.x == 64)
      printf("softmax thread, %d key blocks: wait S %lld, load %lld, max %lld, exp+pack %lld, rescale %lld, store+arrive %lld\n", nkv, ph[0] / nkv, ph[1] / nkv,
             ph[2] / nkv, ph[3] / nkv, ph[4] / nkv, ph[5] / nkv);
#endif
    if (nkv > 0) {
      ku_wait(ku_smem(o_full), (nkv - 1) & 1, failed, status);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
    const float inv = 1.0f / l;
#pragma unroll 1
    for (int c0 = 0; c0 < DH; c0 += 32) {
      float o[32];
      if (nkv > 0) {
        ku_tmem_ld32(lane_addr + 128 + c0, o);
      } else {
#pragma unroll
        for (int c = 0; c < 32; ++c) o[c] = 0.0f;
      }
      if (qrow < S) {
        uint4* dst = (uint4*)((unsigned short*)Op + ((i64)bh * S + qrow) * DH + c0);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 w;
          w.x = ku_pack2(o[g * 8 + 0] * inv, o[g * 8 + 1] * inv); w.y = ku_pack2(o[g * 8 + 2] * inv, o[g * 8 + 3] * inv);
          w.z = ku_pack2(o[g * 8 + 4] * inv, o[g * 8 + 5] * inv); w.w = ku_pack2(o[g * 8 + 6] * inv, o[g * 8 + 7] * inv);
          dst[g] = w;
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256u) : "memory");
}
#endif  // KU_TWIN == 1

#if KU_TWIN == 2
// ---- Two query tiles per CTA -------------------------------------------------------------------------------
// One CTA per (head, 256 queries): two tiles of 128 query rows share every K_j / V_j block (128 keys), each with its
// own softmax warpgroup, score buffer and accumulator in tensor memory:
//   columns [0,128) S_0 (P_0 packed over its first 64 columns), [128,256) S_1 / P_1, [256,384) O_0, [384,512) O_1.
// Each tile has its own MMA-issuing thread (warps 1 and 10), P V of a block followed at once by the tile's next scores:
//   ... P_t V_j, S_t = Q_t K_{j+1}^T, P_t V_{j+1}, ...
// so that one tile's exponentials run while the tensor core works for the other tile. A thread's MMAs execute in
// issue order, which is what lets S_t(j+1) overwrite the P_t(j) that the product issued just before it reads.
// Shared-memory traffic per 128 x 128 block (the bound of the smaller kernels, which re-read Q and P from shared
// memory and load K / V per tile): Q K^T 64 KB + V 32 KB + half a K / V load 32 KB = 128 KB.
// Shared memory (DH = 128): Q 2 x 32 KB, a K ring of NKS and a V ring of NVS stages of 32 KB (2 + 2: 192 KB) + barriers,
// all dynamic. The load into a stage is requested when the MMAs that read its previous content have retired.
#ifndef NKS
#define NKS 2
#endif
#ifndef NVS
#define NVS 2
#endif
#ifndef KU_ISSUERS
#define KU_ISSUERS 1   // 2: a second MMA-issuing warp (warp 10) for tile 1
#endif
#ifndef KU_TURNS
#define KU_TURNS (KU_ISSUERS == 2)   // the tiles' warpgroups take turns at the exponentials
#endif
#undef Q_BYTES
#define Q_BYTES TILE_BYTES

__device__ __forceinline__ void ku_tmem_st32_nowait(unsigned taddr, const unsigned* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, "
      "%24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]),
        "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]),
        "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

extern "C" __global__ void __launch_bounds__(320 + 32 * (KU_ISSUERS - 1), 1)
ku_attention_tc_duo(const __grid_constant__ KuTmap tmap_q, const __grid_constant__ KuTmap tmap_k, const __grid_constant__ KuTmap tmap_v, void* __restrict__ Op,
                    int* __restrict__ status) {
  extern __shared__ __align__(1024) unsigned char smem[];
  const unsigned q_s = ku_smem(smem), k_s = q_s + 2 * Q_BYTES, v_s = k_s + NKS * TILE_BYTES;
  if (q_s & 1023u) {   // never seen; a misplaced tile would corrupt the MMA operands silently
    if (threadIdx.x == 0) atomicExch(status, 7);
    return;
  }
  unsigned long long* bars = (unsigned long long*)(smem + 2 * Q_BYTES + (NKS + NVS) * TILE_BYTES);
  unsigned long long *q_full = bars, *k_full = bars + 1, *k_empty = k_full + NKS, *v_full = k_empty + NKS, *v_empty = v_full + NVS, *s_full = v_empty + NVS,
                     *p_ready = s_full + 2, *o_full = p_ready + 2;
  unsigned* tmem_base_slot = (unsigned*)(o_full + 2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qp = (int)gridDim.x - 1 - (int)blockIdx.x;   // pair of query blocks (2 qp, 2 qp + 1); long (late) pairs first
  const int bh = blockIdx.y;
  const int kv_blocks = (S + BKV - 1) / BKV;
  // key blocks per tile: under the causal mask tile 0 stops one block before tile 1
  const int n0 = CAUSAL ? ((2 * qp + 1) < kv_blocks ? (2 * qp + 1) : kv_blocks) : kv_blocks;
  const int n1 = CAUSAL ? ((2 * qp + 2) < kv_blocks ? (2 * qp + 2) : kv_blocks) : kv_blocks;

  if (threadIdx.x == 0) {
    ku_mbar_init(ku_smem(q_full), 1);
    for (int i = 0; i < NKS; ++i) { ku_mbar_init(ku_smem(&k_full[i]), 1); ku_mbar_init(ku_smem(&k_empty[i]), KU_ISSUERS); }   // released by every MMA issuer
    for (int i = 0; i < NVS; ++i) { ku_mbar_init(ku_smem(&v_full[i]), 1); ku_mbar_init(ku_smem(&v_empty[i]), KU_ISSUERS); }
    for (int i = 0; i < 2; ++i) { ku_mbar_init(ku_smem(&s_full[i]), 1); ku_mbar_init(ku_smem(&p_ready[i]), 128); ku_mbar_init(ku_smem(&o_full[i]), 1); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ku_smem(tmem_base_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = *tmem_base_slot;
  bool failed = false;

  if (warp == 0) {
    if (lane == 0) {  // ---- TMA producer: both Q tiles once, then K_j / V_j for the longer tile's blocks ----
      ku_mbar_expect(ku_smem(q_full), 2 * Q_BYTES);
      for (int t = 0; t < 2; ++t)
        for (int c = 0; c < DCH; ++c) ku_tma_3d(q_s + t * Q_BYTES + c * 16384, &tmap_q, c * 64, (2 * qp + t) * BQ, bh, ku_smem(q_full));
      auto load_k = [&](int j) {
        const int st = j % NKS;
        ku_wait(ku_smem(&k_empty[st]), ((j / NKS) & 1) ^ 1, failed, status);
        ku_mbar_expect(ku_smem(&k_full[st]), TILE_BYTES);
        for (int c = 0; c < DCH; ++c) ku_tma_3d(k_s + st * TILE_BYTES + c * 16384, &tmap_k, c * 64, j * BKV, bh, ku_smem(&k_full[st]));
      };
      auto load_v = [&](int j) {
        const int st = j % NVS;
        ku_wait(ku_smem(&v_empty[st]), ((j / NVS) & 1) ^ 1, failed, status);
        ku_mbar_expect(ku_smem(&v_full[st]), TILE_BYTES);
        for (int c = 0; c < DCH; ++c) ku_tma_3d(v_s + st * TILE_BYTES + c * 16384, &tmap_v, c * 64, j * BKV, bh, ku_smem(&v_full[st]));
      };
      // K_0 first (the first scores need it), then the rings are filled; after that block j's turn requests K_{j+NKS}
      // (free once both tiles' scores of block j have retired) and V_{j+NVS-1} (free since the products of block j-1)
      load_k(0);
      for (int j = 0; j < NVS - 1 && j < n1; ++j) load_v(j);
      for (int j = 1; j < NKS && j < n1; ++j) load_k(j);
      for (int j = 0; j < n1; ++j) {
        if (j + NKS < n1) load_k(j + NKS);
        if (j + NVS - 1 < n1) load_v(j + NVS - 1);
      }
    }
#if KU_ISSUERS == 2
  } else if (warp == 1 || warp == 10) {
    if (lane == 0) {  // ---- MMA issuers: warp 1 for tile 0, warp 10 for tile 1 ----
      // One thread sustained an MMA every ~75 clocks, against the 64 clocks a 128 x 128 x 16 MMA executes in, and the tensor
      // pipe idled between them; two issuing threads halve the instructions each has to prepare. The tiles' MMAs are
      // independent (own score buffer and accumulator), every ordering the algorithm needs is inside one tile.
      const int t = warp == 1 ? 0 : 1;
      const int nt = t ? n1 : n0;
      auto issue_s = [&](int j) {   // S_t = Q_t K_j^T
        const int st = j % NKS;
        ku_wait(ku_smem(&k_full[st]), (j / NKS) & 1, failed, status);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int kk = 0; kk < DH / 16; ++kk) {
          const unsigned off = (kk >> 2) * 16384 + (kk & 3) * 32;
          ku_mma(tmem_base + t * 128, ku_smem_desc(q_s + t * Q_BYTES + off, 16, 1024), ku_smem_desc(k_s + st * TILE_BYTES + off, 16, 1024), IDESC_S, kk != 0);
        }
        ku_mma_commit(ku_smem(&s_full[t]));
      };
      auto issue_pv = [&](int j) {   // O_t += P_t V_j: P_t from tensor memory (16 keys = 8 columns), V MN-major from shared memory
        const int st = j % NVS;
        ku_wait(ku_smem(&v_full[st]), (j / NVS) & 1, failed, status);
        ku_wait(ku_smem(&p_ready[t]), j & 1, failed, status);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk)
          ku_mma_ts(tmem_base + 256 + t * 128, tmem_base + t * 128 + kk * 8, ku_smem_desc(v_s + st * TILE_BYTES + kk * 16 * 128, 16384, 1024), IDESC_O, (j | kk) != 0);
        ku_mma_commit(ku_smem(&o_full[t]));
      };
      ku_wait(ku_smem(q_full), 0, failed, status);
      issue_s(0);
      ku_mma_commit(ku_smem(&k_empty[0]));
      // a stage is released by both issuers, also for a block the shorter tile does not compute (a commit with nothing
      // outstanding arrives at once)
      for (int j = 0; j < n1; ++j) {
        if (j < nt) issue_pv(j);
        ku_mma_commit(ku_smem(&v_empty[j % NVS]));
        if (j + 1 < n1) {
          if (j + 1 < nt) issue_s(j + 1);
          ku_mma_commit(ku_smem(&k_empty[(j + 1) % NKS]));
        }
      }
    }
#else
  } else if (warp == 1) {
    if (lane == 0) {  // ---- MMA issuer ----
#if KU_PHASES
      long long ph[8] = {0, 0, 0, 0, 0, 0, 0, 0}, t_prev = 0;
#endif
      auto issue_s = [&](int t, int j) {   // S_t = Q_t K_j^T (K_j has been waited for by the caller)
        const int st = j % NKS;
#pragma unroll
        for (int kk = 0; kk < DH / 16; ++kk) {
          const unsigned off = (kk >> 2) * 16384 + (kk & 3) * 32;
          ku_mma(tmem_base + t * 128, ku_smem_desc(q_s + t * Q_BYTES + off, 16, 1024), ku_smem_desc(k_s + st * TILE_BYTES + off, 16, 1024), IDESC_S, kk != 0);
        }
        ku_mma_commit(ku_smem(&s_full[t]));
      };
      auto issue_pv = [&](int t, int j) {   // O_t += P_t V_j: P_t from tensor memory (16 keys = 8 columns), V MN-major from shared memory
        const int st = j % NVS;
        ku_wait(ku_smem(&p_ready[t]), j & 1, failed, status);
        KU_TICK(1 + 4 * t)
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk)
          ku_mma_ts(tmem_base + 256 + t * 128, tmem_base + t * 128 + kk * 8, ku_smem_desc(v_s + st * TILE_BYTES + kk * 16 * 128, 16384, 1024), IDESC_O, (j | kk) != 0);
        ku_mma_commit(ku_smem(&o_full[t]));
      };
      ku_wait(ku_smem(q_full), 0, failed, status);
      ku_wait(ku_smem(&k_full[0]), 0, failed, status);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      issue_s(0, 0);
      issue_s(1, 0);
      ku_mma_commit(ku_smem(&k_empty[0]));
#if KU_PHASES
      asm volatile("mov.u64 %0, %%clock64;" : "=l"(t_prev));
      for (int i = 0; i < 8; ++i) ph[i] = 0;
#endif
      for (int j = 0; j < n1; ++j) {
        const int st = j % NVS, nx = (j + 1) % NKS;
#if KU_PHASES
        if (j == 4) { for (int i = 0; i < 8; ++i) ph[i] = 0; asm volatile("mov.u64 %0, %%clock64;" : "=l"(t_prev)); }
#endif
        ku_wait(ku_smem(&v_full[st]), (j / NVS) & 1, failed, status);
        KU_TICK(0)
        if (j < n0) issue_pv(0, j);
        KU_TICK(2)
        if (j + 1 < n1) ku_wait(ku_smem(&k_full[nx]), ((j + 1) / NKS) & 1, failed, status);
        KU_TICK(3)
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (j + 1 < n0) issue_s(0, j + 1);
        KU_TICK(4)
        issue_pv(1, j);
        ku_mma_commit(ku_smem(&v_empty[st]));
        KU_TICK(6)
        if (j + 1 < n1) {
          issue_s(1, j + 1);
          ku_mma_commit(ku_smem(&k_empty[nx]));
        }
        KU_TICK(7)
      }
#if KU_PHASES
      if (blockIdx.x == 0 && blockIdx.y == 40)
        printf("MMA thread, %d key blocks (from the fifth on): wait V %lld, wait P0 %lld, issue PV0 %lld, wait K %lld, issue S0 %lld, wait P1 %lld, issue PV1 %lld, issue S1 %lld\n", n1,
               ph[0] / (n1 - 4), ph[1] / (n1 - 4), ph[2] / (n1 - 4), ph[3] / (n1 - 4), ph[4] / (n1 - 4), ph[5] / (n1 - 4), ph[6] / (n1 - 4), ph[7] / (n1 - 4));
#endif
    }
#endif
  } else {  // ---- softmax: a warpgroup per tile, one thread per query row ----
    const int t = (warp - 2) >> 2;                // the tile
    const int q4 = warp & 3;                      // the TMEM lane quarter this warp may access
    const int r = q4 * 32 + lane;                 // row of the tile == TMEM lane
    const int qb = 2 * qp + t;
    const int qrow = qb * BQ + r;
    const int nkv = t ? n1 : n0;
    const unsigned s_addr = tmem_base + ((unsigned)(q4 * 32) << 16) + t * 128;
    const unsigned o_addr = tmem_base + ((unsigned)(q4 * 32) << 16) + 256 + t * 128;
    float m = -KU_INF, l = 0.0f;   // reference maximum (followed lazily, see the one-CTA kernel) and the row's sum
#if KU_PHASES
    long long ph[6] = {0, 0, 0, 0, 0, 0}, t_prev;
    asm volatile("mov.u64 %0, %%clock64;" : "=l"(t_prev));
#endif
#if KU_TURNS == 1
    if (t == 1) asm volatile("bar.arrive 1, 256;" ::: "memory");   // tile 0 goes first (n0 >= 1)
#endif
    for (int j = 0; j < nkv; ++j) {
#if KU_PHASES
      if (j == 4) { for (int i = 0; i < 6; ++i) ph[i] = 0; asm volatile("mov.u64 %0, %%clock64;" : "=l"(t_prev)); }
#endif
      ku_wait(ku_smem(&s_full[t]), j & 1, failed, status);
      KU_TICK(0)
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const bool need_mask = (CAUSAL && j == qb) || (j * BKV + BKV > S);
      float sc[BKV];
#pragma unroll
      for (int c0 = 0; c0 < BKV; c0 += 32) ku_tmem_ld32_nowait(s_addr + c0, sc + c0);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
      for (int c = 0; c < BKV; ++c) asm volatile("" : "+f"(sc[c]));   // the values may only be read after the wait
      KU_TICK(1)
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < BKV; ++c) {
          const int key = j * BKV + c;
          if ((CAUSAL && key > qrow) || key >= S) sc[c] = -KU_INF;
        }
      }
      float b4[4] = {sc[0], sc[1], sc[2], sc[3]};   // four independent chains
#pragma unroll
      for (int c = 4; c < BKV; ++c) b4[c & 3] = fmaxf(b4[c & 3], sc[c]);
      const float bm = fmaxf(fmaxf(b4[0], b4[1]), fmaxf(b4[2], b4[3])) * SCALE_LOG2E;   // SCALE_LOG2E > 0
      const bool grow = bm > m + 8.0f || (m == -KU_INF && bm != -KU_INF);
      const bool any_grow = __any_sync(0xffffffffu, grow);
      const float alpha = grow ? ku_ex2(m - bm) : 1.0f;
      if (grow) m = bm;
      const float nref = (m == -KU_INF) ? 0.0f : -m;
      KU_TICK(2)
      // The tiles take turns at the exponentials (named barriers 1 and 2: one warpgroup arrives, the other waits):
      // tile 0 block j, tile 1 block j, tile 0 block j+1, ... Left alone both warpgroups reach this phase together,
      // share the special-function unit for twice as long and then leave it idle together while their MMAs run.
#if KU_TURNS == 1
      if (t == 0) asm volatile("bar.sync 1, 256;" ::: "memory");
      else if (j < n0) asm volatile("bar.sync 2, 256;" ::: "memory");
#elif KU_TURNS == 2   // only the first block is ordered: tile 1 starts one exponential phase behind tile 0, then both run free
      if (t == 1 && j == 0) asm volatile("bar.sync 2, 256;" ::: "memory");
#endif
      float s4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      // the probabilities, 64 keys (32 packed columns) at a time, over the first half of the scores they came from
      // (all of this lane's scores are in registers by now)
#pragma unroll
      for (int h = 0; h < BKV / 64; ++h) {
        unsigned pk[32];
#pragma unroll
        for (int c = 0; c < 64; c += 2) {
          const float x0 = fmaf(sc[h * 64 + c], SCALE_LOG2E, nref), x1 = fmaf(sc[h * 64 + c + 1], SCALE_LOG2E, nref);
          const float e0 = ((c & 7) >= 8 - KU_POLY) ? ku_ex2_fma(x0) : ku_ex2(x0);
          const float e1 = (((c + 1) & 7) >= 8 - KU_POLY) ? ku_ex2_fma(x1) : ku_ex2(x1);
          s4[(c >> 1) & 3] += e0 + e1;
          pk[c >> 1] = ku_pack2(e0, e1);
        }
        ku_tmem_st32_nowait(s_addr + h * 32, pk);
      }
#if KU_TURNS == 1
      if (t == 0) asm volatile("bar.arrive 2, 256;" ::: "memory");
      else if (j + 1 < n0) asm volatile("bar.arrive 1, 256;" ::: "memory");
#elif KU_TURNS == 2
      if (t == 0 && j == 0) asm volatile("bar.arrive 2, 256;" ::: "memory");
#endif
      KU_TICK(3)
      // only a rescale of O has to wait for the tile's previous product (its score block was issued after that
      // product, so the wait is over by now; o_full can be at most one phase ahead of it)
      if (any_grow) {
        if (j > 0) {
          ku_wait(ku_smem(&o_full[t]), (j - 1) & 1, failed, status);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
          for (int c0 = 0; c0 < DH; c0 += 32) {
            float v[32];
            ku_tmem_ld32(o_addr + c0, v);
#pragma unroll
            for (int c = 0; c < 32; ++c) v[c] *= alpha;
            ku_tmem_st32(o_addr + c0, v);
          }
        }
        l *= alpha;
      }
      l += (s4[0] + s4[1]) + (s4[2] + s4[3]);
      KU_TICK(4)
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      ku_mbar_arrive(ku_smem(&p_ready[t]));
      KU_TICK(5)
    }
#if KU_PHASES
    if (blockIdx.x == 0 && blockIdx.y == 40 && lane == 0 && q4 == 2)
      printf("softmax thread of tile %d, %d key blocks (from the fifth on): wait S %lld, load %lld, max %lld, exp+pack+store %lld, rescale %lld, wait store+arrive %lld\n", t, nkv,
             ph[0] / (nkv - 4), ph[1] / (nkv - 4), ph[2] / (nkv - 4), ph[3] / (nkv - 4), ph[4] / (nkv - 4), ph[5] / (nkv - 4));
#endif
    if (nkv > 0) {
      ku_wait(ku_smem(&o_full[t]), (nkv - 1) & 1, failed, status);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
    const float inv = 1.0f / l;
#pragma unroll 1
    for (int c0 = 0; c0 < DH; c0 += 32) {
      float o[32];
      if (nkv > 0) {
        ku_tmem_ld32(o_addr + c0, o);
      } else {
#pragma unroll
        for (int c = 0; c < 32; ++c) o[c] = 0.0f;
      }
      if (qrow < S) {
        uint4* dst = (uint4*)((unsigned short*)Op + ((i64)bh * S + qrow) * DH + c0);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 w;
          w.x = ku_pack2(o[g * 8 + 0] * inv, o[g * 8 + 1] * inv); w.y = ku_pack2(o[g * 8 + 2] * inv, o[g * 8 + 3] * inv);
          w.z = ku_pack2(o[g * 8 + 4] * inv, o[g * 8 + 5] * inv); w.w = ku_pack2(o[g * 8 + 6] * inv, o[g * 8 + 7] * inv);
          dst[g] = w;
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
}
#endif  // KU_TWIN == 2
#endif  // KU_TWIN

// Fused scaled-dot-product attention for sm_100a (Op::Sdpa, kurumi_core/src/graph/op.rs:55-58):
// out = softmax(q k^T / sqrt(dh) [+ causal mask]) v over the trailing [S, DH] of [BH, S, DH] bf16 / f16
// tensors, online softmax, no S x S buffer. The math is the interpreter's decomposition
// (kurumi_core/src/interp/nn.rs:125-172): scale = 1/sqrt(dh) as f32, key j > query i masked to -inf,
// softmax in f32; results stay within rel 2e-2 of the f64 run.
//
// One CTA per (head, 256 queries): two tiles of 128 query rows share every K_j / V_j block of 128 keys.
//   warp 0      TMA producer: both Q tiles once, then K_j / V_j (cp.async.bulk.tensor, SWIZZLE_128B, no multicast)
//   warp 1      tcgen05.mma issuer for both tiles: ... P_0 V_j, S_0 = Q_0 K_{j+1}^T, P_1 V_j, S_1 = Q_1 K_{j+1}^T ...
//   warps 2..9  softmax, a warpgroup per tile, one thread per query row: tcgen05.ld the scores, maximum / sum in the
//               log2 domain, P_j packed to bf16 over the first half of the score columns it came from (the second
//               MMA reads its A operand from tensor memory). O accumulates in tensor memory across key blocks; the
//               threads rescale it (tcgen05.ld / st) only when a row's maximum has grown by more than 2^8 since the
//               scale it was accumulated with
// Tensor memory: columns [0,128) S_0 / P_0, [128,256) S_1 / P_1, [256,384) O_0, [384,512) O_1. A thread's MMAs execute in
// issue order, which is what lets S_t(j+1) overwrite the P_t(j) that the product issued just before it reads.
// Shared memory (DH = 128): Q 2 x 32 KB, a K ring of NKS and a V ring of NVS stages of 32 KB (2 + 2: 192 KB) + barriers,
// all dynamic. The load into a stage is requested when the MMAs that read its previous content have retired.
// Causal: key blocks above the diagonal are never loaded (tile 0 stops one block before tile 1); the diagonal block is
// masked per element. Every mbarrier wait is bounded (status word + sticky failure), tensor memory is always released.
//
// Spliced in by the host: BH, S, DH (64 or 128), CAUSAL, SCALE_LOG2E (scale * log2 e as a positive float literal),
// IDESC_S, IDESC_O, KU_IS_BF16, NKS, NVS.
#define BQ 128
#define BKV 128
#define DCH (DH / 64)                    // 64-element (128-byte) chunks along the head dimension
#define TILE_BYTES (128 * 128 * DCH)     // one [128 rows][DH] bf16 tile: DCH chunks of [128][128 bytes]
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


// D += A B with A in tensor memory (row i of A in lane i, two 16-bit elements per 32-bit column) and B through a shared-memory descriptor
__device__ __forceinline__ void ku_mma_ts(unsigned d_tmem, unsigned a_tmem, unsigned long long bdesc, unsigned idesc, unsigned accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
               ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
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

extern "C" __global__ void __launch_bounds__(320, 1)
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
    for (int i = 0; i < NKS; ++i) { ku_mbar_init(ku_smem(&k_full[i]), 1); ku_mbar_init(ku_smem(&k_empty[i]), 1); }
    for (int i = 0; i < NVS; ++i) { ku_mbar_init(ku_smem(&v_full[i]), 1); ku_mbar_init(ku_smem(&v_empty[i]), 1); }
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
        if (!ku_wait(ku_smem(&k_empty[st]), ((j / NKS) & 1) ^ 1, failed, status)) return;   // after a failed wait no copy is started that nothing would wait for
        ku_mbar_expect(ku_smem(&k_full[st]), TILE_BYTES);
        for (int c = 0; c < DCH; ++c) ku_tma_3d(k_s + st * TILE_BYTES + c * 16384, &tmap_k, c * 64, j * BKV, bh, ku_smem(&k_full[st]));
      };
      auto load_v = [&](int j) {
        const int st = j % NVS;
        if (!ku_wait(ku_smem(&v_empty[st]), ((j / NVS) & 1) ^ 1, failed, status)) return;
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
  } else if (warp == 1) {
    if (lane == 0) {  // ---- MMA issuer ----
      // A thread that issues alone runs a handful of clocks per instruction: the descriptors are built once per tile and
      // stepped by constants (the start-address field counts 16-byte units and never carries out of its 14 bits here),
      // so that an MMA costs its issuer two additions, not two descriptor constructions.
      const unsigned long long qd0 = ku_smem_desc(q_s, 16, 1024), qd1 = ku_smem_desc(q_s + Q_BYTES, 16, 1024);
      auto issue_s = [&](int t, int j) {   // S_t = Q_t K_j^T (K_j has been waited for by the caller)
        const int st = j % NKS;
        const unsigned long long qd = t ? qd1 : qd0, kd = ku_smem_desc(k_s + st * TILE_BYTES, 16, 1024);
        const unsigned d = tmem_base + t * 128;
#pragma unroll
        for (int kk = 0; kk < DH / 16; ++kk) {
          const unsigned long long off = (unsigned long long)(((kk >> 2) * 16384 + (kk & 3) * 32) >> 4);
          ku_mma(d, qd + off, kd + off, IDESC_S, kk != 0);
        }
        ku_mma_commit(ku_smem(&s_full[t]));
      };
      auto issue_pv = [&](int t, int j) {   // O_t += P_t V_j: P_t from tensor memory (16 keys = 8 columns), V MN-major from shared memory
        const int st = j % NVS;
        if (!ku_wait(ku_smem(&p_ready[t]), j & 1, failed, status)) return;   // no instruction is issued on operands that may not be there
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned long long vd = ku_smem_desc(v_s + st * TILE_BYTES, 16384, 1024);
        const unsigned d = tmem_base + 256 + t * 128, a = tmem_base + t * 128;
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk)
          ku_mma_ts(d, a + kk * 8, vd + (unsigned long long)((kk * 16 * 128) >> 4), IDESC_O, (j | kk) != 0);
        ku_mma_commit(ku_smem(&o_full[t]));
      };
      ku_wait(ku_smem(q_full), 0, failed, status);
      ku_wait(ku_smem(&k_full[0]), 0, failed, status);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      issue_s(0, 0);
      issue_s(1, 0);
      ku_mma_commit(ku_smem(&k_empty[0]));
      for (int j = 0; j < n1; ++j) {
        const int st = j % NVS, nx = (j + 1) % NKS;
        ku_wait(ku_smem(&v_full[st]), (j / NVS) & 1, failed, status);
        if (j < n0) issue_pv(0, j);
        if (j + 1 < n1) ku_wait(ku_smem(&k_full[nx]), ((j + 1) / NKS) & 1, failed, status);
        if (failed) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (j + 1 < n0) issue_s(0, j + 1);
        issue_pv(1, j);
        ku_mma_commit(ku_smem(&v_empty[st]));
        if (j + 1 < n1) {
          issue_s(1, j + 1);
          ku_mma_commit(ku_smem(&k_empty[nx]));
        }
      }
    }
  } else {  // ---- softmax: a warpgroup per tile, one thread per query row ----
    const int t = (warp - 2) >> 2;                // the tile
    const int q4 = warp & 3;                      // the TMEM lane quarter this warp may access
    const int r = q4 * 32 + lane;                 // row of the tile == TMEM lane
    const int qb = 2 * qp + t;
    const int qrow = qb * BQ + r;
    const int nkv = t ? n1 : n0;
    const unsigned s_addr = tmem_base + ((unsigned)(q4 * 32) << 16) + t * 128;
    const unsigned o_addr = tmem_base + ((unsigned)(q4 * 32) << 16) + 256 + t * 128;
    float m = -KU_INF, l = 0.0f;   // reference maximum (followed lazily: it moves only when the block maximum exceeds it by more than 2^8) and the row's sum
    for (int j = 0; j < nkv; ++j) {
      ku_wait(ku_smem(&s_full[t]), j & 1, failed, status);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const bool need_mask = (CAUSAL && j == qb) || (j * BKV + BKV > S);
      float sc[BKV];
#pragma unroll
      for (int c0 = 0; c0 < BKV; c0 += 32) ku_tmem_ld32_nowait(s_addr + c0, sc + c0);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
      for (int c = 0; c < BKV; ++c) asm volatile("" : "+f"(sc[c]));   // the values may only be read after the wait
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
      float s4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      // the probabilities, 64 keys (32 packed columns) at a time, over the first half of the scores they came from
      // (all of this lane's scores are in registers by now)
#pragma unroll
      for (int h = 0; h < BKV / 64; ++h) {
        unsigned pk[32];
#pragma unroll
        for (int c = 0; c < 64; c += 2) {
          const float x0 = fmaf(sc[h * 64 + c], SCALE_LOG2E, nref), x1 = fmaf(sc[h * 64 + c + 1], SCALE_LOG2E, nref);
          const float e0 = ku_ex2(x0), e1 = ku_ex2(x1);
          s4[(c >> 1) & 3] += e0 + e1;
          pk[c >> 1] = ku_pack2(e0, e1);
        }
        ku_tmem_st32_nowait(s_addr + h * 32, pk);
      }
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
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      ku_mbar_arrive(ku_smem(&p_ready[t]));
    }
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

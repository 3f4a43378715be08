// Tensor-core contraction for sm_100a on PAIRS of SMs: C[b, m, n] = epilogue(round(sum_k A[b, m, k] * B[b, k, n])).
//
// The same pipeline as gemm_tc.cuh (TMA ring -> tcgen05.mma -> TMEM -> fused epilogue), but a cluster of
// two CTAs works on one 256 x BN output tile with tcgen05.mma.cta_group::2: CTA r of the pair stages
// rows [r*128, r*128+128) of the A tile and columns [r*BN/2, (r+1)*BN/2) of the B tile in its own shared
// memory, the MMAs issued by the leader (rank 0) read both halves, and each CTA's tensor memory receives
// its 128 rows of the accumulator. Per k-block a CTA therefore loads (128 + BN/2) rows instead of
// (128 + BN): two thirds of the shared-memory fill per FLOP at BN = 256, and the smaller stage makes the
// ring six deep instead of four.
//   warp 0      one thread issues this CTA's TMA loads (cta_group::2 form, no multicast); they complete on
//               the LEADER's full barrier, which the leader arms with the bytes of both halves
//   warp 1      allocates tensor memory (both CTAs, cta_group::2); in the leader one thread issues the MMAs
//               and commits them to the stage's empty barrier / the accumulator's full barrier of BOTH CTAs
//   warps 2..9  epilogue of this CTA's 128 rows; they release the accumulator on the leader's barrier
// Every mbarrier wait is bounded; a role that gives up raises *status, stops waiting and runs to the end,
// so both CTAs still meet at the closing cluster barrier and tensor memory is released.
//
// Spliced in by the host: M, N, K, BATCH, BM (=128, rows per CTA), BN, BKB (=128 bytes of K per stage),
// ESIZE, STAGES, A_MN, B_MN, IDESC (M = 256), TILES_M (blocks of 256 rows), TILES_N, KU_ROUND(x) and
//   ku_out_t ku_epilogue(float acc, i64 b, i64 m, i64 n KU_EPI_PARAMS).
#define BNH (BN / 2)                     // B-tile columns staged by one CTA
#define BK (BKB / ESIZE)                 // K elements per stage
#define A_STAGE_BYTES (BM * BKB)
#define B_STAGE_BYTES (BNH * BKB)
#define STAGE_BYTES (A_STAGE_BYTES + B_STAGE_BYTES)
#define KBLOCKS ((K + BK - 1) / BK)
#define SPIN_LIMIT (1u << 24)
#define NEPI 8                           // epilogue warps: two per tensor-memory lane quarter, each taking half of the columns

struct alignas(64) KuTmap { unsigned long long opaque[16]; };
template <int BYTES> struct KuBits { typedef unsigned char type; };
template <> struct KuBits<2> { typedef unsigned short type; };
template <> struct KuBits<4> { typedef unsigned type; };

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
// bounded wait: returns false (and raises the status word once) when the barrier never flips
__device__ __forceinline__ bool ku_wait(unsigned a, unsigned parity, bool& failed, int* status) {
  if (failed) return false;
  unsigned spins = 0;
  while (!ku_mbar_try(a, parity)) {
    ++spins;
    if ((spins & 4095u) == 0 && *(volatile int*)status != 0) { failed = true; return false; }  // another role already gave up
    if (spins > SPIN_LIMIT) { failed = true; atomicExch(status, 2); return false; }
  }
  return true;
}
__device__ __forceinline__ void ku_tma_3d(unsigned dst, const KuTmap* map, int x, int y, int z, unsigned mbar) {
  asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(mbar) : "memory");
}
// shared-memory matrix descriptor, SWIZZLE_128B, version 1; offsets in bytes
__device__ __forceinline__ unsigned long long ku_smem_desc(unsigned addr, unsigned lbo, unsigned sbo) {
  return (unsigned long long)((addr & 0x3FFFFu) >> 4) | ((unsigned long long)(lbo >> 4) << 16) | ((unsigned long long)(sbo >> 4) << 32) |
         (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void ku_mma(unsigned d_tmem, unsigned long long adesc, unsigned long long bdesc, unsigned idesc, unsigned accumulate) {
#if ESIZE == 1
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
#else
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
#endif
}
// arrives on the barrier at this shared-memory offset in BOTH CTAs of the pair once the MMAs issued so far retire
__device__ __forceinline__ void ku_mma_commit(unsigned mbar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(mbar), "h"((unsigned short)3) : "memory");
}
__device__ __forceinline__ unsigned ku_cluster_rank() { unsigned r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ unsigned ku_mapa(unsigned a, unsigned rank) { unsigned ra; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(a), "r"(rank)); return ra; }
__device__ __forceinline__ void ku_mbar_arrive_remote(unsigned remote) { asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory"); }
__device__ __forceinline__ void ku_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void ku_tmem_ld32(unsigned taddr, float (&v)[32]) {
  unsigned r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, "
      "%23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
        "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
        "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
}

// tile index -> (batch, block of 256 rows, column block): groups of 8 row blocks, column-major inside a group
__device__ __forceinline__ void ku_tile_coords(int t, int& b, int& mb, int& nb) {
  const int per_batch = TILES_M * TILES_N;
  b = t / per_batch;
  const int r = t - b * per_batch;
  const int group = r / (8 * TILES_N), in_group = r - group * 8 * TILES_N;
  const int rows = (TILES_M - group * 8) < 8 ? (TILES_M - group * 8) : 8;
  mb = group * 8 + in_group % rows;
  nb = in_group / rows;
}

extern "C" __global__ void __launch_bounds__(64 + 32 * NEPI, 1)
ku_gemm_tc2(const __grid_constant__ KuTmap tmap_a, const __grid_constant__ KuTmap tmap_b, void* __restrict__ Cp, int* __restrict__ status KU_EPI_PARAMS) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long full_bar[STAGES], empty_bar[STAGES], tmem_full[2], tmem_empty[2];
  __shared__ unsigned tmem_base_slot;
  unsigned char* smem = smem_raw + ((1024u - (ku_smem(smem_raw) & 1023u)) & 1023u);  // swizzle atoms need 1024-byte alignment
  const unsigned smem_s = ku_smem(smem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned rank = ku_cluster_rank();   // 0 = leader of the pair
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int total_tiles = BATCH * TILES_M * TILES_N;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { ku_mbar_init(ku_smem(&full_bar[s]), 1); ku_mbar_init(ku_smem(&empty_bar[s]), 1); }
    for (int a = 0; a < 2; ++a) { ku_mbar_init(ku_smem(&tmem_full[a]), 1); ku_mbar_init(ku_smem(&tmem_empty[a]), 2 * 32 * NEPI); }  // the epilogue threads of both CTAs
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // 512 columns in each CTA: two BN-wide f32 accumulators of this CTA's 128 rows
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ku_smem(&tmem_base_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  ku_cluster_sync();   // both CTAs' barriers exist before either signals the other
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = tmem_base_slot;
  bool failed = false;

  if (warp == 0) {
    if (lane == 0) {  // ---- TMA producer (both CTAs) ----
      int it = 0;
      for (int t = pair; t < total_tiles && !failed; t += npairs) {
        int b, mb, nb;
        ku_tile_coords(t, b, mb, nb);
        const int row0 = mb * 256 + (int)rank * BM, col0 = nb * BN + (int)rank * BNH;
        for (int kb = 0; kb < KBLOCKS; ++kb, ++it) {
          const int s = it % STAGES;
          const unsigned ph = (it / STAGES) & 1;
          if (!ku_wait(ku_smem(&empty_bar[s]), ph ^ 1, failed, status)) break;  // first pass over the ring: passes at once; after a failed wait no copy is started that nothing would wait for
          const unsigned fb = ku_mapa(ku_smem(&full_bar[s]), 0);    // the leader's barrier collects both halves
          if (rank == 0) ku_mbar_expect(ku_smem(&full_bar[s]), 2 * STAGE_BYTES);
          const unsigned sa = smem_s + s * STAGE_BYTES, sb = sa + A_STAGE_BYTES;
#if A_MN
          for (int c = 0; c < BM * ESIZE / 128; ++c) ku_tma_3d(sa + c * BK * 128, &tmap_a, row0 + c * (128 / ESIZE), kb * BK, b, fb);
#else
          ku_tma_3d(sa, &tmap_a, kb * BK, row0, b, fb);
#endif
#if B_MN
          for (int c = 0; c < BNH * ESIZE / 128; ++c) ku_tma_3d(sb + c * BK * 128, &tmap_b, col0 + c * (128 / ESIZE), kb * BK, b, fb);
#else
          ku_tma_3d(sb, &tmap_b, kb * BK, col0, b, fb);
#endif
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {  // ---- MMA issuer (leader only) ----
      int it = 0, local = 0;
      for (int t = pair; t < total_tiles && !failed; t += npairs, ++local) {
        const int acc = local & 1;
        ku_wait(ku_smem(&tmem_empty[acc]), ((local >> 1) & 1) ^ 1, failed, status);  // both epilogues have drained this accumulator
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < KBLOCKS; ++kb, ++it) {
          const int s = it % STAGES;
          if (!ku_wait(ku_smem(&full_bar[s]), (it / STAGES) & 1, failed, status)) break;   // no instruction is issued on operands that may not be there
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const unsigned sa = smem_s + s * STAGE_BYTES, sb = sa + A_STAGE_BYTES;
#pragma unroll
          for (int k = 0; k < BKB / 32; ++k) {  // 32 bytes of K per instruction
#if A_MN
            const unsigned long long ad = ku_smem_desc(sa + k * (32 / ESIZE) * 128, BK * 128, 1024);
#else
            const unsigned long long ad = ku_smem_desc(sa + k * 32, 16, 1024);
#endif
#if B_MN
            const unsigned long long bd = ku_smem_desc(sb + k * (32 / ESIZE) * 128, BK * 128, 1024);
#else
            const unsigned long long bd = ku_smem_desc(sb + k * 32, 16, 1024);
#endif
            ku_mma(d_tmem, ad, bd, IDESC, (kb | k) != 0);
          }
          ku_mma_commit(ku_smem(&empty_bar[s]));  // the stage is free in both CTAs once these MMAs have read it
        }
        ku_mma_commit(ku_smem(&tmem_full[acc]));  // both halves of the accumulator are complete once all MMAs of the tile retire
      }
    }
  } else {  // ---- epilogue warps: this CTA's 128 rows of the tile ----
    const int q = warp & 3;  // the TMEM lane quarter this warp may read
    const int half = (warp - 2) >> 2;   // which half of the tile's columns this warp handles
    int local = 0;
    for (int t = pair; t < total_tiles; t += npairs, ++local) {
      int b, mb, nb;
      ku_tile_coords(t, b, mb, nb);
      const int acc = local & 1;
      ku_wait(ku_smem(&tmem_full[acc]), (local >> 1) & 1, failed, status);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const i64 m = (i64)mb * 256 + (i64)rank * BM + q * 32 + lane;
      const unsigned taddr = tmem_base + ((unsigned)(q * 32) << 16) + acc * BN;
      ku_out_t* crow = (ku_out_t*)Cp + ((i64)b * M + m) * N;
#pragma unroll 1
      for (int c = half * (BN / 64); c < (half + 1) * (BN / 64); ++c) {
        float v[32];
        ku_tmem_ld32(taddr + c * 32, v);
        const i64 n0 = (i64)nb * BN + c * 32;
        if (m < M && n0 < N) {
          if ((N % (16 / (int)sizeof(ku_out_t))) == 0 && n0 + 32 <= N) {
            // 16 bytes of outputs at a time, packed in registers
            constexpr int PER = 16 / (int)sizeof(ku_out_t);
#pragma unroll
            for (int w = 0; w < 32 / PER; ++w) {
              unsigned pk[4] = {0u, 0u, 0u, 0u};
#pragma unroll
              for (int e = 0; e < PER; ++e) {
                const ku_out_t o = ku_epilogue(KU_ROUND(v[w * PER + e]), (i64)b, m, n0 + w * PER + e KU_EPI_ARGS);
                unsigned bits;
                if (sizeof(ku_out_t) == 4) bits = __float_as_uint(*(const float*)&o); else bits = (unsigned)(*(const typename KuBits<sizeof(ku_out_t)>::type*)&o);
                pk[e * (int)sizeof(ku_out_t) / 4] |= bits << (8 * ((e * (int)sizeof(ku_out_t)) & 3));
              }
              ((uint4*)(crow + n0))[w] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            }
          } else {
            for (int j = 0; j < 32 && n0 + j < N; ++j) crow[n0 + j] = ku_epilogue(KU_ROUND(v[j]), (i64)b, m, n0 + j KU_EPI_ARGS);
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      ku_mbar_arrive_remote(ku_mapa(ku_smem(&tmem_empty[acc]), 0));   // the leader's barrier counts both CTAs' epilogue threads
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  ku_cluster_sync();   // the peer may still be reading this CTA's shared memory or signalling its barriers
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
}

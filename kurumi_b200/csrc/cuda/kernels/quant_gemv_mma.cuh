// Weight-only quantised matmul for a few activation rows (decode) with 16-bit activations and 2- or 4-bit weights:
// out[m][n] = sum_c act[m][c] * W[n][c], W[n][c] = field(n, c) * scale[n][c / GROUP] (+ min)
// (kurumi_core/src/quant.rs:90-113 is the dequantisation, kurumi_core/src/interp/contract.rs:69-99 the op).
//
// The packed weight is the only large operand and crosses HBM once, 16 bytes per lane per load, past L1. What bounded the
// scalar kernel (quant_gemv.cuh) was the work per weight - a field extraction, an integer-to-float step, a shared-memory
// read of the activation and a multiply-add, per weight and thread. Here the products run on mma.sync.m16n8k16: a warp
// owns 16 weight rows, the (up to 8) activation rows are the instruction's N side, and the A operand is the raw field
// values, which are exact in the activation's 16-bit format and cost one logic operation per pair of weights:
//   f16   the field bits are an f16 subnormal already (v * 2^-24): an AND; the factor 2^24 goes into the scale;
//   bf16  (bits | 0x4300) is 128 + v: an AND-OR; 128 * sum a_c comes off after the sum (the sum of a row's activations
//         over the run is needed for the minimum anyway).
// The sum over a group's columns of a_c * field_c accumulates in f32 in the tensor core; scale and minimum are applied in
// f32 afterwards, per group (s * sum a_c field_c + min * sum a_c; for signed fields the field is offset by 2^(bits-1) and
// that offset times sum a_c is taken off again), and one rounding to the activation dtype follows, as in the interpreter.
//
// What bounds it: the kernel issues about one instruction per weight (extraction, operand reads, the per-run scaling),
// and mma.sync itself runs at 32 clocks per instruction and SM sub-core on this architecture (its tensor cores serve
// tcgen05; this is the compatibility path), 26 us for 28672 x 8192 weights whatever their width. Measured there with one
// activation row: 4-bit 51 us (f16) / 60 us (bf16), 2-bit 52 us, against 18 us and 9 us for the bytes alone.
//
// Which column goes to which slot of an instruction is free as long as the activations follow the same order. Lane
// (g, t) (g = lane / 4, t = lane % 4) loads the 16-byte piece t of a run of four pieces of rows g and g + 8; a pair of
// weights is (field i, field i + FPW / 2) of a 32-bit word, which sit 16 bits apart and so come out with one AND; an
// instruction takes two pairs per row. The activations are laid out in shared memory in exactly that order, so that
// the B operand is one 8-byte read per instruction. A run of four pieces must lie in one group: GROUP % (4 * PIECE) == 0.
//
// A CTA is 8 warps: RT tiles of 16 rows, each split over KS warps that take every KS-th run of a row and add their
// partial sums at the end (the host picks the largest KS whose CTAs make up at most two waves). A lane keeps D runs of its two
// rows in flight (a register ring), requested before the activations are staged, so the weight stream never waits for
// the staging. The activations of all K columns are staged once per CTA when they fit (KC == K); otherwise in chunks
// of KC columns, KC a multiple of RUN * KS * D so that the ring's slots line up with the chunk boundaries.
//
// Spliced in by the host: M (<= 8), N, K (a multiple of 4 * PIECE), BITS (2, 4), GROUP, SYM, ACT (1 bf16, 2 f16),
// KC (columns staged at a time), KS (1, 2, 4, 8), D (depth of the ring), RES (CTAs per SM the launch counts on).
#define NT 256
#define NWARP (NT / 32)
#define RT (NWARP / KS)              // 16-row tiles of a CTA
#define RB (K * BITS / 8)            // bytes of a packed row
#define NG (K / GROUP)
#define PIECE (128 / BITS)           // weights in a 16-byte piece
#define RUN (4 * PIECE)              // columns of one step of a quad of lanes
#define NRUN (K / RUN)
#define FPW (32 / BITS)              // fields of a 32-bit word
#define HALF (FPW / 2)
#define ROWP (KC + 16)               // shared-memory row stride in 16-bit elements: rows 32 bytes apart modulo 128
#define FMASK ((1u << BITS) - 1u)

__device__ __forceinline__ void ku_mma_16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
#if ACT == 1
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
#else
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
#endif
}
// the weight stream bypasses L1 (every byte is used once; the scale and minimum sectors, used for many runs, stay there)
__device__ __forceinline__ uint4 ku_ld_stream(const u8* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
// two fields 16 bits apart -> two 16-bit floats, one logic operation: f16 v * 2^-24 (a subnormal), bf16 128 + v (the
// 128 comes off again after the sum, as 128 * sum a_c: a packed bf16 subtraction here would run at a quarter of the rate)
__device__ __forceinline__ unsigned ku_pair(unsigned x) {
#if ACT == 1
  return (x & (FMASK | (FMASK << 16))) | 0x43004300u;
#else
  return x & (FMASK | (FMASK << 16));
#endif
}
#if ACT == 1
#define KU_FIELD_SCALE 1.0f
#define KU_FIELD_BIAS 128.0f
#else
#define KU_FIELD_SCALE 16777216.0f   // 2^24: the fields went in as f16 subnormals
#define KU_FIELD_BIAS 0.0f
#endif

extern "C" __global__ void __launch_bounds__(NT, RES)
ku_quant_gemv_mma(const u8* __restrict__ qw, const u16* __restrict__ scales, const u16* __restrict__ mins, const void* __restrict__ act, void* __restrict__ out) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  u16* a_s = (u16*)smem_raw;                              // [M][ROWP], columns in instruction order
  float* a_sum = (float*)(smem_raw + M * ROWP * 2);       // [M][KC / RUN]: sum of a row's activations over each run
#if KS > 1
  __shared__ float red[KS][RT][32][4];
#endif
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int tile = warp % RT, ks = warp / RT;
  const int blocks = (N + RT * 16 - 1) / (RT * 16);
  // A lane's column of the B operand is activation row g, its results belong to rows 2t and 2t + 1. Rows that do not
  // exist read row M - 1 instead: a column of the result depends on its own column of B only, and those columns are dropped.
  const u16* a_lane = a_s + (g < M ? g : M - 1) * ROWP + t * 4;
  const float* sum0 = a_sum + ((2 * t) < M ? 2 * t : M - 1) * (KC / RUN);
  const float* sum1 = a_sum + ((2 * t + 1) < M ? 2 * t + 1 : M - 1) * (KC / RUN);
  for (int blk = blockIdx.x; blk < blocks; blk += gridDim.x) {
    const int n0 = (blk * RT + tile) * 16;
    const int nlo = (n0 + g) < N ? (n0 + g) : (N - 1), nhi = (n0 + g + 8) < N ? (n0 + g + 8) : (N - 1);   // rows past the end re-read the last row; their results are dropped
    const unsigned olo = (unsigned)nlo * NG, ohi = (unsigned)nhi * NG;   // the rows' offsets into scales and mins
    const u8* rlo = qw + (size_t)nlo * RB + t * 16;
    const u8* rhi = qw + (size_t)nhi * RB + t * 16;
    // the ring: slot d holds run ks + (j + d) * KS of the two rows
    uint4 qlo[D], qhi[D];
#pragma unroll
    for (int d = 0; d < D; ++d) {
      const int r = ks + d * KS;
      qlo[d] = make_uint4(0, 0, 0, 0); qhi[d] = make_uint4(0, 0, 0, 0);
      if (r < NRUN) { qlo[d] = ku_ld_stream(rlo + (size_t)r * (RUN * BITS / 8)); qhi[d] = ku_ld_stream(rhi + (size_t)r * (RUN * BITS / 8)); }
    }
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};              // rows (g, g, g+8, g+8) x activation rows (2t, 2t+1, 2t, 2t+1)
    int j = 0;
    for (int kc0 = 0; kc0 < K; kc0 += KC) {
      const int kc = (K - kc0) < KC ? (K - kc0) : KC;
      if (KC < K || blk == (int)blockIdx.x) {
        __syncthreads();
        // activations of the chunk in instruction order: the four 16-bit values of (run, s, piece) are columns
        // c0, c0 + HALF, c0 + 1, c0 + 1 + HALF with c0 = run * RUN + piece * PIECE + word * FPW + i, pair p = 2 s = word * HALF + i
        // (a thread takes the FPW columns under one 32-bit word of weights, 16 or 32 bytes, and writes them as HALF / 2 groups of four)
        for (int idx = threadIdx.x; idx < M * (kc / FPW); idx += NT) {
          const int m = idx / (kc / FPW), wi = idx - m * (kc / FPW);      // wi = (run * 4 + piece) * (PIECE / FPW) + word
          const int wd = wi % (PIECE / FPW), pc = (wi / (PIECE / FPW)) & 3, run = wi / (4 * (PIECE / FPW));
          const uint4* src = (const uint4*)((const u16*)act + (size_t)m * K + kc0 + wi * FPW);
          unsigned w[FPW / 2];
#pragma unroll
          for (int q = 0; q < FPW / 8; ++q) { const uint4 v = src[q]; w[4 * q] = v.x; w[4 * q + 1] = v.y; w[4 * q + 2] = v.z; w[4 * q + 3] = v.w; }
#define KU_COL(f) ((w[(f) >> 1] >> (16 * ((f) & 1))) & 0xFFFFu)
#pragma unroll
          for (int sn = 0; sn < HALF / 2; ++sn) {
            uint2 v;
            v.x = KU_COL(2 * sn) | (KU_COL(2 * sn + HALF) << 16);
            v.y = KU_COL(2 * sn + 1) | (KU_COL(2 * sn + 1 + HALF) << 16);
            *(uint2*)(a_s + m * ROWP + (((run * (PIECE / 4) + wd * (HALF / 2) + sn) * 4 + pc) * 4)) = v;
          }
#undef KU_COL
        }
        __syncthreads();
        // the sum of each activation row over each run, a warp per (row, run), from the staged copy (the order inside a run is free)
        for (int pr = warp; pr < M * (kc / RUN); pr += NWARP) {
          const int m = pr / (kc / RUN), run = pr - m * (kc / RUN);
          float s = 0.0f;
#pragma unroll
          for (int c = lane; c < RUN; c += 32) {
#if ACT == 1
            s += ku_dec_bf16(a_s[m * ROWP + run * RUN + c]);
#else
            s += ku_dec_f16(a_s[m * ROWP + run * RUN + c]);
#endif
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
          if (lane == 0) a_sum[m * (KC / RUN) + run] = s;
        }
        __syncthreads();
      }
      const int r_end = (kc0 + kc) / RUN, r_base = kc0 / RUN;
      while (ks + j * KS < r_end) {
#pragma unroll
        for (int d = 0; d < D; ++d) {
          const int r = ks + (j + d) * KS;
          if (r < r_end) {
            const uint4 plo = qlo[d], phi = qhi[d];
            if (r + D * KS < NRUN) {
              qlo[d] = ku_ld_stream(rlo + (size_t)(r + D * KS) * (RUN * BITS / 8));
              qhi[d] = ku_ld_stream(rhi + (size_t)(r + D * KS) * (RUN * BITS / 8));
            }
            const int run = r - r_base;                   // the run inside the staged chunk
            const unsigned wlo[4] = {plo.x, plo.y, plo.z, plo.w}, whi[4] = {phi.x, phi.y, phi.z, phi.w};
            float dd[4] = {0.0f, 0.0f, 0.0f, 0.0f}, de[4] = {0.0f, 0.0f, 0.0f, 0.0f};   // two chains of instructions: one does not wait for the other
            const u16* ap = a_lane + run * (PIECE / 4) * 16;
#pragma unroll
            for (int wd = 0; wd < 4; ++wd) {
#if SYM
              const unsigned sb = (1u << (BITS - 1)) * (0xFFFFFFFFu / FMASK);   // the sign bit of every field: two's complement -> offset binary
              const unsigned xl = wlo[wd] ^ sb, xh = whi[wd] ^ sb;
#else
              const unsigned xl = wlo[wd], xh = whi[wd];
#endif
#pragma unroll
              for (int i = 0; i < HALF; i += 2) {
                const int s = (wd * HALF + i) >> 1;
                const uint2 b = *(const uint2*)(ap + s * 16);
                ku_mma_16816((s & 1) ? de : dd, ku_pair(xl >> (BITS * i)), ku_pair(xh >> (BITS * i)), ku_pair(xl >> (BITS * (i + 1))), ku_pair(xh >> (BITS * (i + 1))), b.x, b.y);
              }
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) dd[q] += de[q];
            // the run lies in one group per row: scale, minimum / offset in f32
            const int gi = r * RUN / GROUP;
            const float slo = ku_dec_f16(scales[olo + gi]) * KU_FIELD_SCALE, shi = ku_dec_f16(scales[ohi + gi]) * KU_FIELD_SCALE;
            const float s0 = sum0[run], s1 = sum1[run];
#if SYM
            const float off = ((float)(1u << (BITS - 1)) + KU_FIELD_BIAS) / KU_FIELD_SCALE;      // in the units the fields went in with
            acc[0] = __fmaf_rn(dd[0] - off * s0, slo, acc[0]); acc[1] = __fmaf_rn(dd[1] - off * s1, slo, acc[1]);
            acc[2] = __fmaf_rn(dd[2] - off * s0, shi, acc[2]); acc[3] = __fmaf_rn(dd[3] - off * s1, shi, acc[3]);
#else
            const float mlo = ku_dec_f16(mins[olo + gi]), mhi = ku_dec_f16(mins[ohi + gi]);
            acc[0] = __fmaf_rn(s0, mlo, __fmaf_rn(dd[0] - KU_FIELD_BIAS * s0, slo, acc[0])); acc[1] = __fmaf_rn(s1, mlo, __fmaf_rn(dd[1] - KU_FIELD_BIAS * s1, slo, acc[1]));
            acc[2] = __fmaf_rn(s0, mhi, __fmaf_rn(dd[2] - KU_FIELD_BIAS * s0, shi, acc[2])); acc[3] = __fmaf_rn(s1, mhi, __fmaf_rn(dd[3] - KU_FIELD_BIAS * s1, shi, acc[3]));
#endif
          }
        }
        j += D;
      }
    }
#if KS > 1
    // the KS partial sums of a tile, added in warp order
    __syncthreads();
#pragma unroll
    for (int q = 0; q < 4; ++q) red[ks][tile][lane][q] = acc[q];
    __syncthreads();
    if (ks == 0) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        acc[q] = red[0][tile][lane][q];
#pragma unroll
        for (int w = 1; w < KS; ++w) acc[q] += red[w][tile][lane][q];
      }
    }
#endif
    if (ks == 0) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int n = n0 + g + (q >> 1) * 8, m = 2 * t + (q & 1);
        if (n < N && m < M) {
#if ACT == 1
          ((u16*)out)[(size_t)m * N + n] = ku_enc_bf16(acc[q]);
#else
          ((u16*)out)[(size_t)m * N + n] = ku_enc_f16(acc[q]);
#endif
        }
      }
    }
  }
}

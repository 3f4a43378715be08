// Weight-only quantised matmul for a few activation rows (decode): out[m][n] = sum_c act[m][c] * W[n][c] with
// W[n][c] = field(n, c) * scale[n][c / GROUP] (+ min) read straight from the packed weight
// (kurumi_core/src/quant.rs:90-113 is the dequantisation, kurumi_core/src/interp/contract.rs:69-99 the op).
// The packed weight is the only large operand and is read exactly once, 16 bytes per lane per load: the
// kernel is bound by HBM. A CTA keeps a chunk of the activations in shared memory as f32; each warp owns
// RPW output columns at a time and every lane a 16-byte piece of their packed rows; within a group the sum
// is taken over a_j * field_j and scaled once (s * sum a_j field_j + min * sum a_j), products accumulate in
// f32 and one rounding to the activation dtype follows, as in the interpreter.
//
// Spliced in by the host: M (<= 8), N, K, BITS (2, 4, 8), GROUP, SYM, ACT (0 f32, 1 bf16, 2 f16), KC (columns
// of a shared-memory chunk: a whole number of warp-wide strides of 32 pieces, or K itself when K is smaller), RPW.
#define NT 256
#define NWARP (NT / 32)
#define RB (K * BITS / 8)            // bytes of a packed row
#define NG (K / GROUP)
#define PIECE (128 / BITS)           // weights in a 16-byte piece
#define SUB (PIECE < GROUP ? PIECE : GROUP)   // weights of a piece that share a group

__device__ __forceinline__ float ku_act_at(const void* act, size_t i) {
#if ACT == 0
  return ((const float*)act)[i];
#elif ACT == 1
  return ku_dec_bf16(((const u16*)act)[i]);
#else
  return ku_dec_f16(((const u16*)act)[i]);
#endif
}

extern "C" __global__ void __launch_bounds__(NT)
ku_quant_gemv(const u8* __restrict__ qw, const u16* __restrict__ scales, const u16* __restrict__ mins, const void* __restrict__ act, void* __restrict__ out) {
  extern __shared__ __align__(16) float a_s[];   // [M][KC]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int blocks = (N + NWARP * RPW - 1) / (NWARP * RPW);
  for (int blk = blockIdx.x; blk < blocks; blk += gridDim.x) {
    const int n0 = (blk * NWARP + warp) * RPW;
    float acc[RPW][M];
#pragma unroll
    for (int r = 0; r < RPW; ++r)
#pragma unroll
      for (int m = 0; m < M; ++m) acc[r][m] = 0.0f;
    for (int kc0 = 0; kc0 < K; kc0 += KC) {
      const int kc = (K - kc0) < KC ? (K - kc0) : KC;
      __syncthreads();
      // activations of the chunk as f32, laid out so that the 32 lanes of a warp, each working on its own
      // 16-byte piece (PIECE consecutive columns), read consecutive words: column c of a warp-wide block
      // of 32 * PIECE columns goes to (c % PIECE) * 32 + (c / PIECE)
      for (int i = threadIdx.x; i < M * kc; i += NT) {
        const int m = i / kc, c = i - m * kc;
        const int blkc = c / (32 * PIECE), within = c - blkc * (32 * PIECE);
        a_s[m * KC + blkc * (32 * PIECE) + (within % PIECE) * 32 + within / PIECE] = ku_act_at(act, (size_t)m * K + kc0 + c);
      }
      __syncthreads();
      // the pieces of all RPW rows at a stride position are loaded before any is used, and two stride positions
      // are unrolled: 2 * RPW 16-byte loads in flight per lane keep HBM busy
#pragma unroll 2
      for (int b = lane * 16, blkc = 0; b < kc * BITS / 8; b += 32 * 16, ++blkc) {
        uint4 pks[RPW];
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
          const int n = (n0 + r) < N ? (n0 + r) : (N - 1);   // rows past the end re-read the last row; their results are dropped
          // past L1: every byte of the weight is used once, the scales and minima are used again
          asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(pks[r].x), "=r"(pks[r].y), "=r"(pks[r].z), "=r"(pks[r].w) : "l"(qw + (size_t)n * RB + (size_t)kc0 * BITS / 8 + b));
        }
        const int c0 = b * 8 / BITS;   // first column of the piece inside the chunk
        const float* ap = a_s + blkc * (32 * PIECE) + lane;   // this lane's column f of the block is ap[f * 32]
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
          const int n = (n0 + r) < N ? (n0 + r) : (N - 1);
          const unsigned wds[4] = {pks[r].x, pks[r].y, pks[r].z, pks[r].w};
#pragma unroll
          for (int sb = 0; sb < PIECE / SUB; ++sb) {
            const int gi = (kc0 + c0 + sb * SUB) / GROUP;
            const float s = ku_dec_f16(scales[(size_t)n * NG + gi]);
            // sum_j a_j * (raw_j * s + mn) = s * sum_j a_j raw_j + mn * sum_j a_j: one multiply-add per weight
            float t[M];
#if !SYM
            const float mn = ku_dec_f16(mins[(size_t)n * NG + gi]);
            float u[M];
#endif
#pragma unroll
            for (int m = 0; m < M; ++m) {
              t[m] = 0.0f;
#if !SYM
              u[m] = 0.0f;
#endif
            }
#pragma unroll
            for (int j = 0; j < SUB; ++j) {
              const int f = sb * SUB + j;                      // field index inside the piece
              const unsigned raw = (wds[(f * BITS) >> 5] >> ((f * BITS) & 31)) & ((1u << BITS) - 1u);
              // integer -> float without the quarter-rate conversion instruction: 2^23 + v has v in its low mantissa bits
#if SYM
              const float q = __uint_as_float(0x4B000000u | (raw ^ (1u << (BITS - 1)))) - (8388608.0f + (float)(1u << (BITS - 1)));   // the sign-extended field
#else
              const float q = __uint_as_float(0x4B000000u | raw) - 8388608.0f;
#endif
#pragma unroll
              for (int m = 0; m < M; ++m) {
                const float av = ap[m * KC + f * 32];
                t[m] = __fmaf_rn(av, q, t[m]);
#if !SYM
                u[m] += av;
#endif
              }
            }
#pragma unroll
            for (int m = 0; m < M; ++m) {
#if SYM
              acc[r][m] = __fmaf_rn(t[m], s, acc[r][m]);
#else
              acc[r][m] = __fmaf_rn(u[m], mn, __fmaf_rn(t[m], s, acc[r][m]));
#endif
            }
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < RPW; ++r)
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float v = acc[r][m];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0 && n0 + r < N) {
#if ACT == 0
          ((float*)out)[(size_t)m * N + n0 + r] = v;
#elif ACT == 1
          ((u16*)out)[(size_t)m * N + n0 + r] = ku_enc_bf16(v);
#else
          ((u16*)out)[(size_t)m * N + n0 + r] = ku_enc_f16(v);
#endif
        }
      }
  }
}

// Causal intra-chunk matrix W on CUDA cores, any shape (the general, materialising path).
#include "common.cuh"

namespace fracssm {

// W[t,k] = sum_m c[t,m] * exp(lcr[t,m] - lcr[k,m]) * kappa[k,m] for k <= t, else 0.
// One block of 256 threads owns a 64 x 64 tile of one chunk's W, 4 x 4 entries per thread; the modes
// are swept in slices of 32 staged in shared memory, transposed ([mode][token]) so that a thread
// reads its four tokens with one 16-byte load.
//   * A tile below the diagonal (all its k before all its t) needs no exponential per (t, k, m): with
//     the last token of the k tile as reference point the decay splits into two factors that are both
//     <= 1, exp(lcr[t] - lcr[ref]) and exp(lcr[ref] - lcr[k]); they are applied while staging (one
//     exponential per staged element) and the tile is a plain product of two 64 x 32 operands.
//   * A tile on the diagonal has no such point for all its pairs and keeps one exponential per
//     (t, k, m), on register tiles.
//   * Tiles above the diagonal are written as zeros.
// Padded tokens of a partial chunk reuse the last valid lcr row (their c and kappa are zero), which
// keeps every exponent finite.
constexpr int kWt = 64, kWm = 32;

__global__ void __launch_bounds__(256)
chunk_w_kernel(const void *__restrict__ c, const void *__restrict__ kappa, int ck_dt, int64_t c_sb,
               int64_t c_sl, int64_t k_sb, int64_t k_sl, const float *__restrict__ lcr,
               int64_t g_sb, int64_t g_sl, float *__restrict__ W, int64_t L, int64_t M, int64_t T,
               int64_t N, int tiles) {
  const int ti = blockIdx.x / tiles, tk = blockIdx.x % tiles;
  const int64_t n = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;   // entries t = 4 ty + i, k = 4 tx + j of the tile
  float *out = W + ((b * N + n) * T) * T;
  const int64_t tb = (int64_t)ti * kWt, kb = (int64_t)tk * kWt;
  float acc[4][4] = {};
  float dacc = 0.f;   // diagonal tile: the entry (t, k) = (4d + i, 4d + j), d = tid / 16, of the register tiles on the diagonal
  if (tk <= ti) {
    __shared__ __align__(16) float ct[kWm][kWt + 4], kk[kWm][kWt + 4], gt[kWm][kWt + 4], gk[kWm][kWt + 4],
        kk2[kWm][kWt + 4];
    const int64_t t0 = n * T;
    const int64_t len = min(T, L - t0);
    const bool below = tk < ti;
    const int64_t rref = min(kb + kWt - 1, len - 1);   // reference token of a tile below the diagonal
    for (int64_t m0 = 0; m0 < M; m0 += kWm) {
      __syncthreads();
      for (int i = tid; i < kWt * kWm; i += 256) {
        // a warp takes 8 modes x 4 rows: 32-byte pieces of four rows from memory, 32 distinct banks in the
        // transposed shared-memory arrays (row stride 68 floats)
        const int blk = i >> 5, ln = i & 31;
        const int mm = 8 * (blk & 3) + (ln & 7), rr = 4 * (blk >> 2) + (ln >> 3);
        const int64_t m = m0 + mm;
        const bool mv = m < M;
        const int64_t row_t = tb + rr, row_k = kb + rr;
        const int64_t rt = min(row_t, len - 1), rk = min(row_k, len - 1);
        const float g_t = mv ? lcr[b * g_sb + (t0 + rt) * g_sl + m] * kLog2e : 0.f;
        const float g_k = mv ? lcr[b * g_sb + (t0 + rk) * g_sl + m] * kLog2e : 0.f;
        float c_v = (mv && row_t < len) ? ld_f32(c, b * c_sb + (t0 + row_t) * c_sl + m, ck_dt) : 0.f;
        float k_v = (mv && row_k < len) ? ld_f32(kappa, b * k_sb + (t0 + row_k) * k_sl + m, ck_dt) : 0.f;
        if (below) {
          const float g_r = mv ? lcr[b * g_sb + (t0 + rref) * g_sl + m] * kLog2e : 0.f;
          c_v *= exp2f(g_t - g_r);
          k_v *= exp2f(g_r - g_k);
        } else {
          gt[mm][rr] = g_t;
          gk[mm][rr] = g_k;
          // kappa taken to the last token of its group of four rows (the warp holds the four rows of
          // a group for 8 modes: the group's last row is in lanes 24..31)
          const float g_4 = __shfl_sync(0xffffffffu, g_k, 24 + (ln & 7));
          kk2[mm][rr] = k_v * exp2f(fminf(g_4 - g_k, 0.f));
        }
        ct[mm][rr] = c_v;
        kk[mm][rr] = k_v;
      }
      __syncthreads();
      if (below) {
#pragma unroll 8
        for (int mm = 0; mm < kWm; ++mm) {
          const float4 a4 = *reinterpret_cast<const float4 *>(&ct[mm][4 * ty]);
          const float4 b4 = *reinterpret_cast<const float4 *>(&kk[mm][4 * tx]);
          const float av[4] = {a4.x, a4.y, a4.z, a4.w}, bv[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
      } else {
        // On the diagonal tile: a 4 x 4 register tile strictly below the diagonal (all its k before
        // all its t) takes the last k of its group as reference point: four exponentials per mode for
        // the thread's t rows, the k side comes scaled from the staging.  The 16 register tiles ON the
        // diagonal are done afterwards, one entry per thread, with one exponential per (t, k, m).
        if (tx < ty) {
#pragma unroll 4
          for (int mm = 0; mm < kWm; ++mm) {
            const float4 a4 = *reinterpret_cast<const float4 *>(&ct[mm][4 * ty]);
            const float4 p4 = *reinterpret_cast<const float4 *>(&gt[mm][4 * ty]);
            const float4 b4 = *reinterpret_cast<const float4 *>(&kk2[mm][4 * tx]);
            const float g_r = gk[mm][4 * tx + 3];
            const float av[4] = {a4.x * exp2f(fminf(p4.x - g_r, 0.f)), a4.y * exp2f(fminf(p4.y - g_r, 0.f)),
                                 a4.z * exp2f(fminf(p4.z - g_r, 0.f)), a4.w * exp2f(fminf(p4.w - g_r, 0.f))};
            const float bv[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
              for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
          }
        }
        {
          const int d = tid >> 4, i = (tid >> 2) & 3, j = tid & 3;
          if (j <= i) {
#pragma unroll 8
            for (int mm = 0; mm < kWm; ++mm)
              dacc = fmaf(ct[mm][4 * d + i] * kk[mm][4 * d + j], exp2f(gt[mm][4 * d + i] - gk[mm][4 * d + j]), dacc);
          }
        }
      }
    }
  }
  if (tk != ti || tx != ty) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int64_t t = tb + 4 * ty + i;
      if (t >= T) continue;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int64_t k = kb + 4 * tx + j;
        if (k < T) out[t * T + k] = (k <= t) ? acc[i][j] : 0.f;
      }
    }
  }
  if (tk == ti) {
    const int d = tid >> 4, i = (tid >> 2) & 3, j = tid & 3;
    const int64_t t = tb + 4 * d + i, k = kb + 4 * d + j;
    if (t < T && k < T) out[t * T + k] = (j <= i) ? dacc : 0.f;
  }
}

}  // namespace fracssm

extern "C" int fracssm_chunk_w(const void *c, const void *kappa, int ck_dtype, int64_t c_sb,
                               int64_t c_sl, int64_t k_sb, int64_t k_sl, const float *lcr,
                               int64_t g_sb, int64_t g_sl, float *W, int64_t B, int64_t L, int64_t M,
                               int64_t T, void *stream) {
  using namespace fracssm;
  if (B < 0 || L < 0 || M <= 0 || T <= 0) return fail(FRACSSM_ERR_ARG, "chunk_w: bad sizes");
  if (!known_dtype(ck_dtype)) return fail(FRACSSM_ERR_ARG, "chunk_w: unsupported dtype");
  if (B == 0 || L == 0) return FRACSSM_OK;
  if (!c || !kappa || !lcr || !W) return fail(FRACSSM_ERR_ARG, "chunk_w: null pointer");
  const int64_t N = ceil_div(L, T);
  const int tiles = (int)ceil_div(T, kWt);
  if (B > 65535 || N > 65535) return fail(FRACSSM_ERR_UNSUPPORTED, "chunk_w: B or N too large for one launch");
  dim3 grid((unsigned)(tiles * tiles), (unsigned)N, (unsigned)B), block(256);
  chunk_w_kernel<<<grid, block, 0, (cudaStream_t)stream>>>(c, kappa, ck_dtype, c_sb, c_sl, k_sb, k_sl,
                                                           lcr, g_sb, g_sl, W, L, M, T, N, tiles);
  return check_launch("chunk_w");
}

// Causal intra-chunk matrix W on CUDA cores, any shape (the general, materialising path).
//
// W[t,k] = sum_m c[t,m] * exp(lcr[t,m] - lcr[k,m]) * kappa[k,m] for k <= t, else 0.
// One block of 32x32 threads owns a 32x32 tile of one chunk's W; modes are swept in
// slices of 32 staged in shared memory (lcr pre-multiplied by log2 e).  Tiles above the
// diagonal are written as zeros.  Padded tokens of a partial chunk reuse the last valid
// lcr row (their c and kappa are zero), which keeps every exponent finite.
#include "common.cuh"

namespace fracssm {

__global__ void __launch_bounds__(1024)
chunk_w_kernel(const void *__restrict__ c, const void *__restrict__ kappa, int ck_dt, int64_t c_sb,
               int64_t c_sl, int64_t k_sb, int64_t k_sl, const float *__restrict__ lcr,
               int64_t g_sb, int64_t g_sl, float *__restrict__ W, int64_t L, int64_t M, int64_t T,
               int64_t N, int tiles) {
  const int ti = blockIdx.x / tiles, tk = blockIdx.x % tiles;
  const int64_t n = blockIdx.y, b = blockIdx.z;
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int64_t t = (int64_t)ti * 32 + ty, k = (int64_t)tk * 32 + tx;
  float *out = W + ((b * N + n) * T) * T;
  if (tk > ti) {
    if (t < T && k < T) out[t * T + k] = 0.f;
    return;
  }
  __shared__ float gt[32][33], ct[32][33], gk[32][33], kk[32][33];
  const int64_t t0 = n * T;
  const int64_t len = min(T, L - t0);
  const int64_t row_t = (int64_t)ti * 32 + ty, row_k = (int64_t)tk * 32 + ty;  // staging rows
  float acc = 0.f;
  for (int64_t m0 = 0; m0 < M; m0 += 32) {
    const int64_t m = m0 + tx;
    __syncthreads();
    {
      const bool mv = m < M;
      const int64_t rt = min(row_t, len - 1), rk = min(row_k, len - 1);
      gt[ty][tx] = mv ? lcr[b * g_sb + (t0 + rt) * g_sl + m] * kLog2e : 0.f;
      gk[ty][tx] = mv ? lcr[b * g_sb + (t0 + rk) * g_sl + m] * kLog2e : 0.f;
      ct[ty][tx] = (mv && row_t < len) ? ld_f32(c, b * c_sb + (t0 + row_t) * c_sl + m, ck_dt) : 0.f;
      kk[ty][tx] = (mv && row_k < len) ? ld_f32(kappa, b * k_sb + (t0 + row_k) * k_sl + m, ck_dt) : 0.f;
    }
    __syncthreads();
    if (k <= t) {
#pragma unroll 8
      for (int mm = 0; mm < 32; ++mm)
        acc = fmaf(ct[ty][mm] * kk[tx][mm], exp2f(gt[ty][mm] - gk[tx][mm]), acc);
    }
  }
  if (t < T && k < T) out[t * T + k] = (k <= t) ? acc : 0.f;
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
  const int tiles = (int)ceil_div(T, 32);
  if (B > 65535 || N > 65535) return fail(FRACSSM_ERR_UNSUPPORTED, "chunk_w: B or N too large for one launch");
  dim3 grid((unsigned)(tiles * tiles), (unsigned)N, (unsigned)B), block(32, 32);
  chunk_w_kernel<<<grid, block, 0, (cudaStream_t)stream>>>(c, kappa, ck_dtype, c_sb, c_sl, k_sb, k_sl,
                                                           lcr, g_sb, g_sl, W, L, M, T, N, tiles);
  return check_launch("chunk_w");
}

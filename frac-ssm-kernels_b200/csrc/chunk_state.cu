// Per-chunk state contribution on CUDA cores, any shape and dtype (the general path).
//
// states[b,n,r,m] = sum_t u[t,r] * kappa[t,m] * exp(lcr[last,m] - lcr[t,m])
// One block computes a 64(r) x 64(m) tile of one chunk's state; tokens are swept in
// slices of 32 staged in shared memory, the decay weight is formed while staging.
#include "common.cuh"

namespace fracssm {

constexpr int kStR = 64, kStM = 64, kStT = 32;

__global__ void __launch_bounds__(256)
chunk_state_kernel(const void *__restrict__ u, int u_dt, int64_t u_sb, int64_t u_sl,
                   const void *__restrict__ kappa, int k_dt, int64_t k_sb, int64_t k_sl,
                   const float *__restrict__ lcr, int64_t g_sb, int64_t g_sl,
                   void *__restrict__ states, int s_dt, int64_t L, int64_t R, int64_t M, int64_t T,
                   int64_t N, int m_tiles) {
  const int64_t n = blockIdx.x, b = blockIdx.y;
  const int r0 = (blockIdx.z / m_tiles) * kStR, m0 = (blockIdx.z % m_tiles) * kStM;
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;  // tx: 4 modes, ty: 4 rows
  __shared__ float us[kStT][kStR];
  __shared__ float ws[kStT][kStM];
  __shared__ float g_last[kStM];

  const int64_t t0 = n * T;
  const int64_t len = min(T, L - t0);
  if (tid < kStM) {
    int64_t m = m0 + tid;
    g_last[tid] = (m < M) ? lcr[b * g_sb + (t0 + len - 1) * g_sl + m] : 0.f;
  }
  float acc[4][4] = {};
  for (int64_t ts = 0; ts < len; ts += kStT) {
    __syncthreads();
    for (int i = tid; i < kStT * kStR; i += 256) {
      int tt = i / kStR, rr = i % kStR;
      int64_t t = ts + tt, r = r0 + rr;
      us[tt][rr] = (t < len && r < R) ? ld_f32(u, b * u_sb + (t0 + t) * u_sl + r, u_dt) : 0.f;
    }
    for (int i = tid; i < kStT * kStM; i += 256) {
      int tt = i / kStM, mm = i % kStM;
      int64_t t = ts + tt, m = m0 + mm;
      float w = 0.f;
      if (t < len && m < M) {
        float g = lcr[b * g_sb + (t0 + t) * g_sl + m];
        w = ld_f32(kappa, b * k_sb + (t0 + t) * k_sl + m, k_dt) * __expf(g_last[mm] - g);
      }
      ws[tt][mm] = w;
    }
    __syncthreads();
#pragma unroll 8
    for (int tt = 0; tt < kStT; ++tt) {
      float4 a = *reinterpret_cast<const float4 *>(&us[tt][ty * 4]);
      float4 w = *reinterpret_cast<const float4 *>(&ws[tt][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int64_t r = r0 + ty * 4 + i;
    if (r >= R) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int64_t m = m0 + tx * 4 + j;
      if (m < M) st_f32(states, ((b * N + n) * R + r) * M + m, s_dt, acc[i][j]);
    }
  }
}

}  // namespace fracssm

extern "C" int fracssm_chunk_state(const void *u, int u_dtype, int64_t u_sb, int64_t u_sl,
                                   const void *kappa, int k_dtype, int64_t k_sb, int64_t k_sl,
                                   const float *lcr, int64_t g_sb, int64_t g_sl, void *states,
                                   int states_dtype, int64_t B, int64_t L, int64_t R, int64_t M,
                                   int64_t T, void *stream) {
  using namespace fracssm;
  if (B < 0 || L < 0 || R <= 0 || M <= 0 || T <= 0) return fail(FRACSSM_ERR_ARG, "chunk_state: bad sizes");
  if (!known_dtype(u_dtype) || !known_dtype(k_dtype) ||
      (states_dtype != FRACSSM_F32 && states_dtype != FRACSSM_BF16))
    return fail(FRACSSM_ERR_ARG, "chunk_state: unsupported dtype");
  if (B == 0 || L == 0) return FRACSSM_OK;
  if (!u || !kappa || !lcr || !states) return fail(FRACSSM_ERR_ARG, "chunk_state: null pointer");
  const int64_t N = ceil_div(L, T);
  const int m_tiles = (int)ceil_div(M, kStM), r_tiles = (int)ceil_div(R, kStR);
  if (B > 65535 || (int64_t)m_tiles * r_tiles > 65535)
    return fail(FRACSSM_ERR_UNSUPPORTED, "chunk_state: B, R or M too large for one launch");
  dim3 grid((unsigned)N, (unsigned)B, (unsigned)(m_tiles * r_tiles));
  chunk_state_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(
      u, u_dtype, u_sb, u_sl, kappa, k_dtype, k_sb, k_sl, lcr, g_sb, g_sl, states, states_dtype, L,
      R, M, T, N, m_tiles);
  return check_launch("chunk_state");
}

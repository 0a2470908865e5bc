// Chunk readout on CUDA cores, any shape and dtype (the general path), in two flavours:
//   plain: h = (c * exp(lcr)) . states_acc^T + W . u with W read from memory
//   fused: the 32x32 tiles of W are formed in shared memory and never stored
// One block of 256 threads owns a 32(token) x 64(r) tile of h.  Thread (tx, ty) holds
// tokens {2ty, 2ty+1} x rows {4tx .. 4tx+3}.
#include "common.cuh"

namespace fracssm {

struct ReadoutArgs {
  const void *u; int u_dt; int64_t u_sb, u_sl;
  const void *c; int c_dt; int64_t c_sb, c_sl;
  const void *kappa; int64_t k_sb, k_sl;          // fused only (dtype = c_dt)
  const void *acc; int a_dt;
  const void *W; int w_dt;                        // plain only
  const float *lcr; int64_t g_sb, g_sl;
  void *h;
  int64_t L, R, M, T, N;
  int r_tiles;
};

template <bool FUSED>
__global__ void __launch_bounds__(256) chunk_readout_kernel(const ReadoutArgs a) {
  const int ti = blockIdx.x / a.r_tiles;
  const int r0 = (blockIdx.x % a.r_tiles) * 64;
  const int64_t n = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
  const int64_t t0 = n * a.T;
  const int64_t len = min(a.T, a.L - t0);
  const int64_t M = a.M, R = a.R;

  __shared__ float gt[32][33], ct[32][33], gk[32][33], kk[32][33];
  __shared__ float wt[32][33];
  __shared__ float ss[64][33];
  __shared__ __align__(16) float us[32][64];

  float acc[2][4] = {};

  // carried part: (c * exp(lcr)) . states_acc^T
  for (int64_t m0 = 0; m0 < M; m0 += 32) {
    __syncthreads();
    for (int i = tid; i < 32 * 32; i += 256) {
      int tt = i / 32, mm = i % 32;
      int64_t t = (int64_t)ti * 32 + tt, m = m0 + mm;
      float v = 0.f;
      if (t < len && m < M)
        v = ld_f32(a.c, b * a.c_sb + (t0 + t) * a.c_sl + m, a.c_dt) *
            __expf(a.lcr[b * a.g_sb + (t0 + t) * a.g_sl + m]);
      ct[tt][mm] = v;
    }
    for (int i = tid; i < 64 * 32; i += 256) {
      int rr = i / 32, mm = i % 32;
      int64_t r = r0 + rr, m = m0 + mm;
      ss[rr][mm] = (r < R && m < M) ? ld_f32(a.acc, ((b * a.N + n) * R + r) * M + m, a.a_dt) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int mm = 0; mm < 32; ++mm) {
      const float c0 = ct[2 * ty][mm], c1 = ct[2 * ty + 1][mm];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float s = ss[tx * 4 + j][mm];
        acc[0][j] = fmaf(c0, s, acc[0][j]);
        acc[1][j] = fmaf(c1, s, acc[1][j]);
      }
    }
  }

  // local part: W . u over the token tiles at or before this one
  for (int kt = 0; kt <= ti; ++kt) {
    if (FUSED) {
      float wacc[4] = {0.f, 0.f, 0.f, 0.f};
      const int kx = tid % 32, tyb = tid / 32;  // entries (t = tyb + 8 i, k = kx)
      for (int64_t m0 = 0; m0 < M; m0 += 32) {
        __syncthreads();
        for (int i = tid; i < 32 * 32; i += 256) {
          int rr = i / 32, mm = i % 32;
          int64_t m = m0 + mm;
          int64_t row_t = (int64_t)ti * 32 + rr, row_k = (int64_t)kt * 32 + rr;
          const bool mv = m < M;
          const int64_t rt = min(row_t, len - 1), rk = min(row_k, len - 1);
          gt[rr][mm] = mv ? a.lcr[b * a.g_sb + (t0 + rt) * a.g_sl + m] * kLog2e : 0.f;
          gk[rr][mm] = mv ? a.lcr[b * a.g_sb + (t0 + rk) * a.g_sl + m] * kLog2e : 0.f;
          ct[rr][mm] = (mv && row_t < len) ? ld_f32(a.c, b * a.c_sb + (t0 + row_t) * a.c_sl + m, a.c_dt) : 0.f;
          kk[rr][mm] = (mv && row_k < len) ? ld_f32(a.kappa, b * a.k_sb + (t0 + row_k) * a.k_sl + m, a.c_dt) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int tt = tyb + 8 * i;
          if (kt < ti || kx <= tt) {
#pragma unroll 8
            for (int mm = 0; mm < 32; ++mm)
              wacc[i] = fmaf(ct[tt][mm] * kk[kx][mm], exp2f(gt[tt][mm] - gk[kx][mm]), wacc[i]);
          }
        }
      }
      __syncthreads();
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int tt = tyb + 8 * i;
        wt[tt][kx] = (kt < ti || kx <= tt) ? wacc[i] : 0.f;
      }
    } else {
      __syncthreads();
      for (int i = tid; i < 32 * 32; i += 256) {
        int tt = i / 32, kx = i % 32;
        int64_t t = (int64_t)ti * 32 + tt, k = (int64_t)kt * 32 + kx;
        wt[tt][kx] = (t < a.T && k < a.T)
                         ? ld_f32(a.W, ((b * a.N + n) * a.T + t) * a.T + k, a.w_dt) : 0.f;
      }
    }
    for (int i = tid; i < 32 * 64; i += 256) {
      int kx = i / 64, rr = i % 64;
      int64_t k = (int64_t)kt * 32 + kx, r = r0 + rr;
      us[kx][rr] = (k < len && r < R) ? ld_f32(a.u, b * a.u_sb + (t0 + k) * a.u_sl + r, a.u_dt) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int kx = 0; kx < 32; ++kx) {
      const float w0 = wt[2 * ty][kx], w1 = wt[2 * ty + 1][kx];
      const float4 x = *reinterpret_cast<const float4 *>(&us[kx][tx * 4]);
      acc[0][0] = fmaf(w0, x.x, acc[0][0]); acc[0][1] = fmaf(w0, x.y, acc[0][1]);
      acc[0][2] = fmaf(w0, x.z, acc[0][2]); acc[0][3] = fmaf(w0, x.w, acc[0][3]);
      acc[1][0] = fmaf(w1, x.x, acc[1][0]); acc[1][1] = fmaf(w1, x.y, acc[1][1]);
      acc[1][2] = fmaf(w1, x.z, acc[1][2]); acc[1][3] = fmaf(w1, x.w, acc[1][3]);
    }
  }

#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int64_t t = (int64_t)ti * 32 + 2 * ty + i;
    if (t >= len) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t r = r0 + tx * 4 + j;
      if (r < R) st_f32(a.h, (b * a.L + t0 + t) * R + r, a.u_dt, acc[i][j]);
    }
  }
}

static int launch_readout(bool fused, const ReadoutArgs &a, int64_t B, void *stream) {
  const int tiles = (int)ceil_div(a.T, 32);
  if (B > 65535 || a.N > 65535)
    return fail(FRACSSM_ERR_UNSUPPORTED, "chunk_readout: B or N too large for one launch");
  dim3 grid((unsigned)(tiles * a.r_tiles), (unsigned)a.N, (unsigned)B);
  if (fused) chunk_readout_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>(a);
  else chunk_readout_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>(a);
  return check_launch(fused ? "chunk_fused_readout" : "chunk_readout");
}

}  // namespace fracssm

extern "C" int fracssm_chunk_readout(const void *u, int u_dtype, int64_t u_sb, int64_t u_sl,
                                     const void *c, int c_dtype, int64_t c_sb, int64_t c_sl,
                                     const void *states_acc, int acc_dtype, const void *W,
                                     int w_dtype, const float *lcr, int64_t g_sb, int64_t g_sl,
                                     void *h, int64_t B, int64_t L, int64_t R, int64_t M, int64_t T,
                                     void *stream) {
  using namespace fracssm;
  if (B < 0 || L < 0 || R <= 0 || M <= 0 || T <= 0) return fail(FRACSSM_ERR_ARG, "chunk_readout: bad sizes");
  if (!known_dtype(u_dtype) || !known_dtype(c_dtype) || !known_dtype(acc_dtype) || !known_dtype(w_dtype))
    return fail(FRACSSM_ERR_ARG, "chunk_readout: unsupported dtype");
  if (B == 0 || L == 0) return FRACSSM_OK;
  if (!u || !c || !states_acc || !W || !lcr || !h) return fail(FRACSSM_ERR_ARG, "chunk_readout: null pointer");
  ReadoutArgs a{};
  a.u = u; a.u_dt = u_dtype; a.u_sb = u_sb; a.u_sl = u_sl;
  a.c = c; a.c_dt = c_dtype; a.c_sb = c_sb; a.c_sl = c_sl;
  a.acc = states_acc; a.a_dt = acc_dtype; a.W = W; a.w_dt = w_dtype;
  a.lcr = lcr; a.g_sb = g_sb; a.g_sl = g_sl; a.h = h;
  a.L = L; a.R = R; a.M = M; a.T = T; a.N = ceil_div(L, T); a.r_tiles = (int)ceil_div(R, 64);
  return launch_readout(false, a, B, stream);
}

extern "C" int fracssm_chunk_fused_readout(const void *u, int u_dtype, int64_t u_sb, int64_t u_sl,
                                           const void *c, const void *kappa, int ck_dtype,
                                           int64_t c_sb, int64_t c_sl, int64_t k_sb, int64_t k_sl,
                                           const void *states_acc, int acc_dtype, const float *lcr,
                                           int64_t g_sb, int64_t g_sl, void *h, int64_t B, int64_t L,
                                           int64_t R, int64_t M, int64_t T, void *stream) {
  using namespace fracssm;
  if (B < 0 || L < 0 || R <= 0 || M <= 0 || T <= 0) return fail(FRACSSM_ERR_ARG, "chunk_fused_readout: bad sizes");
  if (!known_dtype(u_dtype) || !known_dtype(ck_dtype) || !known_dtype(acc_dtype))
    return fail(FRACSSM_ERR_ARG, "chunk_fused_readout: unsupported dtype");
  if (B == 0 || L == 0) return FRACSSM_OK;
  if (!u || !c || !kappa || !states_acc || !lcr || !h)
    return fail(FRACSSM_ERR_ARG, "chunk_fused_readout: null pointer");
  ReadoutArgs a{};
  a.u = u; a.u_dt = u_dtype; a.u_sb = u_sb; a.u_sl = u_sl;
  a.c = c; a.c_dt = ck_dtype; a.c_sb = c_sb; a.c_sl = c_sl;
  a.kappa = kappa; a.k_sb = k_sb; a.k_sl = k_sl;
  a.acc = states_acc; a.a_dt = acc_dtype;
  a.lcr = lcr; a.g_sb = g_sb; a.g_sl = g_sl; a.h = h;
  a.L = L; a.R = R; a.M = M; a.T = T; a.N = ceil_div(L, T); a.r_tiles = (int)ceil_div(R, 64);
  return launch_readout(true, a, B, stream);
}

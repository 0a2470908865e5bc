// Chunk readout on CUDA cores, any shape and dtype (the general path), in two flavours:
//   plain: h = (c * exp(lcr)) . states_acc^T + W . u with W read from memory
//          (chunk_readout_kernel: one block of 256 threads owns a 32(token) x 64(r) tile of h, thread
//          (tx, ty) holds tokens {2ty, 2ty+1} x columns {4tx .. 4tx+3})
//   fused: the tiles of W are formed in shared memory and never stored
//          (chunk_fused_readout_kernel, 64-token tiles, described at the kernel)
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

__global__ void __launch_bounds__(256) chunk_readout_kernel(const ReadoutArgs a) {
  const int ti = blockIdx.x / a.r_tiles;
  const int r0 = (blockIdx.x % a.r_tiles) * 64;
  const int64_t n = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
  const int64_t t0 = n * a.T;
  const int64_t len = min(a.T, a.L - t0);
  const int64_t M = a.M, R = a.R;

  __shared__ float ct[32][33];
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
    __syncthreads();
    for (int i = tid; i < 32 * 32; i += 256) {
      int tt = i / 32, kx = i % 32;
      int64_t t = (int64_t)ti * 32 + tt, k = (int64_t)kt * 32 + kx;
      wt[tt][kx] = (t < a.T && k < a.T)
                       ? ld_f32(a.W, ((b * a.N + n) * a.T + t) * a.T + k, a.w_dt) : 0.f;
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

// The fused flavour on 64-token tiles: one block of 256 threads owns a 64(token) x 64(r) tile of h,
// thread (tx, ty) holds tokens 4ty .. 4ty+3 x columns 4tx .. 4tx+3.  Operands are staged transposed
// ([mode][token]) so that a thread reads its four tokens with one 16-byte load.  For every 64-token
// tile of W at or before the block's own: the tile is formed on 4 x 4 register tiles (below the
// diagonal as a plain product of two factors that are both <= 1, reference point = last token of the
// k tile, one exponential per staged element; on the diagonal with one exponential per (t, k, m)),
// written transposed to shared memory, and multiplied with the u tile.  The staging buffers are
// reused for the W tile (the two exponent arrays) and the u tile (the two value arrays).
__global__ void __launch_bounds__(256) chunk_fused_readout_kernel(const ReadoutArgs a) {
  constexpr int kT = 64, kMs = 32, kPad = 68;
  const int ti = blockIdx.x / a.r_tiles;
  const int r0 = (blockIdx.x % a.r_tiles) * 64;
  const int64_t n = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
  const int64_t t0 = n * a.T;
  const int64_t len = min(a.T, a.L - t0);
  const int64_t M = a.M, R = a.R;
  const int64_t tb = (int64_t)ti * kT;

  __shared__ __align__(16) float sm[5][kMs][kPad];
  float (*ct)[kPad] = sm[0], (*kk)[kPad] = sm[1], (*gt)[kPad] = sm[2], (*gk)[kPad] = sm[3], (*kk2)[kPad] = sm[4];
  float (*wT)[kPad] = sm[2];                                      // [k][t], 64 rows: spans sm[2] and sm[3]
  float (*us)[kT] = reinterpret_cast<float (*)[kT]>(&sm[0][0][0]);  // [k][r], 64 x 64 floats inside sm[0..1]

  float acc[4][4] = {};

  // carried part: (c * exp(lcr)) . states_acc^T
  for (int64_t m0 = 0; m0 < M; m0 += kMs) {
    __syncthreads();
    for (int i = tid; i < kT * kMs; i += 256) {
      // a warp takes 8 modes x 4 rows: 32-byte pieces of four rows from memory, 32 distinct banks in the
      // transposed shared-memory arrays (row stride 68 floats)
      const int blk = i >> 5, ln = i & 31;
      const int mm = 8 * (blk & 3) + (ln & 7), rr = 4 * (blk >> 2) + (ln >> 3);
      const int64_t t = tb + rr, m = m0 + mm, r = r0 + rr;
      float v = 0.f;
      if (t < len && m < M)
        v = ld_f32(a.c, b * a.c_sb + (t0 + t) * a.c_sl + m, a.c_dt) * __expf(a.lcr[b * a.g_sb + (t0 + t) * a.g_sl + m]);
      ct[mm][rr] = v;
      kk[mm][rr] = (r < R && m < M) ? ld_f32(a.acc, ((b * a.N + n) * R + r) * M + m, a.a_dt) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int mm = 0; mm < kMs; ++mm) {
      const float4 a4 = *reinterpret_cast<const float4 *>(&ct[mm][4 * ty]);
      const float4 b4 = *reinterpret_cast<const float4 *>(&kk[mm][4 * tx]);
      const float av[4] = {a4.x, a4.y, a4.z, a4.w}, bv[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
  }

  // local part: W . u over the 64-token tiles at or before this one
  for (int kt = 0; kt <= ti; ++kt) {
    const int64_t kb = (int64_t)kt * kT;
    const bool below = kt < ti;
    const int64_t rref = min(kb + kT - 1, len - 1);
    float wacc[4][4] = {};   // W[t = 4ty + i][k = 4tx + j] of this tile
    float dacc = 0.f;        // diagonal tile: entry (4d + i, 4d + j), d = tid / 16, of the register tiles on the diagonal
    for (int64_t m0 = 0; m0 < M; m0 += kMs) {
      __syncthreads();
      for (int i = tid; i < kT * kMs; i += 256) {
        // a warp takes 8 modes x 4 rows: 32-byte pieces of four rows from memory, 32 distinct banks in the
      // transposed shared-memory arrays (row stride 68 floats)
      const int blk = i >> 5, ln = i & 31;
      const int mm = 8 * (blk & 3) + (ln & 7), rr = 4 * (blk >> 2) + (ln >> 3);
        const int64_t m = m0 + mm;
        const bool mv = m < M;
        const int64_t row_t = tb + rr, row_k = kb + rr;
        const int64_t rt = min(row_t, len - 1), rk = min(row_k, len - 1);
        const float g_t = mv ? a.lcr[b * a.g_sb + (t0 + rt) * a.g_sl + m] * kLog2e : 0.f;
        const float g_k = mv ? a.lcr[b * a.g_sb + (t0 + rk) * a.g_sl + m] * kLog2e : 0.f;
        float c_v = (mv && row_t < len) ? ld_f32(a.c, b * a.c_sb + (t0 + row_t) * a.c_sl + m, a.c_dt) : 0.f;
        float k_v = (mv && row_k < len) ? ld_f32(a.kappa, b * a.k_sb + (t0 + row_k) * a.k_sl + m, a.c_dt) : 0.f;
        if (below) {
          const float g_r = mv ? a.lcr[b * a.g_sb + (t0 + rref) * a.g_sl + m] * kLog2e : 0.f;
          c_v *= exp2f(g_t - g_r);
          k_v *= exp2f(g_r - g_k);
        } else {
          gt[mm][rr] = g_t;
          gk[mm][rr] = g_k;
          // kappa taken to the last token of its group of four rows (in lanes 24..31 of this warp)
          const float g_4 = __shfl_sync(0xffffffffu, g_k, 24 + (ln & 7));
          kk2[mm][rr] = k_v * exp2f(fminf(g_4 - g_k, 0.f));
        }
        ct[mm][rr] = c_v;
        kk[mm][rr] = k_v;
      }
      __syncthreads();
      if (below) {
#pragma unroll 8
        for (int mm = 0; mm < kMs; ++mm) {
          const float4 a4 = *reinterpret_cast<const float4 *>(&ct[mm][4 * ty]);
          const float4 b4 = *reinterpret_cast<const float4 *>(&kk[mm][4 * tx]);
          const float av[4] = {a4.x, a4.y, a4.z, a4.w}, bv[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) wacc[i][j] = fmaf(av[i], bv[j], wacc[i][j]);
        }
      } else {
        // the diagonal tile, as in chunk_w.cu: register tiles strictly below the diagonal with the
        // last k of their group as reference point, the 16 register tiles on the diagonal one entry
        // per thread
        if (tx < ty) {
#pragma unroll 4
          for (int mm = 0; mm < kMs; ++mm) {
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
              for (int j = 0; j < 4; ++j) wacc[i][j] = fmaf(av[i], bv[j], wacc[i][j]);
          }
        }
        {
          const int d = tid >> 4, i = (tid >> 2) & 3, j = tid & 3;
          if (j <= i) {
#pragma unroll 8
            for (int mm = 0; mm < kMs; ++mm)
              dacc = fmaf(ct[mm][4 * d + i] * kk[mm][4 * d + j], exp2f(gt[mm][4 * d + i] - gk[mm][4 * d + j]), dacc);
          }
        }
      }
    }
    __syncthreads();   // every thread is done with the staging buffers: they become the W and u tiles
    if (below || tx != ty) {   // (register tiles above the diagonal hold zeros)
#pragma unroll
      for (int j = 0; j < 4; ++j)
        *reinterpret_cast<float4 *>(&wT[4 * tx + j][4 * ty]) = make_float4(wacc[0][j], wacc[1][j], wacc[2][j], wacc[3][j]);
    }
    if (!below) {
      const int d = tid >> 4, i = (tid >> 2) & 3, j = tid & 3;
      wT[4 * d + j][4 * d + i] = (j <= i) ? dacc : 0.f;
    }
    for (int i = tid; i < kT * 64; i += 256) {
      const int kx = i / 64, rr = i % 64;
      const int64_t k = kb + kx, r = r0 + rr;
      us[kx][rr] = (k < len && r < R) ? ld_f32(a.u, b * a.u_sb + (t0 + k) * a.u_sl + r, a.u_dt) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int kx = 0; kx < kT; ++kx) {
      const float4 w4 = *reinterpret_cast<const float4 *>(&wT[kx][4 * ty]);
      const float4 x = *reinterpret_cast<const float4 *>(&us[kx][4 * tx]);
      const float wv[4] = {w4.x, w4.y, w4.z, w4.w}, xv[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(wv[i], xv[j], acc[i][j]);
    }
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t t = tb + 4 * ty + i;
    if (t >= len) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t r = r0 + 4 * tx + j;
      if (r < R) st_f32(a.h, (b * a.L + t0 + t) * R + r, a.u_dt, acc[i][j]);
    }
  }
}

static int launch_readout(bool fused, const ReadoutArgs &a, int64_t B, void *stream) {
  const int tiles = (int)ceil_div(a.T, fused ? 64 : 32);
  if (B > 65535 || a.N > 65535)
    return fail(FRACSSM_ERR_UNSUPPORTED, "chunk_readout: B or N too large for one launch");
  dim3 grid((unsigned)(tiles * a.r_tiles), (unsigned)a.N, (unsigned)B);
  if (fused) chunk_fused_readout_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(a);
  else chunk_readout_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(a);
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

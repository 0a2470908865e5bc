// The two mixer steps next to the scan path that the reference runs in PyTorch:
//   * the causal depthwise convolution + SiLU that produces x_conv
//     (frac_ssm/models/modeling_frac.py:116-140, `_causal_conv_full`);
//   * the single-token state update of the decode loop
//     (frac_ssm/models/modeling_frac.py:159-179, `_update_state`, and the D skip of :236).
// Both are bandwidth kernels: every input element is read once, every output written once.
#include "common.cuh"

namespace fracssm {
namespace {

__device__ __forceinline__ float silu_(float x) { return x / (1.f + __expf(-x)); }

constexpr int kConvMaxK = 8;     // kernel widths 1..8
constexpr int kConvTokens = 32;  // tokens per thread: the window slides in registers

// General path: one channel per thread, any dtype.  grid (ceil(C/128), ceil(L/kConvTokens), B).
__global__ void __launch_bounds__(128)
causal_conv_silu_kernel(const void *__restrict__ x, int x_dt, int64_t x_sb, int64_t x_sl,
                        const float *__restrict__ mask, int64_t m_sb, int64_t m_sl,
                        const void *__restrict__ w, int w_dt, const void *__restrict__ bias, int K,
                        void *__restrict__ y, int y_dt, void *__restrict__ u_heads, int64_t R, int64_t L,
                        int64_t C) {
  const int64_t ch = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (ch >= C) return;
  const int64_t H = u_heads ? C / R : 0, hh = u_heads ? ch / R : 0, rr = u_heads ? ch % R : 0;
  const int64_t b = blockIdx.z, l0 = (int64_t)blockIdx.y * kConvTokens;
  float wk[kConvMaxK], win[kConvMaxK];
#pragma unroll
  for (int k = 0; k < kConvMaxK; ++k) wk[k] = k < K ? ld_f32(w, ch * K + k, w_dt) : 0.f;
  const float bv = bias ? ld_f32(bias, ch, w_dt) : 0.f;
  auto in = [&](int64_t l) -> float {
    if (l < 0) return 0.f;
    float v = ld_f32(x, b * x_sb + l * x_sl + ch, x_dt);
    if (mask) v *= mask[b * m_sb + l * m_sl];
    return v;
  };
  // win[k] pairs with wk[k]: win[K-1] is the current token, win[0] the oldest one
#pragma unroll
  for (int k = 0; k < kConvMaxK; ++k) win[k] = (k < K - 1) ? in(l0 - (K - 1) + k) : 0.f;
  const int64_t l1 = min(l0 + kConvTokens, L);
  for (int64_t l = l0; l < l1; ++l) {
    const float cur = in(l);
    float acc = bv;
#pragma unroll
    for (int k = 0; k < kConvMaxK; ++k) {
      if (k < K - 1) acc = fmaf(wk[k], win[k], acc);
      else if (k == K - 1) acc = fmaf(wk[k], cur, acc);
    }
    const float out = silu_(acc);
    st_f32(y, (b * L + l) * C + ch, y_dt, out);
    if (u_heads) st_f32(u_heads, ((b * H + hh) * L + l) * R + rr, y_dt, out);
#pragma unroll
    for (int k = 0; k < kConvMaxK - 1; ++k) {
      if (k < K - 2) win[k] = win[k + 1];
      else if (k == K - 2) win[k] = cur;
    }
  }
}

// bf16 path for the usual width 4.
__device__ __forceinline__ void unpack8(const uint4 &p, float (&f)[8]) {
  const uint32_t wds[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(wds[i] << 16);
    f[2 * i + 1] = __uint_as_float(wds[i] & 0xFFFF0000u);
  }
}

__device__ __forceinline__ void unpack4(const uint2 &p, float (&f)[4]) {
  f[0] = __uint_as_float(p.x << 16);
  f[1] = __uint_as_float(p.x & 0xFFFF0000u);
  f[2] = __uint_as_float(p.y << 16);
  f[3] = __uint_as_float(p.y & 0xFFFF0000u);
}

// Four channels (8 bytes) per thread, kConvTokens tokens walked with the window in registers, the next
// four tokens requested before the current four are worked on; at most 80 registers, so 6 blocks of
// 128 threads per SM.  At batch 16 x 4096 tokens x 1536 channels: 0.154 ms with 16 tokens per thread and
// the loads of a group issued right before their use, 0.143 ms with 32 tokens (the three window tokens and
// the weights are read once per 32), 0.125 ms with the loads one group ahead.
__global__ void __launch_bounds__(128, 6)
causal_conv4_silu_bf16_kernel(const __nv_bfloat16 *__restrict__ x, int64_t x_sb, int64_t x_sl,
                              const float *__restrict__ mask, int64_t m_sb, int64_t m_sl,
                              const void *__restrict__ w, int w_dt, const void *__restrict__ bias,
                              __nv_bfloat16 *__restrict__ y, __nv_bfloat16 *__restrict__ u_heads, int64_t R,
                              int64_t L, int64_t C) {
  const int64_t ch = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (ch >= C) return;
  // the same four values also go to the head-major copy [Bt * H, L, R] (R a multiple of 4)
  __nv_bfloat16 *u_row = nullptr;
  if (u_heads) u_row = u_heads + ((int64_t)blockIdx.z * (C / R) + ch / R) * L * R + ch % R;
  const int64_t b = blockIdx.z, l0 = (int64_t)blockIdx.y * kConvTokens;
  float wk[4][4], bv[4], w0[4], w1[4], w2[4];
  if (w_dt == FRACSSM_BF16) {   // 4 channels x 4 taps = 32 contiguous bytes (ch is a multiple of 4)
    const uint4 *wp = reinterpret_cast<const uint4 *>(reinterpret_cast<const __nv_bfloat16 *>(w) + ch * 4);
#pragma unroll
    for (int q = 0; q < 2; ++q) {   // piece q holds channels 2q, 2q + 1
      float f[8];
      unpack8(__ldg(wp + q), f);
#pragma unroll
      for (int k = 0; k < 4; ++k) { wk[k][2 * q] = f[k]; wk[k][2 * q + 1] = f[4 + k]; }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
      for (int k = 0; k < 4; ++k) wk[k][i] = ld_f32(w, (ch + i) * 4 + k, w_dt);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) bv[i] = bias ? ld_f32(bias, ch + i, w_dt) : 0.f;
  auto in = [&](int64_t l, float (&f)[4]) {
    if (l < 0) {
#pragma unroll
      for (int i = 0; i < 4; ++i) f[i] = 0.f;
      return;
    }
    unpack4(__ldcs(reinterpret_cast<const uint2 *>(x + b * x_sb + l * x_sl + ch)), f);
    if (mask) {
      const float m = mask[b * m_sb + l * m_sl];
#pragma unroll
      for (int i = 0; i < 4; ++i) f[i] *= m;
    }
  };
  in(l0 - 3, w0);
  in(l0 - 2, w1);
  in(l0 - 1, w2);
  const int64_t l1 = min(l0 + kConvTokens, L);
  // the next four tokens are requested before the current four are worked on
  uint2 nraw[4];
  float nmk[4];
  auto request = [&](int64_t lg) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      nraw[j] = make_uint2(0u, 0u);
      nmk[j] = 1.f;
      if (lg + j < l1) {
        nraw[j] = __ldcs(reinterpret_cast<const uint2 *>(x + b * x_sb + (lg + j) * x_sl + ch));
        if (mask) nmk[j] = mask[b * m_sb + (lg + j) * m_sl];
      }
    }
  };
  request(l0);
  for (int64_t lg = l0; lg < l1; lg += 4) {
    uint2 raw[4];
    float mk[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) { raw[j] = nraw[j]; mk[j] = nmk[j]; }
    if (lg + 4 < l1) request(lg + 4);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (lg + j < l1) {
        const int64_t l = lg + j;
        float cur[4];
        unpack4(raw[j], cur);
        if (mask) {
#pragma unroll
          for (int i = 0; i < 4; ++i) cur[i] *= mk[j];
        }
        uint32_t o[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          float r[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int c = 2 * i + e;
            float acc = bv[c];
            acc = fmaf(wk[0][c], w0[c], acc);
            acc = fmaf(wk[1][c], w1[c], acc);
            acc = fmaf(wk[2][c], w2[c], acc);
            acc = fmaf(wk[3][c], cur[c], acc);
            r[e] = __fdividef(acc, 1.f + __expf(-acc));   // silu, about 2 ulp: the output is bf16
          }
          const __nv_bfloat162 t = __floats2bfloat162_rn(r[0], r[1]);
          o[i] = *reinterpret_cast<const uint32_t *>(&t);
        }
        __stcs(reinterpret_cast<uint2 *>(y + (b * L + l) * C + ch), make_uint2(o[0], o[1]));
        if (u_row) __stcs(reinterpret_cast<uint2 *>(u_row + l * R), make_uint2(o[0], o[1]));
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          w0[i] = w1[i];
          w1[i] = w2[i];
          w2[i] = cur[i];
        }
      }
    }
  }
}

// One token of the recurrence for every (batch, head): state [M, R] float32 updated in place,
//   state[m, r] = rho[m] * state[m, r] + kappa[m] * u[r];  out[r] = sum_m c[m] * state[m, r] + u[r] * D[r].
// One block per (batch, head); thread r-lane strides over R, the modes are walked in the block's
// y dimension and reduced through shared memory.
__global__ void __launch_bounds__(256)
decode_step_kernel(const void *__restrict__ u, int u_dt, const float *__restrict__ c,
                   const float *__restrict__ kappa, const float *__restrict__ rho,
                   const float *__restrict__ Dp, float *__restrict__ state, float *__restrict__ out,
                   int64_t H, int64_t R, int64_t M) {
  extern __shared__ float part[];  // [blockDim.y][R]
  const int64_t bh = blockIdx.x, h = bh % H;
  const int ty = threadIdx.y, ny = blockDim.y;
  float *st = state + bh * M * R;
  for (int64_t r = threadIdx.x; r < R; r += blockDim.x) {
    const float ur = ld_f32(u, bh * R + r, u_dt);
    float acc = 0.f;
    for (int64_t m = ty; m < M; m += ny) {
      const float s = fmaf(rho[bh * M + m], st[m * R + r], kappa[bh * M + m] * ur);
      st[m * R + r] = s;
      acc = fmaf(c[bh * M + m], s, acc);
    }
    part[ty * R + r] = acc;
  }
  __syncthreads();
  if (ty == 0) {
    for (int64_t r = threadIdx.x; r < R; r += blockDim.x) {
      float acc = 0.f;
      for (int y = 0; y < ny; ++y) acc += part[y * R + r];
      out[bh * R + r] = acc + ld_f32(u, bh * R + r, u_dt) * Dp[h * R + r];
    }
  }
}

}  // namespace
}  // namespace fracssm

extern "C" int fracssm_causal_conv_silu(const void *x, int x_dtype, int64_t x_sb, int64_t x_sl,
                                        const float *mask, int64_t m_sb, int64_t m_sl,
                                        const void *weight, const void *bias, int w_dtype, void *y,
                                        int y_dtype, int64_t Bt, int64_t L, int64_t C, int64_t K,
                                        void *stream) {
  return fracssm_causal_conv_silu_heads(x, x_dtype, x_sb, x_sl, mask, m_sb, m_sl, weight, bias, w_dtype, y, y_dtype,
                                        nullptr, 0, Bt, L, C, K, stream);
}

extern "C" int fracssm_causal_conv_silu_heads(const void *x, int x_dtype, int64_t x_sb, int64_t x_sl,
                                              const float *mask, int64_t m_sb, int64_t m_sl,
                                              const void *weight, const void *bias, int w_dtype, void *y,
                                              int y_dtype, void *u_heads, int64_t R, int64_t Bt, int64_t L,
                                              int64_t C, int64_t K, void *stream) {
  using namespace fracssm;
  if (u_heads && (R <= 0 || C % R != 0))
    return fail(FRACSSM_ERR_ARG, "causal_conv_silu: the head width must divide the channel count");
  if (Bt < 0 || L < 0 || C <= 0 || K < 1 || K > kConvMaxK) return fail(FRACSSM_ERR_ARG, "causal_conv_silu: bad sizes (kernel width 1..8)");
  if (!known_dtype(x_dtype) || !known_dtype(w_dtype) || !known_dtype(y_dtype))
    return fail(FRACSSM_ERR_ARG, "causal_conv_silu: unsupported dtype");
  if (Bt == 0 || L == 0) return FRACSSM_OK;
  if (!x || !weight || !y) return fail(FRACSSM_ERR_ARG, "causal_conv_silu: null pointer");
  if (Bt > 65535 || ceil_div(L, kConvTokens) > 65535)
    return fail(FRACSSM_ERR_UNSUPPORTED, "causal_conv_silu: batch or sequence too large for one launch");
  auto al16 = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const dim3 block(128);
  if (K == 4 && x_dtype == FRACSSM_BF16 && y_dtype == FRACSSM_BF16 && C % 8 == 0 && al16(x) && al16(y) &&
      x_sb % 8 == 0 && x_sl % 8 == 0 && (!u_heads || (R % 8 == 0 && al16(u_heads))) &&
      (w_dtype != FRACSSM_BF16 || al16(weight))) {
    const dim3 grid((unsigned)ceil_div(C / 4, 128), (unsigned)ceil_div(L, kConvTokens), (unsigned)Bt);
    causal_conv4_silu_bf16_kernel<<<grid, block, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const __nv_bfloat16 *>(x), x_sb, x_sl, mask, m_sb, m_sl, weight, w_dtype, bias,
        reinterpret_cast<__nv_bfloat16 *>(y), reinterpret_cast<__nv_bfloat16 *>(u_heads), R, L, C);
    return check_launch("causal_conv_silu");
  }
  const dim3 grid((unsigned)ceil_div(C, 128), (unsigned)ceil_div(L, kConvTokens), (unsigned)Bt);
  causal_conv_silu_kernel<<<grid, block, 0, (cudaStream_t)stream>>>(x, x_dtype, x_sb, x_sl, mask, m_sb, m_sl, weight,
                                                                 w_dtype, bias, (int)K, y, y_dtype, u_heads, R, L, C);
  return check_launch("causal_conv_silu");
}

extern "C" int fracssm_decode_step(const void *u, int u_dtype, const float *c, const float *kappa,
                                   const float *rho, const float *D, float *state, float *out,
                                   int64_t Bt, int64_t H, int64_t R, int64_t M, void *stream) {
  using namespace fracssm;
  if (Bt < 0 || H <= 0 || R <= 0 || M <= 0) return fail(FRACSSM_ERR_ARG, "decode_step: bad sizes");
  if (!known_dtype(u_dtype)) return fail(FRACSSM_ERR_ARG, "decode_step: unsupported dtype");
  if (Bt == 0) return FRACSSM_OK;
  if (!u || !c || !kappa || !rho || !D || !state || !out) return fail(FRACSSM_ERR_ARG, "decode_step: null pointer");
  int tx = 32;
  while (tx < R && tx < 256) tx *= 2;
  int ty = 256 / tx;
  if (ty > M) ty = (int)M;
  if (ty < 1) ty = 1;
  const size_t smem = (size_t)ty * R * sizeof(float);
  if (smem > 48 * 1024) return fail(FRACSSM_ERR_UNSUPPORTED, "decode_step: head_dim too large");
  decode_step_kernel<<<(unsigned)(Bt * H), dim3(tx, ty), smem, (cudaStream_t)stream>>>(u, u_dtype, c, kappa, rho, D,
                                                                                     state, out, H, R, M);
  return check_launch("decode_step");
}

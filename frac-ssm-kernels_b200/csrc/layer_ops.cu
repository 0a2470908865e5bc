// Bandwidth-bound layer stages around the scan: parameter prep, skip-mix, gated RMSNorm,
// and the skip-mix + gated-RMSNorm epilogue in one pass.
#include "common.cuh"

namespace fracssm {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float softplusf_(float x) { return x > 20.f ? x : log1pf(expf(x)); }

struct ParamArgs {
  const void *dyn; int dyn_dt; int64_t dyn_sb, dyn_sl;
  const void *rw; int rw_dt; int64_t rw_sb, rw_sl;
  const void *x; int x_dt; int64_t x_sb, x_sl;
  const float *mask; int64_t m_sb, m_sl;
  const float *dt_bias, *log_tau;
  const float *read_logit, *write_logit;   // the two gate parameters, one float each, on the device
  float inv_read_temp, dt_min, dt_max, a_min, a_max, l_min, l_max;
  void *u, *c, *kappa; int ck_dt; float *rho;
  int64_t L, H, R, M;
};

// One warp per (bh, token): lanes stride over the M modes; two softmaxes by warp shuffles.
__global__ void __launch_bounds__(128) compute_params_kernel(const ParamArgs a) {
  const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
  const float read_gate = sigmoidf_(__ldg(a.read_logit)), write_gate = sigmoidf_(__ldg(a.write_logit));
  const int64_t l = (int64_t)blockIdx.x * 4 + warp;
  const int64_t bh = blockIdx.y;
  if (l >= a.L) return;
  const int64_t b = bh / a.H, h = bh % a.H;
  const int64_t H = a.H, M = a.M, R = a.R;

  const int64_t dbase = b * a.dyn_sb + l * a.dyn_sl;
  float dt = softplusf_(ld_f32(a.dyn, dbase + h, a.dyn_dt) + a.dt_bias[h]);
  dt = fminf(fmaxf(dt, a.dt_min), a.dt_max);
  const float alpha = a.a_min + sigmoidf_(ld_f32(a.dyn, dbase + H + h, a.dyn_dt)) * (a.a_max - a.a_min);
  const float lam = a.l_min + sigmoidf_(ld_f32(a.dyn, dbase + 2 * H + h, a.dyn_dt)) * (a.l_max - a.l_min);
  const float rate = powf(fmaxf(lam, 1e-4f), 1.f / fmaxf(alpha, 1e-4f));
  const float keep = a.mask ? a.mask[b * a.m_sb + l * a.m_sl] : 1.f;

  const int64_t rbase = b * a.rw_sb + l * a.rw_sl + h * M;       // read residuals
  const int64_t wbase = rbase + H * M;                            // write residuals
  float rmax = -INFINITY, wmax = -INFINITY;
  for (int64_t m = lane; m < M; m += 32) {
    const float prior = -alpha * a.log_tau[m];
    rmax = fmaxf(rmax, (prior + read_gate * ld_f32(a.rw, rbase + m, a.rw_dt)) * a.inv_read_temp);
    wmax = fmaxf(wmax, prior + write_gate * ld_f32(a.rw, wbase + m, a.rw_dt));
  }
  rmax = warp_max(rmax);
  wmax = warp_max(wmax);
  float rsum = 0.f, wsum = 0.f;
  for (int64_t m = lane; m < M; m += 32) {
    const float prior = -alpha * a.log_tau[m];
    rsum += __expf((prior + read_gate * ld_f32(a.rw, rbase + m, a.rw_dt)) * a.inv_read_temp - rmax);
    wsum += __expf(prior + write_gate * ld_f32(a.rw, wbase + m, a.rw_dt) - wmax);
  }
  const float rinv = 1.f / warp_sum(rsum), winv = 1.f / warp_sum(wsum);
  const int64_t obase = (bh * a.L + l) * M;
  for (int64_t m = lane; m < M; m += 32) {
    const float lt = a.log_tau[m];
    const float prior = -alpha * lt;
    const float cw = __expf((prior + read_gate * ld_f32(a.rw, rbase + m, a.rw_dt)) * a.inv_read_temp - rmax) * rinv;
    const float ww = __expf(prior + write_gate * ld_f32(a.rw, wbase + m, a.rw_dt) - wmax) * winv;
    float rho = expf(-dt * (rate / fmaxf(expf(lt), 1e-6f)));
    rho = fminf(fmaxf(rho, 1e-6f), 1.f - 1e-6f);
    float kap = (1.f - rho) * ww;
    if (a.mask) { kap *= keep; rho = rho * keep + (1.f - keep); }
    st_f32(a.c, obase + m, a.ck_dt, cw);
    st_f32(a.kappa, obase + m, a.ck_dt, kap);
    a.rho[obase + m] = rho;
  }
  if (a.u) {   // (no copy when the caller already holds the head-major u, e.g. from the conv kernel)
    const int64_t xbase = b * a.x_sb + l * a.x_sl + h * R;
    for (int64_t r = lane; r < R; r += 32)
      st_f32(a.u, (bh * a.L + l) * R + r, a.x_dt, ld_f32(a.x, xbase + r, a.x_dt));
  }
}

// The same prep for M = 128 with bf16 projections: one warp walks kPrepTokens tokens of one (b, h);
// each lane owns four consecutive modes, so a token's read / write residuals are one 8-byte load per
// lane each, everything stays in registers (one pass), and c / kappa / rho go out as 8- or 16-byte
// stores.  Same formulas, in the same order, as compute_params_kernel.
constexpr int kPrepTokens = 8;

__device__ __forceinline__ void unpack4(const uint2 &p, float (&f)[4]) {
  f[0] = __uint_as_float(p.x << 16);
  f[1] = __uint_as_float(p.x & 0xFFFF0000u);
  f[2] = __uint_as_float(p.y << 16);
  f[3] = __uint_as_float(p.y & 0xFFFF0000u);
}

__global__ void __launch_bounds__(128) compute_params_m128_kernel(const ParamArgs a) {
  const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
  const float read_gate = sigmoidf_(__ldg(a.read_logit)), write_gate = sigmoidf_(__ldg(a.write_logit));
  const int64_t l0 = ((int64_t)blockIdx.x * 4 + warp) * kPrepTokens;
  const int64_t bh = blockIdx.y;
  if (l0 >= a.L) return;
  const int64_t b = bh / a.H, h = bh % a.H;
  const int64_t H = a.H, R = a.R;
  constexpr int64_t M = 128;
  float lt[4], inv_tau[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    lt[i] = a.log_tau[4 * lane + i];
    inv_tau[i] = 1.f / fmaxf(expf(lt[i]), 1e-6f);
  }
  const float dtb = a.dt_bias[h];
  const __nv_bfloat16 *rw = reinterpret_cast<const __nv_bfloat16 *>(a.rw);
  const int64_t l1 = min(l0 + kPrepTokens, a.L);
  // the per-token scalars (step, alpha, rate, mask) are computed once, by lane t for token l0 + t,
  // and handed to the other lanes by shuffles
  float dt_l = 0.f, alpha_l = 0.f, rate_l = 0.f, keep_l = 1.f;
  if (lane < kPrepTokens && l0 + lane < l1) {
    const int64_t l = l0 + lane, dbase = b * a.dyn_sb + l * a.dyn_sl;
    dt_l = softplusf_(ld_f32(a.dyn, dbase + h, a.dyn_dt) + dtb);
    dt_l = fminf(fmaxf(dt_l, a.dt_min), a.dt_max);
    alpha_l = a.a_min + sigmoidf_(ld_f32(a.dyn, dbase + H + h, a.dyn_dt)) * (a.a_max - a.a_min);
    const float lam = a.l_min + sigmoidf_(ld_f32(a.dyn, dbase + 2 * H + h, a.dyn_dt)) * (a.l_max - a.l_min);
    rate_l = powf(fmaxf(lam, 1e-4f), 1.f / fmaxf(alpha_l, 1e-4f));
    if (a.mask) keep_l = a.mask[b * a.m_sb + l * a.m_sl];
  }
  for (int64_t l = l0; l < l1; ++l) {
    const int src = static_cast<int>(l - l0);
    const float dt = __shfl_sync(0xffffffffu, dt_l, src), alpha = __shfl_sync(0xffffffffu, alpha_l, src);
    const float rate = __shfl_sync(0xffffffffu, rate_l, src), keep = __shfl_sync(0xffffffffu, keep_l, src);

    const __nv_bfloat16 *rp = rw + b * a.rw_sb + l * a.rw_sl + h * M + 4 * lane;
    float rres[4], wres[4], rl[4], wl[4];
    unpack4(__ldcs(reinterpret_cast<const uint2 *>(rp)), rres);
    unpack4(__ldcs(reinterpret_cast<const uint2 *>(rp + H * M)), wres);
    float rmax = -INFINITY, wmax = -INFINITY;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float prior = -alpha * lt[i];
      rl[i] = (prior + read_gate * rres[i]) * a.inv_read_temp;
      wl[i] = prior + write_gate * wres[i];
      rmax = fmaxf(rmax, rl[i]);
      wmax = fmaxf(wmax, wl[i]);
    }
    rmax = warp_max(rmax);
    wmax = warp_max(wmax);
    float rsum = 0.f, wsum = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      rl[i] = __expf(rl[i] - rmax);
      wl[i] = __expf(wl[i] - wmax);
      rsum += rl[i];
      wsum += wl[i];
    }
    const float rinv = 1.f / warp_sum(rsum), winv = 1.f / warp_sum(wsum);
    float cw[4], kap[4], rho[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      cw[i] = rl[i] * rinv;
      float r = expf(-dt * (rate * inv_tau[i]));
      r = fminf(fmaxf(r, 1e-6f), 1.f - 1e-6f);
      float k = (1.f - r) * (wl[i] * winv);
      if (a.mask) { k *= keep; r = r * keep + (1.f - keep); }
      kap[i] = k;
      rho[i] = r;
    }
    const int64_t obase = (bh * a.L + l) * M + 4 * lane;
    __stcs(reinterpret_cast<float4 *>(a.rho + obase), make_float4(rho[0], rho[1], rho[2], rho[3]));
    if (a.ck_dt == FRACSSM_F32) {
      __stcs(reinterpret_cast<float4 *>(reinterpret_cast<float *>(a.c) + obase), make_float4(cw[0], cw[1], cw[2], cw[3]));
      __stcs(reinterpret_cast<float4 *>(reinterpret_cast<float *>(a.kappa) + obase),
             make_float4(kap[0], kap[1], kap[2], kap[3]));
    } else {  // bf16
      const __nv_bfloat162 c0 = __floats2bfloat162_rn(cw[0], cw[1]), c1 = __floats2bfloat162_rn(cw[2], cw[3]);
      const __nv_bfloat162 k0 = __floats2bfloat162_rn(kap[0], kap[1]), k1 = __floats2bfloat162_rn(kap[2], kap[3]);
      __stcs(reinterpret_cast<uint2 *>(reinterpret_cast<__nv_bfloat16 *>(a.c) + obase),
             make_uint2(*reinterpret_cast<const uint32_t *>(&c0), *reinterpret_cast<const uint32_t *>(&c1)));
      __stcs(reinterpret_cast<uint2 *>(reinterpret_cast<__nv_bfloat16 *>(a.kappa) + obase),
             make_uint2(*reinterpret_cast<const uint32_t *>(&k0), *reinterpret_cast<const uint32_t *>(&k1)));
    }
    if (a.u) {
      const int64_t xbase = b * a.x_sb + l * a.x_sl + h * R;
      for (int64_t r = lane; r < R; r += 32)
        st_f32(a.u, (bh * a.L + l) * R + r, a.x_dt, ld_f32(a.x, xbase + r, a.x_dt));
    }
  }
}

// The M = 128 prep with fewer instructions per token: a half-warp owns a token (a lane eight
// consecutive modes: one 16-byte load per residual row, 16- and 32-byte stores), so a warp works on
// two tokens at a time, the softmax reductions take four shuffle steps instead of five, and the
// address arithmetic, the shuffles of the per-token scalars and the loop are paid once per two tokens
// and eight modes per lane.  The kernel above issues about 250 warp instructions per token, of which
// about 50 are the per-mode arithmetic; this one about 95.  Measured at batch 16 x 4096 tokens x 24 heads:
// 0.598 ms for the kernel above, 0.571 with this layout at 8 tokens per warp, 0.508 at 32 tokens per warp
// (the per-warp setup paid less often), 0.470 with the next pair's rows requested one step ahead.
__device__ __forceinline__ float half_warp_max(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ void unpack8(const uint4 &p, float (&f)[8]) {
  const uint32_t w[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t *>(&v);
}

// tokens per warp: one lane computes the per-token scalars of one token, and the per-warp setup (the
// time constants, the gates) is paid once per 32 tokens
constexpr int kPairTokens = 32;

__global__ void __launch_bounds__(128) compute_params_m128_pair_kernel(const ParamArgs a) {
  const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
  const int sub = lane >> 4, q = lane & 15;  // token of the pair; modes 8 q .. 8 q + 7
  const float read_gate = sigmoidf_(__ldg(a.read_logit)), write_gate = sigmoidf_(__ldg(a.write_logit));
  const int64_t l0 = ((int64_t)blockIdx.x * 4 + warp) * kPairTokens;
  const int64_t bh = blockIdx.y;
  if (l0 >= a.L) return;
  const int64_t b = bh / a.H, h = bh % a.H;
  const int64_t H = a.H, R = a.R;
  constexpr int64_t M = 128;
  float lt[8], inv_tau[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    lt[i] = a.log_tau[8 * q + i];
    inv_tau[i] = 1.f / fmaxf(expf(lt[i]), 1e-6f);
  }
  const float dtb = a.dt_bias[h];
  const __nv_bfloat16 *rw = reinterpret_cast<const __nv_bfloat16 *>(a.rw);
  const int64_t l1 = min(l0 + kPairTokens, a.L);
  // per-token scalars: computed once, by lane t for token l0 + t, handed over by shuffles
  float dt_l = 0.f, alpha_l = 0.f, rate_l = 0.f, keep_l = 1.f;
  if (lane < kPairTokens && l0 + lane < l1) {
    const int64_t l = l0 + lane, dbase = b * a.dyn_sb + l * a.dyn_sl;
    dt_l = softplusf_(ld_f32(a.dyn, dbase + h, a.dyn_dt) + dtb);
    dt_l = fminf(fmaxf(dt_l, a.dt_min), a.dt_max);
    alpha_l = a.a_min + sigmoidf_(ld_f32(a.dyn, dbase + H + h, a.dyn_dt)) * (a.a_max - a.a_min);
    const float lam = a.l_min + sigmoidf_(ld_f32(a.dyn, dbase + 2 * H + h, a.dyn_dt)) * (a.l_max - a.l_min);
    rate_l = powf(fmaxf(lam, 1e-4f), 1.f / fmaxf(alpha_l, 1e-4f));
    if (a.mask) keep_l = a.mask[b * a.m_sb + l * a.m_sl];
  }
  // the residual rows of the next pair of tokens are requested before this pair is worked on
  uint4 rnext = make_uint4(0, 0, 0, 0), wnext = make_uint4(0, 0, 0, 0);
  const __nv_bfloat16 *rp0 = rw + b * a.rw_sb + h * M + 8 * q;
  if (l0 + sub < l1) {
    rnext = __ldcs(reinterpret_cast<const uint4 *>(rp0 + (l0 + sub) * a.rw_sl));
    wnext = __ldcs(reinterpret_cast<const uint4 *>(rp0 + (l0 + sub) * a.rw_sl + H * M));
  }
#pragma unroll 1
  for (int it = 0; it < kPairTokens / 2; ++it) {
    if (l0 + 2 * it >= l1) break;
    const int src = 2 * it + sub;
    const int64_t l = l0 + src;
    const bool live = l < l1;
    const float dt = __shfl_sync(0xffffffffu, dt_l, src), alpha = __shfl_sync(0xffffffffu, alpha_l, src);
    const float rate = __shfl_sync(0xffffffffu, rate_l, src), keep = __shfl_sync(0xffffffffu, keep_l, src);
    float rl[8], wl[8];
    {
      const uint4 rraw = rnext, wraw = wnext;
      if (l + 2 < l1 && it + 1 < kPairTokens / 2) {
        rnext = __ldcs(reinterpret_cast<const uint4 *>(rp0 + (l + 2) * a.rw_sl));
        wnext = __ldcs(reinterpret_cast<const uint4 *>(rp0 + (l + 2) * a.rw_sl + H * M));
      }
      unpack8(rraw, rl);
      unpack8(wraw, wl);
    }
    float rmax = -INFINITY, wmax = -INFINITY;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float prior = -alpha * lt[i];
      rl[i] = (prior + read_gate * rl[i]) * a.inv_read_temp;
      wl[i] = prior + write_gate * wl[i];
      rmax = fmaxf(rmax, rl[i]);
      wmax = fmaxf(wmax, wl[i]);
    }
    rmax = half_warp_max(rmax);
    wmax = half_warp_max(wmax);
    float rsum = 0.f, wsum = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      rl[i] = __expf(rl[i] - rmax);
      wl[i] = __expf(wl[i] - wmax);
      rsum += rl[i];
      wsum += wl[i];
    }
    const float rinv = 1.f / half_warp_sum(rsum), winv = 1.f / half_warp_sum(wsum);
    float rho[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      rl[i] *= rinv;                                    // c
      float r = expf(-dt * (rate * inv_tau[i]));
      r = fminf(fmaxf(r, 1e-6f), 1.f - 1e-6f);
      float k = (1.f - r) * (wl[i] * winv);
      if (a.mask) { k *= keep; r = r * keep + (1.f - keep); }
      wl[i] = k;                                        // kappa
      rho[i] = r;
    }
    if (live) {
      const int64_t obase = (bh * a.L + l) * M + 8 * q;
      float4 *rp4 = reinterpret_cast<float4 *>(a.rho + obase);
      __stcs(rp4, make_float4(rho[0], rho[1], rho[2], rho[3]));
      __stcs(rp4 + 1, make_float4(rho[4], rho[5], rho[6], rho[7]));
      if (a.ck_dt == FRACSSM_F32) {
        float4 *cp4 = reinterpret_cast<float4 *>(reinterpret_cast<float *>(a.c) + obase);
        float4 *kp4 = reinterpret_cast<float4 *>(reinterpret_cast<float *>(a.kappa) + obase);
        __stcs(cp4, make_float4(rl[0], rl[1], rl[2], rl[3]));
        __stcs(cp4 + 1, make_float4(rl[4], rl[5], rl[6], rl[7]));
        __stcs(kp4, make_float4(wl[0], wl[1], wl[2], wl[3]));
        __stcs(kp4 + 1, make_float4(wl[4], wl[5], wl[6], wl[7]));
      } else {  // bf16
        __stcs(reinterpret_cast<uint4 *>(reinterpret_cast<__nv_bfloat16 *>(a.c) + obase),
               make_uint4(pack_bf16x2(rl[0], rl[1]), pack_bf16x2(rl[2], rl[3]), pack_bf16x2(rl[4], rl[5]),
                          pack_bf16x2(rl[6], rl[7])));
        __stcs(reinterpret_cast<uint4 *>(reinterpret_cast<__nv_bfloat16 *>(a.kappa) + obase),
               make_uint4(pack_bf16x2(wl[0], wl[1]), pack_bf16x2(wl[2], wl[3]), pack_bf16x2(wl[4], wl[5]),
                          pack_bf16x2(wl[6], wl[7])));
      }
      if (a.u) {
        const int64_t xbase = b * a.x_sb + l * a.x_sl + h * R;
        for (int64_t r = q; r < R; r += 16)
          st_f32(a.u, (bh * a.L + l) * R + r, a.x_dt, ld_f32(a.x, xbase + r, a.x_dt));
      }
    }
  }
}

__global__ void __launch_bounds__(256)
skip_mix_kernel(const void *__restrict__ mf, int mf_dt, int64_t mf_sb, int64_t mf_sl,
                const void *__restrict__ x, int x_dt, int64_t x_sb, int64_t x_sl,
                const float *__restrict__ D, void *__restrict__ out, int o_dt, int64_t L, int64_t H,
                int64_t R) {
  const int64_t HR = H * R;
  const int64_t row = blockIdx.x;  // b * L + l
  const int64_t b = row / L, l = row % L;
  for (int64_t j = threadIdx.x; j < HR; j += blockDim.x) {
    const int64_t h = j / R, r = j % R;
    const float v = ld_f32(mf, (b * H + h) * mf_sb + l * mf_sl + r, mf_dt) +
                    ld_f32(x, b * x_sb + l * x_sl + j, x_dt) * D[j];
    st_f32(out, row * HR + j, o_dt, v);
  }
}

__device__ __forceinline__ float block_sum(float v, float *red) {
  v = warp_sum(v);
  const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (threadIdx.x < blockDim.x / 32) ? red[threadIdx.x] : 0.f;
  if (warp == 0) {
    t = warp_sum(t);
    if (lane == 0) red[0] = t;
  }
  __syncthreads();
  t = red[0];
  __syncthreads();
  return t;
}

// One block per row.
__global__ void __launch_bounds__(256)
rmsnorm_gated_kernel(const void *__restrict__ x, int64_t x_srow, const void *__restrict__ gate,
                     int64_t g_srow, int dt, const void *__restrict__ w, int w_dt, float eps,
                     void *__restrict__ y, float *__restrict__ rstd, int64_t D) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  float ss = 0.f;
  for (int64_t j = threadIdx.x; j < D; j += blockDim.x) {
    float v = ld_f32(x, row * x_srow + j, dt);
    if (gate) { const float z = ld_f32(gate, row * g_srow + j, dt); v *= z * sigmoidf_(z); }
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float rs = rsqrtf(ss / (float)D + eps);
  if (rstd && threadIdx.x == 0) rstd[row] = rs;
  for (int64_t j = threadIdx.x; j < D; j += blockDim.x) {
    float v = ld_f32(x, row * x_srow + j, dt);
    if (gate) { const float z = ld_f32(gate, row * g_srow + j, dt); v *= z * sigmoidf_(z); }
    st_f32(y, row * D + j, dt, v * rs * ld_f32(w, j, w_dt));
  }
}

// bf16 fast path: one warp per row, the row (up to 2048 elements) held in registers as 16-byte
// pieces, so x and the gate are read once; four rows per block.  The weight is read as one or two
// 16-byte pieces per chunk (WVEC 1: bf16, 2: f32; 0: element by element, any type): eight 2-byte loads
// with a run-time type switch per chunk made the kernel instruction-bound.
template <int WVEC>
__global__ void __launch_bounds__(128)
rmsnorm_gated_bf16_kernel(const __nv_bfloat16 *__restrict__ x, int64_t x_srow,
                          const __nv_bfloat16 *__restrict__ gate, int64_t g_srow, const void *__restrict__ w,
                          int w_dt, float eps, __nv_bfloat16 *__restrict__ y, float *__restrict__ rstd,
                          int64_t rows, int64_t D) {
  const int lane = threadIdx.x % 32;
  const int64_t row = (int64_t)blockIdx.x * 4 + threadIdx.x / 32;
  if (row >= rows) return;
  const int chunks = static_cast<int>(D / 8);
  float v[8][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int ch = lane + 32 * i;
    if (ch < chunks) {
      unpack8(__ldcs(reinterpret_cast<const uint4 *>(x + row * x_srow) + ch), v[i]);
      if (gate) {
        float z[8];
        unpack8(__ldcs(reinterpret_cast<const uint4 *>(gate + row * g_srow) + ch), z);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[i][e] *= z[e] * sigmoidf_(z[e]);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) ss = fmaf(v[i][e], v[i][e], ss);
    }
  }
  ss = warp_sum(ss);
  const float rs = rsqrtf(ss / (float)D + eps);
  if (rstd && lane == 0) rstd[row] = rs;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int ch = lane + 32 * i;
    if (ch < chunks) {
      float wv[8];
      if (WVEC == 1) {
        unpack8(__ldg(reinterpret_cast<const uint4 *>(w) + ch), wv);
      } else if (WVEC == 2) {
        const float4 w0 = __ldg(reinterpret_cast<const float4 *>(w) + 2 * ch);
        const float4 w1 = __ldg(reinterpret_cast<const float4 *>(w) + 2 * ch + 1);
        wv[0] = w0.x; wv[1] = w0.y; wv[2] = w0.z; wv[3] = w0.w; wv[4] = w1.x; wv[5] = w1.y; wv[6] = w1.z; wv[7] = w1.w;
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) wv[e] = ld_f32(w, 8 * ch + e, w_dt);
      }
      uint32_t o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const __nv_bfloat162 t = __floats2bfloat162_rn(v[i][2 * e] * rs * wv[2 * e], v[i][2 * e + 1] * rs * wv[2 * e + 1]);
        o[e] = *reinterpret_cast<const uint32_t *>(&t);
      }
      __stcs(reinterpret_cast<uint4 *>(y + row * D) + ch, make_uint4(o[0], o[1], o[2], o[3]));
    }
  }
}

// Modes of the epilogue kernels.  With the heads of a layer spread over several GPUs the norm spans
// columns on other GPUs: each GPU first computes its own sum of squares per (b, l) row (partial), the
// sums are added across GPUs, and a second pass normalises with the total (apply).
constexpr int kEpilogueFull = 0, kEpiloguePartial = 1, kEpilogueApply = 2;

// One block per (b, l) row of width H*R: un-flatten h, add the D skip, gate, normalise.
__global__ void __launch_bounds__(256)
scan_epilogue_kernel(const void *__restrict__ h, int h_dt, int64_t h_sb, int64_t h_sl,
                     const void *__restrict__ x, int64_t x_sb, int64_t x_sl,
                     const void *__restrict__ gate, int64_t g_sb, int64_t g_sl, int dt,
                     const float *__restrict__ Dp, const void *__restrict__ w, int w_dt,
                     float gate_bias, float eps, void *__restrict__ y, int64_t L, int64_t H,
                     int64_t R, int mode, float *__restrict__ sumsq, int64_t norm_width) {
  __shared__ float red[32];
  const int64_t HR = H * R;
  const int64_t row = blockIdx.x, b = row / L, l = row % L;
  float ss = 0.f;
  for (int64_t j = threadIdx.x; mode != kEpilogueApply && j < HR; j += blockDim.x) {
    const int64_t hh = j / R, r = j % R;
    float v = ld_f32(h, (b * H + hh) * h_sb + l * h_sl + r, h_dt) +
              ld_f32(x, b * x_sb + l * x_sl + j, dt) * Dp[j];
    const float z = ld_f32(gate, b * g_sb + l * g_sl + j, dt) + gate_bias;
    v *= z * sigmoidf_(z);
    ss = fmaf(v, v, ss);
  }
  if (mode == kEpilogueApply) {
    ss = sumsq[row];
  } else {
    ss = block_sum(ss, red);
    if (mode == kEpiloguePartial) {
      if (threadIdx.x == 0) sumsq[row] = ss;
      return;
    }
  }
  const float rs = rsqrtf(ss / (float)norm_width + eps);
  for (int64_t j = threadIdx.x; j < HR; j += blockDim.x) {
    const int64_t hh = j / R, r = j % R;
    float v = ld_f32(h, (b * H + hh) * h_sb + l * h_sl + r, h_dt) +
              ld_f32(x, b * x_sb + l * x_sl + j, dt) * Dp[j];
    const float z = ld_f32(gate, b * g_sb + l * g_sl + j, dt) + gate_bias;
    v *= z * sigmoidf_(z);
    st_f32(y, row * HR + j, dt, v * rs * ld_f32(w, j, w_dt));
  }
}

// bf16 fast path of the epilogue: one block per (b, l) row, 8 elements (16 bytes) per thread held
// in registers, so every tensor is read once and written once.  The kernel is bound by its
// instruction count as much as by memory, hence the fast-math gate (silu(z) = z / (1 + e^-z) with
// the approximate exponential and division: about 2 ulp, the output is bf16) and the norm weight
// read as one or two 16-byte pieces (WVEC 1: bf16, 2: f32; 0: element by element, any type).
template <int WVEC>
__global__ void __launch_bounds__(1024)
scan_epilogue_bf16_kernel(const __nv_bfloat16 *__restrict__ h, int64_t h_sb, int64_t h_sl,
                          const __nv_bfloat16 *__restrict__ x, int64_t x_sb, int64_t x_sl,
                          const __nv_bfloat16 *__restrict__ gate, int64_t g_sb, int64_t g_sl,
                          const float *__restrict__ Dp, const void *__restrict__ w, int w_dt,
                          float gate_bias, float eps, __nv_bfloat16 *__restrict__ y, int64_t L, int64_t H,
                          int64_t R, int mode, float *__restrict__ sumsq, int64_t norm_width) {
  __shared__ float red[32];
  const int HR = (int)(H * R);
  const int64_t row = blockIdx.x;   // fewer than 2^31 rows (the grid's x extent), so the row splits in 32 bits
  const int64_t b = (int)blockIdx.x / (int)L, l = row - b * L;
  const int j = (int)threadIdx.x * 8;   // < 8192
  float v[8];
  float ss = 0.f;
  const bool live = j < HR;
  if (live) {
    const int hh = j / (int)R, r = j - hh * (int)R;
    float hv[8], xv[8], zv[8];
    unpack8(__ldcs(reinterpret_cast<const uint4 *>(h + (b * H + hh) * h_sb + l * h_sl + r)), hv);
    unpack8(__ldcs(reinterpret_cast<const uint4 *>(x + b * x_sb + l * x_sl + j)), xv);
    unpack8(__ldcs(reinterpret_cast<const uint4 *>(gate + b * g_sb + l * g_sl + j)), zv);
    const float4 d0 = __ldg(reinterpret_cast<const float4 *>(Dp + j)), d1 = __ldg(reinterpret_cast<const float4 *>(Dp + j + 4));
    const float dv[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float z = zv[i] + gate_bias;
      v[i] = fmaf(xv[i], dv[i], hv[i]) * __fdividef(z, 1.f + __expf(-z));
      ss = fmaf(v[i], v[i], ss);
    }
  }
  if (mode == kEpilogueApply) {
    ss = sumsq[row];
  } else {
    ss = block_sum(ss, red);
    if (mode == kEpiloguePartial) {
      if (threadIdx.x == 0) sumsq[row] = ss;
      return;
    }
  }
  const float rs = rsqrtf(ss / (float)norm_width + eps);
  if (live) {
    float wv[8];
    if (WVEC == 1) {
      unpack8(__ldg(reinterpret_cast<const uint4 *>(reinterpret_cast<const __nv_bfloat16 *>(w) + j)), wv);
    } else if (WVEC == 2) {
      const float4 w0 = __ldg(reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(w) + j));
      const float4 w1 = __ldg(reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(w) + j + 4));
      wv[0] = w0.x; wv[1] = w0.y; wv[2] = w0.z; wv[3] = w0.w; wv[4] = w1.x; wv[5] = w1.y; wv[6] = w1.z; wv[7] = w1.w;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) wv[i] = ld_f32(w, j + i, w_dt);
    }
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 t = __floats2bfloat162_rn(v[2 * i] * rs * wv[2 * i], v[2 * i + 1] * rs * wv[2 * i + 1]);
      o[i] = *reinterpret_cast<const uint32_t *>(&t);
    }
    __stcs(reinterpret_cast<uint4 *>(y + row * HR + j), make_uint4(o[0], o[1], o[2], o[3]));
  }
}


// Second pass of the fused layer path: the scan kernel has written the gated values g [batch, L, H*R]
// (bf16) and, per (b, l, head), four partial sums of g^2; this normalises a row with the sum over all
// its heads (taken from the partial sums, or from `sumsq` when the heads of the layer are spread over
// several GPUs and the caller has added the per-rank sums).  One block per row, 8 elements per thread.
__global__ void __launch_bounds__(1024)
layer_norm_apply_kernel(const __nv_bfloat16 *__restrict__ g, const float *__restrict__ ss, int64_t n_partial,
                        const float *__restrict__ sumsq, const void *__restrict__ w, int w_dt, float eps,
                        int64_t norm_width, __nv_bfloat16 *__restrict__ y, int64_t HR) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const int64_t j = (int64_t)threadIdx.x * 8;
  float total;
  if (sumsq) {
    total = sumsq[row];
  } else {
    float part = 0.f;
    for (int64_t i = threadIdx.x; i < n_partial; i += blockDim.x) part += ss[row * n_partial + i];
    total = block_sum(part, red);
  }
  const float rs = rsqrtf(total / (float)norm_width + eps);
  if (j < HR) {
    float v[8];
    unpack8(__ldcs(reinterpret_cast<const uint4 *>(g + row * HR + j)), v);
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 t = __floats2bfloat162_rn(v[2 * i] * rs * ld_f32(w, j + 2 * i, w_dt),
                                                     v[2 * i + 1] * rs * ld_f32(w, j + 2 * i + 1, w_dt));
      o[i] = *reinterpret_cast<const uint32_t *>(&t);
    }
    __stcs(reinterpret_cast<uint4 *>(y + row * HR + j), make_uint4(o[0], o[1], o[2], o[3]));
  }
}

// sumsq[row] = sum of the row's partial sums (one warp per row)
__global__ void layer_sumsq_kernel(const float *__restrict__ ss, int64_t n_partial, float *__restrict__ sumsq,
                                   int64_t rows) {
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
  if (row >= rows) return;
  float part = 0.f;
  for (int64_t i = threadIdx.x % 32; i < n_partial; i += 32) part += ss[row * n_partial + i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
  if (threadIdx.x % 32 == 0) sumsq[row] = part;
}

}  // namespace fracssm

extern "C" int fracssm_compute_params(const void *dyn, int dyn_dtype, int64_t dyn_sb, int64_t dyn_sl,
                                      const void *rw, int rw_dtype, int64_t rw_sb, int64_t rw_sl,
                                      const void *x_conv, int x_dtype, int64_t x_sb, int64_t x_sl,
                                      const float *mask, int64_t m_sb, int64_t m_sl,
                                      const float *dt_bias, const float *base_log_tau,
                                      const float *read_gate_logit, const float *write_gate_logit, float read_temp,
                                      float dt_min, float dt_max, float alpha_min, float alpha_max,
                                      float lambda_min, float lambda_max, void *u, void *c,
                                      void *kappa, int ck_dtype, float *rho, int64_t Bt, int64_t L,
                                      int64_t H, int64_t R, int64_t M, void *stream) {
  using namespace fracssm;
  if (Bt < 0 || L < 0 || H <= 0 || R <= 0 || M <= 0) return fail(FRACSSM_ERR_ARG, "compute_params: bad sizes");
  if (!known_dtype(dyn_dtype) || !known_dtype(rw_dtype) || !known_dtype(x_dtype) || !known_dtype(ck_dtype))
    return fail(FRACSSM_ERR_ARG, "compute_params: unsupported dtype");
  if (Bt == 0 || L == 0) return FRACSSM_OK;
  if (!dyn || !rw || (u && !x_conv) || !dt_bias || !base_log_tau || !read_gate_logit || !write_gate_logit || !c ||
      !kappa || !rho)
    return fail(FRACSSM_ERR_ARG, "compute_params: null pointer");
  if (Bt * H > 65535) return fail(FRACSSM_ERR_UNSUPPORTED, "compute_params: batch*heads too large for one launch");
  ParamArgs a{};
  a.dyn = dyn; a.dyn_dt = dyn_dtype; a.dyn_sb = dyn_sb; a.dyn_sl = dyn_sl;
  a.rw = rw; a.rw_dt = rw_dtype; a.rw_sb = rw_sb; a.rw_sl = rw_sl;
  a.x = x_conv; a.x_dt = x_dtype; a.x_sb = x_sb; a.x_sl = x_sl;
  a.mask = mask; a.m_sb = m_sb; a.m_sl = m_sl;
  a.dt_bias = dt_bias; a.log_tau = base_log_tau;
  a.read_logit = read_gate_logit;
  a.write_logit = write_gate_logit;
  a.inv_read_temp = 1.f / read_temp;
  a.dt_min = dt_min; a.dt_max = dt_max; a.a_min = alpha_min; a.a_max = alpha_max;
  a.l_min = lambda_min; a.l_max = lambda_max;
  a.u = u; a.c = c; a.kappa = kappa; a.ck_dt = ck_dtype; a.rho = rho;
  a.L = L; a.H = H; a.R = R; a.M = M;
  auto al = [](const void *p, uintptr_t n) { return (reinterpret_cast<uintptr_t>(p) & (n - 1)) == 0; };
  if (M == 128 && rw_dtype == FRACSSM_BF16 && (ck_dtype == FRACSSM_F32 || ck_dtype == FRACSSM_BF16) && al(rw, 8) &&
      rw_sb % 4 == 0 && rw_sl % 4 == 0 && al(c, 16) && al(kappa, 16) && al(rho, 16)) {
    // 16-byte loads of the residual rows and 16-byte stores of bf16 c / kappa need the wider alignment
    if (al(rw, 16) && rw_sb % 8 == 0 && rw_sl % 8 == 0) {
      dim3 grid((unsigned)ceil_div(L, 4 * kPairTokens), (unsigned)(Bt * H));
      compute_params_m128_pair_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(a);
    } else {
      dim3 grid((unsigned)ceil_div(L, 4 * kPrepTokens), (unsigned)(Bt * H));
      compute_params_m128_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(a);
    }
    return check_launch("compute_params");
  }
  dim3 grid((unsigned)ceil_div(L, 4), (unsigned)(Bt * H));
  compute_params_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(a);
  return check_launch("compute_params");
}

extern "C" int fracssm_skip_mix(const void *mixed_flat, int mf_dtype, int64_t mf_sb, int64_t mf_sl,
                                const void *x_conv, int x_dtype, int64_t x_sb, int64_t x_sl,
                                const float *D, void *out, int out_dtype, int64_t Bt, int64_t L,
                                int64_t H, int64_t R, void *stream) {
  using namespace fracssm;
  if (Bt < 0 || L < 0 || H <= 0 || R <= 0) return fail(FRACSSM_ERR_ARG, "skip_mix: bad sizes");
  if (!known_dtype(mf_dtype) || !known_dtype(x_dtype) || !known_dtype(out_dtype))
    return fail(FRACSSM_ERR_ARG, "skip_mix: unsupported dtype");
  if (Bt == 0 || L == 0) return FRACSSM_OK;
  if (!mixed_flat || !x_conv || !D || !out) return fail(FRACSSM_ERR_ARG, "skip_mix: null pointer");
  skip_mix_kernel<<<(unsigned)(Bt * L), 256, 0, (cudaStream_t)stream>>>(
      mixed_flat, mf_dtype, mf_sb, mf_sl, x_conv, x_dtype, x_sb, x_sl, D, out, out_dtype, L, H, R);
  return check_launch("skip_mix");
}

extern "C" int fracssm_rmsnorm_gated(const void *x, int64_t x_srow, const void *gate, int64_t g_srow,
                                     int xg_dtype, const void *weight, int w_dtype, float eps,
                                     void *y, float *rstd, int64_t rows, int64_t D, void *stream) {
  using namespace fracssm;
  if (rows < 0 || D <= 0) return fail(FRACSSM_ERR_ARG, "rmsnorm_gated: bad sizes");
  if (!known_dtype(xg_dtype) || !known_dtype(w_dtype)) return fail(FRACSSM_ERR_ARG, "rmsnorm_gated: unsupported dtype");
  if (rows == 0) return FRACSSM_OK;
  if (!x || !weight || !y) return fail(FRACSSM_ERR_ARG, "rmsnorm_gated: null pointer");
  auto al16 = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (xg_dtype == FRACSSM_BF16 && D % 8 == 0 && D <= 2048 && al16(x) && al16(y) && x_srow % 8 == 0 &&
      (!gate || (al16(gate) && g_srow % 8 == 0))) {
    const int wvec = !al16(weight) ? 0 : w_dtype == FRACSSM_BF16 ? 1 : w_dtype == FRACSSM_F32 ? 2 : 0;
#define FRACSSM_RMSNORM(WV)                                                                                        \
  rmsnorm_gated_bf16_kernel<WV><<<(unsigned)ceil_div(rows, 4), 128, 0, (cudaStream_t)stream>>>(                    \
      reinterpret_cast<const __nv_bfloat16 *>(x), x_srow, reinterpret_cast<const __nv_bfloat16 *>(gate), g_srow,   \
      weight, w_dtype, eps, reinterpret_cast<__nv_bfloat16 *>(y), rstd, rows, D)
    if (wvec == 1) FRACSSM_RMSNORM(1);
    else if (wvec == 2) FRACSSM_RMSNORM(2);
    else FRACSSM_RMSNORM(0);
#undef FRACSSM_RMSNORM
    return check_launch("rmsnorm_gated");
  }
  rmsnorm_gated_kernel<<<(unsigned)rows, 256, 0, (cudaStream_t)stream>>>(
      x, x_srow, gate, g_srow, xg_dtype, weight, w_dtype, eps, y, rstd, D);
  return check_launch("rmsnorm_gated");
}

namespace fracssm {
namespace {
int scan_epilogue_launch(const char *who, const void *h, int h_dtype, int64_t h_sb, int64_t h_sl,
                         const void *x_conv, int64_t x_sb, int64_t x_sl, const void *gate, int64_t g_sb,
                         int64_t g_sl, int xg_dtype, const float *D, const void *weight, int w_dtype,
                         float gate_bias, float eps, void *y, int64_t Bt, int64_t L, int64_t H, int64_t R,
                         int mode, float *sumsq, int64_t norm_width, void *stream) {
  if (Bt < 0 || L < 0 || H <= 0 || R <= 0) return fail(FRACSSM_ERR_ARG, "%s: bad sizes", who);
  if (!known_dtype(h_dtype) || !known_dtype(xg_dtype) || (mode != kEpiloguePartial && !known_dtype(w_dtype)))
    return fail(FRACSSM_ERR_ARG, "%s: unsupported dtype", who);
  if (mode != kEpilogueFull && norm_width < H * R) return fail(FRACSSM_ERR_ARG, "%s: norm_width smaller than the local width", who);
  if (Bt == 0 || L == 0) return FRACSSM_OK;
  if (!h || !x_conv || !gate || !D) return fail(FRACSSM_ERR_ARG, "%s: null pointer", who);
  if (mode != kEpiloguePartial && (!weight || !y)) return fail(FRACSSM_ERR_ARG, "%s: null pointer", who);
  if (mode != kEpilogueFull && !sumsq) return fail(FRACSSM_ERR_ARG, "%s: null pointer", who);
  auto al16 = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const int64_t HR = H * R;
  if (h_dtype == FRACSSM_BF16 && xg_dtype == FRACSSM_BF16 && R % 8 == 0 && HR <= 8192 && al16(h) && al16(x_conv) &&
      al16(gate) && al16(y) && al16(D) && h_sb % 8 == 0 && h_sl % 8 == 0 && x_sb % 8 == 0 && x_sl % 8 == 0 &&
      g_sb % 8 == 0 && g_sl % 8 == 0) {
    const unsigned threads = (unsigned)(((HR / 8) + 31) / 32 * 32);
    const int wvec = (mode == kEpiloguePartial || !al16(weight)) ? 0 : w_dtype == FRACSSM_BF16 ? 1 : w_dtype == FRACSSM_F32 ? 2 : 0;
#define FRACSSM_EPILOGUE(WV)                                                                                       \
  scan_epilogue_bf16_kernel<WV><<<(unsigned)(Bt * L), threads, 0, (cudaStream_t)stream>>>(                         \
      reinterpret_cast<const __nv_bfloat16 *>(h), h_sb, h_sl, reinterpret_cast<const __nv_bfloat16 *>(x_conv),     \
      x_sb, x_sl, reinterpret_cast<const __nv_bfloat16 *>(gate), g_sb, g_sl, D, weight, w_dtype, gate_bias, eps,   \
      reinterpret_cast<__nv_bfloat16 *>(y), L, H, R, mode, sumsq, norm_width)
    if (wvec == 1) FRACSSM_EPILOGUE(1);
    else if (wvec == 2) FRACSSM_EPILOGUE(2);
    else FRACSSM_EPILOGUE(0);
#undef FRACSSM_EPILOGUE
    return check_launch(who);
  }
  scan_epilogue_kernel<<<(unsigned)(Bt * L), 256, 0, (cudaStream_t)stream>>>(
      h, h_dtype, h_sb, h_sl, x_conv, x_sb, x_sl, gate, g_sb, g_sl, xg_dtype, D, weight, w_dtype,
      gate_bias, eps, y, L, H, R, mode, sumsq, norm_width);
  return check_launch(who);
}
}  // namespace
}  // namespace fracssm

extern "C" int fracssm_scan_epilogue(const void *h, int h_dtype, int64_t h_sb, int64_t h_sl,
                                     const void *x_conv, int64_t x_sb, int64_t x_sl,
                                     const void *gate, int64_t g_sb, int64_t g_sl, int xg_dtype,
                                     const float *D, const void *weight, int w_dtype,
                                     float gate_bias, float eps, void *y, int64_t Bt, int64_t L,
                                     int64_t H, int64_t R, void *stream) {
  using namespace fracssm;
  return scan_epilogue_launch("scan_epilogue", h, h_dtype, h_sb, h_sl, x_conv, x_sb, x_sl, gate, g_sb, g_sl,
                              xg_dtype, D, weight, w_dtype, gate_bias, eps, y, Bt, L, H, R, kEpilogueFull,
                              nullptr, H * R, stream);
}

// Head-sharded layers, first pass: sumsq[b*L + l] = sum over the H local heads of
// ((h + x_conv * D) * silu(gate + gate_bias))^2.
extern "C" int fracssm_scan_epilogue_sumsq(const void *h, int h_dtype, int64_t h_sb, int64_t h_sl,
                                           const void *x_conv, int64_t x_sb, int64_t x_sl,
                                           const void *gate, int64_t g_sb, int64_t g_sl, int xg_dtype,
                                           const float *D, float gate_bias, float *sumsq, int64_t Bt,
                                           int64_t L, int64_t H, int64_t R, void *stream) {
  using namespace fracssm;
  return scan_epilogue_launch("scan_epilogue_sumsq", h, h_dtype, h_sb, h_sl, x_conv, x_sb, x_sl, gate, g_sb,
                              g_sl, xg_dtype, D, nullptr, FRACSSM_F32, gate_bias, 0.f, nullptr, Bt, L, H, R,
                              kEpiloguePartial, sumsq, H * R, stream);
}

// Head-sharded layers, second pass: the local columns normalised with the row's total sum of squares
// over all `norm_width` columns of the layer (sumsq after the sum across GPUs).
extern "C" int fracssm_scan_epilogue_apply(const void *h, int h_dtype, int64_t h_sb, int64_t h_sl,
                                           const void *x_conv, int64_t x_sb, int64_t x_sl,
                                           const void *gate, int64_t g_sb, int64_t g_sl, int xg_dtype,
                                           const float *D, const void *weight, int w_dtype,
                                           float gate_bias, float eps, const float *sumsq,
                                           int64_t norm_width, void *y, int64_t Bt, int64_t L, int64_t H,
                                           int64_t R, void *stream) {
  using namespace fracssm;
  return scan_epilogue_launch("scan_epilogue_apply", h, h_dtype, h_sb, h_sl, x_conv, x_sb, x_sl, gate, g_sb,
                              g_sl, xg_dtype, D, weight, w_dtype, gate_bias, eps, y, Bt, L, H, R, kEpilogueApply,
                              const_cast<float *>(sumsq), norm_width, stream);
}

// ---------------------------------------------------------------------------------------------
// The layer path with the epilogue fused into the scan's output stage: h never reaches memory.
//   pass 1 (fracssm_scan_layer_gated): the single-pass scan kernel writes
//       g = (h + u * D) * silu(gate + gate_bias), un-flattened to [batch, L, H*64], and partial sums of g^2;
//   pass 2 (fracssm_scan_layer_norm):  y = weight * g * rsqrt(mean(g^2) + eps) per (b, l) row.
// u is the head-major copy of x_conv the parameter prep makes, so the skip connection reads it directly.
extern "C" size_t fracssm_scan_layer_workspace_bytes(int64_t Bt, int64_t H, int64_t L, int64_t R, int64_t M) {
  using namespace fracssm;
  if (Bt <= 0 || H <= 0 || L <= 0) return 0;
  return scan_fused_workspace_bytes(Bt * H, L, R, M, 128);
}

extern "C" int fracssm_scan_layer_gated(const void *u, const void *c, const void *kappa, int ck_dtype,
                                        const float *rho, const float *initial_state, const void *gate,
                                        const float *D, float gate_bias, void *gated, float *ss_partial,
                                        void *final_state, int final_dtype, void *workspace,
                                        size_t workspace_bytes, int64_t Bt, int64_t H, int64_t L, int64_t R,
                                        int64_t M, void *stream) {
  using namespace fracssm;
  if (Bt < 0 || H < 1 || L < 0) return fail(FRACSSM_ERR_ARG, "scan_layer_gated: bad sizes");
  if (Bt == 0 || L == 0) return fail(FRACSSM_ERR_UNSUPPORTED, "scan_layer_gated: empty input");
  if (!fracssm_scan_fused_supported(Bt * H, L, R, M, 128, FRACSSM_BF16, ck_dtype))
    return fail(FRACSSM_ERR_UNSUPPORTED, "scan_layer_gated: needs R = 64, M = 128, bfloat16 u and bfloat16 or float32 c / kappa");
  if (!u || !c || !kappa || !rho || !gate || !D || !gated || !ss_partial || !workspace)
    return fail(FRACSSM_ERR_ARG, "scan_layer_gated: null pointer");
  if (final_state && final_dtype != FRACSSM_F32 && final_dtype != FRACSSM_BF16)
    return fail(FRACSSM_ERR_ARG, "scan_layer_gated: final_state dtype must be float32 or bfloat16");
  if ((reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
    return fail(FRACSSM_ERR_ARG, "scan_layer_gated: workspace must be 256-byte aligned");
  ScanLayerOut lo{gate, D, gated, ss_partial, gate_bias, H};
  // h is not written in this mode; the pointer only has to pass the alignment check
  return scan_fused_launch_ex(u, c, kappa, ck_dtype, rho, initial_state, gated, final_state, final_dtype, workspace,
                              workspace_bytes, Bt * H, L, R, M, 128, stream, 0, tile_default_wait_ns(), &lo);
}

extern "C" int fracssm_scan_layer_sumsq(const float *ss_partial, float *sumsq, int64_t Bt, int64_t L, int64_t H,
                                        void *stream) {
  using namespace fracssm;
  if (Bt < 0 || L < 0 || H < 1) return fail(FRACSSM_ERR_ARG, "scan_layer_sumsq: bad sizes");
  if (Bt == 0 || L == 0) return FRACSSM_OK;
  if (!ss_partial || !sumsq) return fail(FRACSSM_ERR_ARG, "scan_layer_sumsq: null pointer");
  const int64_t rows = Bt * L;
  layer_sumsq_kernel<<<(unsigned)ceil_div(rows, 8), 256, 0, (cudaStream_t)stream>>>(ss_partial, 4 * H, sumsq, rows);
  return check_launch("scan_layer_sumsq");
}

extern "C" int fracssm_scan_layer_norm(const void *gated, const float *ss_partial, const float *sumsq,
                                       const void *weight, int w_dtype, float eps, int64_t norm_width, void *y,
                                       int64_t Bt, int64_t L, int64_t H, int64_t R, void *stream) {
  using namespace fracssm;
  if (Bt < 0 || L < 0 || H < 1 || R < 1) return fail(FRACSSM_ERR_ARG, "scan_layer_norm: bad sizes");
  if (Bt == 0 || L == 0) return FRACSSM_OK;
  if (!gated || !weight || !y || (!ss_partial && !sumsq)) return fail(FRACSSM_ERR_ARG, "scan_layer_norm: null pointer");
  if (!known_dtype(w_dtype)) return fail(FRACSSM_ERR_ARG, "scan_layer_norm: unsupported weight dtype");
  const int64_t HR = H * R;
  if (HR % 8 != 0 || HR > 8192 || norm_width < HR)
    return fail(FRACSSM_ERR_UNSUPPORTED, "scan_layer_norm: row width must be a multiple of 8, at most 8192, and norm_width >= H * R");
  if (((reinterpret_cast<uintptr_t>(gated) | reinterpret_cast<uintptr_t>(y)) & 15) != 0)
    return fail(FRACSSM_ERR_ARG, "scan_layer_norm: gated and y must be 16-byte aligned");
  const unsigned threads = (unsigned)(((HR / 8) + 31) / 32 * 32);
  layer_norm_apply_kernel<<<(unsigned)(Bt * L), threads, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const __nv_bfloat16 *>(gated), ss_partial, 4 * H, sumsq, weight, w_dtype, eps, norm_width,
      reinterpret_cast<__nv_bfloat16 *>(y), HR);
  return check_launch("scan_layer_norm");
}

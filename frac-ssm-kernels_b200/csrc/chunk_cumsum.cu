// Within-chunk running sum of the log-decay (bandwidth-bound stage).
//
// Fast path (chunk_cumsum_vec_kernel; chunks of up to 256 tokens, M a multiple of 4, 16-byte aligned
// rows): one block of 16 warps owns one (chunk, bh, 128-mode column group).  A lane owns four
// consecutive modes, so a warp reads one 512-byte token row per 16-byte load; the 16 warps split the
// chunk's tokens into 16 consecutive segments of at most 16 tokens, each kept in registers.  Every
// element is read once and written once: the running sum inside a segment is a register chain, the
// segments' totals are exchanged through shared memory and their exclusive prefix is added before
// the 16-byte stores.
//
// General path: one block owns one (chunk, bh, 32-mode column group).  Lanes run across modes, so a
// warp reads 128 contiguous bytes per token; the 8 warps split the chunk's tokens into
// 8 consecutive segments.  Pass 1 sums each segment, the segment sums are exchanged in
// shared memory, pass 2 rescans each segment (an L1/L2 hit) from its offset and writes.
// With src_is_rho the logarithm and the 1e-6 floor are applied on load.
#include "common.cuh"

namespace fracssm {

constexpr int kCsWarps = 8;

__global__ void __launch_bounds__(32 * kCsWarps)
chunk_cumsum_kernel(const float *__restrict__ src, int64_t sb, int64_t sl, int src_is_rho,
                    float *__restrict__ lcr, float *__restrict__ chunk_decay, int64_t L, int64_t M,
                    int64_t T, int64_t N) {
  const int64_t n = blockIdx.x, b = blockIdx.y;
  const int64_t m = (int64_t)blockIdx.z * 32 + threadIdx.x;
  const int w = threadIdx.y;
  __shared__ float seg_sum[kCsWarps][32];

  const int64_t t0 = n * T;
  const int64_t len = min(T, L - t0);            // valid tokens of this chunk
  const int64_t seg = (T + kCsWarps - 1) / kCsWarps;
  const int64_t lo = w * seg, hi = min(lo + seg, len);
  const bool live = m < M;

  float acc = 0.f;
  if (live) {
    const float *p = src + b * sb + m;
    for (int64_t t = lo; t < hi; ++t) {
      float x = p[(t0 + t) * sl];
      if (src_is_rho) x = logf(fmaxf(x, kRhoFloor));
      acc += x;
    }
  }
  seg_sum[w][threadIdx.x] = acc;
  __syncthreads();
  float offset = 0.f, total = 0.f;
#pragma unroll
  for (int j = 0; j < kCsWarps; ++j) {
    float s = seg_sum[j][threadIdx.x];
    if (j < w) offset += s;
    total += s;
  }
  if (!live) return;
  if (w == 0) chunk_decay[(b * N + n) * M + m] = total;
  const float *p = src + b * sb + m;
  float *q = lcr + (b * L + t0) * M + m;
  float run = offset;
  for (int64_t t = lo; t < hi; ++t) {
    float x = p[(t0 + t) * sl];
    if (src_is_rho) x = logf(fmaxf(x, kRhoFloor));
    run += x;
    q[t * M] = run;
  }
}

constexpr int kVecWarps = 16, kVecSeg = 16;   // 16 warps x up to 16 tokens = chunks of up to 256 tokens

__global__ void __launch_bounds__(32 * kVecWarps)
chunk_cumsum_vec_kernel(const float *__restrict__ src, int64_t sb, int64_t sl, int src_is_rho,
                        float *__restrict__ lcr, float *__restrict__ chunk_decay, int64_t L, int64_t M,
                        int64_t T, int64_t N) {
  const int64_t n = blockIdx.x, b = blockIdx.y;
  const int lane = threadIdx.x, w = threadIdx.y;
  const int64_t m = ((int64_t)blockIdx.z * 32 + lane) * 4;
  __shared__ float4 seg_sum[kVecWarps][32];

  const int64_t t0 = n * T;
  const int len = (int)min(T, L - t0);                      // valid tokens of this chunk
  const int seg = (int)((T + kVecWarps - 1) / kVecWarps);   // <= kVecSeg
  const int lo = w * seg, cnt = max(0, min(seg, len - lo));
  const bool live = m < M;

  float4 v[kVecSeg];
  float4 run = make_float4(0.f, 0.f, 0.f, 0.f);
  if (live) {
    const float *p = src + b * sb + (t0 + lo) * sl + m;
#pragma unroll
    for (int i = 0; i < kVecSeg; ++i)
      if (i < cnt) v[i] = __ldcs(reinterpret_cast<const float4 *>(p + i * sl));
#pragma unroll
    for (int i = 0; i < kVecSeg; ++i) {
      if (i < cnt) {
        float4 x = v[i];
        if (src_is_rho) {
          x.x = logf(fmaxf(x.x, kRhoFloor)); x.y = logf(fmaxf(x.y, kRhoFloor));
          x.z = logf(fmaxf(x.z, kRhoFloor)); x.w = logf(fmaxf(x.w, kRhoFloor));
        }
        run.x += x.x; run.y += x.y; run.z += x.z; run.w += x.w;
        v[i] = run;                                          // inclusive sum from the segment's start
      }
    }
  }
  seg_sum[w][lane] = run;
  __syncthreads();
  if (!live) return;
  float4 off = make_float4(0.f, 0.f, 0.f, 0.f), tot = off;
#pragma unroll
  for (int j = 0; j < kVecWarps; ++j) {
    const float4 s = seg_sum[j][lane];
    if (j < w) { off.x += s.x; off.y += s.y; off.z += s.z; off.w += s.w; }
    tot.x += s.x; tot.y += s.y; tot.z += s.z; tot.w += s.w;
  }
  if (w == 0) *reinterpret_cast<float4 *>(chunk_decay + (b * N + n) * M + m) = tot;
  float *q = lcr + (b * L + t0 + lo) * M + m;
#pragma unroll
  for (int i = 0; i < kVecSeg; ++i)
    if (i < cnt)
      __stcs(reinterpret_cast<float4 *>(q + i * M),
             make_float4(v[i].x + off.x, v[i].y + off.y, v[i].z + off.z, v[i].w + off.w));
}

}  // namespace fracssm

extern "C" int fracssm_chunk_cumsum(const float *src, int64_t sb, int64_t sl, int src_is_rho,
                                    float *lcr, float *chunk_decay, int64_t B, int64_t L, int64_t M,
                                    int64_t T, void *stream) {
  using namespace fracssm;
  if (B < 0 || L < 0 || M <= 0 || T <= 0) return fail(FRACSSM_ERR_ARG, "chunk_cumsum: bad sizes");
  if (B == 0 || L == 0) return FRACSSM_OK;
  if (!src || !lcr || !chunk_decay) return fail(FRACSSM_ERR_ARG, "chunk_cumsum: null pointer");
  const int64_t N = ceil_div(L, T);
  if (B > 65535 || ceil_div(M, 32) > 65535)
    return fail(FRACSSM_ERR_UNSUPPORTED, "chunk_cumsum: B or M too large for one launch");
  const bool aligned = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(lcr) |
                         reinterpret_cast<uintptr_t>(chunk_decay)) & 15) == 0;
  if (T <= kVecWarps * kVecSeg && M % 4 == 0 && sl % 4 == 0 && sb % 4 == 0 && aligned && ceil_div(M, 128) <= 65535) {
    dim3 vgrid((unsigned)N, (unsigned)B, (unsigned)ceil_div(M, 128)), vblock(32, kVecWarps);
    chunk_cumsum_vec_kernel<<<vgrid, vblock, 0, (cudaStream_t)stream>>>(src, sb, sl, src_is_rho, lcr, chunk_decay,
                                                                        L, M, T, N);
    return check_launch("chunk_cumsum");
  }
  dim3 grid((unsigned)N, (unsigned)B, (unsigned)ceil_div(M, 32)), block(32, kCsWarps);
  chunk_cumsum_kernel<<<grid, block, 0, (cudaStream_t)stream>>>(src, sb, sl, src_is_rho, lcr,
                                                                chunk_decay, L, M, T, N);
  return check_launch("chunk_cumsum");
}

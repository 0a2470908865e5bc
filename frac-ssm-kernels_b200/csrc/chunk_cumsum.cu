// Within-chunk running sum of the log-decay (bandwidth-bound stage).
//
// One block owns one (chunk, bh, 32-mode column group).  Lanes run across modes, so a
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
  dim3 grid((unsigned)N, (unsigned)B, (unsigned)ceil_div(M, 32)), block(32, kCsWarps);
  chunk_cumsum_kernel<<<grid, block, 0, (cudaStream_t)stream>>>(src, sb, sl, src_is_rho, lcr,
                                                                chunk_decay, L, M, T, N);
  return check_launch("chunk_cumsum");
}

// Self-test of the tcgen05 / TMA building blocks: one 128-row MMA tile with the operand
// layouts the scan kernel uses, checked by the GPU tests against a host matmul.
//   D[128, N] = A[128, 128] * B[N, 128]^T   (bf16 operands, fp32 accumulation in TMEM)
#include "common.cuh"
#include "tmap.cuh"
#include "umma.cuh"
#include "fracssm_selftest.h"

namespace fracssm {

struct SelfTestArgs {
  const float *A, *B;   // tiles as [128 rows][128 cols] float32, rounded to bf16 on staging
  float *D;             // [128][N]
  int *status;          // device word: 0 ok, 1 = MMA wait timed out
  int a_mn, b_mn, N, b_group0, b_sbo, b_tma;
  int m_rows;           // 128, or 64 (then D holds all 128 TMEM lanes as they are)
};

__global__ void __launch_bounds__(128)
umma_selftest_kernel(const SelfTestArgs a, const __grid_constant__ CUtensorMap b_map) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t *tileA = smem, *tileB = smem + 32768;
  __shared__ __align__(8) uint64_t bar_mma, bar_tma;
  __shared__ uint32_t tmem_base_s;
  const int tid = threadIdx.x, warp = tid / 32;

  if (tid == 0) {
    umma::mbar_init(&bar_mma, 1);
    umma::mbar_init(&bar_tma, 1);
    umma::fence_mbar_init();
  }
  if (warp == 0) umma::tmem_alloc(&tmem_base_s, 128);
  for (int i = tid; i < 128 * 128; i += 128) {
    const int row = i / 128, col = i % 128;
    *reinterpret_cast<__nv_bfloat16 *>(tileA + umma::tile_off(row, col, 16384)) = __float2bfloat16_rn(a.A[i]);
    if (!a.b_tma && (!a.b_mn || col < a.N))
      *reinterpret_cast<__nv_bfloat16 *>(tileB + umma::tile_off(row, col, 16384)) = __float2bfloat16_rn(a.B[i]);
  }
  umma::fence_async_smem();
  umma::tc_fence_before();
  __syncthreads();
  umma::tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  bool ok = true;
  if (tid == 0) {
    if (a.b_tma) {
      umma::mbar_expect_tx(&bar_tma, 128 * 64 * 2);
      umma::tma_load_3d(tileB, &b_map, &bar_tma, 0, 0, 0);
      ok = umma::mbar_wait(&bar_tma, 0, 1000000000ull);
    }
    const uint32_t idesc = umma::make_idesc(a.m_rows, a.N, a.a_mn != 0, a.b_mn != 0);
    const uint32_t sa = umma::smem_u32(tileA), sb = umma::smem_u32(tileB);
    for (int ks = 0; ks < 8; ++ks) {
      const uint64_t da = a.a_mn ? umma::make_sdesc(sa + ks * 2048, 16384, 1024)
                                 : umma::make_sdesc(sa + (ks / 4) * 16384 + (ks % 4) * 32, 16, 1024);
      const uint64_t db = a.b_mn ? umma::make_sdesc(sb + ks * 2048, 16384, 1024)
                                 : umma::make_sdesc(sb + a.b_group0 * 1024 + (ks / 4) * 16384 + (ks % 4) * 32,
                                                    16, a.b_sbo);
      umma::mma_ss(tmem_base, da, db, idesc, ks > 0 ? 1u : 0u);
    }
    umma::mma_commit(&bar_mma);
  }
  ok = umma::mbar_wait(&bar_mma, 0, 1000000000ull) && ok;
  umma::tc_fence_after();
  if (!ok && tid == 0) *a.status = 1;
  if (ok) {
    const int row = tid;
    for (int c0 = 0; c0 < a.N; c0 += 8) {
      float v[8];
      umma::tmem_ld8(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + c0, v);
      umma::tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 8; ++j) a.D[row * a.N + c0 + j] = v[j];
    }
  }
  umma::tc_fence_before();
  __syncthreads();
  if (warp == 0) umma::tmem_dealloc(tmem_base, 128);
}

}  // namespace fracssm

extern "C" int fracssm_selftest_umma(const float *A, const float *B, const void *B_bf16, float *D,
                                     int *status, int a_mn_major, int b_mn_major, int N,
                                     int b_row_group0, int b_sbo_bytes, int b_via_tma, void *stream) {
  using namespace fracssm;
  if (!A || !B || !D || !status) return fail(FRACSSM_ERR_ARG, "selftest_umma: null pointer");
  if (N < 16 || N > 128 || N % 16) return fail(FRACSSM_ERR_ARG, "selftest_umma: N must be a multiple of 16 in 16..128");
  if (b_mn_major && N != 64 && N != 128)
    return fail(FRACSSM_ERR_ARG, "selftest_umma: MN-major B is one or two 64-wide atoms");
  if (b_via_tma && N != 64) return fail(FRACSSM_ERR_ARG, "selftest_umma: the TMA path loads one 64-wide atom");
  if (!b_mn_major && (b_sbo_bytes % 1024 || b_sbo_bytes <= 0 ||
                      (int64_t)b_row_group0 * 1024 + (int64_t)(N / 8 - 1) * b_sbo_bytes + 1024 > 16384))
    return fail(FRACSSM_ERR_ARG, "selftest_umma: B row groups leave the tile");
  if (b_via_tma && (!b_mn_major || !B_bf16)) return fail(FRACSSM_ERR_ARG, "selftest_umma: TMA path loads the MN-major B");
  SelfTestArgs a{A, B, D, status, a_mn_major, b_mn_major, N, b_row_group0, b_sbo_bytes, b_via_tma, 128};
  CUtensorMap map{};
  if (b_via_tma) {
    int rc = make_tmap_bf16_3d(&map, B_bf16, 64, 128, 1, 64, 128);
    if (rc) return rc;
  }
  const int smem = 65536 + 1024;
  cudaError_t e = cudaFuncSetAttribute(umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return fail(FRACSSM_ERR_CUDA, "selftest_umma: %s", cudaGetErrorString(e));
  umma_selftest_kernel<<<1, 128, smem, (cudaStream_t)stream>>>(a, map);
  return check_launch("selftest_umma");
}

// Diagnostic: the same tile with a 64-row MMA (A rows 0..63).  D [128][N] receives all 128 tensor-
// memory lanes as they are after the MMA (lanes the MMA does not write keep what they held), which
// shows where the hardware puts the 64 result rows.  No counterpart in the reference.
extern "C" int fracssm_selftest_umma_m64(const float *A, const float *B, float *D, int *status, int N,
                                         void *stream) {
  using namespace fracssm;
  if (!A || !B || !D || !status) return fail(FRACSSM_ERR_ARG, "selftest_umma_m64: null pointer");
  if (N < 8 || N > 128 || N % 8) return fail(FRACSSM_ERR_ARG, "selftest_umma_m64: N must be a multiple of 8 in 8..128");
  SelfTestArgs a{A, B, D, status, 0, 0, N, 0, 1024, 0, 64};
  CUtensorMap map{};
  const int smem = 65536 + 1024;
  cudaError_t e = cudaFuncSetAttribute(umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return fail(FRACSSM_ERR_CUDA, "selftest_umma_m64: %s", cudaGetErrorString(e));
  umma_selftest_kernel<<<1, 128, smem, (cudaStream_t)stream>>>(a, map);
  return check_launch("selftest_umma_m64");
}

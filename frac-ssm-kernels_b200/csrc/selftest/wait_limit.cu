// Test-only entry points (built into libfracssm_selftest.so, not into the product library):
// launches of the single-pass scan and of the segment-summary kernel whose first tile waits for a
// predecessor that is not part of the launch, with a short wait limit.  The kernels must return by
// themselves, report FRACSSM_ERR_WAIT through the status call and mark their outputs with NaN.
#include "common.cuh"
#include "fracssm_selftest.h"

namespace fracssm {
int segment_summary_launch_ex(const void *u, const void *kappa, int k_dtype, const float *rho,
                              const float *initial_state, float *final_state, float *decay, void *workspace,
                              size_t workspace_bytes, int64_t B, int64_t L, int64_t R, int64_t M, void *stream,
                              int first_tile, unsigned long long wait_ns, int64_t group);
}  // namespace fracssm

extern "C" int fracssm_selftest_scan_wait_limit(const void *u, const void *c, const void *kappa, const float *rho,
                                                void *h, void *final_state, void *workspace,
                                                size_t workspace_bytes, int64_t B, int64_t L,
                                                unsigned long long wait_ns, void *stream) {
  using namespace fracssm;
  if (L <= 128 || B < 1) return fail(FRACSSM_ERR_ARG, "selftest_scan_wait_limit: needs at least two tiles");
  return scan_fused_launch_ex(u, c, kappa, FRACSSM_BF16, rho, nullptr, h, final_state, FRACSSM_F32, workspace,
                              workspace_bytes, B, L, 64, 128, 128, stream, /*first_tile=*/1, wait_ns, nullptr);
}

extern "C" int fracssm_selftest_summary_wait_limit(const void *u, const void *kappa, const float *rho,
                                                   float *final_state, float *decay, void *workspace,
                                                   size_t workspace_bytes, int64_t B, int64_t L,
                                                   unsigned long long wait_ns, void *stream) {
  using namespace fracssm;
  if (L <= 128 || B < 1) return fail(FRACSSM_ERR_ARG, "selftest_summary_wait_limit: needs at least two tiles");
  return segment_summary_launch_ex(u, kappa, FRACSSM_BF16, rho, nullptr, final_state, decay, workspace,
                                   workspace_bytes, B, L, 64, 128, stream, /*first_tile=*/1, wait_ns, /*group=*/1);
}

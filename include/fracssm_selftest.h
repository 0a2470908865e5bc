/*
 * fracssm_selftest.h -- test-only entry points.  They are built into libfracssm_selftest.so (the
 * product sources plus csrc/selftest), never into libfracssm.so, and exist for the GPU tests only.
 * None has a counterpart in quorbix/frac-ssm-kernels.
 */
#ifndef FRACSSM_SELFTEST_H
#define FRACSSM_SELFTEST_H

#include "fracssm.h"

#ifdef __cplusplus
extern "C" {
#endif

/*
 * one 128-row tcgen05 MMA tile, D[128,N] = A[128,128] * B[N,128]^T, with the
 * shared-memory operand layouts the scan kernel uses (K-major / MN-major, strided row groups,
 * TMA-loaded B).  A and B are float32 [128][128] tiles rounded to bf16 on staging; B_bf16
 * (bf16 [128][64], dense) is only read when b_via_tma != 0.  status: device int, 0 = ok.
 * No counterpart in the reference; used by the GPU tests.
 */
int fracssm_selftest_umma(const float *A, const float *B, const void *B_bf16, float *D, int *status,
                          int a_mn_major, int b_mn_major, int N, int b_row_group0, int b_sbo_bytes,
                          int b_via_tma, void *stream);

/*
 * as fracssm_selftest_umma with K-major operands but a 64-row MMA; D [128][N] receives
 * all 128 tensor-memory lanes, which shows where the 64 result rows land.  No counterpart in the
 * reference.
 */
int fracssm_selftest_umma_m64(const float *A, const float *B, float *D, int *status, int N, void *stream);

/*
 * Bounded device-side waits, exercised without faulting anything: a launch of the single-pass scan
 * (bf16 u / c / kappa, R = 64, M = 128, L > 128) that starts at the SECOND tile of every row, so each
 * row's first item waits for a predecessor that is not part of the launch.  The wait runs out after
 * wait_ns nanoseconds, the kernel returns by itself, fracssm_scan_fused_status(workspace) then
 * reports FRACSSM_ERR_WAIT, and h (tokens 128..L-1) and final_state are NaN.
 */
int fracssm_selftest_scan_wait_limit(const void *u, const void *c, const void *kappa, const float *rho,
                                     void *h, void *final_state, void *workspace, size_t workspace_bytes,
                                     int64_t B, int64_t L, unsigned long long wait_ns, void *stream);
/* The same for the segment-summary kernel (final_state and decay come out as NaN). */
int fracssm_selftest_summary_wait_limit(const void *u, const void *kappa, const float *rho,
                                        float *final_state, float *decay, void *workspace,
                                        size_t workspace_bytes, int64_t B, int64_t L,
                                        unsigned long long wait_ns, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* FRACSSM_SELFTEST_H */

/*
 * fracssm.h — C ABI of the B200 (sm_100a) implementation of the FRAC fractional-SSM
 * chunked scan, forward pass.
 *
 * Every entry point takes raw DEVICE pointers (unless it says "host"), sizes, element
 * strides and a CUDA stream (cudaStream_t passed as void*), owns nothing, allocates
 * nothing unless stated, launches asynchronously on the given stream and returns an
 * int status (0 = ok).  fracssm_last_error() returns the text of the last failure on
 * the calling thread.  Tensors are row-major with a contiguous last dimension; "sb"
 * and "sl" arguments are the strides (in elements) of dim 0 and dim 1.  Outputs are
 * dense.  Dim 0 is the flattened (batch, head) index, bh = b * H + h.
 *
 * Each declaration names the interface of quorbix/frac-ssm-kernels it stands behind
 * (path within that project : line).
 */
#ifndef FRACSSM_H
#define FRACSSM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FRACSSM_ABI_VERSION 2

/* element types */
#define FRACSSM_F32 0
#define FRACSSM_BF16 1
#define FRACSSM_F16 2

/* status codes */
#define FRACSSM_OK 0
#define FRACSSM_ERR_ARG 1         /* bad size, null pointer, unsupported dtype combination */
#define FRACSSM_ERR_CUDA 2        /* a CUDA runtime call or launch failed */
#define FRACSSM_ERR_UNSUPPORTED 3 /* shape outside what a specialised kernel covers */
#define FRACSSM_ERR_WAIT 4        /* a bounded device-side wait ran out */

int fracssm_abi_version(void);
const char *fracssm_last_error(void);

/* 1 if the shape is covered by the tcgen05 single-pass scan kernel, else 0. */
int fracssm_scan_fused_supported(int64_t B, int64_t L, int64_t R, int64_t M, int64_t T,
                                 int u_dtype, int ck_dtype);

/*
 * Within-chunk inclusive running sum of the log-decay, and per-chunk totals.
 * src_is_rho = 0: src is log_rho;  1: src is rho and log(max(rho, 1e-6)) is fused in.
 * lcr [B, L, M] f32, chunk_decay [B, ceil(L/T), M] f32.
 * Replaces frac_ssm/ops/triton/chunk_cumsum.py:189 `chunk_cumsum(log_rho, chunk_size)`
 * and, with src_is_rho, also frac_ssm/ops/triton/frac_scan.py:40.
 */
int fracssm_chunk_cumsum(const float *src, int64_t sb, int64_t sl, int src_is_rho, float *lcr,
                         float *chunk_decay, int64_t B, int64_t L, int64_t M, int64_t T,
                         void *stream);

/*
 * Per-chunk state contribution, states [B, N, R, M] (states_dtype f32 or bf16):
 *   states[b,n,r,m] = sum_t u[t,r] * kappa[t,m] * exp(lcr[last,m] - lcr[t,m]).
 * Replaces frac_ssm/ops/triton/chunk_state.py:305
 * `chunk_state(u, kappa, log_cum_rho, chunk_size, state_fp32)`.
 */
int fracssm_chunk_state(const void *u, int u_dtype, int64_t u_sb, int64_t u_sl, const void *kappa,
                        int k_dtype, int64_t k_sb, int64_t k_sl, const float *lcr, int64_t g_sb,
                        int64_t g_sl, void *states, int states_dtype, int64_t B, int64_t L,
                        int64_t R, int64_t M, int64_t T, void *stream);

/*
 * Inter-chunk recurrence: states_acc[n] = run; run = exp(chunk_decay[n]) * run + states[n].
 * initial_state may be NULL (zero).  The carry is kept in float32 whatever the I/O types.
 * states, states_acc [B, N, R, M]; chunk_decay [B, N, M] f32; initial/final [B, R, M].
 * Replaces frac_ssm/ops/triton/state_passing.py:322
 * `state_passing(states, chunk_decay, initial_state)`.
 */
int fracssm_state_passing(const void *states, int states_dtype, const float *chunk_decay,
                          const void *initial_state, int init_dtype, void *states_acc,
                          int acc_dtype, void *final_state, int final_dtype, int64_t B, int64_t N,
                          int64_t R, int64_t M, void *stream);

/*
 * Causal intra-chunk matrix W [B, N, T, T] f32 (zero above the diagonal):
 *   W[t,k] = sum_m c[t,m] * exp(lcr[t,m] - lcr[k,m]) * kappa[k,m],  k <= t.
 * Replaces frac_ssm/ops/triton/chunk_w.py:418 `chunk_w(c, kappa, log_cum_rho, chunk_size)`.
 */
int fracssm_chunk_w(const void *c, const void *kappa, int ck_dtype, int64_t c_sb, int64_t c_sl,
                    int64_t k_sb, int64_t k_sl, const float *lcr, int64_t g_sb, int64_t g_sl,
                    float *W, int64_t B, int64_t L, int64_t M, int64_t T, void *stream);

/*
 * h = (c * exp(lcr)) . states_acc^T + W . u per chunk; h [B, L, R] in u's dtype.
 * Replaces frac_ssm/ops/triton/chunk_readout.py:657
 * `chunk_readout(u, c, states_acc, W, log_cum_rho, chunk_size)`.
 */
int fracssm_chunk_readout(const void *u, int u_dtype, int64_t u_sb, int64_t u_sl, const void *c,
                          int c_dtype, int64_t c_sb, int64_t c_sl, const void *states_acc,
                          int acc_dtype, const void *W, int w_dtype, const float *lcr, int64_t g_sb,
                          int64_t g_sl, void *h, int64_t B, int64_t L, int64_t R, int64_t M,
                          int64_t T, void *stream);

/*
 * chunk_w and chunk_readout in one kernel; W never reaches memory.
 * Replaces frac_ssm/ops/cute/chunk_fused_readout.py:150
 * `chunk_fused_readout(u, c, kappa, states_acc, log_cum_rho, chunk_size)`.
 */
int fracssm_chunk_fused_readout(const void *u, int u_dtype, int64_t u_sb, int64_t u_sl,
                                const void *c, const void *kappa, int ck_dtype, int64_t c_sb,
                                int64_t c_sl, int64_t k_sb, int64_t k_sl, const void *states_acc,
                                int acc_dtype, const float *lcr, int64_t g_sb, int64_t g_sl,
                                void *h, int64_t B, int64_t L, int64_t R, int64_t M, int64_t T,
                                void *stream);

/*
 * The composed forward scan.  u [B,L,R]; c, kappa [B,L,M] (same dtype: u's or f32);
 * rho [B,L,M] f32; initial_state [B,R,M] f32 or NULL; h [B,L,R] in u's dtype;
 * final_state [B,R,M] (final_dtype f32 or bf16) or NULL.  workspace: device scratch of at
 * least fracssm_frac_scan_workspace_bytes(...) bytes, 256-byte aligned, caller-owned.
 * path: 0 = pick (single-pass tcgen05 kernel when the shape is covered, else staged),
 *       1 = staged kernels, 2 = single-pass kernel (error if the shape is not covered).
 * Replaces frac_ssm/ops/frac_scan.py:53 `frac_scan(...)` /
 * frac_ssm/ops/triton/frac_scan.py:102.
 */
size_t fracssm_frac_scan_workspace_bytes(int64_t B, int64_t L, int64_t R, int64_t M, int64_t T,
                                         int path);
int fracssm_frac_scan_fwd(const void *u, int u_dtype, int64_t u_sb, int64_t u_sl, const void *c,
                          const void *kappa, int ck_dtype, int64_t c_sb, int64_t c_sl,
                          int64_t k_sb, int64_t k_sl, const float *rho, int64_t r_sb, int64_t r_sl,
                          const float *initial_state, void *h, void *final_state, int final_dtype,
                          void *workspace, size_t workspace_bytes, int64_t B, int64_t L, int64_t R,
                          int64_t M, int64_t T, int path, void *stream);

/*
 * The composed forward scan for callers that can neither allocate device memory nor let the
 * library do so (allocator callbacks of another framework, serving loops that forbid
 * cudaMalloc after start-up, bindings without a device allocator).  Same math and kernel as
 * fracssm_frac_scan_fwd with path = 2, but the kernel's scratch is a fixed array inside the
 * library's device image (about 2.1 MB per GPU that loads the library, held until exit), so
 * there is no workspace argument.  Limits: dense tensors, R = 64, M = 128, bf16 u/c/kappa,
 * fp32 rho, 16-byte aligned pointers, and batch*heads B <= 64; larger B is rejected with
 * FRACSSM_ERR_UNSUPPORTED.
 * Calls no cudaMalloc / cudaFree.  The first call on a device looks up the array's device
 * address (once, with that device current): make that first call outside any stream capture.
 * All calls on a device share the array: the ticket and progress counters are cleared on the
 * stream before each launch, and two calls whose kernels overlap on the GPU (different
 * streams) race on it: serialise them.  No counterpart in the reference.
 */
int fracssm_frac_scan_fwd_noalloc(const void *u, const void *c, const void *kappa, const float *rho,
                                  const float *initial_state, void *h, void *final_state,
                                  int final_dtype, int64_t B, int64_t L, int64_t R, int64_t M,
                                  void *stream);

/*
 * Segment summary for sequence sharding: for a segment of L tokens per row, the state it leaves
 * from `initial_state` (or zero) and the product of its decays, so that it acts on any incoming
 * state S as S -> decay (.) S + final_state.  u bf16 [B,L,64]; kappa bf16 or f32 [B,L,128]; rho f32;
 * final_state f32 [B,64,128]; decay f32 [B,128]; dense tensors; workspace of
 * fracssm_segment_summary_workspace_bytes bytes, 256-byte aligned.  Reads u, kappa, rho once.
 * New with respect to the reference (it has no sequence parallelism); the composition rule is the
 * segment summary of frac_ssm/ops/cute/state_passing.py:144-199.
 */
size_t fracssm_segment_summary_workspace_bytes(int64_t B, int64_t R, int64_t M);
int fracssm_segment_summary(const void *u, const void *kappa, int k_dtype, const float *rho,
                            const float *initial_state, float *final_state, float *decay,
                            void *workspace, size_t workspace_bytes, int64_t B, int64_t L, int64_t R,
                            int64_t M, void *stream);

/*
 * The same for rows that come in groups of `group` consecutive rows (the sub-segments of one
 * sequence, in order): the last row of every group is left out and its final_state and decay entries
 * are not written.  A process that cuts its own sequence into sub-segments needs the summaries of all
 * but the last one.  group <= 1: every row; otherwise B must be a multiple of group.  The state starts
 * from zero.  Same workspace as fracssm_segment_summary.  New with respect to the reference.
 */
int fracssm_segment_summary_grouped(const void *u, const void *kappa, int k_dtype, const float *rho,
                                    float *final_state, float *decay, void *workspace,
                                    size_t workspace_bytes, int64_t B, int64_t L, int64_t R, int64_t M,
                                    int64_t group, void *stream);

/*
 * Reads back the error word of the last single-pass launch that used `workspace` (this call
 * synchronises the stream).  Returns 0, or FRACSSM_ERR_WAIT when a bounded device-side wait
 * (for a predecessor tile's state, a TMA load or an MMA) ran out; the outputs the launch still wrote
 * for the affected rows are NaN, and tiles it no longer got to are left unwritten: after this status
 * the outputs of the whole launch are to be discarded.
 * No counterpart in the reference (its kernels have no cross-CTA waits).
 */
int fracssm_scan_fused_status(const void *workspace, void *stream);

/*
 * The same read-back for fracssm_frac_scan_fwd_noalloc, whose scratch the caller never sees: error
 * word of the last such launch on the current device (synchronises the stream).  No counterpart in
 * the reference.
 */
int fracssm_frac_scan_noalloc_status(void *stream);

/*
 * Elementwise scan-parameter prep after the two projections.
 * dyn [Bt, L, 3H] (dt, alpha, lambda logits), rw [Bt, L, 2*H*M] (read then write residuals),
 * x_conv [Bt, L, H*R]; mask [Bt, L] f32 or NULL; dt_bias [H], base_log_tau [M] f32;
 * read_gate_logit, write_gate_logit: the two scalar parameters as DEVICE pointers to one float32 each,
 * as the reference passes them (frac_ssm/layers/compute_params.py:199-202): no host read of a
 * parameter, hence no synchronisation in the forward; the sigmoid is applied in the kernel.
 * Outputs head-major: u [Bt*H, L, R] (x dtype; NULL when the caller already has it, see
 * fracssm_causal_conv_silu_heads: x_conv is then not read), rho [Bt*H, L, M] f32, c and kappa [Bt*H, L, M] in
 * ck_dtype (f32 is what the reference emits; bf16 halves the scan's coefficient traffic).
 * Replaces the kernel behind frac_ssm/layers/compute_params.py:583
 * `frac_compute_scan_params(model, x_conv, x, attention_mask)` (:165-213).
 */
int fracssm_compute_params(const void *dyn, int dyn_dtype, int64_t dyn_sb, int64_t dyn_sl,
                           const void *rw, int rw_dtype, int64_t rw_sb, int64_t rw_sl,
                           const void *x_conv, int x_dtype, int64_t x_sb, int64_t x_sl,
                           const float *mask, int64_t m_sb, int64_t m_sl, const float *dt_bias,
                           const float *base_log_tau, const float *read_gate_logit,
                           const float *write_gate_logit, float read_temp, float dt_min, float dt_max,
                           float alpha_min, float alpha_max, float lambda_min, float lambda_max,
                           void *u, void *c, void *kappa, int ck_dtype, float *rho, int64_t Bt,
                           int64_t L, int64_t H, int64_t R, int64_t M, void *stream);

/*
 * out[b, l, h*R + r] = mixed_flat[b*H + h, l, r] + x_conv[b, l, h*R + r] * D[h, r].
 * Replaces frac_ssm/layers/output_mix.py:232 `frac_skip_mix(model, mixed_flat, x_conv, out_dtype)`.
 */
int fracssm_skip_mix(const void *mixed_flat, int mf_dtype, int64_t mf_sb, int64_t mf_sl,
                     const void *x_conv, int x_dtype, int64_t x_sb, int64_t x_sl, const float *D,
                     void *out, int out_dtype, int64_t Bt, int64_t L, int64_t H, int64_t R,
                     void *stream);

/*
 * y = w * rmsnorm(x * silu(gate)) over rows of width D; gate may be NULL; rstd [rows] f32 or NULL.
 * Replaces frac_ssm/modules/rmsnorm_gated.py:65 `rmsnorm_gated_fwd` behind
 * `MambaRMSNormGated.forward` (:292-299).
 */
int fracssm_rmsnorm_gated(const void *x, int64_t x_srow, const void *gate, int64_t g_srow,
                          int xg_dtype, const void *weight, int w_dtype, float eps, void *y,
                          float *rstd, int64_t rows, int64_t D, void *stream);

/*
 * Skip-mix and gated RMSNorm in one pass over the scan output:
 *   y[b,l,:] = w * rmsnorm((h[bh,l,:] + x_conv[b,l,:] * D) * silu(gate[b,l,:])).
 * Replaces the pair frac_ssm/models/modeling_frac.py:213-214.
 */
int fracssm_scan_epilogue(const void *h, int h_dtype, int64_t h_sb, int64_t h_sl,
                          const void *x_conv, int64_t x_sb, int64_t x_sl, const void *gate,
                          int64_t g_sb, int64_t g_sl, int xg_dtype, const float *D,
                          const void *weight, int w_dtype, float gate_bias, float eps, void *y,
                          int64_t Bt, int64_t L, int64_t H, int64_t R, void *stream);

/*
 * Scan, skip-mix and gated RMSNorm of one layer with the epilogue fused into the scan's output stage:
 * h never reaches memory.  Replaces the sequence frac_ssm/models/modeling_frac.py:203-214
 * (frac_scan -> frac_skip_mix, frac_ssm/layers/output_mix.py:232 -> MambaRMSNormGated,
 * frac_ssm/modules/rmsnorm_gated.py:292) for R = 64, M = 128, bf16 u / gate, dense tensors.
 *   fracssm_scan_layer_gated: the single-pass scan kernel writes
 *       gated[b, l, head*64 + r] = (h[b*H + head, l, r] + u[b*H + head, l, r] * D[head, r])
 *                                  * silu(gate[b, l, head*64 + r] + gate_bias)          (bf16, [Bt, L, H*64])
 *     and ss_partial [Bt, L, H, 4] float32, four partial sums of gated^2 per (b, l, head).  u [Bt*H, L, 64] is
 *     the head-major copy of x_conv that the parameter prep makes, so the skip term reads it directly.
 *     workspace: fracssm_scan_layer_workspace_bytes bytes, 256-byte aligned.
 *   fracssm_scan_layer_norm: y[b, l, :] = weight * gated[b, l, :] * rsqrt(sum / norm_width + eps), where sum
 *     is the row's total of ss_partial, or sumsq[b*L + l] when sumsq is not NULL (a layer whose heads are
 *     spread over several GPUs: the caller adds the per-rank sums from fracssm_scan_layer_sumsq with one
 *     all-reduce and passes the layer's full width as norm_width).
 */
size_t fracssm_scan_layer_workspace_bytes(int64_t Bt, int64_t H, int64_t L, int64_t R, int64_t M);
int fracssm_scan_layer_gated(const void *u, const void *c, const void *kappa, int ck_dtype, const float *rho,
                             const float *initial_state, const void *gate, const float *D, float gate_bias,
                             void *gated, float *ss_partial, void *final_state, int final_dtype,
                             void *workspace, size_t workspace_bytes, int64_t Bt, int64_t H, int64_t L,
                             int64_t R, int64_t M, void *stream);
int fracssm_scan_layer_sumsq(const float *ss_partial, float *sumsq, int64_t Bt, int64_t L, int64_t H,
                             void *stream);
int fracssm_scan_layer_norm(const void *gated, const float *ss_partial, const float *sumsq, const void *weight,
                            int w_dtype, float eps, int64_t norm_width, void *y, int64_t Bt, int64_t L,
                            int64_t H, int64_t R, void *stream);

/*
 * The same epilogue for a layer whose heads are spread over several GPUs (the norm then spans columns
 * held by other GPUs).  Pass 1 writes, per (b, l) row, the sum of squares of the gated values of the H
 * local heads; the caller adds these [Bt*L] float32 vectors across GPUs (one all-reduce); pass 2
 * normalises the local columns with the total over all `norm_width` columns of the layer.
 * The reference has no head-sharded layer; single-GPU semantics are those of fracssm_scan_epilogue
 * (frac_ssm/models/modeling_frac.py:213-214, frac_ssm/modules/rmsnorm_gated.py:8-24).
 */
int fracssm_scan_epilogue_sumsq(const void *h, int h_dtype, int64_t h_sb, int64_t h_sl,
                                const void *x_conv, int64_t x_sb, int64_t x_sl, const void *gate,
                                int64_t g_sb, int64_t g_sl, int xg_dtype, const float *D,
                                float gate_bias, float *sumsq, int64_t Bt, int64_t L, int64_t H,
                                int64_t R, void *stream);
int fracssm_scan_epilogue_apply(const void *h, int h_dtype, int64_t h_sb, int64_t h_sl,
                                const void *x_conv, int64_t x_sb, int64_t x_sl, const void *gate,
                                int64_t g_sb, int64_t g_sl, int xg_dtype, const float *D,
                                const void *weight, int w_dtype, float gate_bias, float eps,
                                const float *sumsq, int64_t norm_width, void *y, int64_t Bt, int64_t L,
                                int64_t H, int64_t R, void *stream);

/*
 * Causal depthwise convolution + SiLU over channels-last activations:
 *   y[b,l,ch] = silu(bias[ch] + sum_k weight[ch,k] * xm[b, l-(K-1)+k, ch]),  xm = x * mask (zero before
 * the sequence start).  x [Bt,L,C] with batch / token strides in elements, mask float32 [Bt,L] or NULL,
 * weight [C,K] and bias [C] (or NULL) of w_dtype, y [Bt,L,C] dense, K in 1..8.
 * Replaces frac_ssm/models/modeling_frac.py:116-131 (`FracMixer._causal_conv_full`: nn.Conv1d with
 * left padding K-1 followed by the activation, or causal_conv1d_fn).
 */
int fracssm_causal_conv_silu(const void *x, int x_dtype, int64_t x_sb, int64_t x_sl, const float *mask,
                             int64_t m_sb, int64_t m_sl, const void *weight, const void *bias,
                             int w_dtype, void *y, int y_dtype, int64_t Bt, int64_t L, int64_t C,
                             int64_t K, void *stream);

/*
 * The same convolution, which also writes its result as the scan's head-major input
 *   u_heads[(b*H + h), l, r] = y[b, l, h*R + r]   (H = C / R; same dtype as y; NULL: only y is written),
 * so that fracssm_compute_params can be called with u = NULL and skips its copy of x_conv.
 * Replaces frac_ssm/models/modeling_frac.py:116-140 together with the head-major copy of
 * frac_ssm/layers/compute_params.py:154-164.
 */
int fracssm_causal_conv_silu_heads(const void *x, int x_dtype, int64_t x_sb, int64_t x_sl, const float *mask,
                                   int64_t m_sb, int64_t m_sl, const void *weight, const void *bias,
                                   int w_dtype, void *y, int y_dtype, void *u_heads, int64_t R, int64_t Bt,
                                   int64_t L, int64_t C, int64_t K, void *stream);

/*
 * One decode token for every (batch, head): state [Bt*H, M, R] float32 is updated in place,
 *   state[m,r] = rho[m] * state[m,r] + kappa[m] * u[r];  out[r] = sum_m c[m] * state[m,r] + u[r] * D[h,r].
 * u [Bt*H, R] (u_dtype), c / kappa / rho [Bt*H, M] float32, D [H, R] float32, out [Bt*H, R] float32.
 * Replaces frac_ssm/models/modeling_frac.py:159-179 (`FracMixer._update_state`) and the skip of :236.
 */
int fracssm_decode_step(const void *u, int u_dtype, const float *c, const float *kappa, const float *rho,
                        const float *D, float *state, float *out, int64_t Bt, int64_t H, int64_t R,
                        int64_t M, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* FRACSSM_H */

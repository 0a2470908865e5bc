// The composed forward scan behind one C entry point.
//
// Staged path: log+cumsum -> chunk_state -> state_passing -> fused readout, with the
// intermediates (lcr, chunk_decay, states, states_acc) in caller-provided scratch.
// Single-pass path: the tcgen05 kernel in scan_fused.cu when the shape is covered.
#include "common.cuh"

namespace fracssm {

struct ScanScratch {
  float *lcr, *chunk_decay, *states, *states_acc;
  size_t bytes;
};

static size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

static ScanScratch staged_layout(void *base, int64_t B, int64_t L, int64_t R, int64_t M, int64_t T) {
  const int64_t N = ceil_div(L, T);
  ScanScratch s{};
  size_t off = 0;
  char *p = reinterpret_cast<char *>(base);
  s.lcr = reinterpret_cast<float *>(p + off);          off += align256((size_t)B * L * M * 4);
  s.chunk_decay = reinterpret_cast<float *>(p + off);  off += align256((size_t)B * N * M * 4);
  s.states = reinterpret_cast<float *>(p + off);       off += align256((size_t)B * N * R * M * 4);
  s.states_acc = reinterpret_cast<float *>(p + off);   off += align256((size_t)B * N * R * M * 4);
  s.bytes = off;
  return s;
}

// defined in scan_fused.cu
size_t scan_fused_workspace_bytes(int64_t B, int64_t L, int64_t R, int64_t M, int64_t T);
int scan_fused_launch(const void *u, const void *c, const void *kappa, int ck_dtype, const float *rho,
                      const float *initial_state, void *h, void *final_state, int final_dtype,
                      void *workspace, size_t workspace_bytes, int64_t B, int64_t L, int64_t R,
                      int64_t M, int64_t T, void *stream);

}  // namespace fracssm

extern "C" size_t fracssm_frac_scan_workspace_bytes(int64_t B, int64_t L, int64_t R, int64_t M,
                                                    int64_t T, int path) {
  using namespace fracssm;
  if (B <= 0 || L <= 0 || R <= 0 || M <= 0 || T <= 0) return 0;
  const size_t staged = staged_layout(nullptr, B, L, R, M, T).bytes;
  const size_t fused = scan_fused_workspace_bytes(B, L, R, M, T);
  if (path == 1) return staged;
  if (path == 2) return fused;
  return staged > fused ? staged : fused;
}

extern "C" int fracssm_frac_scan_fwd(const void *u, int u_dtype, int64_t u_sb, int64_t u_sl,
                                     const void *c, const void *kappa, int ck_dtype, int64_t c_sb,
                                     int64_t c_sl, int64_t k_sb, int64_t k_sl, const float *rho,
                                     int64_t r_sb, int64_t r_sl, const float *initial_state,
                                     void *h, void *final_state, int final_dtype, void *workspace,
                                     size_t workspace_bytes, int64_t B, int64_t L, int64_t R,
                                     int64_t M, int64_t T, int path, void *stream) {
  using namespace fracssm;
  if (B < 0 || L < 0 || R <= 0 || M <= 0 || T <= 0) return fail(FRACSSM_ERR_ARG, "frac_scan: bad sizes");
  if (!known_dtype(u_dtype) || !known_dtype(ck_dtype)) return fail(FRACSSM_ERR_ARG, "frac_scan: unsupported dtype");
  if (ck_dtype != u_dtype && ck_dtype != FRACSSM_F32)
    return fail(FRACSSM_ERR_ARG, "frac_scan: c and kappa dtype must match u dtype or be float32");
  if (final_state && final_dtype != FRACSSM_F32 && final_dtype != FRACSSM_BF16)
    return fail(FRACSSM_ERR_ARG, "frac_scan: final_state dtype must be float32 or bfloat16");
  if (path < 0 || path > 2) return fail(FRACSSM_ERR_ARG, "frac_scan: path must be 0, 1 or 2");
  if (B == 0) return FRACSSM_OK;
  if (L == 0) {
    // no tokens: the final state is the initial state
    if (final_state) {
      if (initial_state && final_dtype == FRACSSM_F32) {
        cudaError_t e = cudaMemcpyAsync(final_state, initial_state, (size_t)B * R * M * 4,
                                        cudaMemcpyDeviceToDevice, (cudaStream_t)stream);
        if (e != cudaSuccess) return fail(FRACSSM_ERR_CUDA, "frac_scan: %s", cudaGetErrorString(e));
      } else if (!initial_state) {
        cudaError_t e = cudaMemsetAsync(final_state, 0, (size_t)B * R * M * dtype_size(final_dtype),
                                        (cudaStream_t)stream);
        if (e != cudaSuccess) return fail(FRACSSM_ERR_CUDA, "frac_scan: %s", cudaGetErrorString(e));
      } else {
        return fail(FRACSSM_ERR_UNSUPPORTED, "frac_scan: L == 0 with a bfloat16 final_state");
      }
    }
    return FRACSSM_OK;
  }
  if (!u || !c || !kappa || !rho || !h || !workspace) return fail(FRACSSM_ERR_ARG, "frac_scan: null pointer");
  if ((reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
    return fail(FRACSSM_ERR_ARG, "frac_scan: workspace must be 256-byte aligned");

  const bool dense = u_sl == R && u_sb == L * R && c_sl == M && c_sb == L * M && k_sl == M &&
                     k_sb == L * M && r_sl == M && r_sb == L * M;
  // the single-pass kernel moves its inputs with bulk copies and 16-byte accesses
  const bool aligned16 = ((reinterpret_cast<uintptr_t>(u) | reinterpret_cast<uintptr_t>(c) |
                           reinterpret_cast<uintptr_t>(kappa) | reinterpret_cast<uintptr_t>(rho) |
                           reinterpret_cast<uintptr_t>(h)) & 15) == 0;
  const bool fused_ok = dense && aligned16 && fracssm_scan_fused_supported(B, L, R, M, T, u_dtype, ck_dtype);
  if (path == 2 && !fused_ok)
    return fail(FRACSSM_ERR_UNSUPPORTED, "frac_scan: shape, dtype, strides or alignment not covered by the single-pass kernel");
  if (fused_ok && path != 1) {
    if (workspace_bytes < scan_fused_workspace_bytes(B, L, R, M, T))
      return fail(FRACSSM_ERR_ARG, "frac_scan: workspace too small");
    return scan_fused_launch(u, c, kappa, ck_dtype, rho, initial_state, h, final_state, final_dtype,
                             workspace, workspace_bytes, B, L, R, M, T, stream);
  }

  ScanScratch s = staged_layout(workspace, B, L, R, M, T);
  if (workspace_bytes < s.bytes) return fail(FRACSSM_ERR_ARG, "frac_scan: workspace too small");
  const int64_t N = ceil_div(L, T);
  int rc = fracssm_chunk_cumsum(rho, r_sb, r_sl, 1, s.lcr, s.chunk_decay, B, L, M, T, stream);
  if (rc) return rc;
  rc = fracssm_chunk_state(u, u_dtype, u_sb, u_sl, kappa, ck_dtype, k_sb, k_sl, s.lcr, L * M, M,
                           s.states, FRACSSM_F32, B, L, R, M, T, stream);
  if (rc) return rc;
  rc = fracssm_state_passing(s.states, FRACSSM_F32, s.chunk_decay, initial_state, FRACSSM_F32,
                             s.states_acc, FRACSSM_F32, final_state, final_dtype, B, N, R, M, stream);
  if (rc) return rc;
  return fracssm_chunk_fused_readout(u, u_dtype, u_sb, u_sl, c, kappa, ck_dtype, c_sb, c_sl, k_sb,
                                     k_sl, s.states_acc, FRACSSM_F32, s.lcr, L * M, M, h, B, L, R, M,
                                     T, stream);
}

// Shared helpers for the fracssm kernels: status/error plumbing, dtype-generic loads.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "fracssm.h"

namespace fracssm {

// Records a message for fracssm_last_error() and returns `code`.
int fail(int code, const char *fmt, ...);

inline int check_launch(const char *what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(FRACSSM_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  return FRACSSM_OK;
}

inline bool known_dtype(int dt) { return dt == FRACSSM_F32 || dt == FRACSSM_BF16 || dt == FRACSSM_F16; }
inline size_t dtype_size(int dt) { return dt == FRACSSM_F32 ? 4 : 2; }

__device__ __forceinline__ float ld_f32(const void *p, int64_t i, int dt) {
  if (dt == FRACSSM_F32) return reinterpret_cast<const float *>(p)[i];
  if (dt == FRACSSM_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p)[i]);
  return __half2float(reinterpret_cast<const __half *>(p)[i]);
}

__device__ __forceinline__ void st_f32(void *p, int64_t i, int dt, float v) {
  if (dt == FRACSSM_F32) reinterpret_cast<float *>(p)[i] = v;
  else if (dt == FRACSSM_BF16) reinterpret_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(v);
  else reinterpret_cast<__half *>(p)[i] = __float2half_rn(v);
}

constexpr float kRhoFloor = 1e-6f;
constexpr float kLog2e = 1.4426950408889634f;

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Output stage of the single-pass scan in layer mode: skip connection and gate applied to the
// accumulator rows, un-flattened to [batch, L, H * 64], with partial sums of squares for the norm.
struct ScanLayerOut {
  const void *gate;   // bf16 [batch, L, H * 64]
  const float *D;     // [H, 64]
  void *gated;        // bf16 [batch, L, H * 64]
  float *ss;          // [batch, L, H, 4]
  float gate_bias;
  int64_t H;
};

// default limit of a device-side wait, in nanoseconds
inline unsigned long long tile_default_wait_ns() { return 2000000000ull; }

// defined in scan_fused.cu
size_t scan_fused_workspace_bytes(int64_t B, int64_t L, int64_t R, int64_t M, int64_t T);
int scan_fused_launch_ex(const void *u, const void *c, const void *kappa, int ck_dtype, const float *rho,
                         const float *initial_state, void *h, void *final_state, int final_dtype,
                         void *workspace, size_t workspace_bytes, int64_t B, int64_t L, int64_t R,
                         int64_t M, int64_t T, void *stream, int first_tile, unsigned long long wait_ns,
                         const ScanLayerOut *layer);

}  // namespace fracssm

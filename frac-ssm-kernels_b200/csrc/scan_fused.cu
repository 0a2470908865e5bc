// Single-pass tcgen05 scan kernel: entry points used by frac_scan.cu.
#include "common.cuh"

namespace fracssm {

size_t scan_fused_workspace_bytes(int64_t, int64_t, int64_t, int64_t, int64_t) { return 0; }

int scan_fused_launch(const void *, const void *, const void *, int, const float *, const float *,
                      void *, void *, int, void *, size_t, int64_t, int64_t, int64_t, int64_t,
                      int64_t, void *) {
  return fail(FRACSSM_ERR_UNSUPPORTED, "single-pass scan kernel not built");
}

}  // namespace fracssm

extern "C" int fracssm_scan_fused_supported(int64_t, int64_t, int64_t, int64_t, int64_t, int, int) {
  return 0;
}

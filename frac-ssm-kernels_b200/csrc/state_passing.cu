// Inter-chunk recurrence (latency-bound stage): one thread per (bh, r, m) lane walks the
// chunks in order with a float32 carry.
//   states_acc[n] = run;  run = exp(chunk_decay[n]) * run + states[n]
#include "common.cuh"

namespace fracssm {

__global__ void __launch_bounds__(256)
state_passing_kernel(const void *__restrict__ states, int s_dt, const float *__restrict__ cd,
                     const void *__restrict__ init, int i_dt, void *__restrict__ acc, int a_dt,
                     void *__restrict__ fin, int f_dt, int64_t N, int64_t RM, int64_t M) {
  const int64_t b = blockIdx.y;
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // r * M + m
  if (e >= RM) return;
  const int64_t m = e % M;
  float run = init ? ld_f32(init, b * RM + e, i_dt) : 0.f;
  for (int64_t n = 0; n < N; ++n) {
    const int64_t at = (b * N + n) * RM + e;
    st_f32(acc, at, a_dt, run);
    run = fmaf(__expf(cd[(b * N + n) * M + m]), run, ld_f32(states, at, s_dt));
  }
  if (fin) st_f32(fin, b * RM + e, f_dt, run);
}

}  // namespace fracssm

extern "C" int fracssm_state_passing(const void *states, int states_dtype, const float *chunk_decay,
                                     const void *initial_state, int init_dtype, void *states_acc,
                                     int acc_dtype, void *final_state, int final_dtype, int64_t B,
                                     int64_t N, int64_t R, int64_t M, void *stream) {
  using namespace fracssm;
  if (B < 0 || N < 0 || R <= 0 || M <= 0) return fail(FRACSSM_ERR_ARG, "state_passing: bad sizes");
  auto ok = [](int dt) { return dt == FRACSSM_F32 || dt == FRACSSM_BF16; };
  if (!ok(states_dtype) || !ok(acc_dtype) || !ok(final_dtype) || (initial_state && !ok(init_dtype)))
    return fail(FRACSSM_ERR_ARG, "state_passing: dtypes must be float32 or bfloat16");
  if (B == 0) return FRACSSM_OK;
  if ((N > 0 && (!states || !chunk_decay || !states_acc)))
    return fail(FRACSSM_ERR_ARG, "state_passing: null pointer");
  if (B > 65535) return fail(FRACSSM_ERR_UNSUPPORTED, "state_passing: B too large for one launch");
  const int64_t RM = R * M;
  dim3 grid((unsigned)ceil_div(RM, 256), (unsigned)B);
  state_passing_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(
      states, states_dtype, chunk_decay, initial_state, init_dtype, states_acc, acc_dtype,
      final_state, final_dtype, N, RM, M);
  return check_launch("state_passing");
}

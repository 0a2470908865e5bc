// Segment summary on sm_100a: what a stretch of tokens does to the state, without the readout.
//
// For every row (batch x head) of a segment of L tokens:
//   final[r, m] = state left by the segment when it starts from a zero (or a given) state
//   decay[m]    = product of max(rho, 1e-6) over the segment
// so that the segment acts on any incoming state S as  S -> decay (.) S + final.  Sequence sharding
// composes these pairs across ranks.  Only u, kappa and rho are read (70 % of the scan's bytes).
//
// Same skeleton as the single-pass scan kernel with the readout removed: persistent CTAs, tickets
// in tile-major order, 16 worker warps forming Khat = kappa * (decay to the tile's end) as bf16
// high + low operand tiles, one control warp issuing the TMA load of u and the two tcgen05
// products Khat^T u, the state handed from tile to tile through scratch and a per-row counter
// with bounded waits.
#include <mutex>
#include <type_traits>

#include "common.cuh"
#include "scan_tile.cuh"
#include "tmap.cuh"
#include "umma.cuh"

namespace fracssm {
namespace {

using namespace tile;
constexpr int kWorkers = 512, kThreads = 640;
constexpr uint32_t kOffKhi = 0, kOffKlo = 32768, kOffU = 65536, kOffSeg = 81920, kOffGt = 90112, kOffMisc = 90624;
constexpr uint32_t kSmemBytes = kOffMisc + 128 + 1024;
constexpr uint32_t kTmemCols = 64;
constexpr size_t kCtrlBytes = 256;

struct SummaryArgs {
  const void *kappa;  // bf16 or f32 [BH, L, 128]
  const float *rho, *init;
  float *fin;    // [BH, 64, 128]
  float *decay;  // [BH, 128]
  int *ctrl, *flags;
  float *state;  // running state per row (worker access order)
  float *dec;    // running decay product per row [BH, 128]
  int BH, L, ntiles, total;
  int rows, group;             // rows the launch works on; group > 1: the last row of every `group` rows is left out
  int first_tile;              // tile index of the first ticket (0 except in the wait-limit self-test)
  unsigned long long wait_ns;  // limit of every device-side wait
};

// Row of the q-th row that the launch works on (rows come in groups of a.group; the last of each is skipped).
__device__ __forceinline__ int summary_row(const SummaryArgs &a, int q) {
  return a.group > 1 ? q + q / (a.group - 1) : q;
}

template <bool KF32>
__global__ void __launch_bounds__(kThreads, 1)
scan_summary_kernel(const SummaryArgs a, const __grid_constant__ CUtensorMap u_map) {
  using CK = typename std::conditional<KF32, float4, uint2>::type;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t *khi = smem + kOffKhi, *klo = smem + kOffKlo, *u_tile = smem + kOffU;
  float *seg = reinterpret_cast<float *>(smem + kOffSeg);
  float *gt_s = reinterpret_cast<float *>(smem + kOffGt);
  // mbarriers, each completed once per tile: cb (tcgen05.commit), barU (TMA), full (16 worker
  // warps), item_bar / state_bar (control warp), out_bar (16 worker warps)
  uint64_t *cb = reinterpret_cast<uint64_t *>(smem + kOffMisc);
  uint64_t *barU = cb + 1, *full = cb + 2, *item_bar = cb + 3, *state_bar = cb + 4, *out_bar = cb + 5;
  uint32_t *tmem_s = reinterpret_cast<uint32_t *>(cb + 6);
  volatile int *items = reinterpret_cast<volatile int *>(tmem_s + 1);
  volatile int *failed = reinterpret_cast<volatile int *>(tmem_s + 3);  // a wait of this CTA ran out

  const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    umma::mbar_init(cb, 1);
    umma::mbar_init(barU, 1);
    umma::mbar_init(full, 16);
    umma::mbar_init(item_bar, 1);
    umma::mbar_init(state_bar, 1);
    umma::mbar_init(out_bar, 16);
    umma::fence_mbar_init();
    umma::prefetch_tmap(&u_map);
    *failed = 0;
  }
  if (w == 0) umma::tmem_alloc(tmem_s, kTmemCols);
  umma::tc_fence_before();
  __syncthreads();
  umma::tc_fence_after();
  const uint32_t tmem = *tmem_s;
  const uint64_t wait_ns = a.wait_ns;
  bool ok = true;  // cleared when a bounded wait runs out; later waits are then skipped
#define FRACSSM_WAIT(bar, parity)                                \
  if (ok) {                                                      \
    ok = umma::mbar_wait_parked(bar, (parity) & 1u, wait_ns);    \
    if (!ok) *failed = 1;                                        \
  }

  if (w > 16) {
    // spare warps: nothing to do
  } else if (w == 16) {
    // =========================== control warp ===========================
    const uint32_t sKhi = umma::smem_u32(khi), sKlo = umma::smem_u32(klo), sU = umma::smem_u32(u_tile);
    constexpr uint32_t kIdMnMn64 = umma::make_idesc(128, 64, true, true);
    int item = 0;
    if (lane == 0) {
      item = atomicAdd(&a.ctrl[0], 1);
      items[0] = item;
      umma::mbar_arrive(item_bar);
    }
    item = __shfl_sync(0xffffffffu, item, 0);
#pragma unroll 1
    for (uint32_t n = 0; item < a.total; ++n) {
      const int j = item / a.rows + a.first_tile, bh = summary_row(a, item % a.rows);
      // The next ticket is taken a tile ahead and published through item_bar.  For the first tile it
      // has to wait until the workers have read the first item (their arrival on `full`): two
      // completions of item_bar in a row would flip its parity twice, and a worker that had not
      // looked yet would wait for a phase that never comes.  From the second tile on the workers have
      // read item n before the control warp can get here (their out_bar arrival comes after it).
      int next = 0;
      auto take_next = [&]() {
        if (lane == 0) {
          next = atomicAdd(&a.ctrl[0], 1);
          items[(n + 1) & 1] = next;
          umma::mbar_arrive(item_bar);
        }
        next = __shfl_sync(0xffffffffu, next, 0);
        if (lane == 1 && next < a.total) {  // pull the next item's inputs into L2 a whole tile ahead
          const int nj = next / a.rows + a.first_tile, nb = summary_row(a, next % a.rows);
          const int ntok = min(kTile, a.L - nj * kTile);
          const int64_t tok = static_cast<int64_t>(nb) * a.L + nj * kTile;
          constexpr int kKb = KF32 ? 4 : 2;
          umma::prefetch_l2(a.rho + tok * kM, ntok * kM * 4);
          umma::prefetch_l2(reinterpret_cast<const char *>(a.kappa) + tok * kM * kKb, ntok * kM * kKb);
        }
      };
      if (n > 0) take_next();
      if (n > 0) { FRACSSM_WAIT(cb, n - 1); }  // the previous tile's MMAs no longer read u
      if (lane == 0) {
        umma::mbar_expect_tx(barU, kTile * kR * 2);
        umma::tma_load_3d(u_tile, &u_map, barU, 0, j * kTile, bh);
      }
      FRACSSM_WAIT(full, n);
      if (n == 0) take_next();
      FRACSSM_WAIT(barU, n);
      umma::tc_fence_after();
      if (lane == 0) {
        const bool early = j == 0 || ld_acquire(a.flags + bh) >= j;
        if (early) umma::mbar_arrive(state_bar);
        // Sacc[m, r] = sum_k (Khi + Klo)[k, m] u[k, r]   (MN-major operands, 8 steps of 16 tokens)
        const uint64_t dh = umma::make_sdesc(sKhi, kAtom, 1024), dl = umma::make_sdesc(sKlo, kAtom, 1024);
        const uint64_t du = umma::make_sdesc(sU, kAtom, 1024);
#pragma unroll
        for (uint32_t s = 0; s < 8; ++s) umma::mma_ss(tmem, dh + s * 128, du + s * 128, kIdMnMn64, s > 0);
#pragma unroll
        for (uint32_t s = 0; s < 8; ++s) umma::mma_ss(tmem, dl + s * 128, du + s * 128, kIdMnMn64, 1u);
        umma::mma_commit(cb);
        if (!early) {
          if (ok) {
            const uint64_t t_start = umma::global_ns();
            while (ld_acquire(a.flags + bh) < j) {
              __nanosleep(100);
              if (umma::global_ns() - t_start > wait_ns) { ok = false; *failed = 1; break; }
            }
          }
          umma::mbar_arrive(state_bar);
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      FRACSSM_WAIT(out_bar, n);  // the workers' stores of the outgoing state precede their arrivals
      if (lane == 0 && j + 1 < a.ntiles) st_release(a.flags + bh, j + 1);
      __syncwarp();
      item = next;
    }
  } else {
    // =========================== worker warps ===========================
    const int Q = w & 3, P = w >> 2;  // TMEM lane quarter of this warp, and its column part
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>(32 * Q) << 16);
    const uint32_t th_off = (lane >> 4) * kAtom + ((lane & 1) << 3) + w * 1024;
    const uint32_t c16 = ((lane & 15) >> 1) << 4;
    const uint32_t sKhi = umma::smem_u32(khi), sKlo = umma::smem_u32(klo);
    const CK *kp = reinterpret_cast<const CK *>(a.kappa);

    FRACSSM_WAIT(item_bar, 0);
    int item = items[0];
    for (uint32_t n = 0; item < a.total; ++n) {
      const int j = item / a.rows + a.first_tile, bh = summary_row(a, item % a.rows);
      const int t0 = j * kTile + 8 * w;
      const int64_t tok0 = static_cast<int64_t>(bh) * a.L + t0;
      float4 rr[8];
      CK kk[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        rr[i] = make_float4(1.f, 1.f, 1.f, 1.f);
        kk[i] = CK{};
        if (t0 + i < a.L) {
          rr[i] = __ldcs(reinterpret_cast<const float4 *>(a.rho + (tok0 + i) * kM) + lane);
          kk[i] = __ldcs(kp + (tok0 + i) * 32 + lane);
        }
      }
      // ks[i] = kappa[i] * product of rho over the tokens after i inside this 8-token segment
      float2 ks[8][2];
      float g8[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float suf = 1.f;
#pragma unroll
        for (int i = 7; i >= 0; --i) {
          float &dst = (q & 1) ? ks[i][q >> 1].y : ks[i][q >> 1].x;
          dst = ck_get(kk[i], q) * suf;
          const float4 v = rr[i];
          suf *= fmaxf(q == 0 ? v.x : q == 1 ? v.y : q == 2 ? v.z : v.w, kRhoFloor);
        }
        g8[q] = suf;
      }
      *reinterpret_cast<float4 *>(seg + w * kM + 4 * lane) = make_float4(g8[0], g8[1], g8[2], g8[3]);
      umma::named_barrier(1, kWorkers);  // segment products visible to every worker
      {
        float2 f[2];
        seg_prod(seg, w + 1, 16, lane, f);
        if (w == 0)
          *reinterpret_cast<float4 *>(gt_s + 4 * lane) =
              make_float4(g8[0] * f[0].x, g8[1] * f[0].y, g8[2] * f[1].x, g8[3] * f[1].y);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float2 kh[2], kl[2];
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            const float2 full_k = __fmul2_rn(ks[i][hf], f[hf]);
            kh[hf] = bf16_round2(full_k);
            kl[hf] = __fadd2_rn(full_k, make_float2(-kh[hf].x, -kh[hf].y));
          }
          emit_row(sKhi, th_off, c16, i, kh[0], kh[1]);
          emit_row(sKlo, th_off, c16, i, kl[0], kl[1]);
        }
      }
      warp_arrive(full, lane);

      // the next item; read before this warp's arrival on out_bar lets the control warp move on
      FRACSSM_WAIT(item_bar, n + 1);
      const int next = items[(n + 1) & 1];

      // ---- incoming state -> outgoing state
      FRACSSM_WAIT(state_bar, n);
      umma::named_barrier(2, kWorkers);  // also orders warp 0's write of gt_s before its readers
      const int m_row = 32 * Q + lane;
      float sj[16];
      float dec_in = 1.f;
      {
        const float4 *sp = reinterpret_cast<const float4 *>(a.state) +
                           (static_cast<int64_t>(bh) * 4 + P) * 4 * kM + m_row;
        if (j > 0) {
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            const float4 v = __ldcg(sp + x * kM);
            sj[4 * x] = v.x; sj[4 * x + 1] = v.y; sj[4 * x + 2] = v.z; sj[4 * x + 3] = v.w;
          }
          if (P == 0) dec_in = __ldcg(a.dec + static_cast<int64_t>(bh) * kM + m_row);
        } else if (a.init) {
#pragma unroll
          for (int x = 0; x < 16; ++x)
            sj[x] = a.init[(static_cast<int64_t>(bh) * kR + 16 * P + x) * kM + m_row];
        } else {
#pragma unroll
          for (int x = 0; x < 16; ++x) sj[x] = 0.f;
        }
      }
      FRACSSM_WAIT(cb, n);
      umma::tc_fence_after();
      {
        float acc[16];
        umma::tmem_ld16(lane_addr + 16 * P, acc);
        umma::tmem_ld_wait();
        const float gt = gt_s[m_row];
        // a wait that ran out leaves no valid state: NaN marks everything computed from it
        const float mark = *failed == 0 ? 0.f : __int_as_float(0x7fc00000);
#pragma unroll
        for (int x = 0; x < 16; ++x) acc[x] = fmaf(gt, sj[x], acc[x]) + mark;
        if (j + 1 < a.ntiles) {
          float4 *sp = reinterpret_cast<float4 *>(a.state) + (static_cast<int64_t>(bh) * 4 + P) * 4 * kM + m_row;
#pragma unroll
          for (int x = 0; x < 4; ++x)
            __stcg(sp + x * kM, make_float4(acc[4 * x], acc[4 * x + 1], acc[4 * x + 2], acc[4 * x + 3]));
          if (P == 0) __stcg(a.dec + static_cast<int64_t>(bh) * kM + m_row, dec_in * gt + mark);
        } else {
#pragma unroll
          for (int x = 0; x < 16; ++x)
            a.fin[(static_cast<int64_t>(bh) * kR + 16 * P + x) * kM + m_row] = acc[x];
          if (P == 0) a.decay[static_cast<int64_t>(bh) * kM + m_row] = dec_in * gt + mark;
        }
      }
      umma::tc_fence_before();
      __syncwarp();
      if (lane == 0) umma::mbar_arrive(out_bar);
      item = next;
    }
  }
#undef FRACSSM_WAIT

  if (!ok) atomicExch(&a.ctrl[1], 1);
  umma::tc_fence_before();
  __syncthreads();
  if (w == 0) umma::tmem_dealloc(tmem, kTmemCols);
}

size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

}  // namespace
}  // namespace fracssm

extern "C" size_t fracssm_segment_summary_workspace_bytes(int64_t B, int64_t R, int64_t M) {
  using namespace fracssm;
  if (B <= 0 || R <= 0 || M <= 0) return 0;
  return kCtrlBytes + align256((size_t)B * 4) + (size_t)B * R * M * 4 + align256((size_t)B * M * 4);
}

namespace fracssm {
// first_tile / wait_ns: 0 and the default limit, except in the wait-limit self-test, which starts at a
// tile whose predecessor is not part of the launch.
int segment_summary_launch_ex(const void *u, const void *kappa, int k_dtype, const float *rho,
                              const float *initial_state, float *final_state, float *decay, void *workspace,
                              size_t workspace_bytes, int64_t B, int64_t L, int64_t R, int64_t M, void *stream,
                              int first_tile, unsigned long long wait_ns, int64_t group) {
  if (B < 0 || L < 0) return fail(FRACSSM_ERR_ARG, "segment_summary: bad sizes");
  if (group < 0 || (group > 1 && B % group != 0))
    return fail(FRACSSM_ERR_ARG, "segment_summary: the row count must be a multiple of the group size");
  if (R != kR || M != kM || (k_dtype != FRACSSM_BF16 && k_dtype != FRACSSM_F32))
    return fail(FRACSSM_ERR_UNSUPPORTED, "segment_summary: needs R = 64, M = 128, bfloat16 u and bfloat16 or float32 kappa");
  if (B == 0) return FRACSSM_OK;
  if (L == 0) return fail(FRACSSM_ERR_UNSUPPORTED, "segment_summary: empty segment");
  if (B * ceil_div(L, kTile) >= (int64_t(1) << 30) || L >= (int64_t(1) << 30))
    return fail(FRACSSM_ERR_UNSUPPORTED, "segment_summary: too many tiles for one launch");
  if (!u || !kappa || !rho || !final_state || !decay || !workspace)
    return fail(FRACSSM_ERR_ARG, "segment_summary: null pointer");
  if ((reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
    return fail(FRACSSM_ERR_ARG, "segment_summary: workspace must be 256-byte aligned");
  // the kernel reads kappa and rho with 8- and 16-byte accesses, u by TMA
  if (((reinterpret_cast<uintptr_t>(u) | reinterpret_cast<uintptr_t>(kappa) | reinterpret_cast<uintptr_t>(rho)) & 15) != 0)
    return fail(FRACSSM_ERR_ARG, "segment_summary: u, kappa and rho must be 16-byte aligned");
  if (workspace_bytes < fracssm_segment_summary_workspace_bytes(B, R, M))
    return fail(FRACSSM_ERR_ARG, "segment_summary: workspace too small");

  static std::mutex mu;
  static int sm_count[64] = {};
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
    return fail(FRACSSM_ERR_CUDA, "segment_summary: cannot identify the current device");
  {
    std::lock_guard<std::mutex> lock(mu);
    if (sm_count[dev] == 0) {
      cudaError_t ae = cudaFuncSetAttribute(scan_summary_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
      if (ae == cudaSuccess)
        ae = cudaFuncSetAttribute(scan_summary_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
      if (ae != cudaSuccess) return fail(FRACSSM_ERR_CUDA, "segment_summary: %s", cudaGetErrorString(ae));
      int n = 0;
      cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
      if (n <= 0) return fail(FRACSSM_ERR_CUDA, "segment_summary: cannot query the SM count");
      sm_count[dev] = n;
    }
    sms = sm_count[dev];
  }
  char *ws = reinterpret_cast<char *>(workspace);
  SummaryArgs a{};
  a.kappa = kappa;
  a.rho = rho;
  a.init = initial_state;
  a.fin = final_state;
  a.decay = decay;
  a.ctrl = reinterpret_cast<int *>(ws);
  a.flags = reinterpret_cast<int *>(ws + kCtrlBytes);
  a.state = reinterpret_cast<float *>(ws + kCtrlBytes + align256((size_t)B * 4));
  a.dec = reinterpret_cast<float *>(ws + kCtrlBytes + align256((size_t)B * 4) + (size_t)B * R * M * 4);
  a.BH = (int)B;
  a.L = (int)L;
  a.ntiles = (int)ceil_div(L, kTile);
  a.first_tile = first_tile;
  a.group = group > 1 ? (int)group : 1;
  a.rows = group > 1 ? (int)(B / group * (group - 1)) : (int)B;
  a.total = (a.ntiles - first_tile) * a.rows;
  a.wait_ns = wait_ns;
  CUtensorMap map;
  int rc = make_tmap_bf16_3d(&map, u, kR, (uint64_t)L, (uint64_t)B, kR, kTile);
  if (rc) return rc;
  cudaError_t e = cudaMemsetAsync(ws, 0, kCtrlBytes + align256((size_t)B * 4), (cudaStream_t)stream);
  if (e != cudaSuccess) return fail(FRACSSM_ERR_CUDA, "segment_summary: %s", cudaGetErrorString(e));
  const int grid = a.total < sms ? a.total : sms;
  if (k_dtype == FRACSSM_F32) scan_summary_kernel<true><<<grid, kThreads, kSmemBytes, (cudaStream_t)stream>>>(a, map);
  else scan_summary_kernel<false><<<grid, kThreads, kSmemBytes, (cudaStream_t)stream>>>(a, map);
  return check_launch("segment_summary");
}
}  // namespace fracssm

extern "C" int fracssm_segment_summary(const void *u, const void *kappa, int k_dtype, const float *rho,
                                       const float *initial_state, float *final_state, float *decay,
                                       void *workspace, size_t workspace_bytes, int64_t B, int64_t L,
                                       int64_t R, int64_t M, void *stream) {
  return fracssm::segment_summary_launch_ex(u, kappa, k_dtype, rho, initial_state, final_state, decay, workspace,
                                            workspace_bytes, B, L, R, M, stream, 0, fracssm::tile::kWaitNs, 1);
}

extern "C" int fracssm_segment_summary_grouped(const void *u, const void *kappa, int k_dtype, const float *rho,
                                               float *final_state, float *decay, void *workspace,
                                               size_t workspace_bytes, int64_t B, int64_t L, int64_t R, int64_t M,
                                               int64_t group, void *stream) {
  return fracssm::segment_summary_launch_ex(u, kappa, k_dtype, rho, nullptr, final_state, decay, workspace,
                                            workspace_bytes, B, L, R, M, stream, 0, fracssm::tile::kWaitNs, group);
}

// Single-pass FRAC scan on sm_100a: every input is read once, the state stays on chip or
// in L2, all contractions run on tcgen05 with accumulators in tensor memory.
//
// Shapes covered: R = 64, M = 128, bf16 u, bf16 or f32 c / kappa, fp32 rho, dense tensors, any L.
//
// Work item = (bh, tile of 128 tokens), handed out by an atomic ticket in tile-major order
// (all bh of tile 0, then tile 1, ...).  The item (bh, j) needs the state left by (bh, j-1);
// it waits on a per-bh counter in global memory with a time limit.  A ticket is only taken
// by a running CTA (one item ahead of the one it is working on) and dependencies point to
// lower tickets, so the lowest unfinished item is always being worked on and never waits.
//
// One CTA per SM, 20 warps (three of them only pad the control warp's register group).  Warps 0-15 ("workers") turn the raw inputs into bf16 operand tiles
// in shared memory and run the epilogues; warp 16 ("control") takes tickets, issues the TMA
// load of u and every tcgen05.mma, and polls the state counter.  Workers hand a batch of tiles
// over by arriving on a "full" mbarrier (one arrival per warp, after a proxy fence); the
// control warp hands buffers and accumulators back through tcgen05.commit mbarriers.  The next
// ticket is taken a whole tile ahead, so its inputs can be pulled into L2 exactly.
//
// Math per tile (tokens t, k in 0..127; modes m; rho floored at 1e-6, 1 beyond L):
//   h[t]   = sum_m Chat[t,m] S[m,:]  +  sum_{k<=t} W[t,k] u[k,:]
//   S_next = Gt (.) S + sum_k Khat[k,:]^T u[k,:]
//   W[t,k] = sum_m c[t,m] kappa[k,m] prod_{k<j<=t} rho[j,m]
// The decay product inside W is never formed as a ratio of two long products (which would
// overflow).  W is assembled from pieces whose two factors are each <= 1:
//   * sibling levels s = 64, 32, 16, 8: for t in the second half and k in the first half of a
//     block of 2s tokens, the reference point is the boundary between the halves:
//       A_s[t] = c[t] prod_{bnd<=j<=t} rho[j],  B_s[k] = kappa[k] prod_{k<j<bnd} rho[j]
//     A-role and B-role rows share one operand tile X_s (every token has exactly one role);
//   * base: the 8x8 diagonal blocks use the middle of the block as reference, which keeps
//     the reciprocal products below 1e24.
// Every piece is a bf16 tcgen05 GEMM over the modes; an epilogue picks, for each (t, k), the
// accumulator of the one level that holds it.  Chat / Khat are the same factors taken to the
// tile's start / end; Khat is split into bf16 high and low parts so that the state keeps
// float32-level accuracy.
#include <cstdlib>
#include <mutex>
#include <type_traits>

#include "common.cuh"
#include "tmap.cuh"
#include "scan_tile.cuh"
#include "umma.cuh"

namespace fracssm {
namespace {

using namespace tile;
constexpr int kWorkers = 512, kThreads = 640;
// Registers are re-divided after launch (setmaxnreg): the 16 worker warps grow to kWorkerRegs,
// the control warp's group of four shrinks to kControlRegs.  The launch allocation per thread
// (checked on the host) must cover both, or the growing warps would wait forever.
constexpr int kWorkerRegs = 112, kControlRegs = 32;
constexpr int kLaunchRegsNeeded = (kWorkers * kWorkerRegs + (kThreads - kWorkers) * kControlRegs + kThreads - 1) / kThreads;
// shared memory map (bytes from the 1024-aligned base)
constexpr uint32_t kOffArea0 = 0, kOffArea1 = 65536;
constexpr uint32_t kOffChatLo = 131072;                  // low part of Chat, one operand tile
constexpr uint32_t kOffS = 163840, kOffSlo = 180224;     // incoming state, bf16 high and low parts
constexpr uint32_t kOffU = 196608;
constexpr uint32_t kOffSeg = 212992;    // float [16][128]: decay product of each 8-token segment
constexpr uint32_t kOffGt = 221184;     // float [128]: decay product of the whole tile
constexpr uint32_t kOffMisc = 221696;   // mbarriers, TMEM base, tickets
constexpr uint32_t kSmemBytes = kOffMisc + 192 + 128 + 1024;
// tensor-memory columns (fp32, 128 lanes each)
constexpr uint32_t kColH = 0, kColS = 64, kColBase = 128, kColL8 = 256, kColL16 = 320, kColL32 = 384,
                   kColL64 = 448;
constexpr int kProfCtas = 256, kProfPhases = 16;
constexpr size_t kCtrlBytes = 256, kProfBytes = kProfCtas * kProfPhases * sizeof(long long);

struct FusedArgs {
  const void *c, *kappa;  // bf16 or f32 [BH, L, 128], see the kernel's CKF32 parameter
  const float *rho, *init;
  __nv_bfloat16 *h;
  void *fin;
  int fin_dt;
  int *ctrl;     // [0] ticket counter, [1] error word
  long long *prof;  // [kProfCtas][16] cycles spent per phase by worker thread 0 of each CTA
  int *flags;    // [BH] tiles finished per bh
  float *state;  // running state per row, 128 m x 64 r floats in the order the workers access it
  int BH, L, ntiles, total;
};

// Raw inputs of one item for one worker thread, one group of 4 tokens x 4 modes.
// c and kappa arrive as bf16 (4 values in a uint2) or as f32 (a float4).
template <bool CKF32>
struct RawRegs {
  using CK = typename std::conditional<CKF32, float4, uint2>::type;
  float4 r[4];
  CK c[4], k[4];
};

template <bool CKF32>
__device__ __forceinline__ void load_raw(RawRegs<CKF32> &raw, const FusedArgs &a, int item, int w, int lane,
                                         int grp) {
  using CK = typename RawRegs<CKF32>::CK;
  const int j = item / a.BH, bh = item - j * a.BH;
  const int t0 = j * kTile + 8 * w + 4 * grp;
  const int64_t tok0 = static_cast<int64_t>(bh) * a.L + t0;
  const CK *cp = reinterpret_cast<const CK *>(a.c), *kp = reinterpret_cast<const CK *>(a.kappa);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    raw.r[i] = make_float4(1.f, 1.f, 1.f, 1.f);
    raw.c[i] = CK{};
    raw.k[i] = CK{};
    if (t0 + i < a.L) {
      raw.r[i] = __ldcs(reinterpret_cast<const float4 *>(a.rho + (tok0 + i) * kM) + lane);
      raw.c[i] = __ldcs(cp + (tok0 + i) * 32 + lane);   // 32 pieces of 4 modes per token row
      raw.k[i] = __ldcs(kp + (tok0 + i) * 32 + lane);
    }
  }
}

// PROF: worker thread 0 of each CTA also charges its cycles to 16 phases of the tile loop (a
// diagnostic build of the same kernel: the bookkeeping costs about 7 % of the run time, because the
// one warp that does it is on every hand-over's critical path).
template <bool CKF32, bool PROF>
__global__ void __launch_bounds__(kThreads, 1)
scan_fused_kernel(const FusedArgs a, const __grid_constant__ CUtensorMap u_map) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t *area0 = smem + kOffArea0, *area1 = smem + kOffArea1;
  uint8_t *s_tile = smem + kOffS, *slo_tile = smem + kOffSlo, *u_tile = smem + kOffU;
  uint8_t *chat_lo = smem + kOffChatLo;
  float *seg = reinterpret_cast<float *>(smem + kOffSeg);
  float *gt_s = reinterpret_cast<float *>(smem + kOffGt);
  // mbarriers: cb[0..4] / barH are completed by tcgen05.commit (each once per tile), barU by the TMA load,
  // full[0..5] by the 16 worker warps, item_bar and state_bar by the control warp.
  uint64_t *cb = reinterpret_cast<uint64_t *>(smem + kOffMisc);  // cb[0..3]: one per MMA batch (cb[4] unused)
  uint64_t *barH = cb + 5, *barU = cb + 6, *full = cb + 7;
  uint64_t *item_bar = cb + 13, *state_bar = cb + 14, *out_bar = cb + 15;
  uint32_t *tmem_s = reinterpret_cast<uint32_t *>(cb + 16);
  volatile int *items = reinterpret_cast<volatile int *>(tmem_s + 1);  // [2], by tile parity
  long long *prof = reinterpret_cast<long long *>(smem + kOffMisc + 192);  // worker thread 0 only

  const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int i = 0; i < 5; ++i) umma::mbar_init(cb + i, 1);
    umma::mbar_init(barH, 1);
    umma::mbar_init(barU, 1);
    for (int i = 0; i < 6; ++i) umma::mbar_init(full + i, 16);
    umma::mbar_init(item_bar, 1);
    umma::mbar_init(state_bar, 1);
    umma::mbar_init(out_bar, 16);
    umma::fence_mbar_init();
    umma::prefetch_tmap(&u_map);
    for (int i = 0; i < kProfPhases; ++i) prof[i] = 0;
  }
  if (w == 0) umma::tmem_alloc(tmem_s, 512);
  umma::tc_fence_before();
  __syncthreads();
  umma::tc_fence_after();
  const uint32_t tmem = *tmem_s;
  bool ok = true;  // cleared when a bounded wait runs out; later waits are then skipped
  // Bounded waits.  The control warp polls (it is one warp and every hand-over of the tile passes
  // through it: a parked wait wakes up several hundred cycles after the barrier completes); the 16
  // worker warps park, which leaves the issue slots to the warps that have work.
  // (each setmaxnreg sits inside its role's branch: the register limit must not merge across roles)
  if (w > 16) {
    // spare warps of the control warp's register group: give the registers back, nothing else
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kControlRegs));
  } else if (w == 16) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kControlRegs));
#define FRACSSM_WAIT(bar, parity) \
  if (ok) ok = umma::mbar_wait(bar, (parity) & 1u, kWaitNs)
    // =========================== control warp ===========================
    const uint32_t sA0 = umma::smem_u32(area0), sA1 = umma::smem_u32(area1);
    const uint32_t sS = umma::smem_u32(s_tile), sSlo = umma::smem_u32(slo_tile), sU = umma::smem_u32(u_tile);
    const uint32_t sClo = umma::smem_u32(chat_lo);
    constexpr uint32_t kIdKK128 = umma::make_idesc(128, 128, false, false);
    constexpr uint32_t kIdKK64 = umma::make_idesc(128, 64, false, false);
    constexpr uint32_t kIdKK32 = umma::make_idesc(128, 32, false, false);
    constexpr uint32_t kIdKMn64 = umma::make_idesc(128, 64, false, true);
    constexpr uint32_t kIdMnMn64 = umma::make_idesc(128, 64, true, true);
    // One GEMM piece = 8 contraction steps of 16.  A K-major 128-column tile advances by 32 bytes
    // inside a 64-column atom and by one atom after 4 steps; an MN-major tile by 16 rows (2048 B).
    // The loop is kept rolled so the control warp needs few registers.
    auto piece = [&](uint32_t d_col, uint32_t a_addr, bool a_mn, uint32_t b_addr, bool b_mn, uint32_t b_sbo,
                     uint32_t idesc, uint32_t acc_first) {
      const uint64_t da = umma::make_sdesc(a_addr, a_mn ? kAtom : 16, 1024);
      const uint64_t db = umma::make_sdesc(b_addr, b_mn ? kAtom : 16, b_sbo);
#pragma unroll
      for (uint32_t s = 0; s < 8; ++s) {
        const uint32_t k_step = ((s >> 2) * kAtom + (s & 3) * 32) >> 4, mn_step = (s * 2048) >> 4;
        umma::mma_ss(tmem + d_col, da + (a_mn ? mn_step : k_step), db + (b_mn ? mn_step : k_step), idesc,
                     s > 0 ? 1u : acc_first);
      }
    };

    int item = 0;
    if (lane == 0) {
      item = atomicAdd(&a.ctrl[0], 1);
      items[0] = item;
      umma::mbar_arrive(item_bar);
    }
    item = __shfl_sync(0xffffffffu, item, 0);
#pragma unroll 1
    for (uint32_t n = 0; item < a.total; ++n) {
      const int j = item / a.BH, bh = item - j * a.BH;
      // The next ticket is taken a tile ahead (the workers read it in the second half of this tile,
      // and its inputs are pulled into L2 now) and published through item_bar.  In the first tile of
      // a CTA this has to wait until the workers have read the first item, i.e. until their arrival
      // on full[0]: two completions of item_bar in a row would flip its parity twice, and a worker
      // that had not looked yet would wait for a phase that never comes.  From the second tile on
      // every worker has read item n before the control warp can get here (the read precedes the
      // worker's arrival on out_bar of the previous tile).
      int next = 0;
      auto take_next = [&]() {
        if (lane == 0) {
          next = atomicAdd(&a.ctrl[0], 1);
          items[(n + 1) & 1] = next;
          umma::mbar_arrive(item_bar);
        }
        next = __shfl_sync(0xffffffffu, next, 0);
        if (lane == 1 && next < a.total) {  // pull the next item's inputs into L2 a whole tile ahead
          const int nj = next / a.BH, nb = next - nj * a.BH;
          const int ntok = min(kTile, a.L - nj * kTile);
          const int64_t tok = static_cast<int64_t>(nb) * a.L + nj * kTile;
          umma::prefetch_l2(a.rho + tok * kM, ntok * kM * 4);
          constexpr int kCkBytes = CKF32 ? 4 : 2;
          umma::prefetch_l2(reinterpret_cast<const char *>(a.c) + tok * kM * kCkBytes, ntok * kM * kCkBytes);
          umma::prefetch_l2(reinterpret_cast<const char *>(a.kappa) + tok * kM * kCkBytes, ntok * kM * kCkBytes);
        }
      };
      if (n > 0) take_next();
      if (n > 0) { FRACSSM_WAIT(barH, n - 1); }  // every MMA of the previous tile has finished
      if (lane == 0) {
        umma::mbar_expect_tx(barU, kTile * kR * 2);
        umma::tma_load_3d(u_tile, &u_map, barU, 0, j * kTile, bh);
      }
      // base: D[t,k] = A0[t,:] . B0[k,:]
      FRACSSM_WAIT(full + 0, n);
      umma::tc_fence_after();
      if (lane == 0) {
        piece(kColBase, sA0, false, sA0 + kTileBytes, false, 1024, kIdKK128, 0u);
        umma::mma_commit(cb + 0);
      }
      if (n == 0) take_next();
      // levels 8 and 16 (area1): first halves are picked by the B descriptor's row-group stride
      FRACSSM_WAIT(full + 1, n);
      umma::tc_fence_after();
      if (lane == 0) {
        piece(kColL8, sA1, false, sA1, false, 2048, kIdKK64, 0u);                      // every other 8-row group
        piece(kColL16, sA1 + kTileBytes, false, sA1 + kTileBytes, false, 4096, kIdKK32, 0u);   // groups 0,4,8,12
        piece(kColL16 + 32, sA1 + kTileBytes, false, sA1 + kTileBytes + 1024, false, 4096, kIdKK32, 0u);  // 1,5,9,13
        umma::mma_commit(cb + 1);
      }
      // levels 32 and 64 (the Chat-low and state slots, idle until late in the tile)
      FRACSSM_WAIT(full + 2, n);
      umma::tc_fence_after();
      if (lane == 0) {
        piece(kColL32, sClo, false, sClo, false, 1024, kIdKK32, 0u);                   // rows 0..31
        piece(kColL32 + 32, sClo, false, sClo + 8192, false, 1024, kIdKK32, 0u);       // rows 64..95
        piece(kColL64, sS, false, sS, false, 1024, kIdKK64, 0u);                       // rows 0..63
        umma::mma_commit(cb + 2);
      }
      // Sacc[m,r] = sum_k (Khi + Klo)[k,m] u[k,r]: the tile's own contribution to the state
      // the state left by the previous tile of this (batch, head) row is usually there already:
      // look before the wait for the workers, when this warp has nothing else to do
      bool early = false;
      if (lane == 0) {
        early = j == 0 || ld_acquire(a.flags + bh) >= j;
        if (early) umma::mbar_arrive(state_bar);
      }
      FRACSSM_WAIT(full + 3, n);
      FRACSSM_WAIT(barU, n);
      umma::tc_fence_after();
      if (lane == 0) {
        piece(kColS, sA0 + kTileBytes, true, sU, true, 1024, kIdMnMn64, 0u);
        piece(kColS, sA1 + kTileBytes, true, sU, true, 1024, kIdMnMn64, 1u);
        umma::mma_commit(cb + 3);
        if (!early) {
          if (ok) {
            const uint64_t t_start = umma::global_ns();
            while (ld_acquire(a.flags + bh) < j) {
              __nanosleep(100);
              if (umma::global_ns() - t_start > kWaitNs) { ok = false; break; }
            }
          }
          umma::mbar_arrive(state_bar);
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      // publish the outgoing state as soon as the workers have stored it: their stores are ordered
      // before their arrivals on out_bar, this release makes them visible to the next tile's CTA
      FRACSSM_WAIT(out_bar, n);
      if (lane == 0 && j + 1 < a.ntiles) st_release(a.flags + bh, j + 1);
      // H = Chat S, both factors split into bf16 high and low parts (low x low dropped)
      FRACSSM_WAIT(full + 5, n);
      umma::tc_fence_after();
      if (lane == 0) {
        piece(kColH, sA0, false, sS, true, 1024, kIdKMn64, 0u);    // Chat(high) S(high)
        piece(kColH, sA1, false, sS, true, 1024, kIdKMn64, 1u);    // Chat(low)  S(high)
        piece(kColH, sA0, false, sSlo, true, 1024, kIdKMn64, 1u);  // Chat(high) S(low)
      }
      // H += W u
      FRACSSM_WAIT(full + 4, n);
      umma::tc_fence_after();
      if (lane == 0) {
        piece(kColH, sClo, false, sU, true, 1024, kIdKMn64, 1u);
        umma::mma_commit(barH);
      }
      __syncwarp();
      item = next;
    }
  } else {
    // =========================== worker warps ===========================
#undef FRACSSM_WAIT
#define FRACSSM_WAIT(bar, parity) \
  if (ok) ok = umma::mbar_wait_parked(bar, (parity) & 1u, kWaitNs)
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kWorkerRegs));
    const int Q = w & 3, P = w >> 2;  // TMEM lane quarter of this warp, and its column part
    // operand-tile addressing of this thread: rows 8w..8w+7, modes 4*lane..4*lane+3
    const uint32_t th_off = (lane >> 4) * kAtom + ((lane & 1) << 3) + w * 1024;
    const uint32_t c16 = ((lane & 15) >> 1) << 4;
    const uint32_t sArea0 = umma::smem_u32(area0), sArea1 = umma::smem_u32(area1);
    const uint32_t sChatLo = umma::smem_u32(chat_lo), sSt = umma::smem_u32(s_tile);
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>(32 * Q) << 16);
    // worker thread 0 charges the cycles since the last mark to a phase (diagnostic)
    long long t_mark = clock64();
#define FRACSSM_MARK(phase)                         \
  if (PROF && tid == 0) {                           \
    const long long now_ = clock64();               \
    prof[phase] += now_ - t_mark;                   \
    t_mark = now_;                                  \
  }

    FRACSSM_WAIT(item_bar, 0);
    int item = items[0];
    int prev_bh = 0, prev_t0 = 0;
    // Output rows of tile number n_done (its H accumulator is complete when barH fires).  It runs at
    // the start of the next tile, after that tile's input loads have been issued, so the loads'
    // latency is covered by this work.
    auto write_rows = [&](uint32_t n_done) {
      FRACSSM_WAIT(barH, n_done);
      umma::tc_fence_after();
      FRACSSM_MARK(13)
      float acc[16];
      umma::tmem_ld16(lane_addr + kColH + 16 * P, acc);
      umma::tmem_ld_wait();
      const int t = prev_t0 + 32 * Q + lane;
      if (t < a.L) {
        uint4 lo, hi;
        lo.x = pack2(acc[0], acc[1]); lo.y = pack2(acc[2], acc[3]); lo.z = pack2(acc[4], acc[5]); lo.w = pack2(acc[6], acc[7]);
        hi.x = pack2(acc[8], acc[9]); hi.y = pack2(acc[10], acc[11]); hi.z = pack2(acc[12], acc[13]); hi.w = pack2(acc[14], acc[15]);
        uint4 *dst = reinterpret_cast<uint4 *>(a.h + (static_cast<int64_t>(prev_bh) * a.L + t) * kR + 16 * P);
        __stcs(dst, lo);
        __stcs(dst + 1, hi);
      }
      umma::tc_fence_before();
      FRACSSM_MARK(14)
    };

    uint32_t n_tiles_done = 0;
    for (uint32_t n = 0; item < a.total; ++n, ++n_tiles_done) {
      const int j = item / a.BH, bh = item - j * a.BH;
      const int t0 = j * kTile;

      // ---- segment products and the base tiles, from the raw registers; one group of 4 tokens
      // at a time to keep few values live
      float2 cp[8][2], ks[8][2];
      float g8[4];
      {
        // the inputs were pulled into L2 a tile ahead; both groups are requested at once
        RawRegs<CKF32> raw0, raw1;
        load_raw(raw0, a, item, w, lane, 0);
        load_raw(raw1, a, item, w, lane, 1);
        if (n > 0) write_rows(n - 1);  // the previous tile's output, while the loads are in flight
        float ga[4], gb[4];
#pragma unroll
        for (int grp = 0; grp < 2; ++grp) {
          const RawRegs<CKF32> &raw = grp ? raw1 : raw0;
          float a0[4][4], b0[4][4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            float rr[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float4 v = raw.r[i];
              rr[i] = fmaxf(q == 0 ? v.x : q == 1 ? v.y : q == 2 ? v.z : v.w, kRhoFloor);
            }
            // p4: running product from the start of the group (inclusive)
            // s4: product of the tokens after t up to the end of the group (exclusive)
            float p4[4], s4[4];
            p4[0] = rr[0]; p4[1] = p4[0] * rr[1]; p4[2] = p4[1] * rr[2]; p4[3] = p4[2] * rr[3];
            s4[3] = 1.f; s4[2] = rr[3]; s4[1] = s4[2] * rr[2]; s4[0] = s4[1] * rr[1];
            if (grp == 0) ga[q] = p4[3]; else gb[q] = p4[3];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float cf = ck_get(raw.c[i], q), kf = ck_get(raw.k[i], q);
              float &cpv = (q & 1) ? cp[4 * grp + i][q >> 1].y : cp[4 * grp + i][q >> 1].x;
              float &ksv = (q & 1) ? ks[4 * grp + i][q >> 1].y : ks[4 * grp + i][q >> 1].x;
              if (grp == 0) {  // base reference point: between token 3 and token 4 of the segment
                a0[i][q] = __fdividef(cf, s4[i]);
                b0[i][q] = kf * s4[i];
                cpv = cf * p4[i];
                ksv = kf * s4[i];          // times gb, below
              } else {
                a0[i][q] = cf * p4[i];
                b0[i][q] = __fdividef(kf, p4[i]);
                cpv = cf * ga[q] * p4[i];
                ksv = kf * s4[i];
              }
            }
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            emit_row(sArea0, th_off, c16, 4 * grp + i, make_float2(a0[i][0], a0[i][1]), make_float2(a0[i][2], a0[i][3]));
            emit_row(sArea0 + kTileBytes, th_off, c16, 4 * grp + i, make_float2(b0[i][0], b0[i][1]),
                     make_float2(b0[i][2], b0[i][3]));
          }
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) g8[q] = ga[q] * gb[q];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          ks[i][0] = __fmul2_rn(ks[i][0], make_float2(gb[0], gb[1]));
          ks[i][1] = __fmul2_rn(ks[i][1], make_float2(gb[2], gb[3]));
        }
        *reinterpret_cast<float4 *>(seg + w * kM + 4 * lane) = make_float4(g8[0], g8[1], g8[2], g8[3]);
      }
      warp_arrive(full + 0, lane);
      umma::named_barrier(1, kWorkers);  // segment products visible to every worker
      FRACSSM_MARK(0)

      // One sibling level: every token row holds its A-role or B-role value.
      auto produce_level = [&](uint32_t tile_s, int hseg) {
        float2 sig[2];
        const bool role_a = (w & hseg) != 0;
        const int first = w - (w & (hseg - 1));
        if (role_a) seg_prod(seg, first, w, lane, sig);
        else seg_prod(seg, w + 1, first + hseg, lane, sig);
#pragma unroll
        for (int i = 0; i < 8; ++i)
          emit_row(tile_s, th_off, c16, i, __fmul2_rn(role_a ? cp[i][0] : ks[i][0], sig[0]),
                   __fmul2_rn(role_a ? cp[i][1] : ks[i][1], sig[1]));
      };

      // ---- levels 8 and 16 -> area1
      produce_level(sArea1, 1);
      produce_level(sArea1 + kTileBytes, 2);
      warp_arrive(full + 1, lane);
      FRACSSM_MARK(1)

      // ---- levels 32 and 64 -> the Chat-low and state slots (their readers finished with the
      // previous tile), so nothing has to be waited for here
      produce_level(sChatLo, 4);
      produce_level(sSt, 8);
      warp_arrive(full + 2, lane);
      FRACSSM_MARK(3)

      // ---- Chat (high) and Khat (high) -> area0 (after the base MMAs), Chat (low) -> area1 tile 0
      // (after the level-8/16 MMAs)
      FRACSSM_WAIT(cb + 0, n);
      FRACSSM_MARK(2)
      FRACSSM_WAIT(cb + 1, n);
      FRACSSM_MARK(4)
      {
        float2 e[2], f[2];
        seg_prod(seg, 0, w, lane, e);
        seg_prod(seg, w + 1, 16, lane, f);
        if (w == 0)
          *reinterpret_cast<float4 *>(gt_s + 4 * lane) =
              make_float4(g8[0] * f[0].x, g8[1] * f[0].y, g8[2] * f[1].x, g8[3] * f[1].y);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float2 cl[2], kl[2];
          uint32_t pch[2], pkh[2];  // the high parts, already packed
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            const float2 chat = __fmul2_rn(cp[i][hf], e[hf]);
            const float2 ch = bf16_round2(chat, pch[hf]);
            cl[hf] = __fadd2_rn(chat, make_float2(-ch.x, -ch.y));
            const float2 full_k = __fmul2_rn(ks[i][hf], f[hf]);
            const float2 kh = bf16_round2(full_k, pkh[hf]);
            kl[hf] = __fadd2_rn(full_k, make_float2(-kh.x, -kh.y));
          }
          emit_row_packed(sArea0, th_off, c16, i, pch[0], pch[1]);
          emit_row(sArea1, th_off, c16, i, cl[0], cl[1]);
          emit_row_packed(sArea0 + kTileBytes, th_off, c16, i, pkh[0], pkh[1]);
          emit_row(sArea1 + kTileBytes, th_off, c16, i, kl[0], kl[1]);
        }
      }
      warp_arrive(full + 3, lane);
      FRACSSM_MARK(5)

      // the next item (published by the control warp at the start of this tile); it must be read
      // here, before this warp's arrival on out_bar lets the control warp move on and publish again
      FRACSSM_WAIT(item_bar, n + 1);
      const int next = items[(n + 1) & 1];
      FRACSSM_MARK(7)

      // ---- the chain first: incoming state -> outgoing state, published for the next tile of the row
      FRACSSM_WAIT(state_bar, n);
      umma::named_barrier(2, kWorkers);  // also orders warp 0's write of gt_s before its readers
      FRACSSM_MARK(9)
      const int m_row = 32 * Q + lane;
      float sj[16];
      {
        // scratch layout [bh][P][x][m][4]: the lanes of a warp touch consecutive 16-byte pieces
        const float4 *sp = reinterpret_cast<const float4 *>(a.state) +
                           (static_cast<int64_t>(bh) * 4 + P) * 4 * kM + m_row;
        if (j > 0) {
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            const float4 v = __ldcg(sp + x * kM);
            sj[4 * x] = v.x; sj[4 * x + 1] = v.y; sj[4 * x + 2] = v.z; sj[4 * x + 3] = v.w;
          }
        } else if (a.init) {
#pragma unroll
          for (int x = 0; x < 16; ++x)
            sj[x] = a.init[(static_cast<int64_t>(bh) * kR + 16 * P + x) * kM + m_row];
        } else {
#pragma unroll
          for (int x = 0; x < 16; ++x) sj[x] = 0.f;
        }
      }
      FRACSSM_WAIT(cb + 3, n);  // Khat(high) and Khat(low) MMAs: Sacc is complete
      umma::tc_fence_after();
      FRACSSM_MARK(11)
      {
        // S_next = Gt * S + Sacc
        float acc[16];
        umma::tmem_ld16(lane_addr + kColS + 16 * P, acc);
        umma::tmem_ld_wait();
        const float gt = gt_s[m_row];
#pragma unroll
        for (int x = 0; x < 16; ++x) acc[x] = fmaf(gt, sj[x], acc[x]);
        float4 *sp = reinterpret_cast<float4 *>(a.state) + (static_cast<int64_t>(bh) * 4 + P) * 4 * kM + m_row;
        if (j + 1 < a.ntiles) {
#pragma unroll
          for (int x = 0; x < 4; ++x)
            __stcg(sp + x * kM, make_float4(acc[4 * x], acc[4 * x + 1], acc[4 * x + 2], acc[4 * x + 3]));
        } else if (a.fin) {
#pragma unroll
          for (int x = 0; x < 16; ++x)
            st_f32(a.fin, (static_cast<int64_t>(bh) * kR + 16 * P + x) * kM + m_row, a.fin_dt, acc[x]);
        }
      }
      umma::tc_fence_before();
      __syncwarp();
      if (lane == 0) umma::mbar_arrive(out_bar);  // the control warp releases the row counter
      FRACSSM_MARK(12)

      // ---- every level MMA has completed: the state slot and the W slot are free
      FRACSSM_WAIT(cb + 2, n);
      umma::tc_fence_after();
      FRACSSM_MARK(6)
      // incoming state as MMA operands, bf16 high / low parts
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t ph[4], pl[4];
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const float2 v = make_float2(sj[8 * half + 2 * x], sj[8 * half + 2 * x + 1]);
          const float2 hi = bf16_round2(v, ph[x]);
          pl[x] = pack2(v.x - hi.x, v.y - hi.y);
        }
        const uint32_t off = m_row * 128 + (((2 * P + half) ^ (m_row & 7)) << 4);
        *reinterpret_cast<uint4 *>(s_tile + off) = make_uint4(ph[0], ph[1], ph[2], ph[3]);
        *reinterpret_cast<uint4 *>(slo_tile + off) = make_uint4(pl[0], pl[1], pl[2], pl[3]);
      }
      warp_arrive(full + 5, lane);
      FRACSSM_MARK(10)

      // ---- W -> the Chat-low slot
      {
        uint8_t *wt = chat_lo;
        const int t = 32 * Q + lane;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          float v[8];
          if (P > Q) {
#pragma unroll
            for (int x = 0; x < 8; ++x) v[x] = 0.f;
          } else if (P < Q) {
            const uint32_t col = ((Q >> 1) != (P >> 1)) ? (kColL64 + 32 * P + 8 * g)
                                                        : (kColL32 + (P >> 1) * 32 + 8 * g);
            umma::tmem_ld8(lane_addr + col, v);
            umma::tmem_ld_wait();
          } else {
            float b[8], l8[8], l16[8];
#pragma unroll
            for (int x = 0; x < 8; ++x) l8[x] = l16[x] = 0.f;
            umma::tmem_ld8(lane_addr + kColBase + 32 * Q + 8 * g, b);
            if ((g & 1) == 0) umma::tmem_ld8(lane_addr + kColL8 + (2 * Q + (g >> 1)) * 8, l8);
            if (g < 2) umma::tmem_ld8(lane_addr + kColL16 + (g & 1) * 32 + Q * 8, l16);
            umma::tmem_ld_wait();
            const int tb = lane >> 3;  // 8-token block of this row inside its 32-token block
#pragma unroll
            for (int x = 0; x < 8; ++x) {
              float r = 0.f;
              if (g == tb) r = (x <= (lane & 7)) ? b[x] : 0.f;
              else if (g < tb) r = ((tb ^ g) >= 2) ? l16[x] : l8[x];
              v[x] = r;
            }
          }
          uint4 pk;
          pk.x = pack2(v[0], v[1]); pk.y = pack2(v[2], v[3]); pk.z = pack2(v[4], v[5]); pk.w = pack2(v[6], v[7]);
          const uint32_t chunk = (4 * P + g) & 7;
          *reinterpret_cast<uint4 *>(wt + (P >> 1) * kAtom + t * 128 + ((chunk ^ (t & 7)) << 4)) = pk;
        }
      }
      warp_arrive(full + 4, lane);
      FRACSSM_MARK(8)

      prev_bh = bh;
      prev_t0 = t0;
      item = next;
    }
    if (n_tiles_done > 0) write_rows(n_tiles_done - 1);
    if (PROF && tid == 0 && a.prof && blockIdx.x < kProfCtas) {
      for (int i = 0; i < kProfPhases; ++i) a.prof[blockIdx.x * kProfPhases + i] = prof[i];
    }
  }

  if (!ok) atomicExch(&a.ctrl[1], 1);
  umma::tc_fence_before();
  __syncthreads();
  if (w == 0) umma::tmem_dealloc(tmem, 512);
}

size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

}  // namespace

size_t scan_fused_workspace_bytes(int64_t B, int64_t, int64_t R, int64_t M, int64_t) {
  return kCtrlBytes + kProfBytes + align256((size_t)B * 4) + (size_t)B * R * M * 4;
}

int scan_fused_launch(const void *u, const void *c, const void *kappa, int ck_dtype, const float *rho,
                      const float *initial_state, void *h, void *final_state, int final_dtype,
                      void *workspace, size_t workspace_bytes, int64_t B, int64_t L, int64_t R,
                      int64_t M, int64_t T, void *stream) {
  (void)T;
  const bool ckf32 = ck_dtype == FRACSSM_F32;
  if (workspace_bytes < scan_fused_workspace_bytes(B, L, R, M, T))
    return fail(FRACSSM_ERR_ARG, "frac_scan: workspace too small");
  // per device, once: opt in to the large dynamic shared memory and remember the SM count
  static std::mutex mu;
  static int sm_count[64] = {};
  auto prepare = [](const void *kernel) -> int {
    cudaError_t ae = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (ae != cudaSuccess) return fail(FRACSSM_ERR_CUDA, "frac_scan: %s", cudaGetErrorString(ae));
    cudaFuncAttributes fa{};
    ae = cudaFuncGetAttributes(&fa, kernel);
    if (ae != cudaSuccess) return fail(FRACSSM_ERR_CUDA, "frac_scan: %s", cudaGetErrorString(ae));
    if (fa.numRegs < kLaunchRegsNeeded)
      return fail(FRACSSM_ERR_UNSUPPORTED,
                  "frac_scan: the single-pass kernel was built with %d registers per thread, needs %d",
                  fa.numRegs, kLaunchRegsNeeded);
    return FRACSSM_OK;
  };
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
    return fail(FRACSSM_ERR_CUDA, "frac_scan: cannot identify the current device");
  {
    std::lock_guard<std::mutex> lock(mu);
    if (sm_count[dev] == 0) {
      int prc = prepare(reinterpret_cast<const void *>(&scan_fused_kernel<false, false>));
      if (prc == FRACSSM_OK) prc = prepare(reinterpret_cast<const void *>(&scan_fused_kernel<true, false>));
      if (prc == FRACSSM_OK) prc = prepare(reinterpret_cast<const void *>(&scan_fused_kernel<false, true>));
      if (prc == FRACSSM_OK) prc = prepare(reinterpret_cast<const void *>(&scan_fused_kernel<true, true>));
      if (prc) return prc;
      int n = 0;
      cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
      if (n <= 0) return fail(FRACSSM_ERR_CUDA, "frac_scan: cannot query the SM count");
      sm_count[dev] = n;
    }
    sms = sm_count[dev];
  }

  char *ws = reinterpret_cast<char *>(workspace);
  FusedArgs a{};
  a.c = c;
  a.kappa = kappa;
  a.rho = rho;
  a.init = initial_state;
  a.h = reinterpret_cast<__nv_bfloat16 *>(h);
  a.fin = final_state;
  a.fin_dt = final_dtype;
  a.ctrl = reinterpret_cast<int *>(ws);
  a.prof = reinterpret_cast<long long *>(ws + kCtrlBytes);
  a.flags = reinterpret_cast<int *>(ws + kCtrlBytes + kProfBytes);
  a.state = reinterpret_cast<float *>(ws + kCtrlBytes + kProfBytes + align256((size_t)B * 4));
  a.BH = (int)B;
  a.L = (int)L;
  a.ntiles = (int)ceil_div(L, kTile);
  a.total = a.ntiles * a.BH;
  CUtensorMap map;
  int rc = make_tmap_bf16_3d(&map, u, kR, (uint64_t)L, (uint64_t)B, kR, kTile);
  if (rc) return rc;
  cudaError_t e = cudaMemsetAsync(ws, 0, kCtrlBytes + kProfBytes + align256((size_t)B * 4), (cudaStream_t)stream);
  if (e != cudaSuccess) return fail(FRACSSM_ERR_CUDA, "frac_scan: %s", cudaGetErrorString(e));
  const int grid = a.total < sms ? a.total : sms;
  // FRACSSM_SCAN_PROFILE=1 in the environment selects the build that records per-phase cycles
  const char *pe = getenv("FRACSSM_SCAN_PROFILE");
  const bool prof = pe && pe[0] != '\0' && pe[0] != '0';
  const cudaStream_t st = (cudaStream_t)stream;
  if (ckf32 && prof) scan_fused_kernel<true, true><<<grid, kThreads, kSmemBytes, st>>>(a, map);
  else if (ckf32) scan_fused_kernel<true, false><<<grid, kThreads, kSmemBytes, st>>>(a, map);
  else if (prof) scan_fused_kernel<false, true><<<grid, kThreads, kSmemBytes, st>>>(a, map);
  else scan_fused_kernel<false, false><<<grid, kThreads, kSmemBytes, st>>>(a, map);
  return check_launch("frac_scan (single-pass kernel)");
}

}  // namespace fracssm

extern "C" int fracssm_scan_fused_supported(int64_t B, int64_t L, int64_t R, int64_t M, int64_t T,
                                            int u_dtype, int ck_dtype) {
  (void)T;
  using namespace fracssm;
  return B >= 1 && L >= 1 && R == kR && M == kM && u_dtype == FRACSSM_BF16 &&
         (ck_dtype == FRACSSM_BF16 || ck_dtype == FRACSSM_F32) &&
         B * ceil_div(L, kTile) < (int64_t(1) << 30) && L < (int64_t(1) << 30);
}

// Reads back the error word of the last single-pass launch that used `workspace`
// (synchronises the stream).  0 = ok, FRACSSM_ERR_WAIT if a device-side wait ran out.
extern "C" int fracssm_scan_fused_status(const void *workspace, void *stream) {
  using namespace fracssm;
  if (!workspace) return fail(FRACSSM_ERR_ARG, "scan_fused_status: null workspace");
  int ctrl[2] = {0, 0};
  cudaError_t e = cudaMemcpyAsync(ctrl, workspace, sizeof(ctrl), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) return fail(FRACSSM_ERR_CUDA, "scan_fused_status: %s", cudaGetErrorString(e));
  if (ctrl[1] != 0) return fail(FRACSSM_ERR_WAIT, "single-pass scan: a device-side wait ran out");
  return FRACSSM_OK;
}

// Diagnostic: cycles thread 0 of each CTA spent in each of the 16 phases of the tile loop during
// the last single-pass launch that used `workspace`, summed over CTAs (synchronises the stream).
extern "C" int fracssm_scan_fused_phase_cycles(const void *workspace, long long *out16, void *stream) {
  using namespace fracssm;
  if (!workspace || !out16) return fail(FRACSSM_ERR_ARG, "scan_fused_phase_cycles: null pointer");
  static long long host[kProfCtas * kProfPhases];
  cudaError_t e = cudaMemcpyAsync(host, reinterpret_cast<const char *>(workspace) + kCtrlBytes, kProfBytes,
                                  cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) return fail(FRACSSM_ERR_CUDA, "scan_fused_phase_cycles: %s", cudaGetErrorString(e));
  for (int p = 0; p < kProfPhases; ++p) {
    out16[p] = 0;
    for (int cta = 0; cta < kProfCtas; ++cta) out16[p] += host[cta * kProfPhases + p];
  }
  return FRACSSM_OK;
}

// ---------------------------------------------------------------------------------------------
// Single-pass scan without any allocation by caller or library.
//
// Some callers cannot provide scratch memory: code that runs where the CUDA allocator must not
// be touched (inside another framework's memory-pool callback, in a latency-critical serving
// loop that forbids cudaMalloc after start-up, or in a host language binding that has no
// device allocator of its own).  For them the scratch of the single-pass kernel (ticket, error
// word, per-row progress counters and the running state) lives in a fixed array in the
// library's device image.  The array exists once per GPU that loads the library and stays until
// the process exits; it bounds the batch*heads count to kNoAllocMaxRows.
namespace fracssm {
namespace {
constexpr int64_t kNoAllocMaxRows = 64;
constexpr size_t kNoAllocBytes =
    kCtrlBytes + kProfBytes + ((kNoAllocMaxRows * 4 + 255) / 256) * 256 + kNoAllocMaxRows * kR * kM * 4;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

constexpr int kMaxDevices = 64;
std::mutex g_noalloc_mutex;
void *g_noalloc_ptr[kMaxDevices] = {};  // device address of g_noalloc_scratch on each device

// Device address of the scratch array on the current device.  The array's name is only a
// host-side handle; the address a kernel can use comes from cudaGetSymbolAddress, asked once
// per device with that device current.
int noalloc_scratch(void **out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(FRACSSM_ERR_CUDA, "frac_scan (no-alloc): %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(FRACSSM_ERR_UNSUPPORTED, "frac_scan (no-alloc): device index too large");
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (!g_noalloc_ptr[dev]) {
    void *p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || !p)
      return fail(FRACSSM_ERR_CUDA, "frac_scan (no-alloc): cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    g_noalloc_ptr[dev] = p;
  }
  *out = g_noalloc_ptr[dev];
  return FRACSSM_OK;
}
}  // namespace
}  // namespace fracssm

extern "C" int fracssm_frac_scan_fwd_noalloc(const void *u, const void *c, const void *kappa,
                                             const float *rho, const float *initial_state, void *h,
                                             void *final_state, int final_dtype, int64_t B, int64_t L,
                                             int64_t R, int64_t M, void *stream) {
  using namespace fracssm;
  if (B < 0 || L < 0) return fail(FRACSSM_ERR_ARG, "frac_scan (no-alloc): bad sizes");
  if (B == 0 || L == 0) return fail(FRACSSM_ERR_UNSUPPORTED, "frac_scan (no-alloc): empty input");
  if (B > kNoAllocMaxRows)
    return fail(FRACSSM_ERR_UNSUPPORTED,
                "frac_scan (no-alloc): batch*heads = %lld exceeds the built-in scratch (max %lld rows); "
                "use fracssm_frac_scan_fwd with a caller-provided workspace",
                (long long)B, (long long)kNoAllocMaxRows);
  if (!fracssm_scan_fused_supported(B, L, R, M, 128, FRACSSM_BF16, FRACSSM_BF16))
    return fail(FRACSSM_ERR_UNSUPPORTED, "frac_scan (no-alloc): needs R = 64, M = 128 and bfloat16 u, c, kappa");
  if (!u || !c || !kappa || !rho || !h) return fail(FRACSSM_ERR_ARG, "frac_scan (no-alloc): null pointer");
  if (final_state && final_dtype != FRACSSM_F32 && final_dtype != FRACSSM_BF16)
    return fail(FRACSSM_ERR_ARG, "frac_scan (no-alloc): final_state dtype must be float32 or bfloat16");
  void *scratch = nullptr;
  int rc = noalloc_scratch(&scratch);
  if (rc) return rc;
  // scan_fused_launch clears the ticket, error word and progress counters on the stream before
  // the kernel; the state rows are written before they are read.
  return scan_fused_launch(u, c, kappa, FRACSSM_BF16, rho, initial_state, h, final_state, final_dtype,
                           scratch, kNoAllocBytes, B, L, R, M, 128, stream);
}

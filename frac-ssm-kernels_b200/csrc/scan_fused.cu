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
// One CTA per SM, 20 warps (three of them only pad the control warp's register group).  Warps
// 0-15 ("workers") turn the raw inputs into bf16 operand tiles in shared memory and run the
// epilogues; warp 16 ("control") takes tickets, issues the TMA load of u and every tcgen05.mma,
// and polls the state counter.  Workers hand a batch of tiles over by arriving on a "full"
// mbarrier (one arrival per warp, after a proxy fence); the control warp hands buffers and
// accumulators back through tcgen05.commit mbarriers.
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
//     Every token has exactly one role per level.  The A rows of two levels are stacked into one
//     128-row operand tile and their B rows into another, so one 128 x 128 product serves two
//     levels (its two diagonal 64 x 64 quadrants; the other two are never read);
//   * base: the 8x8 diagonal blocks use the middle of the block as reference, which keeps
//     the reciprocal products below 1e24.
// Every piece is a bf16 tcgen05 GEMM over the modes; an epilogue copies each block of accumulators
// to its place in W.  Chat / Khat are the same factors taken to the tile's start / end, split into
// bf16 high and low parts so that the state keeps float32-level accuracy.
//
// Shared memory: six 32 KB operand slots, each used twice per tile:
//   slot 0 / 1: base A / B factors        -> Khat high / low   (after the base product)
//   slot 2 / 3: levels 8+16, A / B rows   -> Chat high / low   (after the level-8/16 product)
//   slot 4 / 5: levels 64+32, A / B rows  -> W / incoming state high|low (after that product)
// Tensor memory (fp32 columns): base 0..127, tile's own state contribution 128..191, levels 8+16
// 192..319, levels 64+32 320..447; the output accumulator H re-uses 320..447 (columns 384..447
// take the product with the state's low part and are added when the rows are written).
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
// the control warp's group of four shrinks to kControlRegs.  Each SM sub-partition holds four
// worker warps and one warp of the control group: 4 * 112 + 32 = 5 * 96, the launch allocation
// (checked on the host: it must cover both, or the growing warps would wait forever).
constexpr int kWorkerRegs = 112, kControlRegs = 32;
constexpr int kLaunchRegsNeeded = (kWorkers * kWorkerRegs + (kThreads - kWorkers) * kControlRegs + kThreads - 1) / kThreads;
// shared memory map (bytes from the 1024-aligned base)
constexpr uint32_t kSlot = 32768;
constexpr uint32_t kOffA0 = 0, kOffB0 = kSlot, kOffY1 = 2 * kSlot, kOffZ1 = 3 * kSlot, kOffY2 = 4 * kSlot,
                   kOffZ2 = 5 * kSlot;
constexpr uint32_t kOffKhi = kOffA0, kOffKlo = kOffB0, kOffChi = kOffY1, kOffClo = kOffZ1, kOffW = kOffY2,
                   kOffS = kOffZ2;              // second use of each slot
constexpr uint32_t kOffU = 6 * kSlot;           // u tile, 128 tokens x 64 bf16
constexpr uint32_t kOffSeg = kOffU + 16384;     // float [16][128]: decay product of each 8-token segment
constexpr uint32_t kOffMisc = kOffSeg + 8192;   // mbarriers, TMEM base, tickets, failure flag
constexpr uint32_t kSmemBytes = kOffMisc + 256 + 1024;
// tensor-memory columns (fp32, 128 lanes each)
constexpr uint32_t kColBase = 0, kColS = 128, kColL1 = 192, kColL2 = 320, kColH = 320;
constexpr size_t kCtrlBytes = 256;

struct FusedArgs {
  const void *c, *kappa;  // bf16 or f32 [BH, L, 128], see the kernel's CKF32 parameter
  const float *rho, *init;
  __nv_bfloat16 *h;
  void *fin;
  int fin_dt;
  int *ctrl;     // [0] ticket counter, [1] error word
  int *flags;    // [BH] tiles finished per bh
  float *state;  // running state per row, 128 m x 64 r floats in the order the workers access it
  int BH, L, ntiles, total;
  int first_tile;              // tile index of the first ticket (0 except in the wait-limit self-test)
  unsigned long long wait_ns;  // limit of every device-side wait
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
  const int t0 = (j + a.first_tile) * kTile + 8 * w + 4 * grp;
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

// The two floored decay pairs of one token.
__device__ __forceinline__ void rho_pairs(const float4 &v, f2 (&out)[2]) {
  out[0] = mk2(fmaxf(v.x, kRhoFloor), fmaxf(v.y, kRhoFloor));
  out[1] = mk2(fmaxf(v.z, kRhoFloor), fmaxf(v.w, kRhoFloor));
}

template <bool CKF32>
__global__ void __launch_bounds__(kThreads, 1)
scan_fused_kernel(const FusedArgs a, const __grid_constant__ CUtensorMap u_map) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // mbarriers, each completed exactly once per tile:
  //   cb0 / cb1 / cb2 / cbK / barH by tcgen05.commit, barU by the TMA load,
  //   fA / fL1 / fL2 / fK / fW / fS / out_bar by the 16 worker warps, item_bar / state_bar by the control warp
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kOffMisc);
  uint64_t *cb0 = bars + 0, *cb1 = bars + 1, *cb2 = bars + 2, *cbK = bars + 3, *barH = bars + 4, *barU = bars + 5;
  uint64_t *fA = bars + 6, *fL1 = bars + 7, *fL2 = bars + 8, *fK = bars + 9, *fW = bars + 10, *fS = bars + 11;
  uint64_t *item_bar = bars + 12, *state_bar = bars + 13, *out_bar = bars + 14;
  uint32_t *tmem_s = reinterpret_cast<uint32_t *>(bars + 15);
  volatile int *items = reinterpret_cast<volatile int *>(tmem_s + 1);  // [2], by tile parity
  volatile int *failed = reinterpret_cast<volatile int *>(tmem_s + 3);  // a wait of this CTA ran out

  const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int i = 0; i < 6; ++i) umma::mbar_init(bars + i, 1);
    for (int i = 6; i < 12; ++i) umma::mbar_init(bars + i, 16);
    umma::mbar_init(item_bar, 1);
    umma::mbar_init(state_bar, 1);
    umma::mbar_init(out_bar, 16);
    umma::fence_mbar_init();
    umma::prefetch_tmap(&u_map);
    *failed = 0;
  }
  if (w == 0) umma::tmem_alloc(tmem_s, 512);
  umma::tc_fence_before();
  __syncthreads();
  umma::tc_fence_after();
  const uint32_t tmem = *tmem_s;
  const uint64_t wait_ns = a.wait_ns;
  bool ok = true;  // cleared when a bounded wait runs out; later waits are then skipped
  // Bounded waits.  The control warp polls (it is one warp and every hand-over of the tile passes
  // through it: a parked wait wakes up several hundred cycles after the barrier completes); the 16
  // worker warps park, which leaves the issue slots to the warps that have work.  A wait that runs
  // out marks the CTA as failed: its remaining outputs are written as NaN and the error word is set.
  // (each setmaxnreg sits inside its role's branch: the register limit must not merge across roles)
  if (w > 16) {
    // spare warps of the control warp's register group: give the registers back, nothing else
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kControlRegs));
  } else if (w == 16) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kControlRegs));
#define FRACSSM_WAIT(bar, parity)                                  \
  if (ok) {                                                        \
    ok = umma::mbar_wait(bar, (parity) & 1u, wait_ns);             \
    if (!ok) *failed = 1;                                          \
  }
    // =========================== control warp ===========================
    const uint32_t sb = umma::smem_u32(smem);
    const uint32_t sA0 = sb + kOffA0, sB0 = sb + kOffB0, sY1 = sb + kOffY1, sZ1 = sb + kOffZ1, sY2 = sb + kOffY2,
                   sZ2 = sb + kOffZ2, sU = sb + kOffU;
    const uint32_t sKhi = sb + kOffKhi, sKlo = sb + kOffKlo, sChi = sb + kOffChi, sClo = sb + kOffClo,
                   sW = sb + kOffW, sS = sb + kOffS;
    constexpr uint32_t kIdKK128 = umma::make_idesc(128, 128, false, false);
    constexpr uint32_t kIdKMn64 = umma::make_idesc(128, 64, false, true);
    constexpr uint32_t kIdKMn128 = umma::make_idesc(128, 128, false, true);
    constexpr uint32_t kIdMnMn64 = umma::make_idesc(128, 64, true, true);
    // One GEMM piece = 8 contraction steps of 16.  A K-major 128-column tile advances by 32 bytes
    // inside a 64-column atom and by one atom after 4 steps; an MN-major tile by 16 rows (2048 B).
    auto piece = [&](uint32_t d_col, uint32_t a_addr, bool a_mn, uint32_t b_addr, bool b_mn, uint32_t idesc,
                     uint32_t acc_first) {
      const uint64_t da = umma::make_sdesc(a_addr, a_mn ? kAtom : 16, 1024);
      const uint64_t db = umma::make_sdesc(b_addr, b_mn ? kAtom : 16, 1024);
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
      const int jt = j + a.first_tile;  // tile index inside the row
      // The next ticket is taken a tile ahead (the workers read it in the second half of this tile,
      // and its inputs are pulled into L2 now) and published through item_bar.  In the first tile of
      // a CTA this has to wait until the workers have read the first item, i.e. until their arrival
      // on fA: two completions of item_bar in a row would flip its parity twice, and a worker
      // that had not looked yet would wait for a phase that never comes.  From the second tile on
      // every worker has read item n before the control warp can get here (the read precedes the
      // worker's arrival on fW of the previous tile).
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
          const int tk0 = (nj + a.first_tile) * kTile;
          const int ntok = min(kTile, a.L - tk0);
          const int64_t tok = static_cast<int64_t>(nb) * a.L + tk0;
          umma::prefetch_l2(a.rho + tok * kM, ntok * kM * 4);
          constexpr int kCkBytes = CKF32 ? 4 : 2;
          umma::prefetch_l2(reinterpret_cast<const char *>(a.c) + tok * kM * kCkBytes, ntok * kM * kCkBytes);
          umma::prefetch_l2(reinterpret_cast<const char *>(a.kappa) + tok * kM * kCkBytes, ntok * kM * kCkBytes);
        }
      };
      if (n > 0) take_next();
      // base: D[t,k] = A0[t,:] . B0[k,:]
      FRACSSM_WAIT(fA, n);
      umma::tc_fence_after();
      if (lane == 0) {
        piece(kColBase, sA0, false, sB0, false, kIdKK128, 0u);
        umma::mma_commit(cb0);
      }
      if (n == 0) take_next();
      // the u tile is free once every MMA of the previous tile has finished
      if (n > 0) { FRACSSM_WAIT(barH, n - 1); }
      if (lane == 0) {
        umma::mbar_expect_tx(barU, kTile * kR * 2);
        umma::tma_load_3d(smem + kOffU, &u_map, barU, 0, jt * kTile, bh);
      }
      // levels 8 + 16, then 64 + 32: A rows x B rows of the stacked tiles
      FRACSSM_WAIT(fL1, n);
      umma::tc_fence_after();
      if (lane == 0) {
        piece(kColL1, sY1, false, sZ1, false, kIdKK128, 0u);
        umma::mma_commit(cb1);
      }
      FRACSSM_WAIT(fL2, n);
      umma::tc_fence_after();
      if (lane == 0) {
        piece(kColL2, sY2, false, sZ2, false, kIdKK128, 0u);
        umma::mma_commit(cb2);
      }
      // the state left by the previous tile of this (batch, head) row is usually there already:
      // look before the wait for the workers, when this warp has nothing else to do
      bool early = false;
      if (lane == 0) {
        early = jt == 0 || ld_acquire(a.flags + bh) >= jt;
        if (early) umma::mbar_arrive(state_bar);
      }
      // Sacc[m,r] = sum_k (Khi + Klo)[k,m] u[k,r]: the tile's own contribution to the state
      FRACSSM_WAIT(fK, n);
      FRACSSM_WAIT(barU, n);
      umma::tc_fence_after();
      if (lane == 0) {
        piece(kColS, sKhi, true, sU, true, kIdMnMn64, 0u);
        piece(kColS, sKlo, true, sU, true, kIdMnMn64, 1u);
        umma::mma_commit(cbK);
        if (!early) {
          if (ok) {
            const uint64_t t_start = umma::global_ns();
            while (ld_acquire(a.flags + bh) < jt) {
              __nanosleep(100);
              if (umma::global_ns() - t_start > wait_ns) { ok = false; *failed = 1; break; }
            }
          }
          umma::mbar_arrive(state_bar);
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      FRACSSM_WAIT(fW, n);
      FRACSSM_WAIT(fS, n);
      // Publish the outgoing state as soon as the workers have stored it: their stores are ordered
      // before their arrivals on out_bar, this release makes them visible to the next tile's CTA.
      // If they are not done yet, the output MMAs go first.
      bool released = false;
      if (umma::mbar_test(out_bar, n & 1u)) {
        if (lane == 0 && jt + 1 < a.ntiles) st_release(a.flags + bh, jt + 1);
        released = true;
      }
      // H = Chat S (both split into bf16 high and low parts, low x low dropped) + W u
      umma::tc_fence_after();
      if (lane == 0) {
        piece(kColH, sChi, false, sS, true, kIdKMn128, 0u);   // Chat(high) [S(high) | S(low)], 128 columns
        piece(kColH, sClo, false, sS, true, kIdKMn64, 1u);    // Chat(low) S(high)
        piece(kColH, sW, false, sU, true, kIdKMn64, 1u);      // W u
        umma::mma_commit(barH);
      }
      if (!released) {
        FRACSSM_WAIT(out_bar, n);
        if (lane == 0 && jt + 1 < a.ntiles) st_release(a.flags + bh, jt + 1);
      }
      __syncwarp();
      item = next;
    }
  } else {
    // =========================== worker warps ===========================
#undef FRACSSM_WAIT
#define FRACSSM_WAIT(bar, parity)                                         \
  if (ok) {                                                               \
    ok = umma::mbar_wait_parked(bar, (parity) & 1u, wait_ns);             \
    if (!ok) *failed = 1;                                                 \
  }
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kWorkerRegs));
    const int Q = w & 3, P = w >> 2;  // TMEM lane quarter of this warp, and its share of the columns
    const uint32_t sb = umma::smem_u32(smem);
    // operand-tile addressing of this thread: modes 4*lane..4*lane+3 of a row; the row group and the
    // row inside it are added per store (emit_words)
    const uint32_t th_fix = (lane >> 4) * kAtom + ((lane & 1) << 3) + (((lane & 15) >> 1) << 4);
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>(32 * Q) << 16);
    const uint32_t seg_s = sb + kOffSeg + 16 * lane;  // this lane's four modes of segment 0
    const float kNaN = __int_as_float(0x7fc00000);

    FRACSSM_WAIT(item_bar, 0);
    int item = items[0];
    int prev_bh = 0, prev_t0 = 0;
    // Output rows of the previous tile (its H accumulator is complete when barH fires).  It runs in
    // the middle of the next tile, so that tile's first phase overlaps the output MMAs.
    auto write_rows = [&](uint32_t n_done) {
      FRACSSM_WAIT(barH, n_done);
      umma::tc_fence_after();
      const bool bad = *failed != 0;
      const int t = prev_t0 + 32 * Q + lane;
      uint4 *dst = reinterpret_cast<uint4 *>(a.h + (static_cast<int64_t>(prev_bh) * a.L + t) * kR + 16 * P);
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        float hi[8], lo[8];
        umma::tmem_ld8(lane_addr + kColH + 16 * P + 8 * half, hi);
        umma::tmem_ld8(lane_addr + kColH + 64 + 16 * P + 8 * half, lo);
        umma::tmem_ld_wait();
#pragma unroll
        for (int x = 0; x < 8; ++x) hi[x] = bad ? kNaN : hi[x] + lo[x];
        if (t < a.L) {
          uint4 o;
          o.x = pack2(hi[0], hi[1]); o.y = pack2(hi[2], hi[3]); o.z = pack2(hi[4], hi[5]); o.w = pack2(hi[6], hi[7]);
          __stcs(dst + half, o);
        }
      }
      umma::tc_fence_before();
    };

    RawRegs<CKF32> raw0;
    if (item < a.total) load_raw(raw0, a, item, w, lane, 0);
    uint32_t n_tiles_done = 0;
    for (uint32_t n = 0; item < a.total; ++n, ++n_tiles_done) {
      const int j = item / a.BH, bh = item - j * a.BH;
      const int jt = j + a.first_tile;
      const int t0 = jt * kTile;

      // ---- segment products, the base tiles and the per-token factors cp / ks:
      //   cp[i] = c[i] * (decay from the segment's start to token i, inclusive)
      //   ks[i] = kappa[i] * (decay after token i to the segment's end)
      f2 cp[8][2], ks[8][2];
      f2 g8[2];
      {
        RawRegs<CKF32> raw1;
        load_raw(raw1, a, item, w, lane, 1);   // second half of the segment; the first half is in raw0
        const uint32_t rowsA = sb + kOffA0 + w * 1024 + th_fix, rowsB = sb + kOffB0 + w * 1024 + th_fix;
        f2 g4a[2], g4b[2];
        uint32_t wa[4][2], wb[4][2];
        // tokens 0..3: reference point just after token 3
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          f2 r[4], cc[4], kk[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            f2 rp[2], cq[2], kq[2];
            rho_pairs(raw0.r[i], rp);
            ck_pairs(raw0.c[i], cq);
            ck_pairs(raw0.k[i], kq);
            r[i] = rp[hf]; cc[i] = cq[hf]; kk[i] = kq[hf];
          }
          const f2 q2 = r[3], q1 = mul2(r[3], r[2]), q0 = mul2(q1, r[1]);    // decay after token i up to token 3
          const f2 p1 = mul2(r[0], r[1]), p2 = mul2(p1, r[2]), p3 = mul2(p2, r[3]);
          const f2 iq0 = rcp2(q0), iq1 = mul2(iq0, r[1]), iq2 = mul2(iq1, r[2]);
          g4a[hf] = p3;
          const f2 b0 = mul2(kk[0], q0), b1 = mul2(kk[1], q1), b2 = mul2(kk[2], q2);
          wa[0][hf] = cvt_bf2(mul2(cc[0], iq0));
          wa[1][hf] = cvt_bf2(mul2(cc[1], iq1));
          wa[2][hf] = cvt_bf2(mul2(cc[2], iq2));
          wa[3][hf] = cvt_bf2(cc[3]);
          wb[0][hf] = cvt_bf2(b0); wb[1][hf] = cvt_bf2(b1); wb[2][hf] = cvt_bf2(b2); wb[3][hf] = cvt_bf2(kk[3]);
          cp[0][hf] = mul2(cc[0], r[0]); cp[1][hf] = mul2(cc[1], p1); cp[2][hf] = mul2(cc[2], p2);
          cp[3][hf] = mul2(cc[3], p3);
          ks[0][hf] = b0; ks[1][hf] = b1; ks[2][hf] = b2; ks[3][hf] = kk[3];   // times g4b, below
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          emit_words(rowsA, i, wa[i][0], wa[i][1]);
          emit_words(rowsB, i, wb[i][0], wb[i][1]);
        }
        // tokens 4..7: reference point just before token 4
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          f2 r[4], cc[4], kk[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            f2 rp[2], cq[2], kq[2];
            rho_pairs(raw1.r[i], rp);
            ck_pairs(raw1.c[i], cq);
            ck_pairs(raw1.k[i], kq);
            r[i] = rp[hf]; cc[i] = cq[hf]; kk[i] = kq[hf];
          }
          const f2 q5 = mul2(r[0], r[1]), q6 = mul2(q5, r[2]), q7 = mul2(q6, r[3]);  // decay from token 4 to token i
          const f2 s5 = mul2(r[3], r[2]), s4 = mul2(s5, r[1]);                        // decay after token i to token 7
          const f2 iq7 = rcp2(q7), iq6 = mul2(iq7, r[3]), iq5 = mul2(iq6, r[2]), iq4 = mul2(iq5, r[1]);
          g4b[hf] = q7;
          const f2 a4 = mul2(cc[0], r[0]), a5 = mul2(cc[1], q5), a6 = mul2(cc[2], q6), a7 = mul2(cc[3], q7);
          wa[0][hf] = cvt_bf2(a4); wa[1][hf] = cvt_bf2(a5); wa[2][hf] = cvt_bf2(a6); wa[3][hf] = cvt_bf2(a7);
          wb[0][hf] = cvt_bf2(mul2(kk[0], iq4));
          wb[1][hf] = cvt_bf2(mul2(kk[1], iq5));
          wb[2][hf] = cvt_bf2(mul2(kk[2], iq6));
          wb[3][hf] = cvt_bf2(mul2(kk[3], iq7));
          cp[4][hf] = mul2(a4, g4a[hf]); cp[5][hf] = mul2(a5, g4a[hf]); cp[6][hf] = mul2(a6, g4a[hf]);
          cp[7][hf] = mul2(a7, g4a[hf]);
          ks[4][hf] = mul2(kk[0], s4); ks[5][hf] = mul2(kk[1], s5); ks[6][hf] = mul2(kk[2], r[3]); ks[7][hf] = kk[3];
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          emit_words(rowsA, 4 + i, wa[i][0], wa[i][1]);
          emit_words(rowsB, 4 + i, wb[i][0], wb[i][1]);
        }
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
#pragma unroll
          for (int i = 0; i < 4; ++i) ks[i][hf] = mul2(ks[i][hf], g4b[hf]);
          g8[hf] = mul2(g4a[hf], g4b[hf]);
        }
        asm volatile("st.shared.v2.b64 [%0], {%1, %2};" ::"r"(seg_s + w * (kM * 4)), "l"(g8[0]), "l"(g8[1]) : "memory");
      }
      warp_arrive(fA, lane);
      umma::named_barrier(1, kWorkers);  // segment products visible to every worker
      if (n > 0) write_rows(n - 1);  // also: every MMA of the previous tile is done, slots 2..5 are free

      // ---- products of whole segments: back from this segment to the start of its 16 / 32 / 64 /
      // 128-token block (bk), forward from it to the end of that block (fw).  A level uses bk when
      // this segment sits in the second half of the level's block (A role), else fw (B role).  The
      // products grow level by level, interleaved with the levels' operand rows.
      f2 bk[2] = {one2(), one2()}, fw[2] = {one2(), one2()};
      auto mulseg = [&](f2 (&acc)[2], int s) {
        f2 x, y;
        lds_f2x2(seg_s + s * (kM * 4), x, y);
        acc[0] = mul2(acc[0], x);
        acc[1] = mul2(acc[1], y);
      };
      // One sibling level: this segment's 8 rows go to the A-role or the B-role tile of its stack.
      auto emit_level = [&](uint32_t rows_s, const f2 (&src)[8][2], const f2 (&sig)[2], bool scale) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const f2 v0 = scale ? mul2(src[i][0], sig[0]) : src[i][0];
          const f2 v1 = scale ? mul2(src[i][1], sig[1]) : src[i][1];
          emit_words(rows_s, i, cvt_bf2(v0), cvt_bf2(v1));
        }
      };
      // ---- levels 8 (rows 0..63 of the stack) and 16 (rows 64..127) -> slots 2 / 3
      {
        const uint32_t rg8 = w >> 1, rg16 = 8 + (((w >> 2) << 1) | (w & 1));
        if (w & 1) emit_level(sb + kOffY1 + rg8 * 1024 + th_fix, cp, bk, false);
        else emit_level(sb + kOffZ1 + rg8 * 1024 + th_fix, ks, bk, false);
        if (w & 1) mulseg(bk, w - 1); else mulseg(fw, w + 1);
        if (w & 2) emit_level(sb + kOffY1 + rg16 * 1024 + th_fix, cp, bk, true);
        else emit_level(sb + kOffZ1 + rg16 * 1024 + th_fix, ks, fw, true);
      }
      warp_arrive(fL1, lane);
      // ---- levels 32 (rows 64..127) and 64 (rows 0..63) -> slots 4 / 5
      {
        const uint32_t rg64 = w & 7, rg32 = 8 + (((w >> 3) << 2) | (w & 3));
        const int b4 = w & ~3, b8 = w & ~7;
        if (w & 2) { mulseg(bk, b4); mulseg(bk, b4 + 1); } else { mulseg(fw, b4 + 2); mulseg(fw, b4 + 3); }
        if (w & 4) emit_level(sb + kOffY2 + rg32 * 1024 + th_fix, cp, bk, true);
        else emit_level(sb + kOffZ2 + rg32 * 1024 + th_fix, ks, fw, true);
        if (w & 4) {
#pragma unroll
          for (int s = 0; s < 4; ++s) mulseg(bk, b8 + s);
        } else {
#pragma unroll
          for (int s = 4; s < 8; ++s) mulseg(fw, b8 + s);
        }
        if (w & 8) emit_level(sb + kOffY2 + rg64 * 1024 + th_fix, cp, bk, true);
        else emit_level(sb + kOffZ2 + rg64 * 1024 + th_fix, ks, fw, true);
      }
      warp_arrive(fL2, lane);
      // to the tile's start (E) and end (F)
      if (w & 8) {
#pragma unroll
        for (int s = 0; s < 8; ++s) mulseg(bk, s);
      } else {
#pragma unroll
        for (int s = 8; s < 16; ++s) mulseg(fw, s);
      }
      const f2 (&E)[2] = bk, (&F)[2] = fw;
      // decay of the whole tile for the mode this thread owns in the state update (m = 32 Q + lane):
      // every warp holds the full vector, four modes per lane
      float gt_row;
      {
        float g[4];
        un2(mul2(mul2(E[0], g8[0]), F[0]), g[0], g[1]);
        un2(mul2(mul2(E[1], g8[1]), F[1]), g[2], g[3]);
        const int src = 8 * Q + (lane >> 2);
#pragma unroll
        for (int x = 0; x < 4; ++x) g[x] = __shfl_sync(0xffffffffu, g[x], src);
        const int cmp = lane & 3;
        gt_row = cmp == 0 ? g[0] : cmp == 1 ? g[1] : cmp == 2 ? g[2] : g[3];
      }

      // ---- Khat = ks * (decay to the tile's end), high and low parts -> slots 0 / 1 (base product done)
      FRACSSM_WAIT(cb0, n);
      {
        const uint32_t rowsH = sb + kOffKhi + w * 1024 + th_fix, rowsL = sb + kOffKlo + w * 1024 + th_fix;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const f2 k0 = mul2(ks[i][0], F[0]), k1 = mul2(ks[i][1], F[1]);
          const uint32_t h0 = cvt_bf2(k0), h1 = cvt_bf2(k1);
          emit_words(rowsH, i, h0, h1);
          emit_words(rowsL, i, cvt_bf2(sub2(k0, widen_bf2(h0))), cvt_bf2(sub2(k1, widen_bf2(h1))));
        }
      }
      // ---- Chat = cp * (decay from the tile's start) -> slots 2 / 3 (level-8/16 product done)
      FRACSSM_WAIT(cb1, n);
      {
        const uint32_t rowsH = sb + kOffChi + w * 1024 + th_fix, rowsL = sb + kOffClo + w * 1024 + th_fix;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const f2 c0 = mul2(cp[i][0], E[0]), c1 = mul2(cp[i][1], E[1]);
          const uint32_t h0 = cvt_bf2(c0), h1 = cvt_bf2(c1);
          emit_words(rowsH, i, h0, h1);
          emit_words(rowsL, i, cvt_bf2(sub2(c0, widen_bf2(h0))), cvt_bf2(sub2(c1, widen_bf2(h1))));
        }
      }
      warp_arrive(fK, lane);

      // the next item (published by the control warp at the start of this tile); it must be read
      // here, before this warp's arrival on fW lets the control warp move on and publish again.
      // Its first four token rows are requested now and arrive while the tile finishes.
      FRACSSM_WAIT(item_bar, n + 1);
      const int next = items[(n + 1) & 1];
      if (next < a.total) load_raw(raw0, a, next, w, lane, 0);

      // ---- W -> slot 4: each block of accumulators goes to its place (levels 64+32 product done)
      FRACSSM_WAIT(cb2, n);
      umma::tc_fence_after();
      {
        const uint32_t sW = sb + kOffW;
        // 8 accumulators of row t, columns 8 kc .. 8 kc + 7 of W, as one 16-byte store
        auto put8 = [&](int t, int kc, const auto &v, int o) {
          uint4 pk;
          pk.x = pack2(v[o], v[o + 1]); pk.y = pack2(v[o + 2], v[o + 3]); pk.z = pack2(v[o + 4], v[o + 5]);
          pk.w = pack2(v[o + 6], v[o + 7]);
          const uint32_t addr = sW + (kc >> 3) * kAtom + t * 128 + (((kc & 7) ^ (t & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pk.x), "r"(pk.y), "r"(pk.z), "r"(pk.w)
                       : "memory");
        };
        const int grp = lane >> 3;  // row group of this lane inside the warp's 32 accumulator rows
        float v[32];
        if (P == 0) {
          // base: row t = 32 Q + lane, its own segment's 8 columns, masked above the diagonal
          umma::tmem_ld32(lane_addr + kColBase + 32 * Q, v);
          umma::tmem_ld_wait();
          float o[8];
#pragma unroll
          for (int x = 0; x < 8; ++x) {
            const float s = grp == 0 ? v[x] : grp == 1 ? v[8 + x] : grp == 2 ? v[16 + x] : v[24 + x];
            o[x] = x <= (lane & 7) ? s : 0.f;
          }
          put8(32 * Q + lane, 4 * Q + grp, o, 0);
        } else if (Q < 2) {
          if (P == 1) {
            // level 8: accumulator row 32 Q + lane is token 64 Q + 16 grp + 8 + (lane & 7); its partner
            // segment is the one before it
            umma::tmem_ld32(lane_addr + kColL1 + 32 * Q, v);
            umma::tmem_ld_wait();
            float o[8];
#pragma unroll
            for (int x = 0; x < 8; ++x) o[x] = grp == 0 ? v[x] : grp == 1 ? v[8 + x] : grp == 2 ? v[16 + x] : v[24 + x];
            put8(64 * Q + 16 * grp + 8 + (lane & 7), 8 * Q + 2 * grp, o, 0);
          } else {
            // level 64: accumulator row 32 Q + lane is token 64 + 32 Q + lane; columns = tokens 0..63
            const int c0 = 32 * (P - 2);
            umma::tmem_ld32(lane_addr + kColL2 + c0, v);
            umma::tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 4; ++e) put8(64 + 32 * Q + lane, (c0 >> 3) + e, v, 8 * e);
          }
        } else {
          const int q2 = Q - 2;
          if (P == 1) {
            // level 16: accumulator row 64 + 32 q2 + lane is token 64 q2 + 32 (lane >> 4) + 16 + (lane & 15);
            // its partners are the 16 tokens before its 16-token half
            umma::tmem_ld32(lane_addr + kColL1 + 64 + 32 * q2, v);
            umma::tmem_ld_wait();
            float o[16];
#pragma unroll
            for (int x = 0; x < 16; ++x) o[x] = (lane >> 4) ? v[16 + x] : v[x];
            const int t = 64 * q2 + 32 * (lane >> 4) + 16 + (lane & 15);
            const int kc = 8 * q2 + 4 * (lane >> 4);
            put8(t, kc, o, 0);
            put8(t, kc + 1, o, 8);
          } else {
            // level 32: accumulator row 64 + 32 q2 + lane is token 64 q2 + 32 + lane; partners: the 32
            // tokens before its half
            float u16[16];
            umma::tmem_ld16(lane_addr + kColL2 + 64 + 32 * q2 + 16 * (P - 2), u16);
            umma::tmem_ld_wait();
            const int t = 64 * q2 + 32 + lane, kc = 8 * q2 + 2 * (P - 2);
            put8(t, kc, u16, 0);
            put8(t, kc + 1, u16, 8);
          }
        }
        // zeros above the diagonal: row t = tid / 4 owns the blocks kc > t / 8, four threads share a row
        {
          const int t = tid >> 2;
          for (int kc = (t >> 3) + 1 + (tid & 3); kc < 16; kc += 4) {
            const uint32_t addr = sW + (kc >> 3) * kAtom + t * 128 + (((kc & 7) ^ (t & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(addr), "r"(0u) : "memory");
          }
        }
      }
      warp_arrive(fW, lane);

      // ---- the chain: incoming state -> MMA operand (high | low) -> outgoing state
      FRACSSM_WAIT(state_bar, n);
      const int m_row = 32 * Q + lane;
      float sj[16];
      {
        // scratch layout [bh][P][x][m][4]: the lanes of a warp touch consecutive 16-byte pieces
        const float4 *sp = reinterpret_cast<const float4 *>(a.state) +
                           (static_cast<int64_t>(bh) * 4 + P) * 4 * kM + m_row;
        if (jt > 0) {
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            const float4 s4 = __ldcg(sp + x * kM);
            sj[4 * x] = s4.x; sj[4 * x + 1] = s4.y; sj[4 * x + 2] = s4.z; sj[4 * x + 3] = s4.w;
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
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t ph[4], pl[4];
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const float2 sv = make_float2(sj[8 * half + 2 * x], sj[8 * half + 2 * x + 1]);
          const float2 hi = bf16_round2(sv, ph[x]);
          pl[x] = pack2(sv.x - hi.x, sv.y - hi.y);
        }
        const uint32_t off = m_row * 128 + (((2 * P + half) ^ (m_row & 7)) << 4);
        *reinterpret_cast<uint4 *>(smem + kOffS + off) = make_uint4(ph[0], ph[1], ph[2], ph[3]);
        *reinterpret_cast<uint4 *>(smem + kOffS + kAtom + off) = make_uint4(pl[0], pl[1], pl[2], pl[3]);
      }
      warp_arrive(fS, lane);

      FRACSSM_WAIT(cbK, n);  // Khat(high) and Khat(low) MMAs: Sacc is complete
      umma::tc_fence_after();
      {
        // S_next = Gt * S + Sacc
        float acc[16];
        umma::tmem_ld16(lane_addr + kColS + 16 * P, acc);
        umma::tmem_ld_wait();
        const bool bad = *failed != 0;
#pragma unroll
        for (int x = 0; x < 16; ++x) acc[x] = bad ? kNaN : fmaf(gt_row, sj[x], acc[x]);
        float4 *sp = reinterpret_cast<float4 *>(a.state) + (static_cast<int64_t>(bh) * 4 + P) * 4 * kM + m_row;
        if (jt + 1 < a.ntiles) {
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

      prev_bh = bh;
      prev_t0 = t0;
      item = next;
    }
    if (n_tiles_done > 0) write_rows(n_tiles_done - 1);
  }

  if (!ok) atomicExch(&a.ctrl[1], 1);
  umma::tc_fence_before();
  __syncthreads();
  if (w == 0) umma::tmem_dealloc(tmem, 512);
}

size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

}  // namespace

size_t scan_fused_workspace_bytes(int64_t B, int64_t, int64_t R, int64_t M, int64_t) {
  return kCtrlBytes + align256((size_t)B * 4) + (size_t)B * R * M * 4;
}

// first_tile / wait_ns: 0 and the default limit, except in the wait-limit self-test, which starts
// at a tile whose predecessor is not part of the launch.
int scan_fused_launch_ex(const void *u, const void *c, const void *kappa, int ck_dtype, const float *rho,
                         const float *initial_state, void *h, void *final_state, int final_dtype,
                         void *workspace, size_t workspace_bytes, int64_t B, int64_t L, int64_t R,
                         int64_t M, int64_t T, void *stream, int first_tile, unsigned long long wait_ns) {
  (void)T;
  const bool ckf32 = ck_dtype == FRACSSM_F32;
  if (workspace_bytes < scan_fused_workspace_bytes(B, L, R, M, T))
    return fail(FRACSSM_ERR_ARG, "frac_scan: workspace too small");
  // the kernel reads c / kappa / rho and writes h with 8- and 16-byte accesses
  if (((reinterpret_cast<uintptr_t>(u) | reinterpret_cast<uintptr_t>(c) | reinterpret_cast<uintptr_t>(kappa) |
        reinterpret_cast<uintptr_t>(rho) | reinterpret_cast<uintptr_t>(h)) & 15) != 0)
    return fail(FRACSSM_ERR_ARG, "frac_scan: u, c, kappa, rho and h must be 16-byte aligned");
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
      int prc = prepare(reinterpret_cast<const void *>(&scan_fused_kernel<false>));
      if (prc == FRACSSM_OK) prc = prepare(reinterpret_cast<const void *>(&scan_fused_kernel<true>));
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
  a.flags = reinterpret_cast<int *>(ws + kCtrlBytes);
  a.state = reinterpret_cast<float *>(ws + kCtrlBytes + align256((size_t)B * 4));
  a.BH = (int)B;
  a.L = (int)L;
  a.ntiles = (int)ceil_div(L, kTile);
  a.first_tile = first_tile;
  a.total = (a.ntiles - first_tile) * a.BH;
  a.wait_ns = wait_ns;
  CUtensorMap map;
  int rc = make_tmap_bf16_3d(&map, u, kR, (uint64_t)L, (uint64_t)B, kR, kTile);
  if (rc) return rc;
  cudaError_t e = cudaMemsetAsync(ws, 0, kCtrlBytes + align256((size_t)B * 4), (cudaStream_t)stream);
  if (e != cudaSuccess) return fail(FRACSSM_ERR_CUDA, "frac_scan: %s", cudaGetErrorString(e));
  const int grid = a.total < sms ? a.total : sms;
  const cudaStream_t st = (cudaStream_t)stream;
  if (ckf32) scan_fused_kernel<true><<<grid, kThreads, kSmemBytes, st>>>(a, map);
  else scan_fused_kernel<false><<<grid, kThreads, kSmemBytes, st>>>(a, map);
  return check_launch("frac_scan (single-pass kernel)");
}

int scan_fused_launch(const void *u, const void *c, const void *kappa, int ck_dtype, const float *rho,
                      const float *initial_state, void *h, void *final_state, int final_dtype,
                      void *workspace, size_t workspace_bytes, int64_t B, int64_t L, int64_t R,
                      int64_t M, int64_t T, void *stream) {
  return scan_fused_launch_ex(u, c, kappa, ck_dtype, rho, initial_state, h, final_state, final_dtype, workspace,
                              workspace_bytes, B, L, R, M, T, stream, 0, kWaitNs);
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
    kCtrlBytes + ((kNoAllocMaxRows * 4 + 255) / 256) * 256 + kNoAllocMaxRows * kR * kM * 4;
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
  if (((reinterpret_cast<uintptr_t>(u) | reinterpret_cast<uintptr_t>(c) | reinterpret_cast<uintptr_t>(kappa) |
        reinterpret_cast<uintptr_t>(rho) | reinterpret_cast<uintptr_t>(h)) & 15) != 0)
    return fail(FRACSSM_ERR_ARG, "frac_scan (no-alloc): u, c, kappa, rho and h must be 16-byte aligned");
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

// Error word of the last no-alloc launch on the current device (synchronises the stream).
extern "C" int fracssm_frac_scan_noalloc_status(void *stream) {
  using namespace fracssm;
  void *scratch = nullptr;
  int rc = noalloc_scratch(&scratch);
  if (rc) return rc;
  return fracssm_scan_fused_status(scratch, stream);
}

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
// One CTA per SM, 20 warps.  Warps 0-15 ("workers") turn the raw inputs into bf16 operand tiles in
// shared memory and run the epilogues; warp 16 ("MMA warp") issues the TMA load of u and every
// tcgen05.mma; warp 17 ("chain warp") takes the tickets, pulls the next item into L2 and hands the
// state from tile to tile of a row (polls and releases the per-row counter); warps 18-19 only pad
// the register group of those two.  Workers hand a batch of tiles over by arriving on a "full"
// mbarrier (one arrival per warp, after a proxy fence); the MMA warp hands buffers and accumulators
// back through tcgen05.commit mbarriers.  The MMA warp passes through its code once per tile, so that
// code is kept small (rolled loops over the contraction steps, issued from one elected lane, which
// keeps the descriptor arithmetic on the uniform datapath): as straight-line code it was fetched from
// beyond the instruction cache every tile and the kernel ran 10 % slower.
//
// A tile is processed in two passes over the modes (64 + 64): a worker thread owns 8 token rows x 2
// modes per pass, so its per-token factors (32 registers) and the raw inputs of the other pass
// (32 registers, requested one pass ahead in two batches of four token rows; full tiles use one
// address per thread and immediate row offsets) fit in registers without spilling; each operand tile's two
// 64-column halves are filled by the two passes and the level / base products are issued per pass
// (4 of their 8 contraction steps), accumulating in tensor memory.
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
// 192..319, levels 64+32 320..447, output accumulator H 448..511.
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
// the group of the MMA and chain warps shrinks to kControlRegs.  Each SM sub-partition holds four
// worker warps and one warp of that group: 4 * 112 + 32 = 5 * 96, the launch allocation
// (checked on the host: it must cover both, or the growing warps would wait forever).
constexpr int kWorkerRegs = 112, kControlRegs = 32;
constexpr int kLaunchRegsNeeded = (kWorkers * kWorkerRegs + (kThreads - kWorkers) * kControlRegs + kThreads - 1) / kThreads;
// shared memory map (bytes from the 1024-aligned base)
constexpr uint32_t kSlot = 32768;
static_assert(kSlot == 32768, "emit_pair_next_slot stores 32768 bytes further on");
constexpr uint32_t kOffA0 = 0, kOffB0 = kSlot, kOffY1 = 2 * kSlot, kOffZ1 = 3 * kSlot, kOffY2 = 4 * kSlot,
                   kOffZ2 = 5 * kSlot;
constexpr uint32_t kOffKhi = kOffA0, kOffKlo = kOffB0, kOffChi = kOffY1, kOffClo = kOffZ1, kOffW = kOffY2,
                   kOffS = kOffZ2;              // second use of each slot
constexpr uint32_t kOffU = 6 * kSlot;           // u tile, 128 tokens x 64 bf16
constexpr uint32_t kOffSeg = kOffU + 16384;     // float [16][128]: decay product of each 8-token segment
constexpr uint32_t kOffMisc = kOffSeg + 8192;   // mbarriers, TMEM base, tickets, failure flag
constexpr uint32_t kSmemBytes = kOffMisc + 256 + 1024;
// tensor-memory columns (fp32, 128 lanes each)
constexpr uint32_t kColBase = 0, kColS = 128, kColL1 = 192, kColL2 = 320, kColH = 448;
constexpr size_t kCtrlBytes = 256;

struct FusedArgs {
  const void *c, *kappa;  // bf16 or f32 [BH, L, 128], see the kernel's CKF32 parameter
  const float *rho, *init;
  const __nv_bfloat16 *u;   // [BH, L, 64] (read by TMA; the pointer is only used for the L2 prefetch)
  __nv_bfloat16 *h;
  void *fin;
  int fin_dt;
  int *ctrl;     // [0] ticket counter, [1] error word
  int *flags;    // [BH] tiles finished per bh
  float *state;  // running state per row, 128 m x 64 r floats in the order the workers access it
  int BH, L, ntiles, total;
  int first_tile;              // tile index of the first ticket (0 except in the wait-limit self-test)
  unsigned long long wait_ns;  // limit of every device-side wait
  // Layer mode (gate != null): instead of h, the output stage writes the gated value
  //   g[b, l, head*64 + r] = (h[bh, l, r] + u[bh, l, r] * D[head, r]) * silu(gate[b, l, head*64 + r] + gate_bias)
  // un-flattened to [batch, L, H*64], and per (b, l, head) four partial sums of g^2 (16 columns each).
  const __nv_bfloat16 *gate;
  const float *D;
  __nv_bfloat16 *gated;
  float *ss;
  float gate_bias;
  int H;
};

// Diagnostic build (-DFRACSSM_PHASE_PROF, never the product library): clock stamps of a few warps of
// CTA 0 at the phase boundaries of four consecutive tiles, read back with fracssm_prof_stamps.
#ifdef FRACSSM_PHASE_PROF
constexpr int kProfTile0 = 8, kProfTiles = 4, kProfWarps = 4, kProfMarks = 40;
__device__ long long g_prof[kProfTiles][kProfWarps][kProfMarks];
#define FRACSSM_MARK(slot, id)                                                                   \
  if (blockIdx.x == 0 && lane == 0 && n >= kProfTile0 && n < kProfTile0 + kProfTiles && (slot) >= 0) \
    g_prof[n - kProfTile0][slot][id] = clock64();
#else
#define FRACSSM_MARK(slot, id)
#endif

// Raw inputs of one item for one worker thread and one half of the modes: its 8 token rows x 2 modes.
// rho arrives as two floats; c and kappa as two bf16 (one word) or two floats.
template <bool CKF32>
struct RawHalf {
  using CK = typename std::conditional<CKF32, f2, uint32_t>::type;
  f2 r[8];
  CK c[8], k[8];
};

// The loads do not allocate in L1 (with 222 KB of shared memory per CTA the L1 keeps about 28 KB, a
// tile reads 164 KB) and are volatile so that they stay where they are written.
__device__ __forceinline__ void ldg_stream(f2 &d, const void *p) {
  asm volatile("ld.global.L1::no_allocate.b64 %0, [%1];" : "=l"(d) : "l"(p));
}
__device__ __forceinline__ void ldg_stream(uint32_t &d, const void *p) {
  asm volatile("ld.global.L1::no_allocate.b32 %0, [%1];" : "=r"(d) : "l"(p));
}
__device__ __forceinline__ f2 ck_wide(uint32_t v) { return widen_bf2(v); }
__device__ __forceinline__ f2 ck_wide(f2 v) { return v; }

// Requests token row i (0..7) of this thread's segment of `item`, modes 64 h + 2 lane, + 1.
template <bool CKF32>
__device__ __forceinline__ void load_tok(RawHalf<CKF32> &raw, const FusedArgs &a, int bh, int t0, int w, int lane,
                                         int h, int i) {
  using CK = typename RawHalf<CKF32>::CK;
  const int t = t0 + 8 * w + i;
  raw.r[i] = mk2(1.f, 1.f);
  raw.c[i] = CK{};
  raw.k[i] = CK{};
  if (t < a.L) {
    const int64_t e = (static_cast<int64_t>(bh) * a.L + t) * kM + 64 * h + 2 * lane;   // element index
    ldg_stream(raw.r[i], a.rho + e);
    ldg_stream(raw.c[i], reinterpret_cast<const char *>(a.c) + e * (CKF32 ? 4 : 2));
    ldg_stream(raw.k[i], reinterpret_cast<const char *>(a.kappa) + e * (CKF32 ? 4 : 2));
  }
}

// The same for token rows I and I + 1 of a tile that lies wholly inside the sequence: one element
// offset for the thread, the rows as immediate byte offsets of the loads.
template <int OFF>
__device__ __forceinline__ void ldg_stream_at(f2 &d, const void *p) {
  asm volatile("ld.global.L1::no_allocate.b64 %0, [%1+%2];" : "=l"(d) : "l"(p), "n"(OFF));
}
template <int OFF>
__device__ __forceinline__ void ldg_stream_at(uint32_t &d, const void *p) {
  asm volatile("ld.global.L1::no_allocate.b32 %0, [%1+%2];" : "=r"(d) : "l"(p), "n"(OFF));
}
// 32 bytes per lane in one instruction (sm_100: 256-bit global accesses); the address must be 32-byte aligned
__device__ __forceinline__ void stg_stream_32B(void *p, const uint4 &a, const uint4 &b) {
  asm volatile("st.global.cs.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w),
               "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w) : "memory");
}
__device__ __forceinline__ void ldg_stream_32B(const void *p, uint4 &a, uint4 &b) {
  asm volatile("ld.global.cs.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];" : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w),
               "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(p));
}
template <bool CKF32, bool RAGGED, int I>
__device__ __forceinline__ void load_tok2(RawHalf<CKF32> &raw, const FusedArgs &a, int bh, int t0, int w, int lane,
                                          int h) {
  if (!RAGGED || t0 + kTile <= a.L) {
    constexpr int kCk = CKF32 ? 4 : 2;
    const int64_t e = (static_cast<int64_t>(bh) * a.L + t0 + 8 * w) * kM + 64 * h + 2 * lane;   // row 0 of the segment
    const float *rp = a.rho + e;
    const char *cp = reinterpret_cast<const char *>(a.c) + e * kCk, *kp = reinterpret_cast<const char *>(a.kappa) + e * kCk;
    ldg_stream_at<I * kM * 4>(raw.r[I], rp);
    ldg_stream_at<I * kM * kCk>(raw.c[I], cp);
    ldg_stream_at<I * kM * kCk>(raw.k[I], kp);
    ldg_stream_at<(I + 1) * kM * 4>(raw.r[I + 1], rp);
    ldg_stream_at<(I + 1) * kM * kCk>(raw.c[I + 1], cp);
    ldg_stream_at<(I + 1) * kM * kCk>(raw.k[I + 1], kp);
    return;
  }
  if constexpr (RAGGED) {
    load_tok(raw, a, bh, t0, w, lane, h, I);
    load_tok(raw, a, bh, t0, w, lane, h, I + 1);
  }
}

__device__ __forceinline__ f2 floor2(f2 v) {
  float lo, hi;
  un2(v, lo, hi);
  return mk2(fmaxf(lo, kRhoFloor), fmaxf(hi, kRhoFloor));
}
// One 4-byte store of an operand row: rows_s = tile + 16384 * half + 1024 * row group + the thread's
// fixed offset (bits 4..6 hold its 16-byte chunk index), i = row inside the group.
__device__ __forceinline__ void emit_pair(uint32_t rows_s, int i, uint32_t w0) {
  const uint32_t addr = (rows_s ^ (static_cast<uint32_t>(i) << 4)) + i * 128;
  asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(w0) : "memory");
}

// The same row of the operand tile one slot further on (slots are 32 KB apart, so the swizzled row
// address is the same plus a constant, which the store takes as an immediate).
__device__ __forceinline__ void emit_pair_next_slot(uint32_t rows_s, int i, uint32_t w0) {
  const uint32_t addr = (rows_s ^ (static_cast<uint32_t>(i) << 4)) + i * 128;
  asm volatile("st.shared.b32 [%0+32768], %1;" ::"r"(addr), "r"(w0) : "memory");
}

// CKF32: c and kappa are float32 (else bf16).  LAYER: the output stage applies the skip connection and
// the gate (its code is kept out of the plain kernel, whose loop is fetched once per tile).
// RAGGED: L is not a multiple of the tile, so a row's last tile takes the row-by-row, predicated loads
// (kept out of the other instances: the loop's code is fetched once per tile and its size counts).
template <bool CKF32, bool LAYER, bool RAGGED>
__global__ void __launch_bounds__(kThreads, 1)
scan_fused_kernel(const FusedArgs a, const __grid_constant__ CUtensorMap u_map) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // mbarriers.  Completed once per tile: cb2 / cbK / barH (tcgen05.commit), barU (TMA), fS / fW / out_bar
  // (16 worker warps), item_bar / state_bar (chain warp), read_bar (workers + MMA warp).  Completed once per HALF of the modes,
  // i.e. twice per tile, so the phase parity of half h is simply h: cb0 / cbL (tcgen05.commit) and
  // fA / fL1 / fL / fK (16 worker warps).
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kOffMisc);
  uint64_t *cb0 = bars + 0, *cbL = bars + 1, *cb2 = bars + 2, *cbK = bars + 3, *barH = bars + 4, *barU = bars + 5;
  uint64_t *fA = bars + 6, *fL = bars + 7, *fK = bars + 8, *fW = bars + 9, *fS = bars + 10;
  uint64_t *item_bar = bars + 11, *state_bar = bars + 12, *out_bar = bars + 13, *read_bar = bars + 14;
  uint64_t *fL1 = bars + 15;    // 16 worker warps, once per half: the rows of the levels 8 + 16 are written
  uint32_t *tmem_s = reinterpret_cast<uint32_t *>(bars + 16);
  volatile int *items = reinterpret_cast<volatile int *>(tmem_s + 1);  // [2], by tile parity
  volatile int *failed = reinterpret_cast<volatile int *>(tmem_s + 3);  // a wait of this CTA ran out

  const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int i = 0; i < 6; ++i) umma::mbar_init(bars + i, 1);
    for (int i = 6; i < 11; ++i) umma::mbar_init(bars + i, 16);
    umma::mbar_init(item_bar, 1);
    umma::mbar_init(state_bar, 1);
    umma::mbar_init(out_bar, 16);
    umma::mbar_init(read_bar, 17);   // the 16 worker warps and the MMA warp, once each has read the tile's item
    umma::mbar_init(fL1, 16);
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
  // Bounded waits.  The MMA and chain warps poll (every hand-over of the tile passes through them:
  // a parked wait wakes up several hundred cycles after the barrier completes); the 16 worker
  // warps park, which leaves the issue slots to the warps that have work.  A wait that runs
  // out marks the CTA as failed: its remaining outputs are written as NaN and the error word is set.
  // (each setmaxnreg sits inside its role's branch: the register limit must not merge across roles)
  if (w > 17) {
    // spare warps of the two service warps' register group: give the registers back, nothing else
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kControlRegs));
  } else if (w == 17) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kControlRegs));
#define FRACSSM_WAIT(bar, parity)                                  \
  if (ok) {                                                        \
    ok = umma::mbar_wait(bar, (parity) & 1u, wait_ns);             \
    if (!ok) *failed = 1;                                          \
  }
    // =========================== chain warp ===========================
    // Tickets, the L2 prefetch of the next item, and the hand-over of the state between the tiles of
    // a (batch, head) row: nothing here waits for an MMA, so a row's chain is never held up by them.
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
      // The next ticket is published through item_bar only after every reader holds the current one
      // (read_bar): two completions of item_bar in a row would flip its parity twice, and a reader
      // that had not looked yet would wait for a phase that never comes.
      FRACSSM_WAIT(read_bar, n);
      int next = 0;
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
        umma::prefetch_l2(a.u + tok * kR, ntok * kR * 2);
      }
      // the state left by the previous tile of this row
      if (lane == 0) {
        if (jt > 0 && ok) {
          const uint64_t t_start = umma::global_ns();
          while (ld_acquire(a.flags + bh) < jt) {
            __nanosleep(100);
            if (umma::global_ns() - t_start > wait_ns) { ok = false; *failed = 1; break; }
          }
        }
        umma::mbar_arrive(state_bar);
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      // publish the outgoing state once the workers have stored it: their stores are ordered before
      // their arrivals on out_bar, this release makes them visible to the next tile's CTA
      FRACSSM_WAIT(out_bar, n);
      if (lane == 0 && jt + 1 < a.ntiles) st_release(a.flags + bh, jt + 1);
      __syncwarp();
      item = next;
    }
#undef FRACSSM_WAIT
  } else if (w == 16) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kControlRegs));
#define FRACSSM_WAIT(bar, parity)                                  \
  if (ok) {                                                        \
    ok = umma::mbar_wait(bar, (parity) & 1u, wait_ns);             \
    if (!ok) *failed = 1;                                          \
  }
    // =========================== MMA warp ===========================
    const uint32_t sb = umma::smem_u32(smem);
    const uint32_t sA0 = sb + kOffA0, sB0 = sb + kOffB0, sY1 = sb + kOffY1, sZ1 = sb + kOffZ1, sY2 = sb + kOffY2,
                   sZ2 = sb + kOffZ2, sU = sb + kOffU;
    const uint32_t sKhi = sb + kOffKhi, sKlo = sb + kOffKlo, sChi = sb + kOffChi, sClo = sb + kOffClo,
                   sW = sb + kOffW, sS = sb + kOffS;
    constexpr uint32_t kIdKK128 = umma::make_idesc(128, 128, false, false);
    constexpr uint32_t kIdKMn64 = umma::make_idesc(128, 64, false, true);
    constexpr uint32_t kIdMnMn64 = umma::make_idesc(128, 64, true, true);
    // Contraction steps s0 .. s1-1 (16 modes or tokens each) of one GEMM piece.  A K-major 128-column
    // tile advances by 32 bytes inside a 64-column atom and by one atom after 4 steps (steps 0..3 are
    // the first half of the modes, 4..7 the second); an MN-major tile by 16 rows (2048 B).
    // Called by the one elected lane.
    // The steps run as a real loop (not unrolled): this warp passes through its code once per tile,
    // so straight-line code would be fetched from beyond the instruction cache every time.
    auto piece = [&](uint32_t d_col, uint32_t a_addr, bool a_mn, uint32_t b_addr, bool b_mn, uint32_t idesc,
                     uint32_t acc_first, uint32_t s0, uint32_t s1) {
      const uint32_t k0 = ((s0 >> 2) * kAtom + (s0 & 3) * 32) >> 4, mn0 = (s0 * 2048) >> 4;
      uint64_t da = umma::make_sdesc(a_addr, a_mn ? kAtom : 16, 1024) + (a_mn ? mn0 : k0);
      uint64_t db = umma::make_sdesc(b_addr, b_mn ? kAtom : 16, 1024) + (b_mn ? mn0 : k0);
      uint32_t acc = acc_first;
#pragma unroll 1
      for (uint32_t s = s0; s < s1; ++s) {
        umma::mma_ss(tmem + d_col, da, db, idesc, acc);
        acc = 1u;
        const uint32_t k_inc = (s & 3) == 3 ? (kAtom - 96) >> 4 : 2u, mn_inc = 2048 >> 4;
        da += a_mn ? mn_inc : k_inc;
        db += b_mn ? mn_inc : k_inc;
      }
    };

#pragma unroll 1
    for (uint32_t n = 0;; ++n) {
      FRACSSM_WAIT(item_bar, n);
      const int item = items[n & 1];
      __syncwarp();
      if (lane == 0) umma::mbar_arrive(read_bar);
      if (item >= a.total) break;
      const int j = item / a.BH, bh = item - j * a.BH;
      const int jt = j + a.first_tile;  // tile index inside the row
      FRACSSM_MARK(3, 0)
#pragma unroll
      for (uint32_t h = 0; h < 2; ++h) {
        // base: D[t,k] += A0[t, modes of half h] . B0[k, the same modes]
        FRACSSM_WAIT(fA, h);
        FRACSSM_MARK(3, 1 + 4 * h)
        umma::tc_fence_after();
        if (umma::elect_one()) {
          piece(kColBase, sA0, false, sB0, false, kIdKK128, h, 4 * h, 4 * h + 4);
          umma::mma_commit(cb0);
        }
        __syncwarp();
        if (h == 0) {
          // the u tile is free once every MMA of the previous tile has finished
          if (n > 0) { FRACSSM_WAIT(barH, n - 1); }
          FRACSSM_MARK(3, 2)
          if (lane == 0) {
            umma::mbar_expect_tx(barU, kTile * kR * 2);
            umma::tma_load_3d(smem + kOffU, &u_map, barU, 0, jt * kTile, bh);
          }
        }
        // levels 8 + 16, then 64 + 32: A rows x B rows of the stacked tiles, this half of the modes
        FRACSSM_WAIT(fL1, h);
        umma::tc_fence_after();
        if (umma::elect_one()) {
          piece(kColL1, sY1, false, sZ1, false, kIdKK128, h, 4 * h, 4 * h + 4);
          umma::mma_commit(cbL);
        }
        __syncwarp();
        FRACSSM_WAIT(fL, h);
        FRACSSM_MARK(3, 3 + 4 * h)
        umma::tc_fence_after();
        if (umma::elect_one()) {
          piece(kColL2, sY2, false, sZ2, false, kIdKK128, h, 4 * h, 4 * h + 4);
          if (h == 1) umma::mma_commit(cb2);
        }
        __syncwarp();
        FRACSSM_MARK(3, 4 + 4 * h)
      }
      // Sacc[m,r] = sum_k (Khi + Klo)[k,m] u[k,r]: the tile's own contribution to the state
      // (fK completes once per half.  Its first completion of this tile is known to have happened:
      // the workers arrive on it before they arrive on fA for the second half, which was waited for
      // above.  Waiting for it here again could miss it: once BOTH completions are in, the barrier's
      // parity is back where it started.)
      FRACSSM_WAIT(fK, 1);
      FRACSSM_WAIT(barU, n);
      FRACSSM_MARK(3, 9)
      umma::tc_fence_after();
      if (umma::elect_one()) {
        piece(kColS, sKhi, true, sU, true, kIdMnMn64, 0u, 0, 8);
        piece(kColS, sKlo, true, sU, true, kIdMnMn64, 1u, 0, 8);
        umma::mma_commit(cbK);
      }
      __syncwarp();
      FRACSSM_MARK(3, 10)
      // H = Chat S (both split into bf16 high and low parts, low x low dropped: with single bf16
      // roundings the output misses its tolerance where large terms cancel) ...
      FRACSSM_WAIT(fS, n);
      FRACSSM_MARK(3, 11)
      umma::tc_fence_after();
      if (umma::elect_one()) {
        piece(kColH, sChi, false, sS, true, kIdKMn64, 0u, 0, 8);           // Chat(high) S(high)
        piece(kColH, sClo, false, sS, true, kIdKMn64, 1u, 0, 8);           // Chat(low)  S(high)
        piece(kColH, sChi, false, sS + kAtom, true, kIdKMn64, 1u, 0, 8);   // Chat(high) S(low)
      }
      __syncwarp();
      // ... + W u
      FRACSSM_WAIT(fW, n);
      FRACSSM_MARK(3, 12)
      umma::tc_fence_after();
      if (umma::elect_one()) {
        piece(kColH, sW, false, sU, true, kIdKMn64, 1u, 0, 8);
        umma::mma_commit(barH);
      }
      __syncwarp();
      FRACSSM_MARK(3, 13)
      __syncwarp();
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
    // operand-tile addressing of this thread inside one half (64 modes = one 64-column atom) of a row:
    // modes 2*lane, 2*lane+1 -> 16-byte chunk lane / 4, bytes 4 * (lane % 4); the half, the row group
    // and the row inside it are added per store (emit_pair)
    const uint32_t th_fix = ((lane >> 2) << 4) + ((lane & 3) << 2);
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>(32 * Q) << 16);
    const uint32_t seg_s = sb + kOffSeg + 8 * lane;  // this lane's two modes of segment 0, half 0
    const float kNaN = __int_as_float(0x7fc00000);
#ifdef FRACSSM_PHASE_PROF
    const int pslot = w == 0 ? 0 : w == 5 ? 1 : w == 15 ? 2 : -1;
#endif

    FRACSSM_WAIT(item_bar, 0);
    int item = items[0];
    __syncwarp();
    if (lane == 0) umma::mbar_arrive(read_bar);
    int prev_bh = 0, prev_t0 = 0;
    // 32-byte accesses of the output stage need 32-byte aligned rows (a row is 128 bytes: the bases decide)
    const bool io32 = ((LAYER ? (reinterpret_cast<uintptr_t>(a.u) | reinterpret_cast<uintptr_t>(a.gate))
                              : reinterpret_cast<uintptr_t>(a.h)) & 31) == 0;
    // Output rows of the previous tile (its H accumulator is complete when barH fires).  It runs in
    // the middle of the next tile's first phase, which so overlaps the output MMAs.
    auto write_rows = [&](uint32_t n_done) {
      const int t = prev_t0 + 32 * Q + lane;
      if constexpr (!LAYER) {
        FRACSSM_WAIT(barH, n_done);
        umma::tc_fence_after();
        const bool bad = *failed != 0;
        uint4 *dst = reinterpret_cast<uint4 *>(a.h + (static_cast<int64_t>(prev_bh) * a.L + t) * kR + 16 * P);
        float acc[16];
        umma::tmem_ld16(lane_addr + kColH + 16 * P, acc);
        umma::tmem_ld_wait();
        if (t < a.L) {
          uint4 o0, o1;
          if (bad) {
#pragma unroll
            for (int x = 0; x < 16; ++x) acc[x] = kNaN;
          }
          o0.x = pack2(acc[0], acc[1]); o0.y = pack2(acc[2], acc[3]); o0.z = pack2(acc[4], acc[5]); o0.w = pack2(acc[6], acc[7]);
          o1.x = pack2(acc[8], acc[9]); o1.y = pack2(acc[10], acc[11]); o1.z = pack2(acc[12], acc[13]); o1.w = pack2(acc[14], acc[15]);
          // one 32-byte store per row where the rows are 32-byte aligned: a lane's 32 bytes are one
          // sector, and two 16-byte stores made the warp touch its 32 lines twice
          if (io32) {
            stg_stream_32B(dst, o0, o1);
          } else {
            __stcs(dst, o0);
            __stcs(dst + 1, o1);
          }
        }
      } else {
        // layer mode: skip connection, gate and the partial sum of squares, 8 columns at a time; the
        // row's u and gate values are requested before the wait for the accumulator
        const int b = prev_bh / a.H, head = prev_bh - b * a.H;
        const bool live = t < a.L;
        const int64_t urow = (static_cast<int64_t>(prev_bh) * a.L + t) * kR + 16 * P;
        const int64_t grow = ((static_cast<int64_t>(b) * a.L + t) * a.H + head) * kR + 16 * P;
        uint4 uv[2] = {}, gv[2] = {};
        if (live) {
          const uint4 *up = reinterpret_cast<const uint4 *>(a.u + urow), *gp = reinterpret_cast<const uint4 *>(a.gate + grow);
          if (io32) {
            ldg_stream_32B(up, uv[0], uv[1]);
            ldg_stream_32B(gp, gv[0], gv[1]);
          } else {
            uv[0] = __ldcs(up); uv[1] = __ldcs(up + 1);
            gv[0] = __ldcs(gp); gv[1] = __ldcs(gp + 1);
          }
        }
        FRACSSM_WAIT(barH, n_done);
        umma::tc_fence_after();
        const bool bad = *failed != 0;
        float ss = 0.f;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          float acc[8];
          umma::tmem_ld8(lane_addr + kColH + 16 * P + 8 * half, acc);
          umma::tmem_ld_wait();
          const float4 d0 = __ldg(reinterpret_cast<const float4 *>(a.D + head * kR + 16 * P + 8 * half));
          const float4 d1 = __ldg(reinterpret_cast<const float4 *>(a.D + head * kR + 16 * P + 8 * half + 4));
          const float dv[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
          const uint32_t uw[4] = {uv[half].x, uv[half].y, uv[half].z, uv[half].w};
          const uint32_t gw[4] = {gv[half].x, gv[half].y, gv[half].z, gv[half].w};
          uint32_t o[4];
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            float v[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const float uf = __uint_as_float(e ? (uw[x] & 0xFFFF0000u) : (uw[x] << 16));
              const float z = __uint_as_float(e ? (gw[x] & 0xFFFF0000u) : (gw[x] << 16)) + a.gate_bias;
              const float mixed = fmaf(uf, dv[2 * x + e], acc[2 * x + e]);
              v[e] = bad ? kNaN : mixed * __fdividef(z, 1.f + __expf(-z));
              ss = fmaf(v[e], v[e], ss);
            }
            o[x] = pack2(v[0], v[1]);
          }
          if (live) __stcs(reinterpret_cast<uint4 *>(a.gated + grow) + half, make_uint4(o[0], o[1], o[2], o[3]));
        }
        if (live) a.ss[((static_cast<int64_t>(b) * a.L + t) * a.H + head) * 4 + P] = ss;
      }
      umma::tc_fence_before();
    };

    // The raw inputs of one half of the modes live in registers from their request to their use:
    // half 0 of an item is requested during the second part of the previous tile, half 1 during
    // half 0's own pass, right after half 0's registers have been used.
    RawHalf<CKF32> raw;
    if (item < a.total) {
      const int j0 = item / a.BH;
#pragma unroll
      for (int i = 0; i < 8; ++i) load_tok(raw, a, item - j0 * a.BH, (j0 + a.first_tile) * kTile, w, lane, 0, i);
    }
    uint32_t n_tiles_done = 0;
    for (uint32_t n = 0; item < a.total; ++n, ++n_tiles_done) {
      const int j = item / a.BH, bh = item - j * a.BH;
      const int jt = j + a.first_tile;
      const int t0 = jt * kTile;
      FRACSSM_MARK(pslot, 0)
      float gt_row = 0.f;   // decay of the whole tile for the mode this thread owns in the state update
      const int m_row = 32 * Q + lane;
      float sj[16];         // incoming state: row m_row, columns 16 P .. 16 P + 15
      auto load_state = [&]() {
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
      };

#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t half_off = h * kAtom + th_fix;
        // ---- segment products, the base tiles and the per-token factors cp / ks of this half:
        //   cp[i] = c[i] * (decay from the segment's start to token i, inclusive)
        //   ks[i] = kappa[i] * (decay after token i to the segment's end)
        f2 cp[8], ks[8], g8;
        {
          const uint32_t rowsA = sb + kOffA0 + half_off + w * 1024;   // B0 is the next slot
          f2 g4a, g4b;
          {
            // tokens 0..3: reference point just after token 3
            const f2 r0 = floor2(raw.r[0]), r1 = floor2(raw.r[1]), r2 = floor2(raw.r[2]), r3 = floor2(raw.r[3]);
            const f2 c0 = ck_wide(raw.c[0]), c1 = ck_wide(raw.c[1]), c2 = ck_wide(raw.c[2]), c3 = ck_wide(raw.c[3]);
            const f2 k0 = ck_wide(raw.k[0]), k1 = ck_wide(raw.k[1]), k2 = ck_wide(raw.k[2]), k3 = ck_wide(raw.k[3]);
            const f2 q1 = mul2(r3, r2), q0 = mul2(q1, r1);                   // decay after token i up to token 3
            const f2 p1 = mul2(r0, r1), p2 = mul2(p1, r2), p3 = mul2(p2, r3);
            const f2 iq0 = rcp2(q0), iq1 = mul2(iq0, r1), iq2 = mul2(iq1, r2);
            g4a = p3;
            const f2 b0 = mul2(k0, q0), b1 = mul2(k1, q1), b2 = mul2(k2, r3);
            emit_pair(rowsA, 0, cvt_bf2(mul2(c0, iq0)));
            emit_pair(rowsA, 1, cvt_bf2(mul2(c1, iq1)));
            emit_pair(rowsA, 2, cvt_bf2(mul2(c2, iq2)));
            emit_pair(rowsA, 3, cvt_bf2(c3));
            emit_pair_next_slot(rowsA, 0, cvt_bf2(b0));
            emit_pair_next_slot(rowsA, 1, cvt_bf2(b1));
            emit_pair_next_slot(rowsA, 2, cvt_bf2(b2));
            emit_pair_next_slot(rowsA, 3, cvt_bf2(k3));
            cp[0] = mul2(c0, r0); cp[1] = mul2(c1, p1); cp[2] = mul2(c2, p2); cp[3] = mul2(c3, p3);
            ks[0] = b0; ks[1] = b1; ks[2] = b2; ks[3] = k3;   // times g4b, below
          }
          {
            // tokens 4..7: reference point just before token 4
            const f2 r4 = floor2(raw.r[4]), r5 = floor2(raw.r[5]), r6 = floor2(raw.r[6]), r7 = floor2(raw.r[7]);
            const f2 c4 = ck_wide(raw.c[4]), c5 = ck_wide(raw.c[5]), c6 = ck_wide(raw.c[6]), c7 = ck_wide(raw.c[7]);
            const f2 k4 = ck_wide(raw.k[4]), k5 = ck_wide(raw.k[5]), k6 = ck_wide(raw.k[6]), k7 = ck_wide(raw.k[7]);
            const f2 q5 = mul2(r4, r5), q6 = mul2(q5, r6), q7 = mul2(q6, r7);  // decay from token 4 to token i
            const f2 s5 = mul2(r7, r6), s4 = mul2(s5, r5);                      // decay after token i to token 7
            const f2 iq7 = rcp2(q7), iq6 = mul2(iq7, r7), iq5 = mul2(iq6, r6), iq4 = mul2(iq5, r5);
            g4b = q7;
            const f2 a4 = mul2(c4, r4), a5 = mul2(c5, q5), a6 = mul2(c6, q6), a7 = mul2(c7, q7);
            emit_pair(rowsA, 4, cvt_bf2(a4));
            emit_pair(rowsA, 5, cvt_bf2(a5));
            emit_pair(rowsA, 6, cvt_bf2(a6));
            emit_pair(rowsA, 7, cvt_bf2(a7));
            emit_pair_next_slot(rowsA, 4, cvt_bf2(mul2(k4, iq4)));
            emit_pair_next_slot(rowsA, 5, cvt_bf2(mul2(k5, iq5)));
            emit_pair_next_slot(rowsA, 6, cvt_bf2(mul2(k6, iq6)));
            emit_pair_next_slot(rowsA, 7, cvt_bf2(mul2(k7, iq7)));
            cp[4] = mul2(a4, g4a); cp[5] = mul2(a5, g4a); cp[6] = mul2(a6, g4a); cp[7] = mul2(a7, g4a);
            ks[4] = mul2(k4, s4); ks[5] = mul2(k5, s5); ks[6] = mul2(k6, r7); ks[7] = k7;
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) ks[i] = mul2(ks[i], g4b);
          g8 = mul2(g4a, g4b);
          asm volatile("st.shared.b64 [%0], %1;" ::"r"(seg_s + h * 4096 + w * 256), "l"(g8) : "memory");
        }
        FRACSSM_MARK(pslot, 1 + 10 * h)
        warp_arrive(fA, lane);
        // The other half's inputs (or, in the second pass, nothing: the next item's first half is
        // requested in the tile's last part) are requested now that this half's registers are free.
        // (two token rows at a time, between phases: measured faster than one batch)
        // (in two batches of four token rows: one batch, and four batches of two, measured slower)
        auto request_other_half = [&](auto i) {
          if (h == 0) {
            load_tok2<CKF32, RAGGED, decltype(i)::value>(raw, a, bh, t0, w, lane, 1);
            load_tok2<CKF32, RAGGED, decltype(i)::value + 2>(raw, a, bh, t0, w, lane, 1);
          }
        };
        request_other_half(std::integral_constant<int, 0>{});
        umma::named_barrier(1, kWorkers);  // segment products visible to every worker
        FRACSSM_MARK(pslot, 2 + 10 * h)
        if (h == 0 && n > 0) write_rows(n - 1);  // also: every MMA of the previous tile is done, slots 2..5 are free
        request_other_half(std::integral_constant<int, 4>{});
        FRACSSM_MARK(pslot, 3 + 10 * h)

        // ---- products of whole segments: back from this segment to the start of its 16 / 32 / 64 /
        // 128-token block (bk), forward from it to the end of that block (fw).  A level uses bk when
        // this segment sits in the second half of the level's block (A role), else fw (B role).  The
        // products grow level by level, interleaved with the levels' operand rows.
        f2 bk = one2(), fw = one2();
        const uint32_t seg_h = seg_s + h * 4096;
        auto mulseg = [&](f2 &acc, int s) {
          f2 x;
          asm volatile("ld.shared.b64 %0, [%1];" : "=l"(x) : "r"(seg_h + s * 256));
          acc = mul2(acc, x);
        };
        // One sibling level: this segment's 8 rows go to the A-role or the B-role tile of its stack.
        auto emit_level = [&](uint32_t rows_s, const f2 (&src)[8], f2 sig, bool scale) {
#pragma unroll
          for (int i = 0; i < 8; ++i) emit_pair(rows_s, i, cvt_bf2(scale ? mul2(src[i], sig) : src[i]));
        };
        // ---- levels 8 (rows 0..63 of the stack) and 16 (rows 64..127) -> slots 2 / 3
        {
          const uint32_t rg8 = w >> 1, rg16 = 8 + (((w >> 2) << 1) | (w & 1));
          if (w & 1) emit_level(sb + kOffY1 + half_off + rg8 * 1024, cp, bk, false);
          else emit_level(sb + kOffZ1 + half_off + rg8 * 1024, ks, bk, false);
          if (w & 1) mulseg(bk, w - 1); else mulseg(fw, w + 1);
          if (w & 2) emit_level(sb + kOffY1 + half_off + rg16 * 1024, cp, bk, true);
          else emit_level(sb + kOffZ1 + half_off + rg16 * 1024, ks, fw, true);
        }
        warp_arrive(fL1, lane);
        // ---- levels 32 (rows 64..127) and 64 (rows 0..63) -> slots 4 / 5
        {
          const uint32_t rg64 = w & 7, rg32 = 8 + (((w >> 3) << 2) | (w & 3));
          const int b4 = w & ~3, b8 = w & ~7;
          if (w & 2) { mulseg(bk, b4); mulseg(bk, b4 + 1); } else { mulseg(fw, b4 + 2); mulseg(fw, b4 + 3); }
          if (w & 4) emit_level(sb + kOffY2 + half_off + rg32 * 1024, cp, bk, true);
          else emit_level(sb + kOffZ2 + half_off + rg32 * 1024, ks, fw, true);
          if (w & 4) {
#pragma unroll
            for (int s = 0; s < 4; ++s) mulseg(bk, b8 + s);
          } else {
#pragma unroll
            for (int s = 4; s < 8; ++s) mulseg(fw, b8 + s);
          }
          if (w & 8) emit_level(sb + kOffY2 + half_off + rg64 * 1024, cp, bk, true);
          else emit_level(sb + kOffZ2 + half_off + rg64 * 1024, ks, fw, true);
        }
        warp_arrive(fL, lane);
        FRACSSM_MARK(pslot, 4 + 10 * h)
        // to the tile's start (bk becomes E) and end (fw becomes F)
        if (w & 8) {
#pragma unroll
          for (int s = 0; s < 8; ++s) mulseg(bk, s);
        } else {
#pragma unroll
          for (int s = 8; s < 16; ++s) mulseg(fw, s);
        }
        // Every warp holds the tile's decay for all 64 modes of this half, two per lane; this thread
        // needs the one of mode m = 32 Q + lane, which lies in half Q / 2.
        {
          float g0, g1;
          un2(mul2(mul2(bk, g8), fw), g0, g1);
          const int src = (32 * (Q & 1) + lane) >> 1;
          g0 = __shfl_sync(0xffffffffu, g0, src);
          g1 = __shfl_sync(0xffffffffu, g1, src);
          if (h == (Q >> 1)) gt_row = (lane & 1) ? g1 : g0;
        }
        FRACSSM_MARK(pslot, 5 + 10 * h)

        // ---- Khat = ks * (decay to the tile's end), high and low parts -> slots 0 / 1 (this half's
        // base product done)
        FRACSSM_WAIT(cb0, h);
        FRACSSM_MARK(pslot, 6 + 10 * h)
        {
          const uint32_t rowsH = sb + kOffKhi + half_off + w * 1024;   // the low part is the next slot
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const f2 kf = mul2(ks[i], fw);
            const uint32_t hi = cvt_bf2(kf);
            emit_pair(rowsH, i, hi);
            emit_pair_next_slot(rowsH, i, cvt_bf2(sub2(kf, widen_bf2(hi))));
          }
        }
        // ---- Chat = cp * (decay from the tile's start) -> slots 2 / 3 (this half's level-8/16 product done)
        FRACSSM_WAIT(cbL, h);
        FRACSSM_MARK(pslot, 7 + 10 * h)
        {
          const uint32_t rowsH = sb + kOffChi + half_off + w * 1024;   // the low part is the next slot
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const f2 cf = mul2(cp[i], bk);
            const uint32_t hi = cvt_bf2(cf);
            emit_pair(rowsH, i, hi);
            emit_pair_next_slot(rowsH, i, cvt_bf2(sub2(cf, widen_bf2(hi))));
          }
        }
        warp_arrive(fK, lane);
        FRACSSM_MARK(pslot, 8 + 10 * h)
      }

      // the next item (published by the control warp at the start of this tile); it must be read
      // here, before this warp's arrivals on fS / fW let the control warp move on and publish again.
      // The first half of its inputs is requested now and arrives while the tile finishes.
      FRACSSM_WAIT(item_bar, n + 1);
      const int next = items[(n + 1) & 1];
      __syncwarp();
      if (lane == 0) umma::mbar_arrive(read_bar);
      const bool more = next < a.total;
      const int nj = more ? next / a.BH : 0;
      const int nbh = next - nj * a.BH, nt0 = (nj + a.first_tile) * kTile;
      auto request_next = [&](auto i) {   // four token rows of the next item's first half
        if (more) {
          load_tok2<CKF32, RAGGED, decltype(i)::value>(raw, a, nbh, nt0, w, lane, 0);
          load_tok2<CKF32, RAGGED, decltype(i)::value + 2>(raw, a, nbh, nt0, w, lane, 0);
        }
      };
      request_next(std::integral_constant<int, 0>{});

      auto w_epilogue = [&]() {
      // ---- W -> slot 4: each block of accumulators goes to its place, 8 columns at a time
      umma::tc_fence_after();
      {
        const uint32_t sW = sb + kOffW;
        // 8 accumulators of row t, columns 8 kc .. 8 kc + 7 of W, as one 16-byte store
        auto put8 = [&](int t, int kc, const float (&v)[8]) {
          uint4 pk;
          pk.x = pack2(v[0], v[1]); pk.y = pack2(v[2], v[3]); pk.z = pack2(v[4], v[5]); pk.w = pack2(v[6], v[7]);
          const uint32_t addr = sW + (kc >> 3) * kAtom + t * 128 + (((kc & 7) ^ (t & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pk.x), "r"(pk.y), "r"(pk.z), "r"(pk.w)
                       : "memory");
        };
        // (each role reads its accumulator columns with ONE tcgen05.ld and one wait)
        auto slice8 = [&](const float (&v)[32], int e, float (&o)[8]) {
#pragma unroll
          for (int x = 0; x < 8; ++x) o[x] = v[8 * e + x];
        };
        // of the warp's 32 accumulator rows, row group g (8 rows) owns the g-th block of 8 columns
        auto own_block = [&](uint32_t col0, float (&o)[8]) {
          const int grp = lane >> 3;
          float v[32];
          umma::tmem_ld32(lane_addr + col0, v);
          umma::tmem_ld_wait();
#pragma unroll
          for (int x = 0; x < 8; ++x) {
            const float lo = (grp & 1) ? v[8 + x] : v[x], hi = (grp & 1) ? v[24 + x] : v[16 + x];
            o[x] = (grp & 2) ? hi : lo;
          }
        };
        if (P == 0) {
          // base: row t = 32 Q + lane, its own segment's 8 columns, masked above the diagonal
          float o[8];
          own_block(kColBase + 32 * Q, o);
#pragma unroll
          for (int x = 0; x < 8; ++x) o[x] = x <= (lane & 7) ? o[x] : 0.f;
          put8(32 * Q + lane, 4 * Q + (lane >> 3), o);
        } else if (Q < 2) {
          if (P == 1) {
            // level 8: accumulator row 32 Q + lane is token 64 Q + 16 (lane / 8) + 8 + lane % 8; its
            // partner segment is the one before it
            float o[8];
            own_block(kColL1 + 32 * Q, o);
            put8(64 * Q + 16 * (lane >> 3) + 8 + (lane & 7), 8 * Q + 2 * (lane >> 3), o);
          } else {
            // level 64: accumulator row 32 Q + lane is token 64 + 32 Q + lane; columns = tokens 0..63
            float v[32];
            umma::tmem_ld32(lane_addr + kColL2 + 32 * (P - 2), v);
            umma::tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float b[8];
              slice8(v, e, b);
              put8(64 + 32 * Q + lane, 4 * (P - 2) + e, b);
            }
          }
        } else {
          const int q2 = Q - 2;
          if (P == 1) {
            // level 16: accumulator row 64 + 32 q2 + lane is token 64 q2 + 32 (lane / 16) + 16 + lane % 16;
            // its partners are the 16 tokens before its 16-token half
            const int t = 64 * q2 + 32 * (lane >> 4) + 16 + (lane & 15);
            float v[32];
            umma::tmem_ld32(lane_addr + kColL1 + 64 + 32 * q2, v);
            umma::tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              float b0[8];
#pragma unroll
              for (int x = 0; x < 8; ++x) b0[x] = (lane >> 4) ? v[16 + 8 * e + x] : v[8 * e + x];
              put8(t, 8 * q2 + 4 * (lane >> 4) + e, b0);
            }
          } else {
            // level 32: accumulator row 64 + 32 q2 + lane is token 64 q2 + 32 + lane; partners: the 32
            // tokens before its half
            float v[16];
            umma::tmem_ld16(lane_addr + kColL2 + 64 + 32 * q2 + 16 * (P - 2), v);
            umma::tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              float b[8];
#pragma unroll
              for (int x = 0; x < 8; ++x) b[x] = v[8 * e + x];
              put8(64 * q2 + 32 + lane, 8 * q2 + 2 * (P - 2) + e, b);
            }
          }
        }
        request_next(std::integral_constant<int, 4>{});
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
      FRACSSM_MARK(pslot, 24)
      };
      // ---- the chain: incoming state -> MMA operand (high | low) -> outgoing state
      FRACSSM_WAIT(state_bar, n);
      load_state();
      FRACSSM_WAIT(cb2, n);  // levels 64+32 product done: slots 4 / 5 are free, its accumulators complete
      FRACSSM_MARK(pslot, 20)
      // the incoming state as the MMA operand [high | low] of H = Chat S
      auto state_operand = [&]() {
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
        FRACSSM_MARK(pslot, 21)
      };
      // S_next = Gt * S + Sacc, stored for the next tile of the row (or as the final state)
      auto state_update = [&]() {
        FRACSSM_WAIT(cbK, n);  // Khat(high) and Khat(low) MMAs: Sacc is complete
        umma::tc_fence_after();
        FRACSSM_MARK(pslot, 22)
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
        umma::tc_fence_before();
        __syncwarp();
        if (lane == 0) umma::mbar_arrive(out_bar);  // the chain warp releases the row counter
        FRACSSM_MARK(pslot, 23)
      };
      // The outgoing state goes first when its own part (Sacc) is already complete: that is the case
      // when the tile had to wait for the incoming state, i.e. when the row's chain of tiles is what
      // limits the run; otherwise the operand goes first and the MMA warp gets to work earlier.
      const bool chain_first = __shfl_sync(0xffffffffu, umma::mbar_test(cbK, n & 1u) ? 1 : 0, 0) != 0;
      if (chain_first) {
        state_update();
        state_operand();
      } else {
        state_operand();
        state_update();
      }

      w_epilogue();


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
                         int64_t M, int64_t T, void *stream, int first_tile, unsigned long long wait_ns,
                         const ScanLayerOut *layer) {
  (void)T;
  const bool ckf32 = ck_dtype == FRACSSM_F32;
  if (workspace_bytes < scan_fused_workspace_bytes(B, L, R, M, T))
    return fail(FRACSSM_ERR_ARG, "frac_scan: workspace too small");
  // the kernel reads c / kappa / rho and writes h with 8- and 16-byte accesses
  if (((reinterpret_cast<uintptr_t>(u) | reinterpret_cast<uintptr_t>(c) | reinterpret_cast<uintptr_t>(kappa) |
        reinterpret_cast<uintptr_t>(rho) | reinterpret_cast<uintptr_t>(h)) & 15) != 0)
    return fail(FRACSSM_ERR_ARG, "frac_scan: u, c, kappa, rho and h must be 16-byte aligned");
  if (layer && (((reinterpret_cast<uintptr_t>(layer->gate) | reinterpret_cast<uintptr_t>(layer->gated) |
                  reinterpret_cast<uintptr_t>(layer->D)) & 15) != 0 || layer->H < 1 || B % layer->H != 0))
    return fail(FRACSSM_ERR_ARG, "scan_layer: gate, gated and D must be 16-byte aligned and rows = batch * heads");
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
      int prc = prepare(reinterpret_cast<const void *>(&scan_fused_kernel<false, false, false>));
      if (prc == FRACSSM_OK) prc = prepare(reinterpret_cast<const void *>(&scan_fused_kernel<true, false, false>));
      if (prc == FRACSSM_OK) prc = prepare(reinterpret_cast<const void *>(&scan_fused_kernel<false, false, true>));
      if (prc == FRACSSM_OK) prc = prepare(reinterpret_cast<const void *>(&scan_fused_kernel<true, false, true>));
      if (prc == FRACSSM_OK) prc = prepare(reinterpret_cast<const void *>(&scan_fused_kernel<false, true, true>));
      if (prc == FRACSSM_OK) prc = prepare(reinterpret_cast<const void *>(&scan_fused_kernel<true, true, true>));
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
  a.u = reinterpret_cast<const __nv_bfloat16 *>(u);
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
  if (layer) {
    a.gate = reinterpret_cast<const __nv_bfloat16 *>(layer->gate);
    a.D = layer->D;
    a.gated = reinterpret_cast<__nv_bfloat16 *>(layer->gated);
    a.ss = layer->ss;
    a.gate_bias = layer->gate_bias;
    a.H = (int)layer->H;
  }
  CUtensorMap map;
  int rc = make_tmap_bf16_3d(&map, u, kR, (uint64_t)L, (uint64_t)B, kR, kTile);
  if (rc) return rc;
  cudaError_t e = cudaMemsetAsync(ws, 0, kCtrlBytes + align256((size_t)B * 4), (cudaStream_t)stream);
  if (e != cudaSuccess) return fail(FRACSSM_ERR_CUDA, "frac_scan: %s", cudaGetErrorString(e));
  const int grid = a.total < sms ? a.total : sms;
  const cudaStream_t st = (cudaStream_t)stream;
  if (a.gate != nullptr) {
    if (ckf32) scan_fused_kernel<true, true, true><<<grid, kThreads, kSmemBytes, st>>>(a, map);
    else scan_fused_kernel<false, true, true><<<grid, kThreads, kSmemBytes, st>>>(a, map);
  } else {
    const bool ragged = a.L % kTile != 0;
    if (ragged) {
      if (ckf32) scan_fused_kernel<true, false, true><<<grid, kThreads, kSmemBytes, st>>>(a, map);
      else scan_fused_kernel<false, false, true><<<grid, kThreads, kSmemBytes, st>>>(a, map);
    } else {
      if (ckf32) scan_fused_kernel<true, false, false><<<grid, kThreads, kSmemBytes, st>>>(a, map);
      else scan_fused_kernel<false, false, false><<<grid, kThreads, kSmemBytes, st>>>(a, map);
    }
  }
  return check_launch("frac_scan (single-pass kernel)");
}

int scan_fused_launch(const void *u, const void *c, const void *kappa, int ck_dtype, const float *rho,
                      const float *initial_state, void *h, void *final_state, int final_dtype,
                      void *workspace, size_t workspace_bytes, int64_t B, int64_t L, int64_t R,
                      int64_t M, int64_t T, void *stream) {
  return scan_fused_launch_ex(u, c, kappa, ck_dtype, rho, initial_state, h, final_state, final_dtype, workspace,
                              workspace_bytes, B, L, R, M, T, stream, 0, kWaitNs, nullptr);
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

#ifdef FRACSSM_PHASE_PROF
// Diagnostic build only: copies the clock stamps of the last launch to the host.
extern "C" int fracssm_prof_stamps(long long *out, int n) {
  using namespace fracssm;
  if (n != kProfTiles * kProfWarps * kProfMarks) return FRACSSM_ERR_ARG;
  return cudaMemcpyFromSymbol(out, g_prof, sizeof(long long) * n) == cudaSuccess ? FRACSSM_OK : FRACSSM_ERR_CUDA;
}
#endif

// Helpers shared by the single-pass scan kernel and the segment-summary kernel: operand-tile
// emission, packed float pairs, packed rounding, segment products, release/acquire of the per-row
// counters.
// Thread mapping assumed: worker warp w owns token rows 8w..8w+7 of a 128-token tile, lane l owns
// modes 4l..4l+3.
#pragma once

#include "common.cuh"
#include "umma.cuh"

namespace fracssm {
namespace tile {

constexpr int kTile = 128, kR = 64, kM = 128;
constexpr uint32_t kTileBytes = 32768;  // [128 x 128] bf16 operand tile
constexpr uint32_t kAtom = 16384;       // one 64-column block of such a tile
constexpr uint64_t kWaitNs = 2000000000ull;  // default limit of every device-side wait

// ---- two floats in one 64-bit register (sm_100 packed f32x2 arithmetic) --------------------------
using f2 = unsigned long long;
__device__ __forceinline__ f2 mk2(float lo, float hi) {
  f2 d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
  return d;
}
__device__ __forceinline__ void un2(f2 v, float &lo, float &hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f2 mul2(f2 a, f2 b) {
  f2 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f2 sub2(f2 a, f2 b) {
  f2 d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f2 one2() { return mk2(1.f, 1.f); }
// approximate reciprocal of both halves (inputs here are >= 1e-24, results <= 1e24)
__device__ __forceinline__ f2 rcp2(f2 v) {
  float lo, hi;
  un2(v, lo, hi);
  asm("rcp.approx.ftz.f32 %0, %0;" : "+f"(lo));
  asm("rcp.approx.ftz.f32 %0, %0;" : "+f"(hi));
  return mk2(lo, hi);
}
// both halves rounded to bf16, packed (low half = first element)
__device__ __forceinline__ uint32_t cvt_bf2(f2 v) {
  float lo, hi;
  un2(v, lo, hi);
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
// a packed bf16 pair widened back to two floats
__device__ __forceinline__ f2 widen_bf2(uint32_t p) {
  return mk2(__uint_as_float(p << 16), __uint_as_float(p & 0xFFFF0000u));
}
// two packed floats from shared memory in one access
__device__ __forceinline__ void lds_f2x2(uint32_t saddr, f2 &a, f2 &b) {
  asm volatile("ld.shared.v2.b64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "r"(saddr));
}

// Product of the segment decays seg[lo..hi) for this lane's four modes (as two packed pairs).
__device__ __forceinline__ void seg_prod(const float *seg, int lo, int hi, int lane, float2 (&out)[2]) {
  out[0] = out[1] = make_float2(1.f, 1.f);
  for (int s = lo; s < hi; ++s) {
    const float4 g = *reinterpret_cast<const float4 *>(seg + s * kM + 4 * lane);
    out[0] = __fmul2_rn(out[0], make_float2(g.x, g.y));
    out[1] = __fmul2_rn(out[1], make_float2(g.z, g.w));
  }
}

// Store four consecutive modes of token row 8*w + i of an operand tile (32-bit shared address).
// th_off = this thread's fixed part of the swizzled offset, c16 = its 16-byte chunk index << 4.
__device__ __forceinline__ void emit_row(uint32_t tile_s, uint32_t th_off, uint32_t c16, int i, float2 v0,
                                         float2 v1) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v0.x, v0.y), b = __floats2bfloat162_rn(v1.x, v1.y);
  const uint32_t addr = tile_s + th_off + i * 128 + (c16 ^ (static_cast<uint32_t>(i) << 4));
  asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(*reinterpret_cast<const uint32_t *>(&a)),
               "r"(*reinterpret_cast<const uint32_t *>(&b))
               : "memory");
}
// Store four consecutive modes that are already packed bf16 pairs (no second conversion).
__device__ __forceinline__ void emit_row_packed(uint32_t tile_s, uint32_t th_off, uint32_t c16, int i, uint32_t w0,
                                                uint32_t w1) {
  const uint32_t addr = tile_s + th_off + i * 128 + (c16 ^ (static_cast<uint32_t>(i) << 4));
  asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(w0), "r"(w1) : "memory");
}
// The same store with the row group folded into `rows_s` (= tile + 1024 * row group + the thread's
// fixed offset, whose bits 4..6 hold the thread's chunk index): the swizzle is one XOR per row.
__device__ __forceinline__ void emit_words(uint32_t rows_s, int i, uint32_t w0, uint32_t w1) {
  const uint32_t addr = (rows_s ^ (static_cast<uint32_t>(i) << 4)) + i * 128;
  asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(w0), "r"(w1) : "memory");
}
// Half of such a store: the packed pair of modes 2 hf, 2 hf + 1 of the thread's four.
__device__ __forceinline__ void emit_word(uint32_t rows_s, int i, int hf, uint32_t w0) {
  const uint32_t addr = (rows_s ^ (static_cast<uint32_t>(i) << 4)) + i * 128 + 4 * hf;
  asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(w0) : "memory");
}
// Both components rounded to bf16: the packed pair, and the same values as floats.
__device__ __forceinline__ float2 bf16_round2(float2 v, uint32_t &packed) {
  const __nv_bfloat162 t = __floats2bfloat162_rn(v.x, v.y);
  packed = *reinterpret_cast<const uint32_t *>(&t);
  return make_float2(__uint_as_float(packed << 16), __uint_as_float(packed & 0xFFFF0000u));
}
__device__ __forceinline__ float2 bf16_round2(float2 v) {  // each component rounded to bf16, as floats
  const __nv_bfloat162 t = __floats2bfloat162_rn(v.x, v.y);
  const uint32_t u = *reinterpret_cast<const uint32_t *>(&t);
  return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xFFFF0000u));
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  const __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t *>(&t);
}

__device__ __forceinline__ int ld_acquire(const int *p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release(int *p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// bf16 (4 values in a uint2) or f32 (a float4) coefficient pieces
__device__ __forceinline__ float ck_get(const uint2 &v, int q) {
  const uint32_t wd = (q < 2) ? v.x : v.y;
  return __uint_as_float((q & 1) ? (wd & 0xFFFF0000u) : (wd << 16));
}
__device__ __forceinline__ float ck_get(const float4 &v, int q) {
  return q == 0 ? v.x : q == 1 ? v.y : q == 2 ? v.z : v.w;
}
// the same four values as two packed float pairs
__device__ __forceinline__ void ck_pairs(const uint2 &v, f2 (&out)[2]) {
  out[0] = widen_bf2(v.x);
  out[1] = widen_bf2(v.y);
}
__device__ __forceinline__ void ck_pairs(const float4 &v, f2 (&out)[2]) {
  out[0] = mk2(v.x, v.y);
  out[1] = mk2(v.z, v.w);
}

// One arrival per warp on a "full" barrier: every lane's shared-memory writes are fenced for
// the async proxy and its TMEM reads are ordered before the control warp's next MMAs.
__device__ __forceinline__ void warp_arrive(uint64_t *bar, int lane) {
  umma::fence_async_smem();
  umma::tc_fence_before();
  __syncwarp();
  if (lane == 0) umma::mbar_arrive(bar);
}

}  // namespace tile
}  // namespace fracssm

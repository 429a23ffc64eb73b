// Shared declarations of the tensor-core gated-delta kernels (forward: gdn_tc.cu,
// backward: gdn_tc_bwd.cu).
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "umma_tiles.cuh"

namespace mxb {

// [B,T,H,D] bf16 -> tensor map over (D, H, T, B) with 64 x 64 boxes and 128-byte swizzle; false if it cannot be made.
bool make_tma_map_bthd(CUtensorMap* m, const void* base, int B, int T, int H, int D);

namespace tcg {
constexpr int C = 64;     // chunk
constexpr int KD = 128;   // Dk = Dv
constexpr int VS = 64;    // Dv columns per state CTA
constexpr int LDA = 68;   // fp32 row pitch of the 64x64 solve matrix (16-byte aligned rows)
using bf16 = __nv_bfloat16;

struct TcP {
  int B, T, H, n, gate_is_log, save, no_tma;
  int Dk, Dv;    // true widths of q,k and of v,out (multiples of 8 up to KD).  The tiles are always KD wide: the copy
                 // engine zero-fills the columns a narrower tensor does not have and clips them on the way out, so
                 // only the kernels' direct accesses to the fp32 states index with these
  const bf16 *q, *k, *v;
  const float *beta, *gate, *h0;
  bf16* out;
  float* hT;
  const bf16* dO;
  const float* dhT_in;
  bf16 *dq, *dk, *dv;
  float *dbeta, *dgate, *dh0;
  int* status;   // device word: nonzero when a bounded wait gave up
  // workspace, indexed by ci = (b*H+h)*n + chunk
  float* gam;    // [C]
  bf16* Tm;      // [C][C]
  bf16* w;       // [C][KD]
  bf16* u;       // [C][KD]
  bf16* P;       // [C][C]
  // Everything below is stored as the byte image of the blocked shared-memory operand tile it is read into.
  bf16* hs;      // [KD][KD]  state at chunk start   (backward only)
  bf16* vn;      // [C][KD]
  bf16* dhs;     // [KD][KD]  dS at chunk end
  bf16* dvn;     // [C][KD]   -dv_new (the sign the state pass needs as an operand)
};

// Tensor maps of the token-indexed operands: [B,T,H,128] bf16 viewed as (D, H, T, B), boxes of 64 columns x
// 64 time steps with 128-byte swizzle; rows past the end of the sequence are zero-filled by the copy engine.
// o, dq, dk, dv: results written back by tiled stores (rows past the end of the sequence are clipped).
struct alignas(64) RowMaps {
  CUtensorMap k, q, v, dO, o, dq, dk, dv;
};

// Views of a [64][128] tile for tcgen05 and for 16-byte unit access: written by the copy engine with 128-byte
// swizzle (SW = true: two 8 KB slabs of 64 columns) or staged un-swizzled in the blocked layout.
template <bool SW>
__device__ __forceinline__ tc::Tile in_kmajor(const void* ptr) {
  return SW ? tc::kmajor_sw128_tile(ptr, 8192) : tc::kmajor_tile(ptr, KD);
}
template <bool SW>
__device__ __forceinline__ tc::Tile in_mnmajor(const void* ptr) {
  return SW ? tc::mnmajor_sw128_tile(ptr, 8192) : tc::mnmajor_tile(ptr, KD);
}
template <bool SW>
__device__ __forceinline__ uint32_t in_unit(int r, int c8) {
  return SW ? tc::sw128_unit(r, c8) : tc::kmajor_unit(r, c8, KD);
}

__device__ __forceinline__ float log_gate_tc(float g, int gate_is_log) {
  return gate_is_log ? fmaxf(g, kLogGateFloor) : __logf(fmaxf(g, kGateFloor));
}
__device__ __forceinline__ uint4 ldg16(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ void sts16(uint8_t* base, uint32_t off, uint4 v) {
  *reinterpret_cast<uint4*>(base + off) = v;
}
// Staging-loop index u -> (row, 16-byte unit) of a tile with 16 (or 8) units per row, ordered so that the
// eight lanes of one shared-memory write phase fill one contiguous 128-byte row group of the blocked layout
// (no bank conflicts) while each row is still read from global memory in 64-byte pieces.
__device__ __forceinline__ int urow16(int u) { return ((u >> 7) << 3) | (u & 7); }
__device__ __forceinline__ int ucol16(int u) { return (u >> 3) & 15; }
__device__ __forceinline__ int urow8(int u) { return ((u >> 6) << 3) | (u & 7); }
__device__ __forceinline__ int ucol8(int u) { return (u >> 3) & 7; }
__device__ __forceinline__ uint4 zero16() { return make_uint4(0u, 0u, 0u, 0u); }

// Loads 32 fp32 accumulator columns [c0, c0+32) of this thread's TMEM lane.
__device__ __forceinline__ void ld_acc32(uint32_t taddr, int warp, int c0, float (&f)[32]) {
  uint32_t r[32];
  tc::tmem_ld_32x32b_x32(taddr + ((uint32_t)(32 * (warp & 3)) << 16) + (uint32_t)c0, r);
  tc::tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(r[i]);
}
// Two blocks of 32 accumulator columns [c0, c0+32), [c0+32, c0+64) of this thread's TMEM lane, the second load in
// flight while the first block is processed: process(column of the block, values).
template <typename F>
__device__ __forceinline__ void for_acc2x32(uint32_t taddr, int warp, int c0, F&& process) {
  uint32_t r0[32], r1[32];
  const uint32_t base = taddr + ((uint32_t)(32 * (warp & 3)) << 16) + (uint32_t)c0;
  tc::tmem_ld_32x32b_x32(base, r0);
  tc::tmem_ld_wait();
  tc::tmem_ld_32x32b_x32(base + 32u, r1);
  float f[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(r0[i]);
  process(c0, f);
  tc::tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(r1[i]);
  process(c0 + 32, f);
}
// Loads 64 fp32 accumulator columns [0, 64) at taddr of this thread's TMEM lane: both loads in flight, one wait.
__device__ __forceinline__ void ld_acc64(uint32_t taddr, int warp, float (&f)[64]) {
  uint32_t r0[32], r1[32];
  const uint32_t base = taddr + ((uint32_t)(32 * (warp & 3)) << 16);
  tc::tmem_ld_32x32b_x32(base, r0);
  tc::tmem_ld_32x32b_x32(base + 32u, r1);
  tc::tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    f[i] = __uint_as_float(r0[i]);
    f[32 + i] = __uint_as_float(r1[i]);
  }
}
}  // namespace tcg
using namespace tcg;

}  // namespace mxb

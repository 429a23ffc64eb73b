// Shared-memory operand tiles for tcgen05.mma in the two un-swizzled canonical
// layouts, written from registers in 16-byte units (8 bf16).
//
// K-major tile X[R rows][KC cols] (row = M or N index, col = contraction index):
//   byte(r, k) = (r/8)*SBO + (k/8)*128 + (r%8)*16 + (k%8)*2,  SBO = (KC/8)*128, LBO = 128
//   one MMA K-step (16 elements) advances the start address by 256 bytes.
// MN-major tile X[KR rows][MN cols] (row = contraction index, col = M or N index; this is
// the natural row-major layout of an operand whose contraction runs over rows):
//   byte(k, m) = (m/8)*128 + (k/8)*LBO + (k%8)*16 + (m%8)*2,  SBO = 128, LBO = (MN/8)*128
//   one MMA K-step advances the start address by 2*LBO bytes.
#pragma once

#include "tcgen05.cuh"

namespace mxb {
namespace tc {

struct Tile {
  uint32_t saddr;  // shared-memory byte address of the tile
  uint32_t lbo, sbo, kstep;
  int mn_major;
  uint32_t swizzle = kSwizzleNone;
  uint32_t slab_ksteps = 0;   // K-steps per slab (0: the tile is one piece)
  uint32_t slab_stride = 0;   // byte distance between consecutive slabs along K
};

__device__ __forceinline__ Tile kmajor_tile(const void* smem, int kcols) {
  return Tile{smem_u32(smem), 128u, (uint32_t)(kcols / 8) * 128u, 256u, 0};
}
__device__ __forceinline__ Tile mnmajor_tile(const void* smem, int mn) {
  const uint32_t lbo = (uint32_t)(mn / 8) * 128u;
  return Tile{smem_u32(smem), lbo, 128u, 2u * lbo, 1};
}
// Tiles written by TMA with 128-byte swizzle: slabs of [rows][64 bf16] (128-byte rows, 8-row groups
// 1024 bytes apart), slab s holding columns 64 s .. 64 s + 63; slabs are slab_bytes apart and 1024-byte
// aligned.  K-major view: contraction along the columns (4 K-steps of 32 bytes per slab, then the next slab).
__device__ __forceinline__ Tile kmajor_sw128_tile(const void* smem, uint32_t slab_bytes) {
  Tile t{smem_u32(smem), 16u, 1024u, 32u, 0};
  t.swizzle = kSwizzle128;
  t.slab_ksteps = 4;
  t.slab_stride = slab_bytes;
  return t;
}
// MN-major view of the same bytes: contraction along the rows (a K-step = 16 rows = 2048 bytes); the
// 64-column slabs are consecutive blocks of the M/N extent, slab_bytes apart (leading byte offset).
__device__ __forceinline__ Tile mnmajor_sw128_tile(const void* smem, uint32_t slab_bytes) {
  Tile t{smem_u32(smem), slab_bytes, 1024u, 2048u, 1};
  t.swizzle = kSwizzle128;
  return t;
}
// Sub-tile starting at row r0 (multiple of 8) of a K-major tile / at column m0 (multiple
// of 8) of an MN-major tile.
__device__ __forceinline__ Tile kmajor_rows(Tile t, int r0) { t.saddr += (uint32_t)(r0 / 8) * t.sbo; return t; }
__device__ __forceinline__ Tile mnmajor_cols(Tile t, int m0) { t.saddr += (uint32_t)(m0 / 8) * 128u; return t; }
// Skip k0 (multiple of 16) contraction elements.
__device__ __forceinline__ Tile skip_k(Tile t, int k0) { t.saddr += (uint32_t)(k0 / 16) * t.kstep; return t; }

// Byte offset of the 16-byte unit holding elements (r, 8*c8 .. 8*c8+7) of a K-major tile.
__device__ __forceinline__ uint32_t kmajor_unit(int r, int c8, int kcols) {
  return (uint32_t)(r >> 3) * (uint32_t)(kcols / 8) * 128u + (uint32_t)c8 * 128u + (uint32_t)(r & 7) * 16u;
}
// Byte offset of the 16-byte unit holding elements (r, 8*c8 .. 8*c8+7) of a 64-row tile written by TMA with
// 128-byte swizzle (8 KB slabs of 64 columns, 1024-byte aligned): the unit index within a 128-byte row is
// XORed with the row's position in its 8-row group.
__device__ __forceinline__ uint32_t sw128_unit(int r, int c8) {
  return (uint32_t)(c8 >> 3) * 8192u + (uint32_t)r * 128u + (uint32_t)(((c8 & 7) ^ (r & 7)) << 4);
}
// Byte offset of the 16-byte unit holding elements (k, 8*c8 .. 8*c8+7) of an MN-major tile.
__device__ __forceinline__ uint32_t mnmajor_unit(int k, int c8, int mn) {
  return (uint32_t)c8 * 128u + (uint32_t)(k >> 3) * (uint32_t)(mn / 8) * 128u + (uint32_t)(k & 7) * 16u;
}

// D[tmem] (+)= A * B over ktotal contraction elements; one thread issues.
__device__ __forceinline__ void issue_gemm(uint32_t tmem_d, const Tile& a, const Tile& b, int M, int N, int ktotal,
                                           bool accumulate) {
  const uint32_t idesc = make_idesc_bf16(M, N, a.mn_major, b.mn_major);
  const uint64_t da = make_smem_desc(a.saddr, a.lbo, a.sbo, a.swizzle);
  const uint64_t db = make_smem_desc(b.saddr, b.lbo, b.sbo, b.swizzle);
  auto koff = [](const Tile& t, uint32_t ks) {
    return t.slab_ksteps ? (ks / t.slab_ksteps) * t.slab_stride + (ks % t.slab_ksteps) * t.kstep : ks * t.kstep;
  };
  for (int ks = 0; ks < ktotal / 16; ++ks)
    mma_ss(tmem_d, da + (uint64_t)(koff(a, ks) >> 4), db + (uint64_t)(koff(b, ks) >> 4), idesc,
           (accumulate || ks > 0) ? 1u : 0u);
}

// ---- bf16 packing ---------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void unpack_bf16(uint32_t w, float& lo, float& hi) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&w);
  lo = __low2float(v);
  hi = __high2float(v);
}
__device__ __forceinline__ uint4 scale_bf16x8(uint4 v, float s) {
  float a, b;
  uint4 r;
  unpack_bf16(v.x, a, b); r.x = pack_bf16(a * s, b * s);
  unpack_bf16(v.y, a, b); r.y = pack_bf16(a * s, b * s);
  unpack_bf16(v.z, a, b); r.z = pack_bf16(a * s, b * s);
  unpack_bf16(v.w, a, b); r.w = pack_bf16(a * s, b * s);
  return r;
}

}  // namespace tc
}  // namespace mxb

// Gated delta rule, chunked WY/UT form - tensor-core path (tcgen05.mma, TMEM
// accumulators) for bf16 I/O with fp32 state, chunk 64, Dk and Dv up to 128 (tiles are 128 wide; narrower heads ride
// on the copy engine's zero fill and clipping).
//
// Same mathematics as the fp32 path (gdn_simt.cu; reference
// gated_delta_scan_chunked, gpu/ir.cpp:2352-2550).  Every contraction runs as
// tcgen05.mma.kind::f16 on bf16 operands staged in shared memory (token rows by
// TMA in the 128-byte-swizzled layout, workspace tiles as byte images of the
// canonical layouts of umma_tiles.cuh) with fp32 accumulation in tensor memory;
// the triangular inverse, all decay factors, the recurrent state and every
// reduction stay in fp32.
//
//   gdn_tc_prep_kernel       one CTA per chunk (three per SM): [k;q] k^T (M=128), fp32 solve,
//                            (T beta) v and (T beta E(gam)) k (M=64, N=128 each) -> u, w, P, T
//   gdn_tc_state_fwd_kernel  one CTA per (batch, head), sequential over chunks, fp32 state in
//                            registers (thread = state row, 64 columns), operands two chunks ahead:
//                            [w;q] S (M=128) -> v_new, then [0;P] v_new and (r k)^T v_new
#include <cuda.h>

#include <cstring>

#include "gdn_tc.cuh"

namespace mxb {

// ------------------------------------------------------------------ prep
// u = T (v beta) and w = T (k beta E(gam)) are evaluated as (T diag(beta)) v and
// (T diag(beta E(gam))) k: the scaling goes into two column-scaled bf16 copies of T written
// straight from the solve's registers, so k, q and v are staged raw.
//
// A CTA is a chain of dependent steps (copy -> MMA -> epilogue -> solve -> MMA -> epilogue -> stores) that leaves
// the SM idle most of the time, so the kernel is sized for FOUR CTAs per SM: 128 TMEM columns (u and w go through
// the same columns one after the other) and 51 KB of shared memory, every region reused as soon as it is dead:
//   [k;q] (32 KB, two slabs of 64 columns: k box then q box)  ->  v lands in the q boxes once q k^T is done
//                                                              ->  k scaled to diag(d) k in place during the solve
//                                                              ->  u image over v, w image over k
//   A / T fp32 matrix (17 KB): then the bf16 T image on its way out and T diag(beta), the one operand of both
//   products (w = (T diag beta)(diag(d) k)), over it
//   P goes from the accumulator straight to the workspace (a warp's stores fill whole 128-byte lines of the image)
// TMA = true: k, q, v arrive as cp.async.bulk.tensor tiles (boxes of 64 rows x 64 columns, 128-byte
// swizzle; rows past the end of the sequence are zero-filled by the copy engine).  TMA = false: the same
// tiles staged with cp.async into the same swizzled positions (kept as a cross-check and for drivers
// without the tensor-map entry point).
constexpr int kPrepSmem = 32768 + C * LDA * 4 + 3 * C * 4 + 64 + 64 + 1024;
static_assert(C * LDA * 4 >= 2 * 8192, "the T image and T diag(beta) go over the fp32 matrix");
static_assert(4 * (kPrepSmem + 1024) <= 228 * 1024, "four CTAs per SM");

using PrepMaps = RowMaps;

__device__ __forceinline__ uint4 pack8f(const float* e) {
  return make_uint4(tc::pack_bf16(e[0], e[1]), tc::pack_bf16(e[2], e[3]), tc::pack_bf16(e[4], e[5]),
                    tc::pack_bf16(e[6], e[7]));
}

template <bool TMA>
__global__ void __launch_bounds__(128, 4) gdn_tc_prep_kernel(TcP p, const __grid_constant__ PrepMaps maps) {
  extern __shared__ uint8_t raw[];
  uint8_t* sm = raw + ((1024u - (tc::smem_u32(raw) & 1023u)) & 1023u);
  uint8_t* Akq = sm;                    // slab s at 16384 s: k box [64][64], then q box [64][64] (later v, u / w images)
  float* Am = reinterpret_cast<float*>(Akq + 32768);  // [64][LDA]  A, then T in place
  uint8_t* Tt = reinterpret_cast<uint8_t*>(Am);       // [64 i][64 m] T image, over the fp32 matrix once it is dead
  uint8_t* Tb = Tt + 8192;              // [64 i][64 m] T diag(beta), behind it
  float* gam = Am + C * LDA;
  float* bet = gam + C;
  float* dd = bet + C;                  // E(gam)
  uint64_t* mbar = reinterpret_cast<uint64_t*>(dd + C);  // [0] MMA completion, [1] k,q landed, [2] v landed
  uint32_t* tslot = reinterpret_cast<uint32_t*>(mbar + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x, bh = blockIdx.y, b = bh / p.H, h = bh % p.H, t0 = c * C;
  const size_t ci = (size_t)bh * p.n + c;
  auto row = [&](int i) { return ((size_t)(b * p.T + t0 + i) * p.H + h); };
  const int imax = min(C, p.T - t0);
  const uint32_t sAkq = tc::smem_u32(Akq);
  // byte offset in Akq of unit (i, c8) of the k tile; the q (later v) tile sits 8192 bytes further
  auto kq_unit = [](int i, int c8) {
    return (uint32_t)(c8 >> 3) * 16384u + (uint32_t)i * 128u + (uint32_t)(((c8 & 7) ^ (i & 7)) << 4);
  };

  // prologue latencies side by side: warp 0 allocates TMEM, warp 1 reads the gates, one thread of warp 2
  // initialises the barriers and issues the copies that complete on them
  if (tid == 64) {
    tc::mbar_init(&mbar[0], 1);
    tc::mbar_init(&mbar[1], 1);
    tc::mbar_init(&mbar[2], 1);
    tc::mbar_fence_init();
  }
  if (TMA) {
    if (tid == 64) {
      tc::mbar_expect_tx(&mbar[1], 32768);
      for (int sl = 0; sl < 2; ++sl) {
        tc::tma_load_4d(sAkq + sl * 16384, &maps.k, 64 * sl, h, t0, b, &mbar[1]);
        tc::tma_load_4d(sAkq + sl * 16384 + 8192, &maps.q, 64 * sl, h, t0, b, &mbar[1]);
      }
    }
  } else {
    for (int u = tid; u < 64 * 16; u += 128) {
      const int i = urow16(u), c8 = ucol16(u);
      const bool ok = i < imax;
      const size_t g = ok ? row(i) * KD + c8 * 8 : 0;
      tc::cp_async16(sAkq + kq_unit(i, c8), p.k + g, ok);
      tc::cp_async16(sAkq + 8192 + kq_unit(i, c8), p.q + g, ok);
    }
    tc::cp_async_commit();
  }
  if (warp == 0) {
    tc::tmem_alloc(tslot, 128);
    tc::tmem_relinquish();
  }
  if (warp == 1) {  // in-chunk inclusive cumulative sum of the log gate: two elements per lane
    const bool ok0 = 2 * lane < imax, ok1 = 2 * lane + 1 < imax;
    const float g0 = ok0 ? log_gate_tc(p.gate[row(2 * lane)], p.gate_is_log) : 0.f;
    const float g1 = ok1 ? log_gate_tc(p.gate[row(2 * lane + 1)], p.gate_is_log) : 0.f;
    float s = g0 + g1;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, s, o);
      if (lane >= o) s += t;
    }
    const float c1 = s, c0 = s - g1;
    const float b0 = ok0 ? p.beta[row(2 * lane)] : 0.f, b1 = ok1 ? p.beta[row(2 * lane + 1)] : 0.f;
    gam[2 * lane] = c0; gam[2 * lane + 1] = c1;
    bet[2 * lane] = b0; bet[2 * lane + 1] = b1;
    dd[2 * lane] = exp_nonpos(c0); dd[2 * lane + 1] = exp_nonpos(c1);
    p.gam[ci * C + 2 * lane] = c0;
    p.gam[ci * C + 2 * lane + 1] = c1;
  }
  bool ok = true;
  if (TMA) {
    __syncthreads();  // barriers initialised before anyone waits on them
    ok = tc::mbar_wait(&mbar[1], 0);  // [k;q]
  } else {
    tc::cp_async_wait<0>();
  }
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t taddr = *tslot;
  // D0[128 x 64] = [k;q] k^T
  if (tid == 0) {
    const tc::Tile a = tc::kmajor_sw128_tile(Akq, 16384);
    tc::issue_gemm(taddr, a, a, 128, 64, KD, false);  // B = first 64 rows of the same tile
    tc::mma_commit(mbar);
  }
  if (ok) ok = tc::mbar_wait(mbar, 0);
  tc::fence_after_sync();
  // q is dead: v takes its place (needed only for the second MMA, long after the solve)
  if (TMA) {
    if (tid == 64) {
      tc::mbar_expect_tx(&mbar[2], 16384);
      for (int sl = 0; sl < 2; ++sl) tc::tma_load_4d(sAkq + sl * 16384 + 8192, &maps.v, 64 * sl, h, t0, b, &mbar[2]);
    }
  } else {
    for (int u = tid; u < 64 * 16; u += 128) {
      const int i = urow16(u), c8 = ucol16(u);
      const bool okv = i < imax;
      tc::cp_async16(sAkq + 8192 + kq_unit(i, c8), okv ? p.v + row(i) * KD + c8 * 8 : p.v, okv);
    }
    tc::cp_async_commit();
  }
  if (ok) {
    const int i = tid & 63;
    const float gi = gam[i], bi = bet[i];
    for (int c0 = 0; c0 < 64; c0 += 32) {
      float f[32];
      ld_acc32(taddr, warp, c0, f);
      if (tid < 64) {  // A = -(k beta k^T) Gamma, strictly lower
        // all 32 values first, then the stores: a store into A between the loads of gam would pin the order
        // (the compiler must assume the two shared arrays overlap) and the exponentials would run one by one
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) {
          const int j = c0 + jj;
          const float val = -bi * f[jj] * exp_nonpos(gi - gam[j]);
          f[jj] = (j < i) ? val : 0.f;
        }
#pragma unroll
        for (int x = 0; x < 8; ++x)
          *reinterpret_cast<float4*>(Am + i * LDA + c0 + 4 * x) = make_float4(f[4 * x], f[4 * x + 1], f[4 * x + 2], f[4 * x + 3]);
      } else {         // P = (q k^T) Gamma, lower incl. diagonal -> straight into its operand-tile image in the workspace
        uint32_t pk[16];
#pragma unroll
        for (int jj = 0; jj < 32; jj += 2) {
          const int j = c0 + jj;
          const float v0 = f[jj] * exp_nonpos(gi - gam[j]), v1 = f[jj + 1] * exp_nonpos(gi - gam[j + 1]);
          const float x0 = (j <= i) ? v0 : 0.f, x1 = (j + 1 <= i) ? v1 : 0.f;
          pk[jj >> 1] = tc::pack_bf16(x0, x1);
        }
        uint8_t* pimg = reinterpret_cast<uint8_t*>(p.P + ci * C * C);
#pragma unroll
        for (int x = 0; x < 4; ++x)  // eight consecutive rows of a unit column are one 128-byte line of the image
          *reinterpret_cast<uint4*>(pimg + tc::kmajor_unit(i, (c0 >> 3) + x, C)) =
              make_uint4(pk[4 * x], pk[4 * x + 1], pk[4 * x + 2], pk[4 * x + 3]);
      }
    }
  }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  // T = (I - A)^-1 in fp32, in place over A.  The two 32 x 32 diagonal blocks by forward substitution
  // (thread = block and column, the column in registers), then the off-diagonal block
  // T21 = T22 (A21 T11) as two small fp32 products over all 128 threads.
  {
    float Tc[32];
    const int blk = (tid >> 5) & 1, cc = tid & 31, r0 = 32 * blk;
    if (ok && tid < C) {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float* arow = Am + (r0 + i) * LDA + r0;
        float s0 = (i == cc) ? 1.f : 0.f, s1 = 0.f;
#pragma unroll
        for (int j = 0; j + 1 < i; j += 2) {
          s0 = fmaf(arow[j], Tc[j], s0);
          s1 = fmaf(arow[j + 1], Tc[j + 1], s1);
        }
        if (i & 1) s0 = fmaf(arow[i - 1], Tc[i - 1], s0);
        Tc[i] = (i < cc) ? 0.f : s0 + s1;
      }
    } else if (ok) {
      // the other half of the CTA meanwhile turns k into diag(d) k in place (its product with itself is done), so
      // that w = (T diag beta)(diag(d) k) needs no second scaled copy of T
      const int i = tid - C;
      const float di = dd[i];
#pragma unroll
      for (int c8 = 0; c8 < 16; ++c8) {
        uint4* unit = reinterpret_cast<uint4*>(Akq + kq_unit(i, c8));
        *unit = tc::scale_bf16x8(*unit, di);
      }
    }
    __syncthreads();  // every thread has read its block of A
    if (ok && tid < C) {
#pragma unroll
      for (int i = 0; i < 32; ++i) Am[(r0 + i) * LDA + r0 + cc] = Tc[i];
    }
    __syncthreads();
    const int i2 = tid >> 2, jb = (tid & 3) * 8;  // row i2 of the lower-left block, 8 of its columns
    {  // X = A21 T11 -> the unused upper-right block
      float x[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
      for (int k = 0; k < 32; ++k) {
        const float a = Am[(32 + i2) * LDA + k];
        const float4 t0 = *reinterpret_cast<const float4*>(Am + k * LDA + jb);
        const float4 t1 = *reinterpret_cast<const float4*>(Am + k * LDA + jb + 4);
        x[0] = fmaf(a, t0.x, x[0]); x[1] = fmaf(a, t0.y, x[1]); x[2] = fmaf(a, t0.z, x[2]); x[3] = fmaf(a, t0.w, x[3]);
        x[4] = fmaf(a, t1.x, x[4]); x[5] = fmaf(a, t1.y, x[5]); x[6] = fmaf(a, t1.z, x[6]); x[7] = fmaf(a, t1.w, x[7]);
      }
      *reinterpret_cast<float4*>(Am + i2 * LDA + 32 + jb) = make_float4(x[0], x[1], x[2], x[3]);
      *reinterpret_cast<float4*>(Am + i2 * LDA + 32 + jb + 4) = make_float4(x[4], x[5], x[6], x[7]);
    }
    __syncthreads();
    {  // T21 = T22 X -> over A21 (nothing reads A21 any more)
      float y[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
      for (int k = 0; k < 32; ++k) {
        const float a = Am[(32 + i2) * LDA + 32 + k];
        const float4 t0 = *reinterpret_cast<const float4*>(Am + k * LDA + 32 + jb);
        const float4 t1 = *reinterpret_cast<const float4*>(Am + k * LDA + 32 + jb + 4);
        y[0] = fmaf(a, t0.x, y[0]); y[1] = fmaf(a, t0.y, y[1]); y[2] = fmaf(a, t0.z, y[2]); y[3] = fmaf(a, t0.w, y[3]);
        y[4] = fmaf(a, t1.x, y[4]); y[5] = fmaf(a, t1.y, y[5]); y[6] = fmaf(a, t1.z, y[6]); y[7] = fmaf(a, t1.w, y[7]);
      }
      *reinterpret_cast<float4*>(Am + (32 + i2) * LDA + jb) = make_float4(y[0], y[1], y[2], y[3]);
      *reinterpret_cast<float4*>(Am + (32 + i2) * LDA + jb + 4) = make_float4(y[4], y[5], y[6], y[7]);
    }
    __syncthreads();
    // the T image and the bf16 operand tile T diag(beta); the upper triangle (it holds X) reads as zero.  Both go
    // over the fp32 matrix: every thread first reads all its rows, then a barrier, then writes.
    uint4 timg[4], tbimg[4];
#pragma unroll
    for (int m = 0; m < 4; ++m) {
      const int u = tid + 128 * m, i = urow8(u), c8 = ucol8(u);
      const float4 a0 = *reinterpret_cast<const float4*>(Am + i * LDA + 8 * c8);
      const float4 a1 = *reinterpret_cast<const float4*>(Am + i * LDA + 8 * c8 + 4);
      float e[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w}, eb[8];
#pragma unroll
      for (int y = 0; y < 8; ++y) {
        const int mm = 8 * c8 + y;
        e[y] = (mm <= i) ? e[y] : 0.f;
        eb[y] = e[y] * bet[mm];
      }
      timg[m] = pack8f(e);
      tbimg[m] = pack8f(eb);
    }
    __syncthreads();
#pragma unroll
    for (int m = 0; m < 4; ++m) {
      sts16(Tt, 16 * (tid + 128 * m), timg[m]);
      sts16(Tb, 16 * (tid + 128 * m), tbimg[m]);
    }
  }
  if (TMA) { if (ok) ok = tc::mbar_wait(&mbar[2], 0); }  // v
  else tc::cp_async_wait<0>();
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  // D1[64 x 128] = (T beta) v -> u     (v contracted over its rows)
  if (ok && tid == 0) {
    tc::issue_gemm(taddr, tc::kmajor_tile(Tb, C), tc::mnmajor_sw128_tile(Akq + 8192, 16384), 64, KD, C, false);
    tc::mma_commit(mbar);
    tc::bulk_store(p.Tm + ci * C * C, tc::smem_u32(Tt), 8192);  // T leaves as the byte image of its operand tile
    tc::bulk_commit();
  }
  if (ok) ok = tc::mbar_wait(mbar, 1);
  tc::fence_after_sync();
  const int ir = 16 * warp + (lane & 15);  // M=64: row m sits in TMEM lane (m%16) + 32*(m/16)
  if (ok) {
    // the u image (un-swizzled K-major layout; rows 0-31 and 32-63 are its two contiguous halves) over the v boxes
    for (int c0 = 0; c0 < 128; c0 += 32) {
      float f[32];
      ld_acc32(taddr, warp, c0, f);
      if (lane < 16) {
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const uint32_t off = tc::kmajor_unit(ir, (c0 >> 3) + x, KD);
          sts16(Akq, 8192u + (off >> 13) * 16384u + (off & 8191u), pack8f(&f[8 * x]));
        }
      }
    }
  }
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();  // the accumulator columns have been read: the second product may overwrite them
  tc::fence_after_sync();
  // D1[64 x 128] = (T beta)(d k) -> w
  if (ok && tid == 0) {
    tc::issue_gemm(taddr, tc::kmajor_tile(Tb, C), tc::mnmajor_sw128_tile(Akq, 16384), 64, KD, C, false);
    tc::mma_commit(mbar);
    for (int hf = 0; hf < 2; ++hf) tc::bulk_store(p.u + ci * C * KD + hf * 4096, sAkq + 8192 + hf * 16384, 8192);
    tc::bulk_commit();
  }
  if (ok) ok = tc::mbar_wait(mbar, 0);
  tc::fence_after_sync();
  if (ok) {
    // the w image in the 128-byte-swizzled layout of a TMA tile (two 8 KB slabs of 64 columns), over the k boxes, so
    // that the state kernels can put it beside TMA-loaded q rows in one operand
    for (int c0 = 0; c0 < 128; c0 += 32) {
      float f[32];
      ld_acc32(taddr, warp, c0, f);
      if (lane < 16) {
#pragma unroll
        for (int x = 0; x < 4; ++x) sts16(Akq, kq_unit(ir, (c0 >> 3) + x), pack8f(&f[8 * x]));
      }
    }
  } else if (tid == 0) {
    atomicExch(p.status, 1);
  }
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  if (tid == 0) {
    if (ok) {
      for (int sl = 0; sl < 2; ++sl) tc::bulk_store(p.w + ci * C * KD + sl * 4096, sAkq + sl * 16384, 8192);
      tc::bulk_commit();
    }
    tc::bulk_wait_read<0>();  // shared memory must outlive the copies
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(taddr, 128);
}

// ------------------------------------------------------------ state forward
// One CTA (256 threads) per (batch, head).  Thread t owns state row kk = t & 127 and the
// 64 columns of half t >> 7.  The operand tiles are double-buffered (buffer c & 1 for chunk c): the operands of
// chunk c+2 are requested as soon as the MMA (or epilogue) that last read the buffer for chunk c has finished, so
// a copy has more than a whole chunk period to land (a chunk takes ~2.5 us, a copy from HBM up to ~1.5 us):
//   group A  [w;q]      buffer free after MMA1      needed before MMA1
//   group U  u          free after epilogue 1       needed before epilogue 1
//   group PK P and k    free after MMA2/MMA3        needed in the shadow of MMA1 (k is scaled in place there)
// Six groups are outstanding at the top of every chunk, in the order A, U, PK (chunk c), A, U, PK (chunk c+1).
//
// TMA = true: q and k rows arrive as tensor-map boxes (128-byte swizzle) issued by ONE thread and complete on the
// barrier of their group, like the images: no thread spends issue slots on copies (four cp.async per thread and
// group cost every thread ~1.6 k and ~1.1 k cycles per chunk, on the critical path between an MMA and its epilogue).
// TMA = false: the same rows by cp.async into the same swizzled positions.
constexpr int kStateFwdSmem = 2 * 32768 + 32768 + 2 * 16384 + 16384 + 16384 + 2 * 16384 + 2 * 16384 + 2 * C * 4 + 128 + 1024;

template <bool TMA>
__global__ void __launch_bounds__(256) gdn_tc_state_fwd_kernel(TcP p, const __grid_constant__ RowMaps maps) {
  extern __shared__ uint8_t raw[];
  uint8_t* sm = raw + ((1024u - (tc::smem_u32(raw) & 1023u)) & 1023u);
  uint8_t* A1 = sm;                 // x2 [128: w rows 0-63, q rows 64-127][128 kk], two swizzled slabs of 64 columns
  uint8_t* Sop = A1 + 2 * 32768;    // [128 kk][128 j]   bf16 copy of the state
  uint8_t* A2 = Sop + 32768;        // x2 [128: zero rows 0-63, P rows 64-127][64 m]
  uint8_t* Vn = A2 + 2 * 16384;     // [64 i][128 j]     v_new
  uint8_t* Ot = Vn + 16384;         // [64 i][128 j]     output tile on its way out (two swizzled slabs)
  uint8_t* A3 = Ot + 16384;         // x2 [64 i][128 kk] k, then diag(E(gam_last-gam_i)) k  (A = k^T), swizzled slabs
  uint8_t* Ut = A3 + 2 * 16384;     // x2 [64 i][128 j]  u
  float* dd = reinterpret_cast<float*>(Ut + 2 * 16384);
  float* rr = dd + C;
  // [0] MMA completion; per buffer: [1 + buf] w image and q rows, [3 + buf] u image, [5 + buf] P image and k rows landed
  uint64_t* mbar = reinterpret_cast<uint64_t*>(rr + C);
  uint32_t* tslot = reinterpret_cast<uint32_t*>(mbar + 8);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int kk = tid & 127, half = tid >> 7, j0 = 64 * half;
  const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H;
  const uint32_t sA1b = tc::smem_u32(A1), sA2b = tc::smem_u32(A2), sA3b = tc::smem_u32(A3), sUb = tc::smem_u32(Ut);
  const uint32_t sOt = tc::smem_u32(Ot);
  constexpr int kOutThread = 96;  // hands the output tiles to the copy engine (its own bulk-group queue)

  auto grow = [&](int c, int i) { return ((size_t)(b * p.T + c * C + i) * p.H + h); };
  // The workspace tiles (w, u, P) are byte images of the operand layout: one bulk copy each, issued by one
  // thread, completing on an mbarrier.  The raw q and k rows come by cp.async.
  // Slab s of A1 (columns 64 s ..): the w slab (rows 0-63), then the q box (rows 64-127).  The issuing threads sit
  // in warps whose epilogue after the issue point is the short one (tid 64: q rows; tid 32: state update).
  auto issue_A = [&](int c) {  // [w;q] of chunk c
    if (c < p.n) {
      const size_t ci = (size_t)bh * p.n + c;
      const uint32_t sA1 = sA1b + (c & 1) * 32768;
      uint64_t* mb = &mbar[1 + (c & 1)];
      if (tid == 64) {
        tc::mbar_expect_tx(mb, TMA ? 32768 : 16384);
        for (int sl = 0; sl < 2; ++sl) {
          tc::bulk_load(sA1 + sl * 16384, p.w + ci * C * KD + sl * 4096, 8192, mb);
          if (TMA) tc::tma_load_4d(sA1 + sl * 16384 + 8192, &maps.q, 64 * sl, h, c * C, b, mb);
        }
      }
      if (!TMA) {
        const int imax = min(C, p.T - c * C);
        for (int u = tid; u < 64 * 16; u += 256) {
          const int i = urow16(u), c8 = ucol16(u);
          const uint32_t off = (uint32_t)(c8 >> 3) * 16384u + 8192u + (uint32_t)i * 128u + (uint32_t)(((c8 & 7) ^ (i & 7)) << 4);
          tc::cp_async16(sA1 + off, i < imax ? p.q + grow(c, i) * KD + c8 * 8 : p.q, i < imax);
        }
      }
    }
    if (!TMA) tc::cp_async_commit();
  };
  auto issue_U = [&](int c) {
    if (c < p.n && tid == 64) {
      const size_t ci = (size_t)bh * p.n + c;
      tc::mbar_expect_tx(&mbar[3 + (c & 1)], 16384);
      tc::bulk_load(sUb + (c & 1) * 16384, p.u + ci * C * KD, 16384, &mbar[3 + (c & 1)]);
    }
    if (!TMA) tc::cp_async_commit();  // (empty: keeps the group count of the schedule below)
  };
  auto issue_PK = [&](int c) {
    if (c < p.n) {
      const size_t ci = (size_t)bh * p.n + c;
      const uint32_t sA2 = sA2b + (c & 1) * 16384, sA3 = sA3b + (c & 1) * 16384;
      uint64_t* mb = &mbar[5 + (c & 1)];
      if (tid == 32) {
        tc::mbar_expect_tx(mb, TMA ? 8192 + 16384 : 8192);
        tc::bulk_load(sA2 + 8192, p.P + ci * C * C, 8192, mb);  // rows 64..127 of the [128][64] tile
        if (TMA)
          for (int sl = 0; sl < 2; ++sl) tc::tma_load_4d(sA3 + sl * 8192, &maps.k, 64 * sl, h, c * C, b, mb);
      }
      if (!TMA) {
        const int imax = min(C, p.T - c * C);
        for (int u = tid; u < 64 * 16; u += 256) {
          const int i = urow16(u), c8 = ucol16(u);
          tc::cp_async16(sA3 + tc::sw128_unit(i, c8), i < imax ? p.k + grow(c, i) * KD + c8 * 8 : p.k, i < imax);
        }
      }
    }
    if (!TMA) tc::cp_async_commit();
  };

  if (warp == 0) {
    tc::tmem_alloc(tslot, 512);
    tc::tmem_relinquish();
  }
  if (tid == 0) {
    for (int m = 0; m < 7; ++m) tc::mbar_init(&mbar[m], 1);
    tc::mbar_fence_init();
  }
  __syncthreads();  // barriers initialised before the copies can complete on them
  for (int c = 0; c < 2; ++c) {
    issue_A(c);
    issue_U(c);
    issue_PK(c);
  }
  float S[64];  // state row kk, columns j0 .. j0+63 (zero outside the true Dk x Dv state)
  if (p.h0) {
    const float4* src = reinterpret_cast<const float4*>(p.h0 + ((size_t)bh * p.Dk + kk) * p.Dv + j0);
#pragma unroll
    for (int x = 0; x < 16; ++x) {
      const float4 t4 = (kk < p.Dk && j0 + 4 * x < p.Dv) ? __ldg(src + x) : make_float4(0.f, 0.f, 0.f, 0.f);
      S[4 * x] = t4.x; S[4 * x + 1] = t4.y; S[4 * x + 2] = t4.z; S[4 * x + 3] = t4.w;
    }
  } else {
#pragma unroll
    for (int x = 0; x < 64; ++x) S[x] = 0.f;
  }
  for (int u = tid; u < 2 * 64 * 8; u += 256)  // the zero rows of both [0;P] tiles
    sts16(A2 + (u >> 9) * 16384, tc::kmajor_unit((u >> 3) & 63, u & 7, C), zero16());
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t taddr = *tslot;
  uint32_t ph = 0;
  bool ok = true;

  // in-chunk cumulative log decay of the chunk ahead, fetched one chunk early (its latency would otherwise sit
  // at the top of every link of the chain)
  float g_nxt = p.gam[(size_t)bh * p.n * C + (tid & 63)], gl_nxt = p.gam[(size_t)bh * p.n * C + C - 1];
  for (int c = 0; c < p.n; ++c) {
    const size_t ci = (size_t)bh * p.n + c;
    const int t0 = c * C, imax = min(C, p.T - t0);
    const int buf = c & 1;
    const uint32_t lph = (c >> 1) & 1;  // phase of the image barriers of this buffer
    uint8_t* A1c = A1 + buf * 32768;
    uint8_t* A2c = A2 + buf * 16384;
    uint8_t* A3c = A3 + buf * 16384;
    uint8_t* Utc = Ut + buf * 16384;
    const float glast = gl_nxt, g = g_nxt;
    if (c + 1 < p.n) {
      g_nxt = p.gam[(ci + 1) * C + (tid & 63)];
      gl_nxt = p.gam[(ci + 1) * C + C - 1];
    }
    const float L = exp_nonpos(glast);
    if (tid < C) {
      dd[tid] = exp_nonpos(g);
      rr[tid] = exp_nonpos(glast - g);
    }
#pragma unroll
    for (int c8 = 0; c8 < 8; ++c8) {  // state as the MMA operand (and saved for the backward)
      const uint4 val = make_uint4(tc::pack_bf16(S[8 * c8], S[8 * c8 + 1]), tc::pack_bf16(S[8 * c8 + 2], S[8 * c8 + 3]),
                                   tc::pack_bf16(S[8 * c8 + 4], S[8 * c8 + 5]), tc::pack_bf16(S[8 * c8 + 6], S[8 * c8 + 7]));
      sts16(Sop, tc::mnmajor_unit(kk, 8 * half + c8, KD), val);
    }
    if (tid == 0) tc::bulk_wait_read<0>();  // the previous chunk's v_new image has left its tile
    if (!TMA) tc::cp_async_wait<5>();  // group A of this chunk has landed (q rows; the images on the barrier)
    if (ok) ok = tc::mbar_wait(&mbar[1 + buf], lph);
    tc::fence_async_smem();
    tc::fence_before_sync();
    ok = __syncthreads_and(ok);  // the barrier also makes the verdict of the bounded waits uniform, so that all
    if (!ok) break;              // threads leave the loop together
    tc::fence_after_sync();
    if (tid == 0) {  // D1 = [w;q] S
      tc::issue_gemm(taddr, tc::kmajor_sw128_tile(A1c, 16384), tc::mnmajor_tile(Sop, KD), 128, KD, KD, false);
      tc::mma_commit(mbar);
      if (p.save) {  // the state at chunk start, saved for the backward as the byte image of the operand tile
        tc::bulk_store(p.hs + ci * KD * KD, tc::smem_u32(Sop), 32768);
        tc::bulk_commit();
      }
    }
    if (TMA && tid == kOutThread && c > 0) {  // the previous chunk's output tile (complete since the barrier above)
      for (int sl = 0; sl < 2; ++sl)  // a slab that lies wholly past the true width is not stored at all
        if (64 * sl < p.Dv) tc::tma_store_4d(&maps.o, sOt + sl * 8192, 64 * sl, h, t0 - C, b);
      tc::bulk_commit();
    }
    // In the shadow of the MMA: k <- diag(r) k in place, so that the state update contracts it with v_new itself
    // (every thread scales the 16-byte units it would copy in the cp.async variant: no barrier needed for those)
    if (!TMA) tc::cp_async_wait<3>();
    if (ok) ok = tc::mbar_wait(&mbar[5 + buf], lph);  // P image and k rows of this chunk
#pragma unroll
    for (int m = 0; m < 4; ++m) {
      const int u = tid + 256 * m, i = urow16(u);
      uint4* unit = reinterpret_cast<uint4*>(A3c + tc::sw128_unit(i, ucol16(u)));
      *unit = tc::scale_bf16x8(*unit, rr[i]);
    }
    if (ok) ok = tc::mbar_wait(mbar, ph);
    ph ^= 1;
    tc::fence_after_sync();
    issue_A(c + 2);
    if (ok) ok = tc::mbar_wait(&mbar[3 + buf], lph);  // u image of this chunk
    float f[64];  // accumulator row; rows 64-127 keep E(gam_i) (q S) here until P v_new arrives
    if (ok) {
      const int i = kk & 63;
      ld_acc64(taddr + j0, warp, f);
      if (kk < 64) {  // v_new = u - w S
#pragma unroll
        for (int x = 0; x < 8; ++x) {
          const int c8 = 8 * half + x;
          const uint4 uu = *reinterpret_cast<const uint4*>(Utc + tc::kmajor_unit(i, c8, KD));
          float e[8];
          tc::unpack_bf16(uu.x, e[0], e[1]); tc::unpack_bf16(uu.y, e[2], e[3]);
          tc::unpack_bf16(uu.z, e[4], e[5]); tc::unpack_bf16(uu.w, e[6], e[7]);
#pragma unroll
          for (int y = 0; y < 8; ++y) e[y] -= f[8 * x + y];
          sts16(Vn, tc::mnmajor_unit(i, c8, KD), make_uint4(tc::pack_bf16(e[0], e[1]), tc::pack_bf16(e[2], e[3]),
                                                            tc::pack_bf16(e[4], e[5]), tc::pack_bf16(e[6], e[7])));
        }
      } else {
        const float di = dd[i];
#pragma unroll
        for (int jj = 0; jj < 64; ++jj) f[jj] *= di;
      }
    }
    if (tid == 0) tc::bulk_wait_read<0>();  // the state image has left its tile
    if (TMA && tid == kOutThread) tc::bulk_wait_read<0>();  // the previous output tile has left its tile
    tc::fence_async_smem();
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    issue_U(c + 2);  // u has been consumed by every thread
    if (ok && tid == 0) {
      // D2 = [0;P] v_new          D3 = (r k)^T v_new
      tc::issue_gemm(taddr + 128, tc::kmajor_tile(A2c, C), tc::mnmajor_tile(Vn, KD), 128, KD, C, false);
      tc::issue_gemm(taddr + 256, tc::mnmajor_sw128_tile(A3c, 8192), tc::mnmajor_tile(Vn, KD), 128, KD, C, false);
      tc::mma_commit(mbar);
      if (p.save) {
        tc::bulk_store(p.vn + ci * C * KD, tc::smem_u32(Vn), 16384);
        tc::bulk_commit();
      }
    }
    if (ok) {
      ok = tc::mbar_wait(mbar, ph);
      ph ^= 1;
    }
    tc::fence_after_sync();
    issue_PK(c + 2);
    if (ok) {
      const int i = kk & 63;
      float a[64];
      if (kk >= 64) {  // out = E(gam)(q S) + P v_new      (warp-uniform branch)
        ld_acc64(taddr + 128 + j0, warp, a);
        if (TMA) {     // into the swizzled output tile; one thread hands it to the copy engine after the next barrier
#pragma unroll
          for (int x = 0; x < 8; ++x)
            sts16(Ot, tc::sw128_unit(i, 8 * half + x),
                  make_uint4(tc::pack_bf16(f[8 * x] + a[8 * x], f[8 * x + 1] + a[8 * x + 1]),
                             tc::pack_bf16(f[8 * x + 2] + a[8 * x + 2], f[8 * x + 3] + a[8 * x + 3]),
                             tc::pack_bf16(f[8 * x + 4] + a[8 * x + 4], f[8 * x + 5] + a[8 * x + 5]),
                             tc::pack_bf16(f[8 * x + 6] + a[8 * x + 6], f[8 * x + 7] + a[8 * x + 7])));
        } else if (i < imax) {
          uint4* dst = reinterpret_cast<uint4*>(p.out + grow(c, i) * KD + j0);
#pragma unroll
          for (int x = 0; x < 8; ++x)
            dst[x] = make_uint4(tc::pack_bf16(f[8 * x] + a[8 * x], f[8 * x + 1] + a[8 * x + 1]),
                                tc::pack_bf16(f[8 * x + 2] + a[8 * x + 2], f[8 * x + 3] + a[8 * x + 3]),
                                tc::pack_bf16(f[8 * x + 4] + a[8 * x + 4], f[8 * x + 5] + a[8 * x + 5]),
                                tc::pack_bf16(f[8 * x + 6] + a[8 * x + 6], f[8 * x + 7] + a[8 * x + 7]));
        }
      }
      ld_acc64(taddr + 256 + j0, warp, a);  // S <- E(gam_last) S + (r k)^T v_new
#pragma unroll
      for (int jj = 0; jj < 64; ++jj) S[jj] = fmaf(L, S[jj], a[jj]);
    }
    tc::fence_before_sync();
  }
  if (!TMA) tc::cp_async_wait<0>();
  if (TMA) {  // the last chunk's output tile
    tc::fence_async_smem();
    __syncthreads();
    if (ok && tid == kOutThread) {
      for (int sl = 0; sl < 2; ++sl)
        if (64 * sl < p.Dv) tc::tma_store_4d(&maps.o, sOt + sl * 8192, 64 * sl, h, (p.n - 1) * C, b);
      tc::bulk_commit();
    }
    if (tid == kOutThread) tc::bulk_wait_read<0>();
  }
  if (tid == 0) tc::bulk_wait_read<0>();  // shared memory must outlive the copies
  if (!ok && tid == 0) atomicExch(p.status, 2);
  if (ok && p.hT && kk < p.Dk) {
    float4* dst = reinterpret_cast<float4*>(p.hT + ((size_t)bh * p.Dk + kk) * p.Dv + j0);
#pragma unroll
    for (int x = 0; x < 16; ++x)
      if (j0 + 4 * x < p.Dv) dst[x] = make_float4(S[4 * x], S[4 * x + 1], S[4 * x + 2], S[4 * x + 3]);
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(taddr, 512);
}

// ------------------------------------------------------------------ host
size_t gdn_simt_workspace_bytes(const mxb_gdn_desc* d, bool bwd);
mxb_status gdn_simt_bwd(const mxb_gdn_desc*, const void*, const void*, const void*, const float*,
                        const float*, const float*, const void*, const float*, void*, void*, void*,
                        float*, float*, float*, void*, cudaStream_t);

// chunk > 64 is computed with chunks of 64 (the result does not depend on the chunk size).  Heads narrower than the
// 128-wide tiles (64 <= Dk, Dv < 128, multiples of 8 so that rows stay 16-byte aligned) use the same kernels: their
// tensor maps carry the true width, loads of the missing columns return zeros and stores of them are clipped.
bool gdn_tc_supported(const mxb_gdn_desc* d) {
  auto width_ok = [](int w) { return w >= 64 && w <= KD && w % 8 == 0; };
  return d->io_dtype == MXB_BF16 && width_ok(d->Dk) && width_ok(d->Dv) && d->chunk >= C;
}

static size_t carve_tc(TcP& p, void* ws, bool bwd) {
  Carver cv(ws);
  const size_t nc = (size_t)p.B * p.H * p.n;
  p.status = cv.take<int>(64);
  p.gam = cv.take<float>(nc * C);
  p.Tm = cv.take<bf16>(nc * C * C);
  p.w = cv.take<bf16>(nc * C * KD);
  p.u = cv.take<bf16>(nc * C * KD);
  p.P = cv.take<bf16>(nc * C * C);
  if (bwd) {
    p.hs = cv.take<bf16>(nc * KD * KD);
    p.vn = cv.take<bf16>(nc * C * KD);
    p.dhs = cv.take<bf16>(nc * KD * KD);
    p.dvn = cv.take<bf16>(nc * C * KD);
  }
  return cv.bytes();
}

static TcP make_tc(const mxb_gdn_desc* d) {
  TcP p{};
  p.B = d->B; p.T = d->T; p.H = d->H;
  p.Dk = d->Dk; p.Dv = d->Dv;
  p.n = (d->T + C - 1) / C;
  p.gate_is_log = d->gate_is_log;
  return p;
}

size_t gdn_tc_workspace_bytes(const mxb_gdn_desc* d, bool bwd) {
  TcP p = make_tc(d);
  const size_t own = carve_tc(p, nullptr, bwd);
  if (!bwd) return own;
  const size_t simt = gdn_simt_workspace_bytes(d, true);
  return own > simt ? own : simt;
}

template <typename KernelT>
static mxb_status tc_set_smem(KernelT kern, int bytes) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) { set_last_cuda_error((int)e); return MXB_ERR_CUDA; }
  return MXB_OK;
}

mxb_status tc_run_bwd(TcP& p, bool recompute, cudaStream_t st);

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}
// [B,T,H,D] bf16 as a 4-d tensor (D, H, T, B) with boxes of 64 columns x 64 time steps, 128-byte swizzle
// (D a multiple of 8: rows are 16-byte multiples; columns past D and rows past T are zero-filled by the copy engine
// on loads and clipped on stores).  Shared with the Mamba-3 kernels.
bool make_tma_map_bthd(CUtensorMap* m, const void* base, int B, int T, int H, int D) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn || (reinterpret_cast<uintptr_t>(base) & 15) || D % 8 || D <= 0) return false;
  const cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)T, (cuuint64_t)B};
  const cuuint64_t strides[3] = {(cuuint64_t)D * 2, (cuuint64_t)H * D * 2, (cuuint64_t)T * H * D * 2};
  const cuuint32_t box[4] = {64, 1, 64, 1}, estr[4] = {1, 1, 1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static bool g_tc_use_tma = true;
void gdn_tc_set_tma(bool on) { g_tc_use_tma = on; }

mxb_status tc_run_fwd(TcP& p, cudaStream_t st) {
  cudaError_t e = cudaMemsetAsync(p.status, 0, 256, st);
  if (e != cudaSuccess) { set_last_cuda_error((int)e); return MXB_ERR_CUDA; }
  PrepMaps maps;
  std::memset(&maps, 0, sizeof maps);
  // heads narrower than the tiles exist only through the copy engine (the per-thread staging addresses full rows)
  const bool narrow = p.Dk != KD || p.Dv != KD;
  const bool tma = g_tc_use_tma && (!p.no_tma || narrow) && make_tma_map_bthd(&maps.k, p.k, p.B, p.T, p.H, p.Dk) &&
                   make_tma_map_bthd(&maps.q, p.q, p.B, p.T, p.H, p.Dk) && make_tma_map_bthd(&maps.v, p.v, p.B, p.T, p.H, p.Dv) &&
                   make_tma_map_bthd(&maps.o, p.out, p.B, p.T, p.H, p.Dv);
  if (narrow && !tma) return MXB_ERR_UNSUPPORTED;
  if (tma) {
    if (tc_set_smem(gdn_tc_prep_kernel<true>, kPrepSmem) != MXB_OK) return MXB_ERR_CUDA;
    MXB_LAUNCH("gdn_tc_prep_kernel", st,
               (gdn_tc_prep_kernel<true><<<dim3(p.n, p.B * p.H), 128, kPrepSmem, st>>>(p, maps)));
  } else {
    if (tc_set_smem(gdn_tc_prep_kernel<false>, kPrepSmem) != MXB_OK) return MXB_ERR_CUDA;
    MXB_LAUNCH("gdn_tc_prep_kernel", st,
               (gdn_tc_prep_kernel<false><<<dim3(p.n, p.B * p.H), 128, kPrepSmem, st>>>(p, maps)));
  }
  mxb_status s = check_launch("gdn_tc_prep_kernel");
  if (s != MXB_OK) return s;
  if (tma) {
    if (tc_set_smem(gdn_tc_state_fwd_kernel<true>, kStateFwdSmem) != MXB_OK) return MXB_ERR_CUDA;
    MXB_LAUNCH("gdn_tc_state_fwd_kernel", st,
               (gdn_tc_state_fwd_kernel<true><<<dim3(p.B * p.H), 256, kStateFwdSmem, st>>>(p, maps)));
  } else {
    if (tc_set_smem(gdn_tc_state_fwd_kernel<false>, kStateFwdSmem) != MXB_OK) return MXB_ERR_CUDA;
    MXB_LAUNCH("gdn_tc_state_fwd_kernel", st,
               (gdn_tc_state_fwd_kernel<false><<<dim3(p.B * p.H), 256, kStateFwdSmem, st>>>(p, maps)));
  }
  return check_launch("gdn_tc_state_fwd_kernel");
}

mxb_status gdn_tc_fwd(const mxb_gdn_desc* d, const void* q, const void* k, const void* v, const float* beta,
                      const float* gate, const float* h0, void* out, float* hT, void* ws, cudaStream_t st) {
  TcP p = make_tc(d);
  p.q = static_cast<const bf16*>(q); p.k = static_cast<const bf16*>(k); p.v = static_cast<const bf16*>(v);
  p.beta = beta; p.gate = gate; p.h0 = h0; p.out = static_cast<bf16*>(out); p.hT = hT;
  p.save = (d->flags & MXB_GDN_SAVE_FOR_BWD) ? 1 : 0;
  p.no_tma = (d->flags & MXB_GDN_NO_TMA) ? 1 : 0;
  carve_tc(p, ws, p.save != 0);
  return tc_run_fwd(p, st);
}

mxb_status gdn_tc_bwd(const mxb_gdn_desc* d, const void* q, const void* k, const void* v, const float* beta,
                      const float* gate, const float* h0, const void* dO, const float* dhT, void* dq, void* dk,
                      void* dv, float* dbeta, float* dgate, float* dh0, void* ws, cudaStream_t st) {
  if (d->flags & MXB_GDN_BWD_FP32_KERNELS)
    return gdn_simt_bwd(d, q, k, v, beta, gate, h0, dO, dhT, dq, dk, dv, dbeta, dgate, dh0, ws, st);
  TcP p = make_tc(d);
  p.q = static_cast<const bf16*>(q); p.k = static_cast<const bf16*>(k); p.v = static_cast<const bf16*>(v);
  p.beta = beta; p.gate = gate; p.h0 = h0;
  p.dO = static_cast<const bf16*>(dO); p.dhT_in = dhT;
  p.dq = static_cast<bf16*>(dq); p.dk = static_cast<bf16*>(dk); p.dv = static_cast<bf16*>(dv);
  p.dbeta = dbeta; p.dgate = dgate; p.dh0 = dh0;
  p.no_tma = (d->flags & MXB_GDN_NO_TMA) ? 1 : 0;
  carve_tc(p, ws, true);
  return tc_run_bwd(p, !(d->flags & MXB_GDN_BWD_USE_SAVED), st);
}

}  // namespace mxb

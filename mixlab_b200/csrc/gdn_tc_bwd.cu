// Gated delta rule - tensor-core backward (tcgen05.mma, TMEM accumulators),
// bf16 I/O, fp32 state gradient, chunk 64, Dk = Dv = 128.
//
// Hand-derived backward of the chunked form (the reference differentiates
// gpu/ir.cpp:2352-2550 with MLX autograd; its only VJP, tril(T^T dT T^T,-1) of the
// triangular solve, gpu/gated_delta_cuda_primitive.cpp:104-132, is phase C below).
// With d = E(gam), r = E(gam_last-gam), L = E(gam_last), S0 the state at chunk start
// and dS the state gradient at chunk end:
//
//   gdn_tc_state_bwd_kernel  reverse over chunks, one CTA per (batch, head), operands two chunks ahead:
//       dv_new = P^T dO + r (k dS)
//       dS    <- L dS + (d q)^T dO - w^T dv_new
//   gdn_tc_chunk_bwd_kernel  one CTA per chunk, everything else (the contractions with the saved states S0 and dS
//       included):
//       dq = d (dO S0^T) + (dP*Gamma) k                      dP = tril(dO v_new^T)
//       dw = -dv_new S0^T ; dT = dv_new (v beta)^T + dw (k beta d)^T ; dA = tril(T^T dT T^T,-1)
//       dk = (dP*Gamma)^T q + r (v_new dS^T) + beta d (T^T dw) + (Mb + Mb^T) k,  Mb = -beta dA*Gamma
//       dv = beta (T^T dv_new) ; dbeta, dgam from the same pieces ; dg = reverse cumsum of dgam
//
// A 64 x W bf16 tile stored as 8x8-element blocks ("blocked row-major", umma_tiles.cuh)
// can be read by tcgen05.mma either with the contraction along its columns (K-major) or
// along its rows (MN-major); both views are used on the same staged bytes.
#include <cstring>

#include "gdn_tc.cuh"

namespace mxb {

// One CTA (256 threads) per (batch, head); thread t owns row kk = t & 127 of dS and the 64
// columns of half t >> 7.  Chunks run in reverse.  The operand tiles are double-buffered (buffer c & 1 for
// chunk c) and requested two chunks ahead, as soon as the MMA batch that last read the buffer has completed:
//   group A  k, dO, q rows and the P image   free after the first MMA batch
//   group B  the w image                     free after the second MMA batch
// q is scaled in place to diag(E(gam)) q one chunk early, in the shadow of the second MMA batch, so that the
// first batch contracts it with the raw dO tile:  dS <- E(gam_last) dS + (d q)^T dO - w^T dv_new.
//
// TMA = true: the k, dO and q rows arrive as tensor-map boxes (128-byte swizzle, two 8 KB slabs of 64 columns per
// tile) issued by one thread on the barrier of group A; TMA = false: by cp.async into the same swizzled positions
// (twelve copies per thread and chunk).  The w image is stored in the same swizzled layout by the prep kernel.
constexpr int kStateBwdSmem =
    2 * 16384 + 32768 + 2 * 8192 + 2 * 16384 + 2 * 16384 + 2 * 16384 + 16384 + 3 * C * 4 + 128 + 1024;

template <bool TMA>
__global__ void __launch_bounds__(256) gdn_tc_state_bwd_kernel(TcP p, const __grid_constant__ RowMaps maps) {
  extern __shared__ uint8_t raw[];
  uint8_t* sm = raw + ((1024u - (tc::smem_u32(raw) & 1023u)) & 1023u);
  uint8_t* Ak = sm;                  // x2 [64 i][128 kk]   k  (swizzled slabs)
  uint8_t* dSop = Ak + 2 * 16384;    // [128 kk][128 j]     bf16 copy of dS
  uint8_t* Pt = dSop + 32768;        // x2 [64 m][64 i]     P   (A = P^T: contraction over rows)
  uint8_t* dOop = Pt + 2 * 8192;     // x2 [64 m][128 j]    dO (swizzled slabs)
  uint8_t* Aq = dOop + 2 * 16384;    // x2 [64 i][128 kk]   q, then diag(E(gam)) q (swizzled slabs)   (A = q^T)
  uint8_t* Aw = Aq + 2 * 16384;      // x2 [64 i][128 kk]   w image (swizzled slabs)                  (A = w^T)
  uint8_t* Bd = Aw + 2 * 16384;      // [64 i][128 j]       -dv_new
  float* rr = reinterpret_cast<float*>(Bd + 16384);
  float* ddn = rr + C;               // x2 E(gam) of the chunk whose q is scaled next (buffer = chunk & 1)
  // [0] MMA completion; per buffer: [1 + buf] group A landed, [3 + buf] w image landed
  uint64_t* mbar = reinterpret_cast<uint64_t*>(ddn + 2 * C);
  uint32_t* tslot = reinterpret_cast<uint32_t*>(mbar + 8);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kk = tid & 127, half = tid >> 7, j0 = 64 * half;
  const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H;
  const uint32_t sAk = tc::smem_u32(Ak), sPt = tc::smem_u32(Pt), sdO = tc::smem_u32(dOop), sAq = tc::smem_u32(Aq);
  const uint32_t sAw = tc::smem_u32(Aw);

  auto grow = [&](int c, int i) { return ((size_t)(b * p.T + c * C + i) * p.H + h); };
  auto issue_A = [&](int c) {
    if (c >= 0) {
      const size_t ci = (size_t)bh * p.n + c;
      const uint32_t o16 = (c & 1) * 16384;
      if (!TMA) {
        const int imax = min(C, p.T - c * C);
        for (int u = tid; u < 64 * 16; u += 256) {
          const int i = urow16(u), c8 = ucol16(u);
          const bool v = i < imax;
          const size_t g = v ? grow(c, i) * KD + c8 * 8 : 0;
          const uint32_t off = o16 + tc::sw128_unit(i, c8);
          tc::cp_async16(sAk + off, p.k + g, v);
          tc::cp_async16(sdO + off, p.dO + g, v);
          tc::cp_async16(sAq + off, p.q + g, v);
        }
      }
      if (tid == 32) {  // P is a byte image of its operand tile: one bulk copy, completing on the group's barrier
        uint64_t* mb = &mbar[1 + (c & 1)];
        tc::mbar_expect_tx(mb, TMA ? 8192 + 3 * 16384 : 8192);
        tc::bulk_load(sPt + (c & 1) * 8192, p.P + ci * C * C, 8192, mb);
        if (TMA) {
          for (int sl = 0; sl < 2; ++sl) {
            tc::tma_load_4d(sAk + o16 + sl * 8192, &maps.k, 64 * sl, h, c * C, b, mb);
            tc::tma_load_4d(sdO + o16 + sl * 8192, &maps.dO, 64 * sl, h, c * C, b, mb);
            tc::tma_load_4d(sAq + o16 + sl * 8192, &maps.q, 64 * sl, h, c * C, b, mb);
          }
        }
      }
    }
    if (!TMA) tc::cp_async_commit();
  };
  auto issue_B = [&](int c) {
    if (c >= 0 && tid == 32) {
      const size_t ci = (size_t)bh * p.n + c;
      tc::mbar_expect_tx(&mbar[3 + (c & 1)], 16384);
      tc::bulk_load(sAw + (c & 1) * 16384, p.w + ci * C * KD, 16384, &mbar[3 + (c & 1)]);
    }
    if (!TMA) tc::cp_async_commit();  // (empty: keeps the group count of the schedule)
  };
  // q of chunk c <- diag(E(gam)) q in place; every thread scales the 16-byte units it would copy itself
  auto scale_q = [&](int c) {
#pragma unroll
    for (int m = 0; m < 4; ++m) {
      const int u = tid + 256 * m, i = urow16(u);
      uint4* unit = reinterpret_cast<uint4*>(Aq + (c & 1) * 16384 + tc::sw128_unit(i, ucol16(u)));
      *unit = tc::scale_bf16x8(*unit, ddn[(c & 1) * C + i]);
    }
  };

  if (warp == 0) {
    tc::tmem_alloc(tslot, 512);
    tc::tmem_relinquish();
  }
  if (tid == 0) {
    for (int m = 0; m < 5; ++m) tc::mbar_init(&mbar[m], 1);
    tc::mbar_fence_init();
  }
  __syncthreads();  // barriers initialised before the copies can complete on them
  for (int c = p.n - 1; c > p.n - 3; --c) {
    issue_A(c);
    issue_B(c);
  }
  float dS[64];  // row kk of dS, columns j0 .. j0+63
  if (p.dhT_in) {
    const float4* src = reinterpret_cast<const float4*>(p.dhT_in + ((size_t)bh * p.Dk + kk) * p.Dv + j0);
#pragma unroll
    for (int x = 0; x < 16; ++x) {
      const float4 t4 = (kk < p.Dk && j0 + 4 * x < p.Dv) ? __ldg(src + x) : make_float4(0.f, 0.f, 0.f, 0.f);
      dS[4 * x] = t4.x; dS[4 * x + 1] = t4.y; dS[4 * x + 2] = t4.z; dS[4 * x + 3] = t4.w;
    }
  } else {
#pragma unroll
    for (int x = 0; x < 64; ++x) dS[x] = 0.f;
  }
  // in-chunk cumulative log decay: this chunk's, and the next (earlier) one's fetched a chunk early
  const size_t gbase = (size_t)bh * p.n * C;
  float g_cur = p.gam[gbase + (size_t)(p.n - 1) * C + (tid & 63)], gl_cur = p.gam[gbase + (size_t)(p.n - 1) * C + C - 1];
  float g_nxt = 0.f, gl_nxt = 0.f;
  if (p.n > 1) {
    g_nxt = p.gam[gbase + (size_t)(p.n - 2) * C + (tid & 63)];
    gl_nxt = p.gam[gbase + (size_t)(p.n - 2) * C + C - 1];
  }
  if (tid < C) ddn[((p.n - 1) & 1) * C + tid] = exp_nonpos(g_cur);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t taddr = *tslot;
  uint32_t ph = 0;
  bool ok = true;
  {  // the last chunk's q is scaled here; every later one in the shadow of the previous iteration's second batch
    const int c = p.n - 1;
    if (!TMA) tc::cp_async_wait<2>();
    ok = tc::mbar_wait(&mbar[1 + (c & 1)], 0);
    scale_q(c);
  }

  for (int c = p.n - 1; c >= 0; --c) {
    const size_t ci = (size_t)bh * p.n + c;
    const int buf = c & 1;
    const uint32_t lph = ((p.n - 1 - c) >> 1) & 1;  // phase of this buffer's barriers
    const float glast = gl_cur, g = g_cur;
    g_cur = g_nxt; gl_cur = gl_nxt;
    if (c > 1) {
      g_nxt = p.gam[(ci - 2) * C + (tid & 63)];
      gl_nxt = p.gam[(ci - 2) * C + C - 1];
    }
    const float L = exp_nonpos(glast);
    if (tid < C) {
      rr[tid] = exp_nonpos(glast - g);
      if (c > 0) ddn[(buf ^ 1) * C + tid] = exp_nonpos(g_cur);  // for the next chunk's q
    }
#pragma unroll
    for (int c8 = 0; c8 < 8; ++c8) {  // dS at chunk end: MMA operand + saved for the chunk kernel
      const uint4 val = make_uint4(tc::pack_bf16(dS[8 * c8], dS[8 * c8 + 1]), tc::pack_bf16(dS[8 * c8 + 2], dS[8 * c8 + 3]),
                                   tc::pack_bf16(dS[8 * c8 + 4], dS[8 * c8 + 5]), tc::pack_bf16(dS[8 * c8 + 6], dS[8 * c8 + 7]));
      sts16(dSop, tc::mnmajor_unit(kk, 8 * half + c8, KD), val);
    }
    if (tid == 0) tc::bulk_wait_read<0>();  // the previous chunk's -dv_new image has left its tile
    // group A of this chunk was waited for when its q was scaled (previous iteration / prologue)
    tc::fence_async_smem();
    tc::fence_before_sync();
    ok = __syncthreads_and(ok);  // the barrier also makes the verdict of the bounded waits uniform, so that all
    if (!ok) break;              // threads leave the loop together
    tc::fence_after_sync();
    if (tid == 0) {
      tc::issue_gemm(taddr, tc::kmajor_sw128_tile(Ak + buf * 16384, 8192), tc::mnmajor_tile(dSop, KD), 64, KD, KD, false);  // k dS
      tc::issue_gemm(taddr + 128, tc::mnmajor_tile(Pt + buf * 8192, C), tc::mnmajor_sw128_tile(dOop + buf * 16384, 8192), 64, KD,
                     C, false);                                                                                           // P^T dO
      tc::issue_gemm(taddr + 256, tc::mnmajor_sw128_tile(Aq + buf * 16384, 8192), tc::mnmajor_sw128_tile(dOop + buf * 16384, 8192),
                     128, KD, C, false);                                                                                  // (d q)^T dO
      tc::mma_commit(mbar);
      tc::bulk_store(p.dhs + ci * KD * KD, tc::smem_u32(dSop), 32768);  // dS at chunk end, as the operand-tile image
      tc::bulk_commit();
    }
    if (ok) ok = tc::mbar_wait(mbar, ph);
    ph ^= 1;
    tc::fence_after_sync();
    issue_A(c - 2);
    if (ok) {
      const int i = 16 * (warp & 3) + (lane & 15);  // M=64 accumulators: row i in TMEM lane (i%16) + 32*(i/16)
      const float ri = rr[i];
      for (int c0 = 0; c0 < 64; c0 += 32) {
        float fa[32], fb[32];
        ld_acc32(taddr + j0, warp, c0, fa);
        ld_acc32(taddr + 128 + j0, warp, c0, fb);
        if (lane < 16) {
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            float e[8];
#pragma unroll
            for (int y = 0; y < 8; ++y) e[y] = -fmaf(ri, fa[8 * x + y], fb[8 * x + y]);
            const int c8 = 8 * half + (c0 >> 3) + x;
            sts16(Bd, tc::kmajor_unit(i, c8, KD), make_uint4(tc::pack_bf16(e[0], e[1]), tc::pack_bf16(e[2], e[3]),
                                                             tc::pack_bf16(e[4], e[5]), tc::pack_bf16(e[6], e[7])));
          }
        }
      }
    }
    if (tid == 0) tc::bulk_wait_read<0>();  // the dS image has left its tile
    if (ok) ok = tc::mbar_wait(&mbar[3 + buf], lph);  // w image of this chunk
    tc::fence_async_smem();
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    if (ok && tid == 0) {  // ... - w^T dv_new
      tc::issue_gemm(taddr + 256, tc::mnmajor_sw128_tile(Aw + buf * 16384, 8192), tc::mnmajor_tile(Bd, KD), 128, KD, C, true);
      tc::mma_commit(mbar);
      tc::bulk_store(p.dvn + ci * C * KD, tc::smem_u32(Bd), 16384);  // -dv_new as the operand-tile image
      tc::bulk_commit();
    }
    if (c > 0) {  // in the shadow of the MMA: the next chunk's q (its group landed a chunk ago)
      if (!TMA) tc::cp_async_wait<2>();
      if (ok) ok = tc::mbar_wait(&mbar[1 + (buf ^ 1)], ((p.n - c) >> 1) & 1);
      scale_q(c - 1);
    }
    if (ok) {
      ok = tc::mbar_wait(mbar, ph);
      ph ^= 1;
    }
    tc::fence_after_sync();
    issue_B(c - 2);
    if (ok) {
      float a[64];
      ld_acc64(taddr + 256 + j0, warp, a);
#pragma unroll
      for (int jj = 0; jj < 64; ++jj) dS[jj] = fmaf(L, dS[jj], a[jj]);
    }
    tc::fence_before_sync();
  }
  if (!TMA) tc::cp_async_wait<0>();
  if (tid == 0) tc::bulk_wait_read<0>();  // shared memory must outlive the copies
  if (!ok && tid == 0) atomicExch(p.status, 3);
  if (ok && p.dh0 && kk < p.Dk) {
    float4* dst = reinterpret_cast<float4*>(p.dh0 + ((size_t)bh * p.Dk + kk) * p.Dv + j0);
#pragma unroll
    for (int x = 0; x < 16; ++x)
      if (j0 + 4 * x < p.Dv) dst[x] = make_float4(dS[4 * x], dS[4 * x + 1], dS[4 * x + 2], dS[4 * x + 3]);
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(taddr, 512);
}

// ------------------------------------------------- chunk backward
// One CTA per chunk does everything that is not the sequential state pass.  With e = T^T dv_new, z = T^T dw = -e S0^T
// (dw = -dv_new S0^T never needs to be formed), Gamma_ij = E(gam_i - gam_j):
//   batch 1   -e = T^T (-dv_new)                    dP = dO v_new^T                -> dPG = dP*Gamma (lower incl. diagonal)
//   batch 2   DQ = (d dO) S0^T   (stays in TMEM)    z = (-e) S0^T                  (dO is scaled by d in place first)
//   batch 3   r (v_new dS^T) -> dkp                                                 <dS, S0> on the side
//   batch 4   (-e) v^T, z k^T   -> Y = T^T dT = beta_m (e.v_m + d_m z.k_m)
//   batch 5   dA = tril(Y T^T, -1), k k^T           -> M = -dA*Gamma, Mb = beta_i M
//   batch 6   DQ += dPG k                            dPG^T q + Mb k + Mb^T k
//   dq = DQ      dk = dkp + batch 6 + beta d z      dv = beta e      dbeta = e.v + d (k.z) + sum_j M_ij (k_i.k_j)
//   dgam_i = q_i.dq_i - k_i.dk_i + 2 beta_i (d_i (k_i.z_i) + sum_j M_ij (k_i.k_j)),  dgam_last += L <dS,S0> + sum_i k_i.dkp_i
// (the row and column sums over Gamma of the P and A terms are exactly the parts of q.dq and k.dk that come from
// dPG and Mb, so they need no products of their own).
//
// 256 TMEM columns and 107 KB of shared memory: two CTAs share an SM.  Every buffer is reused as soon as it is dead:
//   XdO   dO (TMA tile) -> d dO -> z                      Xe   -dv_new image -> -e -> dv = beta e on its way out
//   Xvn   v_new image -> v (TMA) -> q (TMA) -> dq         R1   S0 image -> dS image -> k (TMA) | dkp -> dk
// TMEM: [0,128) -e, then DQ until the end; [128,256) the other products one after the other.  All accumulators are
// M=64: row i sits in TMEM lane (i%16) + 32*(i/16) and is handled by thread (warp i/16, lane i%16); warps 4-7 take
// the second half of the columns.  Grid = (batch*head, chunk) with batch*head fastest: neighbouring CTAs read
// neighbouring heads of the same time steps (one contiguous row of the token tensors between them), and the chunks
// the reverse state pass wrote last are read first.
constexpr int kChunkBwdSmem = 3 * 16384 + 32768 + 3 * 8192 + 8 * C * 4 + 16 * 4 + 64 + 64 + 1024;

__device__ __forceinline__ void unpack8(uint4 v, float (&e)[8]) {
  tc::unpack_bf16(v.x, e[0], e[1]); tc::unpack_bf16(v.y, e[2], e[3]);
  tc::unpack_bf16(v.z, e[4], e[5]); tc::unpack_bf16(v.w, e[6], e[7]);
}
__device__ __forceinline__ uint4 pack8(const float* e) {
  return make_uint4(tc::pack_bf16(e[0], e[1]), tc::pack_bf16(e[2], e[3]), tc::pack_bf16(e[4], e[5]),
                    tc::pack_bf16(e[6], e[7]));
}
// M=64 accumulators leave lanes 16-31 of every warp without a row.  Where an epilogue does real arithmetic per
// element, the owning lane l hands columns 16..31 of its 32-column block to lane l + 16: both then work on 16
// columns of the same row (16 shuffles buy half of the arithmetic).  h[q] = column c0 + 16 (lane >> 4) + q.
__device__ __forceinline__ void split_block32(const float (&f)[32], int lane, float (&h)[16]) {
  const bool upper = (lane >> 4) != 0;
#pragma unroll
  for (int q = 0; q < 16; ++q) {
    const float up = __shfl_sync(0xffffffffu, f[16 + q], lane & 15);
    h[q] = upper ? up : f[q];
  }
}

__global__ void __launch_bounds__(256, 2) gdn_tc_chunk_bwd_kernel(TcP p, const __grid_constant__ RowMaps maps) {
  extern __shared__ uint8_t raw[];
  uint8_t* sm = raw + ((1024u - (tc::smem_u32(raw) & 1023u)) & 1023u);
  uint8_t* XdO = sm;                // [64][128] dO (swizzled TMA tile), d dO in place, then z (blocked layout)
  uint8_t* Xe = XdO + 16384;        // [64][128] -dv_new image (blocked), then -e and finally dv (swizzled like a TMA tile)
  uint8_t* Xvn = Xe + 16384;        // [64][128] v_new image, then v, then q (swizzled TMA tiles), then dq in place
  uint8_t* R1 = Xvn + 16384;        // [128][128] S0 image, then dS image, then k (swizzled TMA tile) | dkp -> dk (swizzled)
  uint8_t* Xk = R1;
  uint8_t* Xdk = R1 + 16384;
  uint8_t* Xt = R1 + 32768;         // [64][64]  T
  uint8_t* Xpg = Xt + 8192;         // [64][64]  dP*Gamma
  uint8_t* Xy = Xpg + 8192;         // [64][64]  Y, then Mb
  float* gam = reinterpret_cast<float*>(Xy + 8192);
  float* bet = gam + C;
  float* dd = bet + C;
  float* rr = dd + C;
  float* dgo = rr + C;              // [2][C] per-row dgam / dbeta partials of the two column halves
  float* dbo = dgo + 2 * C;
  float* red = dbo + 2 * C;         // [0,8) <dS,S0> per warp, [8,16) sum of k.dkp per warp
  // [0] MMA, [6] second MMA barrier of the last batch; loads: [1] -dv_new/T/dO/v_new, [2] S0, [3] dS, [4] k/v, [5] q
  uint64_t* mbar = reinterpret_cast<uint64_t*>(red + 16);
  uint32_t* tslot = reinterpret_cast<uint32_t*>(mbar + 8);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.x, c = blockIdx.y, b = bh / p.H, h = bh % p.H, t0 = c * C;
  const size_t ci = (size_t)bh * p.n + c;
  const int imax = min(C, p.T - t0);
  auto row = [&](int i) { return ((size_t)(b * p.T + t0 + i) * p.H + h); };
  const bool own = lane < 16;
  const int i = 16 * (warp & 3) + (lane & 15);  // the row this thread owns in every epilogue
  const int hc = warp >> 2;   // warps 0-3 take the first half of an accumulator's columns, warps 4-7 the second
  const int cb = 32 * hc;     // this thread's 32 columns of every [64][64] accumulator
  const int cw = 64 * hc;     // this thread's 64 columns of every [64][128] accumulator
  const int hx = lane >> 4;   // which 16 columns of a shared 32-column block this lane works on (split_block32)

  // prologue latencies side by side: warp 0 allocates TMEM, one thread of warp 1 initialises the barriers and issues
  // the first copies, warps 2-3 fetch the per-row scalars
  if (tid == 32) {
    for (int m = 0; m < 7; ++m) tc::mbar_init(mbar + m, 1);
    tc::mbar_fence_init();
    tc::mbar_expect_tx(mbar + 1, 3 * 16384 + 8192);
    tc::bulk_load(tc::smem_u32(Xe), p.dvn + ci * C * KD, 16384, mbar + 1);  // byte images of the operand tiles
    tc::bulk_load(tc::smem_u32(Xt), p.Tm + ci * C * C, 8192, mbar + 1);
    tc::bulk_load(tc::smem_u32(Xvn), p.vn + ci * C * KD, 16384, mbar + 1);
    for (int sl = 0; sl < 2; ++sl) tc::tma_load_4d(tc::smem_u32(XdO) + 8192 * sl, &maps.dO, 64 * sl, h, t0, b, mbar + 1);
    tc::mbar_expect_tx(mbar + 2, 32768);
    tc::bulk_load(tc::smem_u32(R1), p.hs + ci * KD * KD, 32768, mbar + 2);
    // the operands whose buffers are still occupied are pulled into L2 now, so that their copies find them on chip
    tc::bulk_prefetch_l2(p.dhs + ci * KD * KD, 32768);
    for (int sl = 0; sl < 2; ++sl) {
      tc::tma_prefetch_4d(&maps.k, 64 * sl, h, t0, b);
      tc::tma_prefetch_4d(&maps.v, 64 * sl, h, t0, b);
      tc::tma_prefetch_4d(&maps.q, 64 * sl, h, t0, b);
    }
  }
  if (warp == 0) {
    tc::tmem_alloc(tslot, 256);
    tc::tmem_relinquish();
  }
  if (tid >= 64 && tid < 64 + C) {
    const int r = tid - 64;
    gam[r] = p.gam[ci * C + r];
    bet[r] = r < imax ? p.beta[row(r)] : 0.f;
  }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const float glast = gam[C - 1], L = exp_nonpos(glast);
  if (tid < C) {
    dd[tid] = exp_nonpos(gam[tid]);
    rr[tid] = exp_nonpos(glast - gam[tid]);
  }
  const uint32_t tA = *tslot, tB = tA + 128;
  bool ok = tc::mbar_wait(mbar + 1, 0);
  uint32_t ph = 0;
  // ---- batch 1: -e = T^T (-dv_new) (both operands contracted over their rows), dP = dO v_new^T ----
  if (ok && tid == 0) {
    tc::issue_gemm(tA, tc::mnmajor_tile(Xt, C), tc::mnmajor_tile(Xe, KD), 64, 128, C, false);
    tc::issue_gemm(tB, tc::kmajor_sw128_tile(XdO, 8192), tc::kmajor_tile(Xvn, KD), 64, 64, KD, false);
    tc::mma_commit(mbar);
  }
  __syncthreads();  // dd, rr visible
  const float gi = gam[i], bi = bet[i], di = dd[i], ri = rr[i];
  const float bd_i = bi * di;
  if (ok) ok = tc::mbar_wait(mbar, ph);
  ph ^= 1;
  tc::fence_after_sync();
  ok = __all_sync(0xffffffffu, ok);  // warp-uniform: the epilogues below shuffle with a full mask
  if (ok) {
    // -e goes back over the operand it was computed from (its MMA is complete), in the swizzled layout of a TMA
    // tile: scaled by -beta in place later, the same bytes leave as dv through a tiled store
    for_acc2x32(tA, warp, cw, [&](int c0, const float (&f)[32]) {
      if (own) {
#pragma unroll
        for (int x = 0; x < 4; ++x) sts16(Xe, tc::sw128_unit(i, (c0 >> 3) + x), pack8(&f[8 * x]));
      }
    });
    {  // dP * Gamma, lower triangle incl. diagonal
      float f[32], hq[16];
      ld_acc32(tB, warp, cb, f);
      split_block32(f, lane, hq);
      const int j0 = cb + 16 * hx;
#pragma unroll
      for (int q = 0; q < 16; ++q) {
        const int j = j0 + q;
        const float val = hq[q] * exp_nonpos(gi - gam[j]);  // unconditional: the exponentials overlap
        hq[q] = (j <= i) ? val : 0.f;
      }
#pragma unroll
      for (int x = 0; x < 2; ++x) sts16(Xpg, tc::kmajor_unit(i, (j0 >> 3) + x, C), pack8(&hq[8 * x]));
    }
#pragma unroll
    for (int m = 0; m < 4; ++m) {  // dO <- diag(d) dO in place, so that DQ can take dPG k on top later
      const int u = tid + 256 * m, r = urow16(u);
      uint4* unit = reinterpret_cast<uint4*>(XdO + tc::sw128_unit(r, ucol16(u)));
      *unit = tc::scale_bf16x8(*unit, dd[r]);
    }
  }
  if (ok) ok = tc::mbar_wait(mbar + 2, 0);  // S0
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  // ---- batch 2: DQ = (d dO) S0^T, z = (-e) S0^T ----
  if (ok && tid == 0) {
    tc::issue_gemm(tA, tc::kmajor_sw128_tile(XdO, 8192), tc::kmajor_tile(R1, KD), 64, 128, KD, false);
    tc::issue_gemm(tB, tc::kmajor_sw128_tile(Xe, 8192), tc::kmajor_tile(R1, KD), 64, 128, KD, false);
    tc::mma_commit(mbar);  // one commit: z overwrites d dO and dS overwrites S0, which DQ reads as well
  }
  uint4 s0u[8];  // this thread's 8 units of S0, kept for <dS, S0> (the buffer is about to be reused)
#pragma unroll
  for (int x = 0; x < 8; ++x) s0u[x] = *reinterpret_cast<const uint4*>(R1 + (tid + 256 * x) * 16);
  tc::fence_async_smem();
  __syncthreads();  // every thread has taken its units of S0 before the copy engine overwrites the buffer
  if (ok) ok = tc::mbar_wait(mbar, ph);
  ph ^= 1;
  tc::fence_after_sync();
  ok = __all_sync(0xffffffffu, ok);  // warp-uniform: the epilogues below shuffle with a full mask
  if (ok && tid == 0) {  // S0 is dead in shared memory: dS comes into the same buffer behind the epilogue
    tc::mbar_expect_tx(mbar + 3, 32768);
    tc::bulk_load(tc::smem_u32(R1), p.dhs + ci * KD * KD, 32768, mbar + 3);
  }
  if (ok) {
    for_acc2x32(tB, warp, cw, [&](int c0, const float (&f)[32]) {  // z -> bf16 operand over the dead dO tile (blocked layout)
      if (own) {
#pragma unroll
        for (int x = 0; x < 4; ++x) sts16(XdO, tc::kmajor_unit(i, (c0 >> 3) + x, KD), pack8(&f[8 * x]));
      }
    });
  }
  if (ok) ok = tc::mbar_wait(mbar + 3, 0);  // dS
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  // ---- batch 3: v_new dS^T ----
  if (ok && tid == 0) {
    tc::issue_gemm(tB, tc::kmajor_tile(Xvn, KD), tc::kmajor_tile(R1, KD), 64, 128, KD, false);
    tc::mma_commit(mbar);
  }
  {  // <dS, S0>
    float part = 0.f;
#pragma unroll
    for (int x = 0; x < 8; ++x) {
      float a[8], bq[8];
      unpack8(*reinterpret_cast<const uint4*>(R1 + (tid + 256 * x) * 16), a);
      unpack8(s0u[x], bq);
#pragma unroll
      for (int y = 0; y < 8; ++y) part = fmaf(a[y], bq[y], part);
    }
    part = warp_sum(part);
    if (lane == 0) red[warp] = part;
  }
  tc::fence_async_smem();
  __syncthreads();  // every thread is done with dS before the copy engine overwrites the buffer
  if (ok) ok = tc::mbar_wait(mbar, ph);
  ph ^= 1;
  tc::fence_after_sync();
  ok = __all_sync(0xffffffffu, ok);  // warp-uniform: the epilogues below shuffle with a full mask
  if (ok && tid == 128) {  // v_new and dS are dead: k and v take their places
    tc::mbar_expect_tx(mbar + 4, 2 * 16384);
    for (int sl = 0; sl < 2; ++sl) {
      tc::tma_load_4d(tc::smem_u32(Xk) + 8192 * sl, &maps.k, 64 * sl, h, t0, b, mbar + 4);
      tc::tma_load_4d(tc::smem_u32(Xvn) + 8192 * sl, &maps.v, 64 * sl, h, t0, b, mbar + 4);
    }
  }
  if (ok) {
    for_acc2x32(tB, warp, cw, [&](int c0, float (&f)[32]) {  // dkp = r (v_new dS^T), kept as bf16 where dk will be assembled
      if (own) {
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) f[jj] *= ri;
#pragma unroll
        for (int x = 0; x < 4; ++x) sts16(Xdk, tc::sw128_unit(i, (c0 >> 3) + x), pack8(&f[8 * x]));
      }
    });
  }
  if (ok) ok = tc::mbar_wait(mbar + 4, 0);  // k, v
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  // ---- batch 4: (-e) v^T and z k^T; their column-scaled sum is Y = T^T dT (dT is never formed) ----
  if (ok && tid == 0) {
    tc::issue_gemm(tB, tc::kmajor_sw128_tile(Xe, 8192), tc::kmajor_sw128_tile(Xvn, 8192), 64, 64, KD, false);
    tc::issue_gemm(tB + 64, tc::kmajor_tile(XdO, KD), tc::kmajor_sw128_tile(Xk, 8192), 64, 64, KD, false);
    tc::mma_commit(mbar);
  }
  float vdot = 0.f, kz = 0.f;  // e_i . v_i and k_i . z_i: the diagonals of the two products of this batch
  if (ok) ok = tc::mbar_wait(mbar, ph);
  ph ^= 1;
  tc::fence_after_sync();
  ok = __all_sync(0xffffffffu, ok);  // warp-uniform: the epilogues below shuffle with a full mask
  if (ok) {  // Y[i][m] = beta_m ((e_i . v_m) + d_m (z_i . k_m))
    float f[32], ha[16], hb[16];
    ld_acc32(tB, warp, cb, f);
    split_block32(f, lane, ha);
    ld_acc32(tB + 64, warp, cb, f);
    split_block32(f, lane, hb);
    const int j0 = cb + 16 * hx;
#pragma unroll
    for (int q = 0; q < 16; ++q) {  // the lane whose 16 columns contain column i picks the two row dots off the diagonal
      vdot = (j0 + q == i) ? -ha[q] : vdot;
      kz = (j0 + q == i) ? hb[q] : kz;
    }
    vdot += __shfl_xor_sync(0xffffffffu, vdot, 16);  // one of the two lanes of a row found it (the other holds 0);
    kz += __shfl_xor_sync(0xffffffffu, kz, 16);      // rows whose diagonal lies in the other column half keep 0
#pragma unroll
    for (int q = 0; q < 16; ++q) ha[q] = bet[j0 + q] * fmaf(dd[j0 + q], hb[q], -ha[q]);
#pragma unroll
    for (int x = 0; x < 2; ++x) sts16(Xy, tc::kmajor_unit(i, (j0 >> 3) + x, C), pack8(&ha[8 * x]));
  }
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();  // also: every thread is done with v
  tc::fence_after_sync();
  if (ok && tid == 128) {  // q takes the place of v
    tc::mbar_expect_tx(mbar + 5, 16384);
    for (int sl = 0; sl < 2; ++sl) tc::tma_load_4d(tc::smem_u32(Xvn) + 8192 * sl, &maps.q, 64 * sl, h, t0, b, mbar + 5);
  }
  // ---- batch 5: dA = tril(Y T^T, -1) and k k^T ----
  if (ok && tid == 0) {
    tc::issue_gemm(tB, tc::kmajor_tile(Xy, C), tc::kmajor_tile(Xt, C), 64, 64, C, false);
    tc::issue_gemm(tB + 64, tc::kmajor_sw128_tile(Xk, 8192), tc::kmajor_sw128_tile(Xk, 8192), 64, 64, KD, false);
    tc::mma_commit(mbar);
  }
  if (ok) {  // -e has served as an operand and in the row dots for the last time (barrier above): dv = beta e in place
#pragma unroll
    for (int m = 0; m < 4; ++m) {
      const int u = tid + 256 * m, r = urow16(u);
      uint4* unit = reinterpret_cast<uint4*>(Xe + tc::sw128_unit(r, ucol16(u)));
      *unit = tc::scale_bf16x8(*unit, -bet[r]);
    }
  }
  if (ok) ok = tc::mbar_wait(mbar, ph);
  ph ^= 1;
  tc::fence_after_sync();
  ok = __all_sync(0xffffffffu, ok);  // warp-uniform: the epilogues below shuffle with a full mask
  float db_own = 0.f, dg_own = 0.f;
  if (ok) {  // Xy <- Mb = beta_i M, M = -dA*Gamma strictly lower, zeros elsewhere
    float f[32], ha[16], hk[16];
    ld_acc32(tB, warp, cb, f);
    split_block32(f, lane, ha);
    ld_acc32(tB + 64, warp, cb, f);
    split_block32(f, lane, hk);
    const int j0 = cb + 16 * hx;
    float rs = 0.f;
#pragma unroll
    for (int q = 0; q < 16; ++q) {
      const int j = j0 + q;
      const float mv = -ha[q] * exp_nonpos(gi - gam[j]);  // unconditional: the exponentials overlap
      const float M = (j < i) ? mv : 0.f;
      rs = fmaf(M, hk[q], rs);
      ha[q] = bi * M;
    }
#pragma unroll
    for (int x = 0; x < 2; ++x) sts16(Xy, tc::kmajor_unit(i, (j0 >> 3) + x, C), pack8(&ha[8 * x]));
    rs += __shfl_xor_sync(0xffffffffu, rs, 16);
    if (own) {
      db_own = vdot + di * kz + rs;
      dg_own = 2.f * bi * (di * kz + rs);
    }
  }
  if (ok) ok = tc::mbar_wait(mbar + 5, 0);  // q
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  // ---- batch 6: dPG^T q + Mb k + Mb^T k (one tile read K-major and MN-major), committed first: the dk epilogue
  //      runs while DQ += dPG k is still on the tensor core ----
  if (ok && tid == 0) {
    tc::issue_gemm(tB, tc::mnmajor_tile(Xpg, C), tc::mnmajor_sw128_tile(Xvn, 8192), 64, 128, C, false);
    tc::issue_gemm(tB, tc::kmajor_tile(Xy, C), tc::mnmajor_sw128_tile(Xk, 8192), 64, 128, C, true);
    tc::issue_gemm(tB, tc::mnmajor_tile(Xy, C), tc::mnmajor_sw128_tile(Xk, 8192), 64, 128, C, true);
    tc::mma_commit(mbar + 6);
    tc::issue_gemm(tA, tc::kmajor_tile(Xpg, C), tc::mnmajor_sw128_tile(Xk, 8192), 64, 128, C, true);
    tc::mma_commit(mbar);
  }
  if (ok) ok = tc::mbar_wait(mbar + 6, 0);
  tc::fence_after_sync();
  ok = __all_sync(0xffffffffu, ok);  // warp-uniform: the epilogues below shuffle with a full mask
  float rho = 0.f;
  if (ok) {  // dk = dkp + (dPG^T q + (Mb + Mb^T) k) + beta d z, assembled over dkp (each thread rewrites the units it read)
    float kd = 0.f;
    for (int s = 0; s < 2; ++s) {
      const int c0 = cw + 32 * s;
      float f[32], g2[16];
      ld_acc32(tB, warp, c0, f);
      split_block32(f, lane, g2);
      float r2[2] = {0.f, 0.f}, k2[2] = {0.f, 0.f};
#pragma unroll
      for (int x = 0; x < 2; ++x) {
        const int c8 = (c0 >> 3) + 2 * hx + x;
        float e[8], z[8], kr[8];
        unpack8(*reinterpret_cast<const uint4*>(Xdk + tc::sw128_unit(i, c8)), e);
        unpack8(*reinterpret_cast<const uint4*>(XdO + tc::kmajor_unit(i, c8, KD)), z);
        unpack8(*reinterpret_cast<const uint4*>(Xk + tc::sw128_unit(i, c8)), kr);
#pragma unroll
        for (int y = 0; y < 8; ++y) {
          r2[x] = fmaf(kr[y], e[y], r2[x]);              // k_i . dkp_i
          const float val = g2[8 * x + y] + e[y] + bd_i * z[y];
          k2[x] = fmaf(kr[y], val, k2[x]);               // k_i . dk_i
          g2[8 * x + y] = val;
        }
        sts16(Xdk, tc::sw128_unit(i, c8), pack8(&g2[8 * x]));
      }
      rho += r2[0] + r2[1];
      kd += k2[0] + k2[1];
    }
    rho += __shfl_xor_sync(0xffffffffu, rho, 16);
    kd += __shfl_xor_sync(0xffffffffu, kd, 16);
    dg_own -= kd;
  }
  if (ok) ok = tc::mbar_wait(mbar, ph);  // every product has completed
  ph ^= 1;
  tc::fence_after_sync();
  ok = __all_sync(0xffffffffu, ok);  // warp-uniform: the epilogues below shuffle with a full mask
  if (ok) {  // dq, assembled over q (each thread rewrites the units it read)
    float qd = 0.f;
    for (int s = 0; s < 2; ++s) {
      const int c0 = cw + 32 * s;
      float f[32], hq[16];
      ld_acc32(tA, warp, c0, f);
      split_block32(f, lane, hq);
#pragma unroll
      for (int x = 0; x < 2; ++x) {
        const int c8 = (c0 >> 3) + 2 * hx + x;
        float qr[8];
        unpack8(*reinterpret_cast<const uint4*>(Xvn + tc::sw128_unit(i, c8)), qr);
#pragma unroll
        for (int y = 0; y < 8; ++y) qd = fmaf(qr[y], hq[8 * x + y], qd);
        sts16(Xvn, tc::sw128_unit(i, c8), pack8(&hq[8 * x]));
      }
    }
    qd += __shfl_xor_sync(0xffffffffu, qd, 16);
    dg_own += qd;
  }
  {
    const float tot = warp_sum(own ? rho : 0.f);
    if (lane == 0) red[8 + warp] = tot;  // summed in a fixed order below (deterministic)
  }
  if (own) {  // the two column halves hold partial sums of the same row
    dgo[hc * C + i] = dg_own;
    dbo[hc * C + i] = db_own;
  }
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  if (ok && tid == 64) {  // dq, dk and dv leave by tiled stores (rows past the end of the sequence are clipped)
    for (int sl = 0; sl < 2; ++sl) {  // a slab that lies wholly past the true width is not stored at all
      if (64 * sl < p.Dk) {
        tc::tma_store_4d(&maps.dq, tc::smem_u32(Xvn) + 8192 * sl, 64 * sl, h, t0, b);
        tc::tma_store_4d(&maps.dk, tc::smem_u32(Xdk) + 8192 * sl, 64 * sl, h, t0, b);
      }
      if (64 * sl < p.Dv) tc::tma_store_4d(&maps.dv, tc::smem_u32(Xe) + 8192 * sl, 64 * sl, h, t0, b);
    }
    tc::bulk_commit();
  }
  if (tid < 32) {  // dg = reverse cumulative sum of dgam within the chunk: one warp, two rows per lane
    // d/dgam_last: E(gam_last) <dS, S0> and the sum over the rows of k_i . dkp_i
    float base = 0.f, kp = 0.f;
    for (int wv = 0; wv < 8; ++wv) { base += red[wv]; kp += red[8 + wv]; }
    base = L * base + kp;
    const int ra = C - 1 - 2 * tid, rb = ra - 1;
    float a = dgo[ra] + dgo[C + ra];
    float bq = dgo[rb] + dgo[C + rb];
    warp_rcumsum64(a, bq, tid);
    __syncwarp();  // every lane has read its rows before any lane overwrites them
    dgo[ra] = base + a;
    dgo[rb] = base + bq;
  }
  __syncthreads();
  if (!ok && tid == 0) atomicExch(p.status, 4);
  if (ok && tid < imax) {
    p.dbeta[row(tid)] = dbo[tid] + dbo[C + tid];
    float dg = dgo[tid];
    const float gin = p.gate[row(tid)];
    if (p.gate_is_log) {
      if (gin < kLogGateFloor) dg = 0.f;
    } else {
      dg = (gin > kGateFloor) ? dg / gin : 0.f;
    }
    p.dgate[row(tid)] = dg;
  }
  if (tid == 64) tc::bulk_wait_read<0>();  // shared memory must outlive the stores
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tA, 256);
}

// ------------------------------------------------------------------ host
mxb_status tc_run_fwd(TcP& p, cudaStream_t st);

template <typename KernelT>
static mxb_status bwd_set_smem(KernelT kern, int bytes) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) { set_last_cuda_error((int)e); return MXB_ERR_CUDA; }
  return MXB_OK;
}

// Forward recompute (saving per-chunk states and v_new), reverse state pass, per-chunk pass.
mxb_status tc_run_bwd(TcP& p, bool recompute, cudaStream_t st) {
  p.save = 1;
  mxb_status s = MXB_OK;
  if (recompute) {
    bf16* keep_out = p.out;
    float* keep_hT = p.hT;
    p.out = p.dv;  // the recomputed forward output is not needed; dv is overwritten afterwards
    p.hT = nullptr;
    s = tc_run_fwd(p, st);
    p.out = keep_out;
    p.hT = keep_hT;
    if (s != MXB_OK) return s;
  }
  RowMaps maps;
  std::memset(&maps, 0, sizeof maps);
  const bool narrow = p.Dk != KD || p.Dv != KD;  // narrower heads exist only through the copy engine
  const bool tma = (!p.no_tma || narrow) && make_tma_map_bthd(&maps.k, p.k, p.B, p.T, p.H, p.Dk) &&
                   make_tma_map_bthd(&maps.q, p.q, p.B, p.T, p.H, p.Dk) && make_tma_map_bthd(&maps.v, p.v, p.B, p.T, p.H, p.Dv) &&
                   make_tma_map_bthd(&maps.dO, p.dO, p.B, p.T, p.H, p.Dv);
  if (narrow && !tma) return MXB_ERR_UNSUPPORTED;
  if (tma) {
    if (bwd_set_smem(gdn_tc_state_bwd_kernel<true>, kStateBwdSmem) != MXB_OK) return MXB_ERR_CUDA;
    MXB_LAUNCH("gdn_tc_state_bwd_kernel", st,
               (gdn_tc_state_bwd_kernel<true><<<dim3(p.B * p.H), 256, kStateBwdSmem, st>>>(p, maps)));
  } else {
    if (bwd_set_smem(gdn_tc_state_bwd_kernel<false>, kStateBwdSmem) != MXB_OK) return MXB_ERR_CUDA;
    MXB_LAUNCH("gdn_tc_state_bwd_kernel", st,
               (gdn_tc_state_bwd_kernel<false><<<dim3(p.B * p.H), 256, kStateBwdSmem, st>>>(p, maps)));
  }
  s = check_launch("gdn_tc_state_bwd_kernel");
  if (s != MXB_OK) return s;
  // The chunk kernel is fed and drained by the copy engine only (also under MXB_GDN_NO_TMA, which selects the
  // per-thread staging of the kernels that have one): it needs the tensor maps.
  if (!tma) {
    std::memset(&maps, 0, sizeof maps);
    if (!(make_tma_map_bthd(&maps.k, p.k, p.B, p.T, p.H, p.Dk) && make_tma_map_bthd(&maps.q, p.q, p.B, p.T, p.H, p.Dk) &&
          make_tma_map_bthd(&maps.v, p.v, p.B, p.T, p.H, p.Dv) && make_tma_map_bthd(&maps.dO, p.dO, p.B, p.T, p.H, p.Dv)))
      return MXB_ERR_UNSUPPORTED;
  }
  if (!(make_tma_map_bthd(&maps.dq, p.dq, p.B, p.T, p.H, p.Dk) && make_tma_map_bthd(&maps.dk, p.dk, p.B, p.T, p.H, p.Dk) &&
        make_tma_map_bthd(&maps.dv, p.dv, p.B, p.T, p.H, p.Dv)))
    return MXB_ERR_UNSUPPORTED;
  if (bwd_set_smem(gdn_tc_chunk_bwd_kernel, kChunkBwdSmem) != MXB_OK) return MXB_ERR_CUDA;
  MXB_LAUNCH("gdn_tc_chunk_bwd_kernel", st,
             (gdn_tc_chunk_bwd_kernel<<<dim3(p.B * p.H, p.n), 256, kChunkBwdSmem, st>>>(p, maps)));
  return check_launch("gdn_tc_chunk_bwd_kernel");
}

}  // namespace mxb

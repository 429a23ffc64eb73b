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
//   gdn_tc_chunk_bwd_state_kernel  one CTA per chunk: the contractions with the saved states S0 and dS
//   gdn_tc_chunk_bwd_kernel  one CTA per chunk, everything else:
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
    const float4* src = reinterpret_cast<const float4*>(p.dhT_in + ((size_t)bh * KD + kk) * KD + j0);
#pragma unroll
    for (int x = 0; x < 16; ++x) {
      const float4 t4 = __ldg(src + x);
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
  if (ok && p.dh0) {
    float4* dst = reinterpret_cast<float4*>(p.dh0 + ((size_t)bh * KD + kk) * KD + j0);
#pragma unroll
    for (int x = 0; x < 16; ++x) dst[x] = make_float4(dS[4 * x], dS[4 * x + 1], dS[4 * x + 2], dS[4 * x + 3]);
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(taddr, 512);
}

// ------------------------------------------------- chunk backward, part 2: everything else
// 256 TMEM columns and 108 KB of shared memory: two CTAs share an SM.  TMEM column map (fp32 columns; all
// accumulators are M=64, so row i of every result sits in TMEM lane (i%16) + 32*(i/16) and is handled by
// thread (warp i/16, lane i%16); warps 4-7 take the second half of the columns):
//   1: T^T dv_new [0,128)             z = T^T dw [128,256)      (both rewritten to shared memory as bf16)
//   2: (T^T dv_new) v^T [0,64)        z k^T [64,128)            k k^T [128,192)   q k^T [192,256)
//   3: Y T^T [0,64)   with Y = T^T dT assembled from phase 2
//   4: (dP*Gamma) k [0,128)           (dP*Gamma)^T q + (Mb + Mb^T) k [128,256)
constexpr int kChunkBwdSmem = 5 * 16384 + 3 * 8192 + 13 * C * 4 + 64 + 1024;

__device__ __forceinline__ void unpack8(uint4 v, float (&e)[8]) {
  tc::unpack_bf16(v.x, e[0], e[1]); tc::unpack_bf16(v.y, e[2], e[3]);
  tc::unpack_bf16(v.z, e[4], e[5]); tc::unpack_bf16(v.w, e[6], e[7]);
}
__device__ __forceinline__ uint4 pack8(const float* e) {
  return make_uint4(tc::pack_bf16(e[0], e[1]), tc::pack_bf16(e[2], e[3]), tc::pack_bf16(e[4], e[5]),
                    tc::pack_bf16(e[6], e[7]));
}
// sum_k tile[row][c0 + k] * f[k], k < 32, for a blocked [.][128] bf16 tile in shared memory
template <bool SW>
__device__ __forceinline__ float row_dot32(const uint8_t* tile, int r, int c0, const float (&f)[32]) {
  // the four units are fetched first and summed in four independent chains (one chain of 32 dependent FMAs
  // would cost ~130 cycles of latency on its own)
  uint4 raw[4];
#pragma unroll
  for (int x = 0; x < 4; ++x) raw[x] = *reinterpret_cast<const uint4*>(tile + in_unit<SW>(r, (c0 >> 3) + x));
  float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int x = 0; x < 4; ++x) {
    float e[8];
    unpack8(raw[x], e);
#pragma unroll
    for (int y = 0; y < 8; ++y) s[x] = fmaf(e[y], f[8 * x + y], s[x]);
  }
  return (s[0] + s[1]) + (s[2] + s[3]);
}

// ------------------------------------------------- chunk backward, part 1: state contractions
// Per chunk: everything that needs the saved states.  256 TMEM columns and 97 KB of shared memory, so two
// CTAs share an SM.  S0 and dS use the same shared-memory buffer one after the other.  The four results are
// assembled in shared memory in the blocked operand layout and leave as contiguous 16 KB / 8 KB bulk
// copies; the second kernel loads those byte images back unchanged.
//   phase 1: dO S0^T [0,128), (-dv_new) S0^T [128,256) -> dqp = d (dO S0^T), dw = -dv_new S0^T
//   phase 2: v_new dS^T [0,128), dO v_new^T [128,192) -> dkp = r (v_new dS^T), dP*Gamma, L <dS, S0>
constexpr int kChunkBwdStateSmem = 4 * 16384 + 32768 + 4 * C * 4 + 64 + 1024;

template <bool TMA>
__global__ void __launch_bounds__(256, 2) gdn_tc_chunk_bwd_state_kernel(TcP p, const __grid_constant__ RowMaps maps) {
  extern __shared__ uint8_t raw[];
  uint8_t* sm = raw + ((1024u - (tc::smem_u32(raw) & 1023u)) & 1023u);
  uint8_t* Xdo = sm;                // [64][128] dO            -> later the dkp image
  uint8_t* Xdvn = Xdo + 16384;      // [64][128] -dv_new       -> later the dqp image
  uint8_t* Xvn = Xdvn + 16384;      // [64][128] v_new         -> later the dP*Gamma image (first half)
  uint8_t* Xst = Xvn + 16384;       // the dw image
  uint8_t* Xs = Xst + 16384;        // [128][128] S0, then dS
  float* gam = reinterpret_cast<float*>(Xs + 32768);
  float* dd = gam + C;
  float* rr = dd + C;
  float* red = rr + C;
  uint64_t* mbar = reinterpret_cast<uint64_t*>(red + C);  // [0] MMA, [1] dO/dv_new/S0, [2] v_new, [3] dS
  uint32_t* tslot = reinterpret_cast<uint32_t*>(mbar + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x, bh = blockIdx.y, b = bh / p.H, h = bh % p.H, t0 = c * C;
  const size_t ci = (size_t)bh * p.n + c;
  const int imax = min(C, p.T - t0);
  auto row = [&](int i) { return ((size_t)(b * p.T + t0 + i) * p.H + h); };
  const bool own = lane < 16;
  const int i = 16 * (warp & 3) + (lane & 15), hc = warp >> 2;

  // prologue latencies side by side: warp 0 allocates TMEM, one thread of warp 1 issues the copies, warp 2-3 fetch gam
  if (tid == 32) {
    for (int m = 0; m < 4; ++m) tc::mbar_init(mbar + m, 1);
    tc::mbar_fence_init();
    if (TMA) {  // dO by the copy engine (swizzled tile), the workspace images by bulk copies
      tc::mbar_expect_tx(mbar + 1, 2 * 16384 + 32768);
      tc::tma_load_4d(tc::smem_u32(Xdo), &maps.dO, 0, h, t0, b, mbar + 1);
      tc::tma_load_4d(tc::smem_u32(Xdo) + 8192, &maps.dO, 64, h, t0, b, mbar + 1);
      tc::bulk_load(tc::smem_u32(Xdvn), p.dvn + ci * C * KD, 16384, mbar + 1);
      tc::bulk_load(tc::smem_u32(Xs), p.hs + ci * KD * KD, 32768, mbar + 1);
      tc::mbar_expect_tx(mbar + 2, 16384);
      tc::bulk_load(tc::smem_u32(Xvn), p.vn + ci * C * KD, 16384, mbar + 2);
    }
  }
  if (!TMA) {  // group 0: dO, dv_new, S0   group 1: v_new
    const uint32_t sdo = tc::smem_u32(Xdo), sdvn = tc::smem_u32(Xdvn), svn = tc::smem_u32(Xvn), ss = tc::smem_u32(Xs);
    for (int u = tid; u < 64 * 16; u += 256) {
      const int r = urow16(u), c8 = ucol16(u);
      const uint32_t off = tc::kmajor_unit(r, c8, KD);
      tc::cp_async16(sdo + off, r < imax ? p.dO + row(r) * KD + c8 * 8 : p.dO, r < imax);
      tc::cp_async16(sdvn + 16 * u, p.dvn + ci * C * KD + 8 * u);  // byte images of the operand tiles from here on
    }
    for (int u = tid; u < 128 * 16; u += 256) tc::cp_async16(ss + 16 * u, p.hs + ci * KD * KD + 8 * u);
    tc::cp_async_commit();
    for (int u = tid; u < 64 * 16; u += 256) tc::cp_async16(svn + 16 * u, p.vn + ci * C * KD + 8 * u);
    tc::cp_async_commit();
  }
  if (warp == 0) {
    tc::tmem_alloc(tslot, 256);
    tc::tmem_relinquish();
  }
  if (tid >= 64 && tid < 64 + C) gam[tid - 64] = p.gam[ci * C + tid - 64];
  __syncthreads();
  const float glast = gam[C - 1], L = exp_nonpos(glast);
  if (tid < C) {
    dd[tid] = exp_nonpos(gam[tid]);
    rr[tid] = exp_nonpos(glast - gam[tid]);
  }
  bool ok = true;
  if (TMA) ok = tc::mbar_wait(mbar + 1, 0);
  else tc::cp_async_wait<1>();
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t taddr = *tslot;
  if (tid == 0) {
    tc::issue_gemm(taddr + 0, in_kmajor<TMA>(Xdo), tc::kmajor_tile(Xs, KD), 64, 128, KD, false);          // dO S0^T
    tc::issue_gemm(taddr + 128, tc::kmajor_tile(Xdvn, KD), tc::kmajor_tile(Xs, KD), 64, 128, KD, false);  // -dv_new S0^T
    tc::mma_commit(mbar);
  }
  uint4 s0u[8];  // this thread's 8 units of S0, kept for <dS, S0> (the buffer is about to be reused)
#pragma unroll
  for (int x = 0; x < 8; ++x) s0u[x] = *reinterpret_cast<const uint4*>(Xs + (tid + 256 * x) * 16);
  if (TMA) {  // every thread has taken its units before one thread lets the copy engine overwrite the buffer
    tc::fence_async_smem();
    __syncthreads();
  }
  if (ok) ok = tc::mbar_wait(mbar, 0);
  tc::fence_after_sync();
  // S0 is dead in shared memory: fetch dS into the same buffer behind the epilogue
  if (TMA) {
    if (tid == 0) {
      tc::mbar_expect_tx(mbar + 3, 32768);
      tc::bulk_load(tc::smem_u32(Xs), p.dhs + ci * KD * KD, 32768, mbar + 3);
    }
  } else {
    const uint32_t ss = tc::smem_u32(Xs);
    for (int u = tid; u < 128 * 16; u += 256) tc::cp_async16(ss + 16 * u, p.dhs + ci * KD * KD + 8 * u);
    tc::cp_async_commit();
  }
  const float di = dd[i], ri = rr[i], gi = gam[i];
  if (ok) {
    for (int c0 = 64 * hc; c0 < 64 * hc + 64; c0 += 32) {
      float f[32];
      ld_acc32(taddr + 0, warp, c0, f);
      if (own) {
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) f[jj] *= di;
#pragma unroll
        for (int x = 0; x < 4; ++x) sts16(Xdvn, tc::kmajor_unit(i, (c0 >> 3) + x, KD), pack8(&f[8 * x]));
      }
      ld_acc32(taddr + 128, warp, c0, f);
      if (own) {  // the workspace holds -dv_new, so this is dw = -dv_new S0^T already
#pragma unroll
        for (int x = 0; x < 4; ++x) sts16(Xst, tc::kmajor_unit(i, (c0 >> 3) + x, KD), pack8(&f[8 * x]));
      }
    }
  }
  if (TMA) {  // v_new and dS
    if (ok) ok = tc::mbar_wait(mbar + 2, 0);
    if (ok) ok = tc::mbar_wait(mbar + 3, 0);
  } else {
    tc::cp_async_wait<0>();
  }
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  if (ok && tid == 0) {
    tc::issue_gemm(taddr + 0, tc::kmajor_tile(Xvn, KD), tc::kmajor_tile(Xs, KD), 64, 128, KD, false);    // v_new dS^T
    tc::issue_gemm(taddr + 128, in_kmajor<TMA>(Xdo), tc::kmajor_tile(Xvn, KD), 64, 64, KD, false);     // dO v_new^T
    tc::mma_commit(mbar);
    tc::bulk_store(p.dqp + ci * C * KD, tc::smem_u32(Xdvn), 16384);
    tc::bulk_store(p.dw + ci * C * KD, tc::smem_u32(Xst), 16384);
    tc::bulk_commit();
  }
  {  // <dS, S0>
    float part = 0.f;
#pragma unroll
    for (int x = 0; x < 8; ++x) {
      float a[8], bq[8];
      unpack8(*reinterpret_cast<const uint4*>(Xs + (tid + 256 * x) * 16), a);
      unpack8(s0u[x], bq);
#pragma unroll
      for (int y = 0; y < 8; ++y) part = fmaf(a[y], bq[y], part);
    }
    part = warp_sum(part);
    if (lane == 0) red[warp] = part;
  }
  if (ok) ok = tc::mbar_wait(mbar, 1);
  tc::fence_after_sync();
  if (ok) {
    for (int c0 = 64 * hc; c0 < 64 * hc + 64; c0 += 32) {  // dkp = r (v_new dS^T)   (dO is dead: reuse its tile)
      float f[32];
      ld_acc32(taddr + 0, warp, c0, f);
      if (own) {
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) f[jj] *= ri;
#pragma unroll
        for (int x = 0; x < 4; ++x) sts16(Xdo, tc::kmajor_unit(i, (c0 >> 3) + x, KD), pack8(&f[8 * x]));
      }
    }
    {  // dP * Gamma, lower incl. diagonal (32 columns per half)   (v_new is dead: reuse its tile)
      const int c0 = 32 * hc;
      float f[32];
      ld_acc32(taddr + 128, warp, c0, f);
      if (own) {
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) {
          const int j = c0 + jj;
          const float val = f[jj] * exp_nonpos(gi - gam[j]);  // unconditional: the exponentials overlap
          f[jj] = (j <= i) ? val : 0.f;
        }
#pragma unroll
        for (int x = 0; x < 4; ++x) sts16(Xvn, tc::kmajor_unit(i, (c0 >> 3) + x, C), pack8(&f[8 * x]));
      }
    }
  } else if (tid == 0) {
    atomicExch(p.status, 5);
  }
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  if (tid == 0) {
    if (ok) {
      tc::bulk_store(p.dkp + ci * C * KD, tc::smem_u32(Xdo), 16384);
      tc::bulk_store(p.dpg + ci * C * C, tc::smem_u32(Xvn), 8192);
      tc::bulk_commit();
    }
    float s = 0.f;
    for (int wv = 0; wv < 8; ++wv) s += red[wv];
    p.ls[ci] = L * s;  // d/dgam_last of E(gam_last) <dS, S0>
    tc::bulk_wait_read<0>();  // shared memory must outlive the copies
  }
  if (warp == 0) tc::tmem_dealloc(taddr, 256);
}

// TMA = true: k, q, v by the copy engine (128-byte-swizzled tiles) and every workspace image by bulk copies, all
// completing on mbarriers; TMA = false: cp.async staging in the un-swizzled layout.
template <bool TMA>
__global__ void __launch_bounds__(256, 2) gdn_tc_chunk_bwd_kernel(TcP p, const __grid_constant__ RowMaps maps) {
  extern __shared__ uint8_t raw[];
  uint8_t* sm = raw + ((1024u - (tc::smem_u32(raw) & 1023u)) & 1023u);
  uint8_t* Xk = sm;                 // [64][128] k
  uint8_t* Xq = Xk + 16384;         // [64][128] q
  uint8_t* Xv = Xq + 16384;         // [64][128] v; then Y = T^T dT (first half); then the dqp image -> dq
  uint8_t* X2 = Xv;
  uint8_t* Xdvn = Xv + 16384;       // [64][128] -dv_new, then T^T dv_new in place; then the dkp image -> dk
  uint8_t* Xdw = Xdvn + 16384;      // [64][128] dw, then z = T^T dw in place
  uint8_t* Xt = Xdw + 16384;        // [64][64]  T
  uint8_t* Xpg = Xt + 8192;         // [64][64]  dP*Gamma
  uint8_t* X1 = Xpg + 8192;         // [64][64]  Mb + Mb^T
  float* gam = reinterpret_cast<float*>(X1 + 8192);
  float* bet = gam + C;
  float* dd = bet + C;
  float* rr = dd + C;
  float* dgo = rr + C;              // [2][C] per-row dgam / dbeta partials of the two column halves
  float* dbo = dgo + 2 * C;
  float* red = dbo + 2 * C;
  float* csw = red + C;             // [4 warps][C] per-warp column sums (no atomics)
  uint64_t* mbar = reinterpret_cast<uint64_t*>(csw + 4 * C);  // [0] MMA, [1] dv_new/dw/T, [2] k/q/v/dP*Gamma, [3] dqp/dkp
  uint32_t* tslot = reinterpret_cast<uint32_t*>(mbar + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x, bh = blockIdx.y, b = bh / p.H, h = bh % p.H, t0 = c * C;
  const size_t ci = (size_t)bh * p.n + c;
  const int imax = min(C, p.T - t0);
  auto row = [&](int i) { return ((size_t)(b * p.T + t0 + i) * p.H + h); };
  const bool own = lane < 16;
  const int i = 16 * (warp & 3) + (lane & 15);  // the row this thread owns in every epilogue
  const int hc = warp >> 2;  // warps 0-3 take the first half of an accumulator's columns, warps 4-7 the second

  // The serial latencies of the prologue run side by side on different warps: warp 0 allocates TMEM, one thread
  // each of warps 1 and 4 initialises two barriers and issues the copies that complete on them, warps 2-3 fetch
  // the per-row scalars.
  if (tid == 32) {
    tc::mbar_init(mbar + 0, 1);
    tc::mbar_init(mbar + 5, 1);  // second MMA barrier: a phase with two commits never puts both on one barrier (a waiter
                                 // that falls two phases behind a single barrier would wait for a third)
    tc::mbar_init(mbar + 1, 1);
    tc::mbar_fence_init();
    if (TMA) {
      tc::mbar_expect_tx(mbar + 1, 2 * 16384 + 8192);
      tc::bulk_load(tc::smem_u32(Xdvn), p.dvn + ci * C * KD, 16384, mbar + 1);  // byte images of the operand tiles
      tc::bulk_load(tc::smem_u32(Xdw), p.dw + ci * C * KD, 16384, mbar + 1);
      tc::bulk_load(tc::smem_u32(Xt), p.Tm + ci * C * C, 8192, mbar + 1);
    }
  }
  if (tid == 128) {
    tc::mbar_init(mbar + 2, 1);
    tc::mbar_init(mbar + 3, 1);
    tc::mbar_fence_init();
    if (TMA) {
      tc::mbar_expect_tx(mbar + 2, 3 * 16384 + 8192);
      for (int sl = 0; sl < 2; ++sl) {
        tc::tma_load_4d(tc::smem_u32(Xk) + 8192 * sl, &maps.k, 64 * sl, h, t0, b, mbar + 2);
        tc::tma_load_4d(tc::smem_u32(Xq) + 8192 * sl, &maps.q, 64 * sl, h, t0, b, mbar + 2);
        tc::tma_load_4d(tc::smem_u32(Xv) + 8192 * sl, &maps.v, 64 * sl, h, t0, b, mbar + 2);
      }
      tc::bulk_load(tc::smem_u32(Xpg), p.dpg + ci * C * C, 8192, mbar + 2);
    }
  }
  if (!TMA) {  // group 0: dv_new, dw, T   group 1: k, q, v, dP*Gamma
    const uint32_t sk = tc::smem_u32(Xk), sq = tc::smem_u32(Xq), sv = tc::smem_u32(Xv);
    const uint32_t sdvn = tc::smem_u32(Xdvn), sdw = tc::smem_u32(Xdw);
    const uint32_t st = tc::smem_u32(Xt), spg = tc::smem_u32(Xpg);
    for (int u = tid; u < 64 * 16; u += 256) {
      const int r = urow16(u), c8 = ucol16(u);
      const uint32_t off = tc::kmajor_unit(r, c8, KD);
      tc::cp_async16(sdvn + 16 * u, p.dvn + ci * C * KD + 8 * u);  // byte images of the operand tiles (-dv_new, dw)
      tc::cp_async16(sdw + 16 * u, p.dw + ci * C * KD + 8 * u);
    }
    for (int u = tid; u < 64 * 8; u += 256) {
      const int r = urow8(u), c8 = ucol8(u);
      tc::cp_async16(st + 16 * u, p.Tm + ci * C * C + 8 * u);
    }
    tc::cp_async_commit();
    for (int u = tid; u < 64 * 16; u += 256) {
      const int r = urow16(u), c8 = ucol16(u);
      const uint32_t off = tc::kmajor_unit(r, c8, KD);
      const bool v = r < imax;
      const size_t g = v ? row(r) * KD + c8 * 8 : 0;
      tc::cp_async16(sk + off, p.k + g, v);
      tc::cp_async16(sq + off, p.q + g, v);
      tc::cp_async16(sv + off, p.v + g, v);
    }
    for (int u = tid; u < 64 * 8; u += 256) {
      const int r = urow8(u), c8 = ucol8(u);
      tc::cp_async16(spg + 16 * u, p.dpg + ci * C * C + 8 * u);
      (void)r; (void)c8;
    }
    tc::cp_async_commit();
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
  for (int u = tid; u < 4 * C; u += 256) csw[u] = 0.f;
  __syncthreads();
  const float glast = gam[C - 1];
  if (tid < C) {
    dd[tid] = exp_nonpos(gam[tid]);
    rr[tid] = exp_nonpos(glast - gam[tid]);
  }
  bool ok = true;
  if (TMA) ok = tc::mbar_wait(mbar + 1, 0);
  else tc::cp_async_wait<1>();
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t taddr = *tslot;
  uint32_t ph = 0;
  // ---- phase 1: T^T dv_new and z = T^T dw (both operands contracted over their rows) ----
  if (tid == 0) {
    tc::issue_gemm(taddr + 0, tc::mnmajor_tile(Xt, C), tc::mnmajor_tile(Xdvn, KD), 64, 128, C, false);
    tc::issue_gemm(taddr + 128, tc::mnmajor_tile(Xt, C), tc::mnmajor_tile(Xdw, KD), 64, 128, C, false);
    tc::mma_commit(mbar);
  }
  if (TMA) { if (ok) ok = tc::mbar_wait(mbar + 2, 0); }  // k, q, v, dP*Gamma
  else tc::cp_async_wait<0>();
  __syncthreads();
  if (ok) ok = tc::mbar_wait(mbar, ph);
  ph ^= 1;
  tc::fence_after_sync();
  float dg_own = 0.f, db_own = 0.f;
  const float gi = gam[i], bi = bet[i], di = dd[i], ri = rr[i];
  const float bd_i = bi * di;
  const int cb = 32 * hc;  // this thread's 32 columns of every [64][64] accumulator
  const int cw = 64 * hc;  // this thread's 64 columns of every [64][128] accumulator
  if (ok) {
    // Both products go back to shared memory as bf16 operands of phase 2, over the operands they were
    // computed from (their MMAs are complete); dv = beta (T^T dv_new) leaves from there after phase 2.
    float vdot = 0.f, kz = 0.f;
    for (int s = 0; s < 2; ++s) {
      const int c0 = cw + 32 * s;
      float f[32];
      ld_acc32(taddr + 0, warp, c0, f);
      if (own) {
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) f[jj] = -f[jj];  // the workspace holds -dv_new
        vdot += row_dot32<TMA>(Xv, i, c0, f);
#pragma unroll
        for (int x = 0; x < 4; ++x) sts16(Xdvn, tc::kmajor_unit(i, (c0 >> 3) + x, KD), pack8(&f[8 * x]));
      }
      ld_acc32(taddr + 128, warp, c0, f);
      if (own) {
        kz += row_dot32<TMA>(Xk, i, c0, f);
#pragma unroll
        for (int x = 0; x < 4; ++x) sts16(Xdw, tc::kmajor_unit(i, (c0 >> 3) + x, KD), pack8(&f[8 * x]));
      }
    }
    if (own) {
      db_own += vdot + di * kz;
      dg_own += bd_i * kz;
    }
  }
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  // ---- phase 2: Y = T^T dT = (T^T dv_new)(v beta)^T + z (k beta d)^T, with the column scales applied in the
  //      epilogue; k k^T and q k^T ride along.  Two commits: the Y epilogue (all the next MMA needs) runs while
  //      the tensor core still works on k k^T and q k^T ----
  if (ok && tid == 0) {
    tc::issue_gemm(taddr + 0, tc::kmajor_tile(Xdvn, KD), in_kmajor<TMA>(Xv), 64, 64, KD, false);
    tc::issue_gemm(taddr + 64, tc::kmajor_tile(Xdw, KD), in_kmajor<TMA>(Xk), 64, 64, KD, false);
    tc::mma_commit(mbar);
    tc::issue_gemm(taddr + 128, in_kmajor<TMA>(Xk), in_kmajor<TMA>(Xk), 64, 64, KD, false);  // k k^T
    tc::issue_gemm(taddr + 192, in_kmajor<TMA>(Xq), in_kmajor<TMA>(Xk), 64, 64, KD, false);  // q k^T
    tc::mma_commit(mbar + 5);
  }
  if (ok) {
    ok = tc::mbar_wait(mbar, ph);
    ph ^= 1;
  }
  tc::fence_after_sync();
  if (ok) {  // Y[i][m] = beta_m ((T^T dv_new)_i . v_m) + beta_m d_m (z_i . k_m)   -> X2 (v is dead)
    float f[32], f2[32];
    ld_acc32(taddr + 0, warp, cb, f);
    ld_acc32(taddr + 64, warp, cb, f2);
    if (own) {
#pragma unroll
      for (int jj = 0; jj < 32; ++jj) f[jj] = bet[cb + jj] * fmaf(dd[cb + jj], f2[jj], f[jj]);
#pragma unroll
      for (int x = 0; x < 4; ++x) sts16(X2, tc::kmajor_unit(i, (cb >> 3) + x, C), pack8(&f[8 * x]));
    }
  }
  if (ok) ok = tc::mbar_wait(mbar + 5, 0);
  tc::fence_after_sync();
  float KKr[32];  // (k_i . k_j) for j in [cb, cb+32)
  if (ok) {
    float f[32];
    ld_acc32(taddr + 192, warp, cb, f);  // q k^T: dgam from P
    {
      float rs = 0.f;
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        float e[8];
        unpack8(*reinterpret_cast<const uint4*>(Xpg + tc::kmajor_unit(i, (cb >> 3) + x, C)), e);
#pragma unroll
        for (int y = 0; y < 8; ++y) {
          const int j = cb + 8 * x + y;
          const float X = (own && j <= i) ? e[y] * f[8 * x + y] : 0.f;
          rs += X;
          f[8 * x + y] = X;
        }
      }
      dg_own += rs;
      colsum16(f, lane);  // over the 16 rows this warp owns
      if (own) {
        float* dst = csw + (warp & 3) * C + cb + colsum16_col(lane);
        dst[0] -= f[0];
        dst[1] -= f[1];
      }
    }
    ld_acc32(taddr + 128, warp, cb, KKr);  // k k^T
  }
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  // ---- phase 3: dA = tril(Y T^T, -1) ----
  if (ok && tid == 0) {
    tc::issue_gemm(taddr + 0, tc::kmajor_tile(X2, C), tc::kmajor_tile(Xt, C), 64, 64, C, false);
    tc::mma_commit(mbar);
  }
  if (ok) {  // dv = beta (T^T dv_new), from the bf16 tile, in 64-byte row pieces
    for (int u = tid; u < 64 * 16; u += 256) {
      const int r = urow16(u), c8 = ucol16(u);
      if (r < imax)
        *reinterpret_cast<uint4*>(p.dv + row(r) * KD + c8 * 8) =
            tc::scale_bf16x8(*reinterpret_cast<const uint4*>(Xdvn + tc::kmajor_unit(r, c8, KD)), bet[r]);
    }
  }
  if (ok) {
    ok = tc::mbar_wait(mbar, ph);
    ph ^= 1;
  }
  tc::fence_after_sync();
  tc::fence_async_smem();
  __syncthreads();  // every thread is done with the T^T dv_new tile; Y (over v) has been consumed by the MMA
  // the state contractions from the first kernel land over v and T^T dv_new while phase 3's epilogue runs
  if (TMA) {
    if (tid == 0) {
      tc::mbar_expect_tx(mbar + 3, 2 * 16384);
      tc::bulk_load(tc::smem_u32(Xv), p.dqp + ci * C * KD, 16384, mbar + 3);
      tc::bulk_load(tc::smem_u32(Xdvn), p.dkp + ci * C * KD, 16384, mbar + 3);
    }
  } else {
    const uint32_t sqp = tc::smem_u32(Xv), skp = tc::smem_u32(Xdvn);
    for (int u = tid; u < 64 * 16; u += 256) {
      tc::cp_async16(sqp + 16 * u, p.dqp + ci * C * KD + 8 * u);
      tc::cp_async16(skp + 16 * u, p.dkp + ci * C * KD + 8 * u);
    }
    tc::cp_async_commit();
  }
  if (ok) {  // X1 <- Mb = beta_i M, strictly lower triangle, zeros elsewhere
    float f[32];
    ld_acc32(taddr + 0, warp, cb, f);
    float rs = 0.f;
#pragma unroll
    for (int jj = 0; jj < 32; ++jj) {
      const int j = cb + jj;
      const float mv = -f[jj] * exp_nonpos(gi - gam[j]);  // unconditional: the exponentials overlap
      const float M = (own && j < i) ? mv : 0.f;         // -dA * Gamma
      const float t = M * KKr[jj];
      rs += t;
      KKr[jj] = bi * t;
      f[jj] = bi * M;
    }
    if (own) {
#pragma unroll
      for (int x = 0; x < 4; ++x) sts16(X1, tc::kmajor_unit(i, (cb >> 3) + x, C), pack8(&f[8 * x]));
    }
    db_own += rs;
    dg_own += bi * rs;
    colsum16(KKr, lane);
    if (own) {
      float* dst = csw + (warp & 3) * C + cb + colsum16_col(lane);
      dst[0] -= KKr[0];
      dst[1] -= KKr[1];
    }
  }
  if (TMA) { if (ok) ok = tc::mbar_wait(mbar + 3, 0); }
  else tc::cp_async_wait<0>();
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  // ---- phase 4: (dP*Gamma) k  and  (dP*Gamma)^T q + (Mb + Mb^T) k ----
  if (ok && tid == 0) {
    tc::issue_gemm(taddr + 0, tc::kmajor_tile(Xpg, C), in_mnmajor<TMA>(Xk), 64, 128, C, false);
    tc::mma_commit(mbar);  // the dq epilogue runs while the three products of dk are still on the tensor core
    tc::issue_gemm(taddr + 128, tc::mnmajor_tile(Xpg, C), in_mnmajor<TMA>(Xq), 64, 128, C, false);
    tc::issue_gemm(taddr + 128, tc::kmajor_tile(X1, C), in_mnmajor<TMA>(Xk), 64, 128, C, true);
    tc::issue_gemm(taddr + 128, tc::mnmajor_tile(X1, C), in_mnmajor<TMA>(Xk), 64, 128, C, true);
    tc::mma_commit(mbar + 5);
  }
  if (ok) {
    ok = tc::mbar_wait(mbar, ph);
    ph ^= 1;
  }
  tc::fence_after_sync();
  // dq and dk are assembled over the dqp / dkp images (each thread rewrites the units it read)
  float qdot = 0.f, kdot = 0.f;
  if (ok) {
    for (int s = 0; s < 2; ++s) {
      const int c0 = cw + 32 * s;
      float f[32], g2[32];
      ld_acc32(taddr + 0, warp, c0, g2);  // (dP*Gamma) k
      if (own) {
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          float e[8];
          unpack8(*reinterpret_cast<const uint4*>(Xv + tc::kmajor_unit(i, (c0 >> 3) + x, KD)), e);
#pragma unroll
          for (int y = 0; y < 8; ++y) f[8 * x + y] = e[y];
        }
        qdot += row_dot32<TMA>(Xq, i, c0, f);  // q_i . d_i dqi_i
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) g2[jj] += f[jj];
#pragma unroll
        for (int x = 0; x < 4; ++x) sts16(Xv, tc::kmajor_unit(i, (c0 >> 3) + x, KD), pack8(&g2[8 * x]));
      }
    }
  }
  if (ok) ok = tc::mbar_wait(mbar + 5, 1);
  tc::fence_after_sync();
  if (ok) {
    for (int s = 0; s < 2; ++s) {
      const int c0 = cw + 32 * s;
      float f[32], g2[32];
      ld_acc32(taddr + 128, warp, c0, g2);  // (dP*Gamma)^T q + (Mb+Mb^T) k
      if (own) {
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          float e[8];
          unpack8(*reinterpret_cast<const uint4*>(Xdvn + tc::kmajor_unit(i, (c0 >> 3) + x, KD)), e);
#pragma unroll
          for (int y = 0; y < 8; ++y) f[8 * x + y] = e[y];
        }
        kdot += row_dot32<TMA>(Xk, i, c0, f);  // k_i . r_i dkt_i
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          float z[8];
          unpack8(*reinterpret_cast<const uint4*>(Xdw + tc::kmajor_unit(i, (c0 >> 3) + x, KD)), z);
#pragma unroll
          for (int y = 0; y < 8; ++y) g2[8 * x + y] += f[8 * x + y] + bd_i * z[y];
        }
#pragma unroll
        for (int x = 0; x < 4; ++x) sts16(Xdvn, tc::kmajor_unit(i, (c0 >> 3) + x, KD), pack8(&g2[8 * x]));
      }
    }
    {
      const float rho = own ? kdot : 0.f;
      if (own) dg_own += qdot - rho;
      const float tot = warp_sum(rho);
      if (lane == 0) red[8 + warp] = tot;  // summed in a fixed order at the end (deterministic)
    }
  }
  (void)ri;
  if (own) {  // the two column halves hold partial sums of the same row
    dgo[hc * C + i] = dg_own;
    dbo[hc * C + i] = db_own;
  }
  tc::fence_before_sync();
  __syncthreads();
  if (ok) {  // dq, dk leave in 64-byte row pieces
    for (int u = tid; u < 64 * 16; u += 256) {
      const int r = urow16(u), c8 = ucol16(u);
      if (r < imax) {
        const uint32_t off = tc::kmajor_unit(r, c8, KD);
        *reinterpret_cast<uint4*>(p.dq + row(r) * KD + c8 * 8) = *reinterpret_cast<const uint4*>(Xv + off);
        *reinterpret_cast<uint4*>(p.dk + row(r) * KD + c8 * 8) = *reinterpret_cast<const uint4*>(Xdvn + off);
      }
    }
  }
  if (tid < 32) {  // dg = reverse cumulative sum of dgam within the chunk: one warp, two rows per lane
    // d/dgam_last: E(gam_last) <dS, S0> (from the first kernel) and the sum of rho over the rows
    float base = p.ls[ci];
    for (int wv = 0; wv < 8; ++wv) base += red[8 + wv];
    const int ra = C - 1 - 2 * tid, rb = ra - 1;
    float a = dgo[ra] + dgo[C + ra] + csw[ra] + csw[C + ra] + csw[2 * C + ra] + csw[3 * C + ra];
    float bq = dgo[rb] + dgo[C + rb] + csw[rb] + csw[C + rb] + csw[2 * C + rb] + csw[3 * C + rb];
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
  if (warp == 0) tc::tmem_dealloc(taddr, 256);
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
  const bool tma = !p.no_tma && make_tma_map_bthd(&maps.k, p.k, p.B, p.T, p.H, KD) &&
                   make_tma_map_bthd(&maps.q, p.q, p.B, p.T, p.H, KD) && make_tma_map_bthd(&maps.v, p.v, p.B, p.T, p.H, KD) &&
                   make_tma_map_bthd(&maps.dO, p.dO, p.B, p.T, p.H, KD);
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
  if (tma) {
    if (bwd_set_smem(gdn_tc_chunk_bwd_state_kernel<true>, kChunkBwdStateSmem) != MXB_OK) return MXB_ERR_CUDA;
    MXB_LAUNCH("gdn_tc_chunk_bwd_state_kernel", st,
               (gdn_tc_chunk_bwd_state_kernel<true><<<dim3(p.n, p.B * p.H), 256, kChunkBwdStateSmem, st>>>(p, maps)));
  } else {
    if (bwd_set_smem(gdn_tc_chunk_bwd_state_kernel<false>, kChunkBwdStateSmem) != MXB_OK) return MXB_ERR_CUDA;
    MXB_LAUNCH("gdn_tc_chunk_bwd_state_kernel", st,
               (gdn_tc_chunk_bwd_state_kernel<false><<<dim3(p.n, p.B * p.H), 256, kChunkBwdStateSmem, st>>>(p, maps)));
  }
  s = check_launch("gdn_tc_chunk_bwd_state_kernel");
  if (s != MXB_OK) return s;
  if (tma) {
    if (bwd_set_smem(gdn_tc_chunk_bwd_kernel<true>, kChunkBwdSmem) != MXB_OK) return MXB_ERR_CUDA;
    MXB_LAUNCH("gdn_tc_chunk_bwd_kernel", st,
               (gdn_tc_chunk_bwd_kernel<true><<<dim3(p.n, p.B * p.H), 256, kChunkBwdSmem, st>>>(p, maps)));
  } else {
    if (bwd_set_smem(gdn_tc_chunk_bwd_kernel<false>, kChunkBwdSmem) != MXB_OK) return MXB_ERR_CUDA;
    MXB_LAUNCH("gdn_tc_chunk_bwd_kernel", st,
               (gdn_tc_chunk_bwd_kernel<false><<<dim3(p.n, p.B * p.H), 256, kChunkBwdSmem, st>>>(p, maps)));
  }
  return check_launch("gdn_tc_chunk_bwd_kernel");
}

}  // namespace mxb
